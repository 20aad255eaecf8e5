"""``patch_openfold3()``: swaps the drop-in classes into the reference's own namespaces.

After the call, model code of the reference that builds ``PairFormerStack(**config.architecture.pairformer)``,
``PairBlock(...)`` or ``DiffusionTransformer(...)`` (openfold3/projects/of3_all_atom/model.py:291-302,
openfold3/core/model/latent/template_module.py:148-189, openfold3/core/model/structure/diffusion_module.py:239-249)
constructs the classes of this package instead: same constructor arguments, same parameter names, same forward
keywords, so checkpoints load with ``strict=True``. Every module of the reference that imported one of the classes
by name (``from ... import PairBlock``) is patched too, because such a module holds its own reference to the class.
"""

from __future__ import annotations

import importlib
import sys

from . import modules as _m

# reference module -> class names defined there that this package replaces
_TARGETS = {
    "openfold3.core.model.latent.pairformer": ("PairFormerStack", "PairFormerBlock"),
    "openfold3.core.model.latent.base_blocks": ("PairBlock",),
    "openfold3.core.model.layers.triangular_multiplicative_update": (
        "TriangleMultiplicativeUpdate", "TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming"),
    "openfold3.core.model.layers.triangular_attention": (
        "TriangleAttention", "TriangleAttentionStartingNode", "TriangleAttentionEndingNode"),
    "openfold3.core.model.layers.transition": ("SwiGLUTransition", "ConditionedTransitionBlock"),
    "openfold3.core.model.layers.attention_pair_bias": ("AttentionPairBias",),
    "openfold3.core.model.layers.diffusion_transformer": ("DiffusionTransformer", "DiffusionTransformerBlock"),
}

_originals: dict[tuple[str, str], type] = {}


def patch_openfold3(only: tuple[str, ...] | None = None) -> dict[str, type]:
    """Replaces the reference's hot-path classes by this package's. ``only``: restrict to these class names.
    Returns {class name: original class}. Needs ``openfold3`` importable; idempotent."""
    replaced: dict[str, type] = {}
    for mod_name, names in _TARGETS.items():
        mod = importlib.import_module(mod_name)
        for name in names:
            if only is not None and name not in only:
                continue
            ours = getattr(_m, name)
            orig = getattr(mod, name)
            if orig is ours:
                continue
            _originals.setdefault((mod_name, name), orig)
            replaced[name] = orig
            # the defining module and every loaded openfold3 module that imported the class by name
            for other_name, other in list(sys.modules.items()):
                if other is None or not (other_name == "openfold3" or other_name.startswith("openfold3.")):
                    continue
                for attr, val in list(vars(other).items()):
                    if val is orig:
                        setattr(other, attr, ours)
    return replaced


def unpatch_openfold3() -> None:
    """Puts the reference's own classes back (everywhere ``patch_openfold3`` replaced them)."""
    for (mod_name, name), orig in list(_originals.items()):
        ours = getattr(_m, name)
        for other_name, other in list(sys.modules.items()):
            if other is None or not (other_name == "openfold3" or other_name.startswith("openfold3.")):
                continue
            for attr, val in list(vars(other).items()):
                if val is ours:
                    setattr(other, attr, orig)
        del _originals[(mod_name, name)]
