"""``patch_openfold3()`` against the real reference tree (CPU only; skipped where the tree is not available).

Checks what a maintainer relies on when swapping the classes in: the reference's own model code then constructs
this package's classes, and ``state_dict``s travel both ways with ``strict=True`` (same parameter names and shapes).
The reference tree is looked for in $OPENFOLD3_SRC, else in a directory ``reference`` next to this repository.
"""

import os
import sys
import types
from pathlib import Path

import pytest
import torch

import cases

ROOT = Path(__file__).resolve().parent.parent


def _reference_tree():
    cand = [os.environ.get("OPENFOLD3_SRC"), str(ROOT.parent / "reference")]
    for c in cand:
        if c and (Path(c) / "openfold3" / "core" / "model" / "latent" / "pairformer.py").exists():
            return Path(c)
    return None


@pytest.fixture(scope="module")
def reference():
    tree = _reference_tree()
    if tree is None:
        pytest.skip("the reference's source tree is not available here")
    # stand-ins for three optional packages that take no part in the arithmetic (as in tests/golden/make_golden.py)
    ml = types.ModuleType("ml_collections")

    class ConfigDict(dict):
        def __init__(self, d=None, **kw):
            super().__init__()
            for k, v in dict(d or {}, **kw).items():
                self[k] = ConfigDict(v) if isinstance(v, dict) and not isinstance(v, ConfigDict) else v

        def __getattr__(self, k):
            try:
                return self[k]
            except KeyError:
                raise AttributeError(k) from None

        def __setattr__(self, k, v):
            self[k] = v

    ml.ConfigDict = ConfigDict
    added = {}
    for name, mod in (("ml_collections", ml), ("biotite", types.ModuleType("biotite")),
                      ("biotite.structure", types.ModuleType("biotite.structure")), ("gemmi", types.ModuleType("gemmi"))):
        if name not in sys.modules:
            added[name] = mod
            sys.modules[name] = mod
    sys.modules["biotite.structure"].AtomArray = getattr(sys.modules["biotite.structure"], "AtomArray", type("AtomArray", (), {}))
    sys.modules["biotite"].structure = sys.modules["biotite.structure"]
    if not hasattr(sys.modules["gemmi"], "__version__"):
        sys.modules["gemmi"].__version__ = "0.0.0"
    sys.path.insert(0, str(tree))
    import openfold3.core.model.latent.base_blocks as bb
    import openfold3.core.model.latent.pairformer as pf
    import openfold3.core.model.layers.diffusion_transformer as dt
    yield types.SimpleNamespace(pf=pf, bb=bb, dt=dt)
    cases.pkg.unpatch_openfold3()
    sys.path.remove(str(tree))


PF_KW = dict(transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False, inf=1e9)


def test_state_dicts_travel_both_ways_and_the_swap_reaches_importers(reference):
    pkg = cases.pkg
    ref_stack = reference.pf.PairFormerStack(**cases.OF3, **PF_KW, no_blocks=2, blocks_per_ckpt=None)
    ours = pkg.PairFormerStack(**cases.OF3, **PF_KW, no_blocks=2, blocks_per_ckpt=None)
    sd_ref, sd_ours = ref_stack.state_dict(), ours.state_dict()
    assert list(sd_ref) == list(sd_ours)
    assert all(sd_ref[k].shape == sd_ours[k].shape for k in sd_ref)
    ours.load_state_dict(sd_ref, strict=True)          # a reference checkpoint into the drop-in
    ref_stack.load_state_dict(ours.state_dict(), strict=True)   # and back
    diff_kw = dict(use_ada_layer_norm=True, n_query=None, n_key=None, inf=1e9)
    ref_dt = reference.dt.DiffusionTransformer(**cases.DIFF, **diff_kw, no_blocks=1)
    ours_dt = pkg.DiffusionTransformer(**cases.DIFF, **diff_kw, no_blocks=1)
    ours_dt.load_state_dict(ref_dt.state_dict(), strict=True)
    ref_dt.load_state_dict(ours_dt.state_dict(), strict=True)

    orig_block = reference.bb.PairBlock
    replaced = pkg.patch_openfold3()
    assert {"PairFormerStack", "PairFormerBlock", "PairBlock", "DiffusionTransformer"} <= set(replaced)
    assert reference.pf.PairFormerStack is pkg.PairFormerStack
    assert reference.bb.PairBlock is pkg.PairBlock
    assert reference.dt.DiffusionTransformerBlock is pkg.DiffusionTransformerBlock
    # a module that imported PairBlock by name (the Pairformer module does) now sees the drop-in as well
    assert reference.pf.PairBlock is pkg.PairBlock
    # the reference's own construction path now builds drop-in modules, and a reference checkpoint still loads
    built = reference.pf.PairFormerStack(**cases.OF3, **PF_KW, no_blocks=2, blocks_per_ckpt=None)
    assert isinstance(built, pkg.PairFormerStack) and isinstance(built.blocks[0].pair_stack, pkg.PairBlock)
    built.load_state_dict(sd_ref, strict=True)
    assert pkg.patch_openfold3() == {}                  # idempotent
    pkg.unpatch_openfold3()
    assert reference.bb.PairBlock is orig_block and reference.pf.PairBlock is orig_block


def test_patched_forward_has_no_cpu_fallback(reference):
    """The swapped-in classes run CUDA kernels only: a CPU tensor raises instead of silently computing elsewhere."""
    pkg = cases.pkg
    blk = pkg.PairBlock(**cases.PAIR, **PF_KW).eval()
    with pytest.raises(Exception):
        with torch.no_grad():
            blk(torch.zeros(1, 8, 8, 128), torch.ones(1, 8, 8))
