"""Per-layer ``{bias, init}`` tables for the modules on the Pairformer hot path.

Same keys and values as the reference tables the layer constructors read
(openfold3/core/config/default_linear_init_config.py:27-64 primitives, :70-119 layers,
:157-204 transitions and diffusion transformer, pair / pairformer blocks), restated as plain
attribute dictionaries so the constructors accept either these or the reference's
``ml_collections.ConfigDict`` objects.
"""

from __future__ import annotations


class AttrDict(dict):
    """dict with attribute access, nested dicts wrapped recursively."""

    def __init__(self, d=None, **kw):
        super().__init__()
        for k, v in dict(d or {}, **kw).items():
            self[k] = AttrDict(v) if isinstance(v, dict) and not isinstance(v, AttrDict) else v

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None

    def __setattr__(self, k, v):
        self[k] = v


def _lin(bias, init):
    return {"bias": bias, "init": init}


swiglu_init = AttrDict(linear_a=_lin(False, "relu"), linear_b=_lin(False, "relu"))
ada_ln_init = AttrDict(linear_g=_lin(True, "final"), linear_s=_lin(False, "final"))


def _mha(q_bias, o_init):
    return dict(linear_q=_lin(q_bias, "default"), linear_k=_lin(False, "default"),
                linear_v=_lin(False, "default"), linear_g=_lin(False, "gating"),
                linear_o=_lin(False, o_init))


mha_init = AttrDict(_mha(False, "final"))
att_pair_bias_mha_init = AttrDict(_mha(True, "final"))
att_pair_bias_mha_ada_init = AttrDict(_mha(True, "default"))
tri_att_init = AttrDict(linear_z=_lin(False, "default"), mha=mha_init)
att_pair_bias_init = AttrDict(linear_z=_lin(False, "default"), layer_norm_z={"create_offset": True},
                              mha=att_pair_bias_mha_init)
diffusion_att_pair_bias_init = AttrDict(
    ada_ln=ada_ln_init, linear_ada_out=_lin(True, "gating_ada_zero"), linear_z=_lin(False, "default"),
    layer_norm_z={"create_offset": False}, mha=att_pair_bias_mha_ada_init)
tri_mul_init = AttrDict(linear_a_p=_lin(False, "default"), linear_a_g=_lin(False, "final"),
                        linear_b_p=_lin(False, "default"), linear_b_g=_lin(False, "final"),
                        linear_g=_lin(False, "final"), linear_z=_lin(False, "final"))
swiglu_transition_init = AttrDict(swiglu=swiglu_init, linear_out=_lin(False, "final"))
cond_transition_init = AttrDict(ada_ln=ada_ln_init, swiglu=swiglu_init,
                                linear_g=_lin(True, "gating_ada_zero"), linear_out=_lin(False, "default"))
diffusion_transformer_init = AttrDict(att_pair_bias=diffusion_att_pair_bias_init,
                                      cond_transition=cond_transition_init)
pair_block_init = AttrDict(tri_mul=tri_mul_init, tri_att=tri_att_init,
                           pair_transition={"swiglu": swiglu_transition_init})
pairformer_init = AttrDict(pair_block=pair_block_init, att_pair_bias=att_pair_bias_init,
                           transition=swiglu_transition_init)
