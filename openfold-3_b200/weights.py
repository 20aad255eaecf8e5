"""Seeded random parameters with the reference's ``state_dict`` key names and shapes.

There are no trained weights without network access, and the reference's own initialisers
draw from an unseeded numpy RNG (openfold3/core/model/primitives/initialization.py:48-59)
and zero the gate / output projections (core/config/default_linear_init_config.py), which
would make a fresh block the identity. These helpers draw every tensor from one seeded
``torch.Generator`` instead: fan-in scaled normals for the "default"/"relu" layers and
``N(0, final_std)`` (or fan-in scaled, when ``final_std`` is None) for the layers the
reference zero-initialises, so that every code path contributes to the output.
"""

from __future__ import annotations

import math

import torch


class _Draw:
    def __init__(self, seed: int, final_std: float | None, dtype=torch.float32):
        self.g = torch.Generator(device="cpu")
        self.g.manual_seed(seed)
        self.final_std = final_std
        self.dtype = dtype

    def lecun(self, out_dim, in_dim):
        return (torch.randn(out_dim, in_dim, generator=self.g) / math.sqrt(in_dim)).to(self.dtype)

    def he(self, out_dim, in_dim):
        return (torch.randn(out_dim, in_dim, generator=self.g) * math.sqrt(2.0 / in_dim)).to(self.dtype)

    def final(self, out_dim, in_dim):
        if self.final_std is None:
            return self.lecun(out_dim, in_dim)
        return (torch.randn(out_dim, in_dim, generator=self.g) * self.final_std).to(self.dtype)

    def ln_weight(self, c):
        return (1.0 + 0.1 * torch.randn(c, generator=self.g)).to(self.dtype)

    def ln_bias(self, c):
        return (0.1 * torch.randn(c, generator=self.g)).to(self.dtype)

    def bias(self, c, mean=0.0):
        return (mean + 0.1 * torch.randn(c, generator=self.g)).to(self.dtype)


def _tri_mul(P, p, d: _Draw, c_z, c_h):
    P[p + "linear_g.weight"] = d.final(c_z, c_z)
    P[p + "linear_z.weight"] = d.final(c_z, c_h)
    P[p + "layer_norm_in.weight"] = d.ln_weight(c_z)
    P[p + "layer_norm_in.bias"] = d.ln_bias(c_z)
    P[p + "layer_norm_out.weight"] = d.ln_weight(c_h)
    P[p + "layer_norm_out.bias"] = d.ln_bias(c_h)
    P[p + "linear_a_p.weight"] = d.lecun(c_h, c_z)
    P[p + "linear_a_g.weight"] = d.final(c_h, c_z)
    P[p + "linear_b_p.weight"] = d.lecun(c_h, c_z)
    P[p + "linear_b_g.weight"] = d.final(c_h, c_z)


def _mha(P, p, d: _Draw, c_q, c_hidden, H, q_bias: bool, o_final: bool = True):
    P[p + "linear_q.weight"] = d.lecun(c_hidden * H, c_q)
    if q_bias:
        P[p + "linear_q.bias"] = d.bias(c_hidden * H)
    P[p + "linear_k.weight"] = d.lecun(c_hidden * H, c_q)
    P[p + "linear_v.weight"] = d.lecun(c_hidden * H, c_q)
    P[p + "linear_o.weight"] = d.final(c_q, c_hidden * H) if o_final else d.lecun(c_q, c_hidden * H)
    P[p + "linear_g.weight"] = d.final(c_hidden * H, c_q)


def _tri_att(P, p, d: _Draw, c_z, c_hidden, H):
    P[p + "layer_norm.weight"] = d.ln_weight(c_z)
    P[p + "layer_norm.bias"] = d.ln_bias(c_z)
    P[p + "linear_z.weight"] = d.lecun(H, c_z)
    _mha(P, p + "mha.", d, c_z, c_hidden, H, q_bias=False)


def _swiglu_transition(P, p, d: _Draw, c, n):
    P[p + "layer_norm.weight"] = d.ln_weight(c)
    P[p + "layer_norm.bias"] = d.ln_bias(c)
    P[p + "swiglu.linear_a.weight"] = d.he(n * c, c)
    P[p + "swiglu.linear_b.weight"] = d.he(n * c, c)
    P[p + "linear_out.weight"] = d.final(c, n * c)


def pair_block_params(seed: int, c_z=128, c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=4,
                      transition_n=4, final_std: float | None = 0.02, prefix: str = "",
                      _draw: _Draw | None = None) -> dict[str, torch.Tensor]:
    """Parameters of one ``PairBlock`` (openfold3/core/model/latent/base_blocks.py:219-306)."""
    d = _draw or _Draw(seed, final_std)
    P: dict[str, torch.Tensor] = {}
    _tri_mul(P, prefix + "tri_mul_out.", d, c_z, c_hidden_mul)
    _tri_mul(P, prefix + "tri_mul_in.", d, c_z, c_hidden_mul)
    _tri_att(P, prefix + "tri_att_start.", d, c_z, c_hidden_pair_att, no_heads_pair)
    _tri_att(P, prefix + "tri_att_end.", d, c_z, c_hidden_pair_att, no_heads_pair)
    _swiglu_transition(P, prefix + "pair_transition.", d, c_z, transition_n)
    return P


def pairformer_block_params(seed: int, c_s=384, c_z=128, c_hidden_pair_bias=24, no_heads_pair_bias=16,
                            c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=4, transition_n=4,
                            final_std: float | None = 0.02, prefix: str = "",
                            _draw: _Draw | None = None) -> dict[str, torch.Tensor]:
    """Parameters of one ``PairFormerBlock`` (openfold3/core/model/latent/pairformer.py:38-122)."""
    d = _draw or _Draw(seed, final_std)
    P = pair_block_params(seed, c_z, c_hidden_mul, c_hidden_pair_att, no_heads_pair, transition_n,
                          final_std, prefix + "pair_stack.", d)
    p = prefix + "attn_pair_bias."
    P[p + "layer_norm_a.weight"] = d.ln_weight(c_s)
    P[p + "layer_norm_a.bias"] = d.ln_bias(c_s)
    P[p + "layer_norm_z.weight"] = d.ln_weight(c_z)
    P[p + "layer_norm_z.bias"] = d.ln_bias(c_z)
    P[p + "linear_z.weight"] = d.lecun(no_heads_pair_bias, c_z)
    _mha(P, p + "mha.", d, c_s, c_hidden_pair_bias, no_heads_pair_bias, q_bias=True)
    _swiglu_transition(P, prefix + "single_transition.", d, c_s, transition_n)
    return P


def pair_stack_params(seed: int, no_blocks: int, prefix: str = "", **kw) -> dict[str, torch.Tensor]:
    """Parameters of a ``PairStack`` (keys ``blocks.{i}.…``)."""
    P: dict[str, torch.Tensor] = {}
    for i in range(no_blocks):
        P.update(pair_block_params(seed * 1000 + i, prefix=f"{prefix}blocks.{i}.", **kw))
    return P


def pairformer_stack_params(seed: int, no_blocks: int, prefix: str = "", **kw) -> dict[str, torch.Tensor]:
    """Parameters of a ``PairFormerStack`` (keys ``blocks.{i}.…``)."""
    P: dict[str, torch.Tensor] = {}
    for i in range(no_blocks):
        P.update(pairformer_block_params(seed * 1000 + i, prefix=f"{prefix}blocks.{i}.", **kw))
    return P


def _ada_ln(P, p, d: _Draw, c_a, c_s):
    P[p + "layer_norm_s.weight"] = d.ln_weight(c_s)
    P[p + "linear_g.weight"] = d.final(c_a, c_s)
    P[p + "linear_g.bias"] = d.bias(c_a)
    P[p + "linear_s.weight"] = d.final(c_a, c_s)


def diffusion_block_params(seed: int, c_a=768, c_s=384, c_z=128, c_hidden=48, no_heads=16,
                           n_transition=2, final_std: float | None = 0.02, prefix: str = "",
                           _draw: _Draw | None = None) -> dict[str, torch.Tensor]:
    """Parameters of one ``DiffusionTransformerBlock`` with adaptive LayerNorm
    (openfold3/core/model/layers/diffusion_transformer.py:30-114)."""
    d = _draw or _Draw(seed, final_std)
    P: dict[str, torch.Tensor] = {}
    p = prefix + "attention_pair_bias."
    _ada_ln(P, p + "layer_norm_a.", d, c_a, c_s)
    P[p + "linear_ada_out.weight"] = d.final(c_a, c_s)
    P[p + "linear_ada_out.bias"] = d.bias(c_a, -2.0)
    P[p + "layer_norm_z.weight"] = d.ln_weight(c_z)
    P[p + "linear_z.weight"] = d.lecun(no_heads, c_z)
    _mha(P, p + "mha.", d, c_a, c_hidden, no_heads, q_bias=True, o_final=False)
    p = prefix + "conditioned_transition."
    _ada_ln(P, p + "layer_norm.", d, c_a, c_s)
    P[p + "swiglu.linear_a.weight"] = d.he(n_transition * c_a, c_a)
    P[p + "swiglu.linear_b.weight"] = d.he(n_transition * c_a, c_a)
    P[p + "linear_g.weight"] = d.final(c_a, c_s)
    P[p + "linear_g.bias"] = d.bias(c_a, -2.0)
    P[p + "linear_out.weight"] = d.lecun(c_a, n_transition * c_a)
    return P


def diffusion_stack_params(seed: int, no_blocks: int, prefix: str = "", **kw) -> dict[str, torch.Tensor]:
    P: dict[str, torch.Tensor] = {}
    for i in range(no_blocks):
        P.update(diffusion_block_params(seed * 1000 + i, prefix=f"{prefix}blocks.{i}.", **kw))
    return P
