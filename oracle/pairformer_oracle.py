"""CPU oracle for the Pairformer hot path: TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A plain-PyTorch (CPU, fp32 or fp64) restatement of the reference's stock PyTorch path for
the modules this library accelerates. Only the tests, the smoke check and the benchmark's
CPU-baseline leg may import it; the product never routes through it.

Every function works on a flat ``dict[str, Tensor]`` of parameters that uses the
reference's ``state_dict`` key names (``prefix + "linear_a_p.weight"`` ...), and cites the
reference code it restates (paths relative to the reference project root).

Pinning: `tests/golden/make_golden.py` imports the reference modules themselves, loads the
same seeded parameters and stores their outputs; `tests/test_oracle_golden.py` checks this
file against those stored outputs (and, where the reference tree is present, against the
live modules). Parity of the oracle is therefore pinned to outputs of the reference itself.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

Tensor = torch.Tensor
LN_EPS = 1e-5  # openfold3/core/model/primitives/normalization.py:37


def _ln(x: Tensor, P: dict, prefix: str, c: int) -> Tensor:
    """LayerNorm with optional scale/offset. primitives/normalization.py:33-86."""
    w = P.get(prefix + "weight")
    b = P.get(prefix + "bias")
    return F.layer_norm(x, (c,), w, b, LN_EPS)


def _lin(x: Tensor, P: dict, prefix: str) -> Tensor:
    """Linear without activation. primitives/linear.py:120-138."""
    return F.linear(x, P[prefix + "weight"], P.get(prefix + "bias"))


def triangle_multiplicative_update(z: Tensor, mask: Tensor | None, P: dict, prefix: str,
                                   outgoing: bool) -> Tensor:
    """Returns the update (no residual).

    layers/triangular_multiplicative_update.py:482-503 (forward) and :71-97
    (_combine_projections): a,b = mask * sigmoid(gate) * proj of LN_in(z);
    outgoing x[i,j,c] = sum_k a[i,k,c] b[j,k,c]; incoming x[i,j,c] = sum_k a[k,i,c] b[k,j,c];
    y = sigmoid(linear_g(LN_in z)) * linear_z(LN_out(x)).
    """
    c_z = z.shape[-1]
    if mask is None:
        mask = z.new_ones(z.shape[:-1])
    m = mask.unsqueeze(-1)
    zn = _ln(z, P, prefix + "layer_norm_in.", c_z)
    a = m * torch.sigmoid(_lin(zn, P, prefix + "linear_a_g.")) * _lin(zn, P, prefix + "linear_a_p.")
    b = m * torch.sigmoid(_lin(zn, P, prefix + "linear_b_g.")) * _lin(zn, P, prefix + "linear_b_p.")
    if outgoing:
        x = torch.einsum("...ikc,...jkc->...ijc", a, b)
    else:
        x = torch.einsum("...kic,...kjc->...ijc", a, b)
    x = _ln(x, P, prefix + "layer_norm_out.", x.shape[-1])
    x = _lin(x, P, prefix + "linear_z.")
    g = torch.sigmoid(_lin(zn, P, prefix + "linear_g."))
    return x * g


def attention(q_x: Tensor, kv_x: Tensor, biases: list[Tensor], P: dict, prefix: str,
              no_heads: int) -> Tensor:
    """Gated multi-head attention with additive biases.

    primitives/attention.py:270-310 (_prep_qkv, _wrap_up), :94-135 (_attention):
    q is scaled by 1/sqrt(c_hidden per head) after the projection (bias included);
    softmax over keys of q k^T + sum(biases); output gated by sigmoid(linear_g(q_x)).
    """
    q = _lin(q_x, P, prefix + "linear_q.")
    k = _lin(kv_x, P, prefix + "linear_k.")
    v = _lin(kv_x, P, prefix + "linear_v.")
    H = no_heads
    d = q.shape[-1] // H
    q = q.view(q.shape[:-1] + (H, d)).transpose(-2, -3) / math.sqrt(d)
    k = k.view(k.shape[:-1] + (H, d)).transpose(-2, -3)
    v = v.view(v.shape[:-1] + (H, d)).transpose(-2, -3)
    scores = torch.einsum("...qc,...kc->...qk", q, k)
    for b in biases:
        scores = scores + b
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("...qk,...kc->...qc", p, v).transpose(-2, -3)  # [*, Q, H, d]
    if (prefix + "linear_g.weight") in P:
        g = torch.sigmoid(_lin(q_x, P, prefix + "linear_g."))
        o = o * g.view(g.shape[:-1] + (H, d))
    o = o.reshape(o.shape[:-2] + (H * d,))
    return _lin(o, P, prefix + "linear_o.")


def triangle_attention(x: Tensor, mask: Tensor | None, P: dict, prefix: str, no_heads: int,
                       inf: float = 1e9, starting: bool = True) -> Tensor:
    """Returns the update (no residual). layers/triangular_attention.py:102-167.

    mask bias inf*(mask-1) broadcast over heads and queries; triangle bias
    tb[h, q, k] = linear_z(LN(x))[q, k, h] shared by every row of the leading axis.
    """
    if mask is None:
        mask = x.new_ones(x.shape[:-1])
    if not starting:
        x = x.transpose(-2, -3)
        mask = mask.transpose(-1, -2)
    xn = _ln(x, P, prefix + "layer_norm.", x.shape[-1])
    mask_bias = (inf * (mask - 1))[..., :, None, None, :]
    tb = _lin(xn, P, prefix + "linear_z.")  # [*, I, J, H]
    tb = tb.permute(*range(tb.dim() - 3), -1, -3, -2).unsqueeze(-4)  # [*, 1, H, I, J]
    o = attention(xn, xn, [mask_bias, tb], P, prefix + "mha.", no_heads)
    if not starting:
        o = o.transpose(-2, -3)
    return o


def swiglu_transition(x: Tensor, mask: Tensor | None, P: dict, prefix: str) -> Tensor:
    """Returns the update. layers/transition.py:259-271, primitives/activations.py:57-61."""
    xn = _ln(x, P, prefix + "layer_norm.", x.shape[-1])
    h = F.silu(_lin(xn, P, prefix + "swiglu.linear_a.")) * _lin(xn, P, prefix + "swiglu.linear_b.")
    y = _lin(h, P, prefix + "linear_out.")
    if mask is not None:
        y = y * mask.unsqueeze(-1)
    return y


def pair_block(z: Tensor, pair_mask: Tensor, P: dict, prefix: str, no_heads_pair: int,
               inf: float = 1e9, mask_trans: bool = True) -> Tensor:
    """Returns the updated pair tensor. latent/base_blocks.py:408-480 (forward), :307-406.

    The ending-node layer is a starting-node module applied to z^T with mask^T (:380-404).
    """
    z = z + triangle_multiplicative_update(z, pair_mask, P, prefix + "tri_mul_out.", True)
    z = z + triangle_multiplicative_update(z, pair_mask, P, prefix + "tri_mul_in.", False)
    z = z + triangle_attention(z, pair_mask, P, prefix + "tri_att_start.", no_heads_pair, inf)
    zt = z.transpose(-2, -3)
    zt = zt + triangle_attention(zt, pair_mask.transpose(-1, -2), P, prefix + "tri_att_end.",
                                 no_heads_pair, inf)
    z = zt.transpose(-2, -3)
    z = z + swiglu_transition(z, pair_mask if mask_trans else None, P, prefix + "pair_transition.")
    return z


def ada_ln(a: Tensor, s: Tensor, P: dict, prefix: str) -> Tensor:
    """Adaptive LayerNorm. primitives/normalization.py:126-140."""
    a = F.layer_norm(a, (a.shape[-1],), None, None, LN_EPS)
    s = F.layer_norm(s, (s.shape[-1],), P[prefix + "layer_norm_s.weight"], None, LN_EPS)
    g = torch.sigmoid(_lin(s, P, prefix + "linear_g."))
    return g * a + _lin(s, P, prefix + "linear_s.")


def attention_pair_bias(a: Tensor, z: Tensor, s: Tensor | None, mask: Tensor | None, P: dict,
                        prefix: str, no_heads: int, inf: float = 1e9,
                        use_ada_layer_norm: bool = False) -> Tensor:
    """Returns the update. layers/attention_pair_bias.py:123-227."""
    if use_ada_layer_norm:
        an = ada_ln(a, s, P, prefix + "layer_norm_a.")
    else:
        an = _ln(a, P, prefix + "layer_norm_a.", a.shape[-1])
    if mask is None:
        mask = a.new_ones(a.shape[:-1])
    mask = mask.expand(*a.shape[:-2], -1)
    mask_bias = (inf * (mask - 1))[..., None, None, :]
    zb = _lin(_ln(z, P, prefix + "layer_norm_z.", z.shape[-1]), P, prefix + "linear_z.")
    zb = zb.permute(*range(zb.dim() - 3), -1, -3, -2)  # [*, H, N, N]
    o = attention(an, an, [mask_bias, zb], P, prefix + "mha.", no_heads)
    if use_ada_layer_norm:
        o = torch.sigmoid(_lin(s, P, prefix + "linear_ada_out.")) * o
    return o


def conditioned_transition(a: Tensor, s: Tensor, mask: Tensor | None, P: dict, prefix: str) -> Tensor:
    """Returns the update. layers/transition.py:325-339."""
    an = ada_ln(a, s, P, prefix + "layer_norm.")
    b = F.silu(_lin(an, P, prefix + "swiglu.linear_a.")) * _lin(an, P, prefix + "swiglu.linear_b.")
    y = torch.sigmoid(_lin(s, P, prefix + "linear_g.")) * _lin(b, P, prefix + "linear_out.")
    if mask is not None:
        y = y * mask.unsqueeze(-1)
    return y


def pairformer_block(s: Tensor, z: Tensor, single_mask: Tensor, pair_mask: Tensor, P: dict,
                     prefix: str, no_heads_pair: int, no_heads_pair_bias: int, inf: float = 1e9,
                     mask_trans: bool = True) -> tuple[Tensor, Tensor]:
    """latent/pairformer.py:124-213: pair stack, then the single track on the updated z."""
    z = pair_block(z, pair_mask, P, prefix + "pair_stack.", no_heads_pair, inf, mask_trans)
    s = s + attention_pair_bias(s, z, None, single_mask, P, prefix + "attn_pair_bias.",
                                no_heads_pair_bias, inf, False)
    s = s + swiglu_transition(s, single_mask if mask_trans else None, P, prefix + "single_transition.")
    return s, z


def pairformer_stack(s: Tensor, z: Tensor, single_mask: Tensor, pair_mask: Tensor, P: dict,
                     prefix: str, no_blocks: int, no_heads_pair: int, no_heads_pair_bias: int,
                     inf: float = 1e9, mask_trans: bool = True) -> tuple[Tensor, Tensor]:
    """latent/pairformer.py:398-464."""
    for i in range(no_blocks):
        s, z = pairformer_block(s, z, single_mask, pair_mask, P, f"{prefix}blocks.{i}.",
                                no_heads_pair, no_heads_pair_bias, inf, mask_trans)
    return s, z


def diffusion_transformer_block(a: Tensor, s: Tensor, z: Tensor, mask: Tensor | None, P: dict,
                                prefix: str, no_heads: int, inf: float = 1e9) -> Tensor:
    """layers/diffusion_transformer.py:116-179: a += APB(a, z, s); a += CondTransition(a, s)."""
    a = a + attention_pair_bias(a, z, s, mask, P, prefix + "attention_pair_bias.", no_heads, inf, True)
    a = a + conditioned_transition(a, s, mask, P, prefix + "conditioned_transition.")
    return a


def diffusion_transformer(a: Tensor, s: Tensor, z: Tensor, mask: Tensor | None, P: dict,
                          prefix: str, no_blocks: int, no_heads: int, inf: float = 1e9) -> Tensor:
    """layers/diffusion_transformer.py:263-322."""
    for i in range(no_blocks):
        a = diffusion_transformer_block(a, s, z, mask, P, f"{prefix}blocks.{i}.", no_heads, inf)
    return a
