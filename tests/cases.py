"""Seeded parity cases shared by the golden-vector generator, the oracle tests (CPU) and
the GPU parity tests.

A case is a function returning ``(params, inputs, run_oracle)`` where ``params`` uses the
reference's state_dict key names, ``inputs`` is a dict of CPU fp32 tensors, and
``run_oracle(params, inputs)`` evaluates the CPU oracle and returns a dict of named outputs.
Inputs and weights are regenerated from seeds (same torch build here and on the GPU box), so
the golden files only hold the reference outputs.

Shapes follow the reference's own tests where they exist (openfold3/tests/config.py:17-41:
batch 2, n_res 22; openfold3/tests/test_kernels.py: random 0/1 masks, non outer-product pair
masks, re-drawn zero-initialised weights).
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from __graft_entry__ import load_package  # noqa: E402
from oracle import pairformer_oracle as oracle  # noqa: E402

pkg = load_package()
W = pkg.weights

OF3 = dict(c_s=384, c_z=128, c_hidden_pair_bias=24, no_heads_pair_bias=16, c_hidden_mul=128,
           c_hidden_pair_att=32, no_heads_pair=4, transition_n=4)
PAIR = dict(c_z=128, c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=4, transition_n=4)
DIFF = dict(c_a=768, c_s=384, c_z=128, c_hidden=48, no_heads=16, n_transition=2)


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def rand_mask(shape, g, p_keep=0.8):
    return (torch.rand(shape, generator=g) < p_keep).float()


def token_pair_mask(single_mask):
    return single_mask[..., :, None] * single_mask[..., None, :]


# ----------------------------------------------------------------------------- cases
def block_n64():
    """One PairFormerBlock of the OpenFold3 trunk widths, N=64, all-ones masks, N(0, 0.02) for zero-inits."""
    N = 64
    g = _gen(100)
    inputs = dict(s=torch.randn(1, N, 384, generator=g), z=torch.randn(1, N, N, 128, generator=g),
                  single_mask=torch.ones(1, N), pair_mask=torch.ones(1, N, N))
    P = W.pairformer_block_params(seed=11, **OF3)

    def run(P, x):
        s, z = oracle.pairformer_block(x["s"], x["z"], x["single_mask"], x["pair_mask"], P, "", 4, 16)
        return dict(s=s, z=z)

    return P, inputs, run


def block_n40_padded():
    """PairFormerBlock with the last tokens padded (pair mask = outer product), fan-in scaled weights."""
    N = 40
    g = _gen(101)
    sm = torch.ones(1, N)
    sm[:, -7:] = 0
    inputs = dict(s=torch.randn(1, N, 384, generator=g), z=torch.randn(1, N, N, 128, generator=g),
                  single_mask=sm, pair_mask=token_pair_mask(sm))
    P = W.pairformer_block_params(seed=12, final_std=None, **OF3)

    def run(P, x):
        s, z = oracle.pairformer_block(x["s"], x["z"], x["single_mask"], x["pair_mask"], P, "", 4, 16)
        return dict(s=s, z=z)

    return P, inputs, run


def pair_taps_n24():
    """PairBlock, batch 2, N=24, random non-outer-product pair mask; output after every sub-layer."""
    N = 24
    g = _gen(102)
    inputs = dict(z=torch.randn(2, N, N, 128, generator=g), pair_mask=rand_mask((2, N, N), g))
    P = W.pair_block_params(seed=13, final_std=None, **PAIR)

    def run(P, x):
        z, m = x["z"], x["pair_mask"]
        out = {}
        z = z + oracle.triangle_multiplicative_update(z, m, P, "tri_mul_out.", True)
        out["after_tri_mul_out"] = z
        z = z + oracle.triangle_multiplicative_update(z, m, P, "tri_mul_in.", False)
        out["after_tri_mul_in"] = z
        z = z + oracle.triangle_attention(z, m, P, "tri_att_start.", 4)
        out["after_tri_att_start"] = z
        z = z + oracle.triangle_attention(z, m, P, "tri_att_end.", 4, starting=False)
        out["after_tri_att_end"] = z
        z = z + oracle.swiglu_transition(z, m, P, "pair_transition.")
        out["after_pair_transition"] = z
        return out

    return P, inputs, run


def trimul_n22_b2():
    """Triangle updates alone (updates, no residual), batch 2, N=22 (reference test shape)."""
    N = 22
    g = _gen(103)
    inputs = dict(z=torch.randn(2, N, N, 128, generator=g), mask=rand_mask((2, N, N), g))
    P = W.pair_block_params(seed=14, final_std=None, **PAIR)

    def run(P, x):
        return dict(outgoing=oracle.triangle_multiplicative_update(x["z"], x["mask"], P, "tri_mul_out.", True),
                    incoming=oracle.triangle_multiplicative_update(x["z"], x["mask"], P, "tri_mul_in.", False))

    return P, inputs, run


def triattn_n33_masked_rows():
    """Triangle attention start/end with a random mask that has fully masked rows and columns
    (uniform-softmax rows of the -inf*(1-mask) bias)."""
    N = 33
    g = _gen(104)
    m = rand_mask((1, N, N), g, 0.7)
    m[:, 5, :] = 0
    m[:, :, 9] = 0
    inputs = dict(z=torch.randn(1, N, N, 128, generator=g), mask=m)
    P = W.pair_block_params(seed=15, final_std=None, **PAIR)

    def run(P, x):
        return dict(start=oracle.triangle_attention(x["z"], x["mask"], P, "tri_att_start.", 4),
                    end=oracle.triangle_attention(x["z"], x["mask"], P, "tri_att_end.", 4, starting=False))

    return P, inputs, run


def pair_odd_dims():
    """PairBlock with the odd widths of the reference's shape tests
    (openfold3/tests/test_pairformer.py:24-75: c_hidden_mul 19, 7 heads x 14), c_z 20, N 11."""
    N = 11
    g = _gen(105)
    dims = dict(c_z=20, c_hidden_mul=19, c_hidden_pair_att=14, no_heads_pair=7, transition_n=2)
    inputs = dict(z=torch.randn(2, N, N, 20, generator=g), pair_mask=rand_mask((2, N, N), g))
    P = W.pair_block_params(seed=16, final_std=None, **dims)

    def run(P, x):
        return dict(z=oracle.pair_block(x["z"], x["pair_mask"], P, "", 7))

    return P, inputs, run


def single_track_n50():
    """Single track alone: attention with pair bias + single transition, batch 2, random token mask."""
    N = 50
    g = _gen(106)
    inputs = dict(s=torch.randn(2, N, 384, generator=g), z=torch.randn(2, N, N, 128, generator=g),
                  single_mask=rand_mask((2, N), g))
    P = W.pairformer_block_params(seed=17, final_std=None, **OF3)

    def run(P, x):
        upd = oracle.attention_pair_bias(x["s"], x["z"], None, x["single_mask"], P, "attn_pair_bias.", 16)
        s = x["s"] + upd
        s2 = s + oracle.swiglu_transition(s, x["single_mask"], P, "single_transition.")
        return dict(attn_update=upd, s=s2)

    return P, inputs, run


def stack2_n20():
    """Two-block PairFormerStack, random single mask, random (non outer-product) pair mask, as in
    openfold3/tests/test_kernels.py:387-554."""
    N = 20
    g = _gen(107)
    inputs = dict(s=torch.randn(1, N, 384, generator=g), z=torch.randn(1, N, N, 128, generator=g),
                  single_mask=rand_mask((1, N), g), pair_mask=rand_mask((1, N, N), g))
    P = W.pairformer_stack_params(seed=18, no_blocks=2, final_std=None, **OF3)

    def run(P, x):
        s, z = oracle.pairformer_stack(x["s"], x["z"], x["single_mask"], x["pair_mask"], P, "", 2, 4, 16)
        return dict(s=s, z=z)

    return P, inputs, run


def diffusion_block_n24():
    """One DiffusionTransformerBlock, 3 samples sharing one pair tensor: a [1,3,N,768], s [1,3,N,384],
    z [1,1,N,N,128], mask [1,1,N] (shapes of openfold3/tests/test_kernels.py:556-650)."""
    N = 24
    g = _gen(108)
    m = torch.ones(1, 1, N)
    m[..., -3:] = 0
    inputs = dict(a=torch.randn(1, 3, N, 768, generator=g), s=torch.randn(1, 3, N, 384, generator=g),
                  z=torch.randn(1, 1, N, N, 128, generator=g), mask=m)
    P = W.diffusion_block_params(seed=19, final_std=None, **DIFF)

    def run(P, x):
        upd = oracle.attention_pair_bias(x["a"], x["z"], x["s"], x["mask"], P, "attention_pair_bias.", 16,
                                         use_ada_layer_norm=True)
        a = oracle.diffusion_transformer_block(x["a"], x["s"], x["z"], x["mask"], P, "", 16)
        return dict(attn_update=upd, a=a)

    return P, inputs, run


def diffusion_stack2_n16():
    """Two-block DiffusionTransformer, 2 samples, N(0, 0.02) for the zero-initialised layers."""
    N = 16
    g = _gen(109)
    inputs = dict(a=torch.randn(1, 2, N, 768, generator=g), s=torch.randn(1, 2, N, 384, generator=g),
                  z=torch.randn(1, 1, N, N, 128, generator=g), mask=torch.ones(1, 1, N))
    P = W.diffusion_stack_params(seed=20, no_blocks=2, **DIFF)

    def run(P, x):
        return dict(a=oracle.diffusion_transformer(x["a"], x["s"], x["z"], x["mask"], P, "", 2, 16))

    return P, inputs, run


DEPTHS = (1, 4, 48)


def depth_curve_n64():
    """A 48-block PairFormerStack at N=64 (one padded token), tapped after 1, 4 and 48 blocks: how the bf16 error
    grows with depth. Not a golden case (no stored outputs): the oracle is evaluated where the test runs."""
    N = 64
    g = _gen(110)
    sm = torch.ones(1, N)
    sm[:, -1] = 0
    inputs = dict(s=torch.randn(1, N, 384, generator=g), z=torch.randn(1, N, N, 128, generator=g),
                  single_mask=sm, pair_mask=token_pair_mask(sm))
    P = W.pairformer_stack_params(seed=21, no_blocks=max(DEPTHS), **OF3)

    def run(P, x):
        s, z = x["s"], x["z"]
        out = {}
        for i in range(max(DEPTHS)):
            s, z = oracle.pairformer_block(s, z, x["single_mask"], x["pair_mask"], P, f"blocks.{i}.", 4, 16)
            if i + 1 in DEPTHS:
                out[f"s@{i + 1}"], out[f"z@{i + 1}"] = s, z
        return out

    return P, inputs, run


def run_depth_curve(stack, x: dict) -> dict:
    """Taps a PairFormerStack-like module (``.blocks``) after the depths of ``DEPTHS``."""
    s, z = x["s"], x["z"]
    out = {}
    with torch.no_grad():
        for i, blk in enumerate(stack.blocks):
            s, z = blk(s, z, x["single_mask"], x["pair_mask"])
            if i + 1 in DEPTHS:
                out[f"s@{i + 1}"], out[f"z@{i + 1}"] = s.clone(), z.clone()
    return out


CASES = {f.__name__: f for f in (
    block_n64, block_n40_padded, pair_taps_n24, trimul_n22_b2, triattn_n33_masked_rows, pair_odd_dims,
    single_track_n50, stack2_n20, diffusion_block_n24, diffusion_stack2_n16)}


def rel_err(got: torch.Tensor, ref: torch.Tensor, where: torch.Tensor | None = None) -> float:
    """max |got - ref| / RMS(ref), optionally restricted to positions where ``where`` is true."""
    got, ref = got.double(), ref.double()
    if where is not None:
        got, ref = got[where], ref[where]
    return float((got - ref).abs().max() / ref.pow(2).mean().sqrt())


def rms_err(got: torch.Tensor, ref: torch.Tensor, where: torch.Tensor | None = None) -> float:
    """RMS(got - ref) / RMS(ref): the error of the whole tensor, not of its single worst element."""
    got, ref = got.double(), ref.double()
    if where is not None:
        got, ref = got[where], ref[where]
    return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


# ----------------------------------------------------------------------------- drop-in runners
_PF_KW = dict(transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False, inf=1e9)
_DIFF_KW = dict(use_ada_layer_norm=True, n_query=None, n_key=None, inf=1e9)


def _load(mod, P, device, dtype):
    mod.load_state_dict(P, strict=True)
    return mod.to(device=device, dtype=dtype).eval()


def run_dropin(name: str, P: dict, x: dict, device, dtype) -> dict:
    """Evaluates case ``name`` with the drop-in modules on ``device`` in ``dtype``; mirrors what
    tests/golden/make_golden.py does with the reference modules."""
    x = {k: v.to(device=device, dtype=dtype) for k, v in x.items()}
    with torch.no_grad():
        if name in ("block_n64", "block_n40_padded"):
            blk = _load(pkg.PairFormerBlock(**OF3, **_PF_KW), P, device, dtype)
            s, z = blk(x["s"], x["z"], x["single_mask"], x["pair_mask"])
            return dict(s=s, z=z)
        if name == "pair_taps_n24":
            blk = _load(pkg.PairBlock(**PAIR, **_PF_KW), P, device, dtype)
            z, m = x["z"], x["pair_mask"]
            out = {}
            z = z + blk.tri_mul_out(z, mask=m)
            out["after_tri_mul_out"] = z
            z = z + blk.tri_mul_in(z, mask=m)
            out["after_tri_mul_in"] = z
            z = z + blk.tri_att_start(z, mask=m)
            out["after_tri_att_start"] = z
            zt = z.transpose(-2, -3)
            zt = zt + blk.tri_att_end(zt, mask=m.transpose(-1, -2))
            z = zt.transpose(-2, -3).contiguous()
            out["after_tri_att_end"] = z
            z = z + blk.pair_transition(z, mask=m)
            out["after_pair_transition"] = z
            # the block's own (in-place, transposition-free) forward must give the same result
            out["block_forward"] = blk(x["z"], m)
            out["block_forward_inplace"] = blk(x["z"].clone(), m, inplace_safe=True)
            return out
        if name == "trimul_n22_b2":
            blk = _load(pkg.PairBlock(**PAIR, **_PF_KW), P, device, dtype)
            return dict(outgoing=blk.tri_mul_out(x["z"], mask=x["mask"]),
                        incoming=blk.tri_mul_in(x["z"], mask=x["mask"]))
        if name == "triattn_n33_masked_rows":
            blk = _load(pkg.PairBlock(**PAIR, **_PF_KW), P, device, dtype)
            end_mod = pkg.TriangleAttentionEndingNode(128, 32, 4, inf=1e9)
            end_mod.load_state_dict(blk.tri_att_end.state_dict())
            end_mod = end_mod.to(device=device, dtype=dtype).eval()
            return dict(start=blk.tri_att_start(x["z"], mask=x["mask"]), end=end_mod(x["z"], mask=x["mask"]))
        if name == "pair_odd_dims":
            dims = dict(c_z=20, c_hidden_mul=19, c_hidden_pair_att=14, no_heads_pair=7, transition_n=2)
            blk = _load(pkg.PairBlock(**dims, **_PF_KW), P, device, dtype)
            return dict(z=blk(x["z"], x["pair_mask"]))
        if name == "single_track_n50":
            blk = _load(pkg.PairFormerBlock(**OF3, **_PF_KW), P, device, dtype)
            upd = blk.attn_pair_bias(a=x["s"], z=x["z"], s=None, mask=x["single_mask"])
            s = x["s"] + upd
            s2 = s + blk.single_transition(s, mask=x["single_mask"])
            return dict(attn_update=upd, s=s2)
        if name == "stack2_n20":
            st = _load(pkg.PairFormerStack(**OF3, **_PF_KW, no_blocks=2, blocks_per_ckpt=None), P, device, dtype)
            s, z = st(x["s"], x["z"], x["single_mask"], x["pair_mask"])
            return dict(s=s, z=z)
        if name == "diffusion_block_n24":
            blk = _load(pkg.DiffusionTransformerBlock(**DIFF, **_DIFF_KW), P, device, dtype)
            upd = blk.attention_pair_bias(a=x["a"], z=x["z"], s=x["s"], mask=x["mask"])
            return dict(attn_update=upd, a=blk(x["a"], x["s"], x["z"], mask=x["mask"]))
        if name == "diffusion_stack2_n16":
            st = _load(pkg.DiffusionTransformer(**DIFF, **_DIFF_KW, no_blocks=2), P, device, dtype)
            return dict(a=st(x["a"], x["s"], x["z"], mask=x["mask"]))
    raise KeyError(name)


def golden(name: str) -> dict:
    return torch.load(ROOT / "tests" / "golden" / f"{name}.pt", map_location="cpu")


def golden_view(name: str, key: str, t: torch.Tensor) -> torch.Tensor:
    """Applies the sub-sampling the golden file was stored with."""
    return t[:, ::4] if (name == "block_n64" and key == "z") else t


# Number of bf16 storage roundings each output has been through in bf16 mode (every in-place
# residual write and every separately stored update rounds once). One rounding moves a value x
# by up to 2^-8 |x|, which at the 4-5 sigma tail of a tensor is already ~2e-2 x RMS, i.e. the
# whole bf16 tolerance; the bf16 parity bar is therefore applied to the error in excess of
# this representation floor.
BF16_ROUNDINGS = {
    "block_n64": dict(s=2, z=5), "block_n40_padded": dict(s=2, z=5),
    "pair_taps_n24": dict(after_tri_mul_out=2, after_tri_mul_in=4, after_tri_att_start=6,
                          after_tri_att_end=8, after_pair_transition=10),
    "trimul_n22_b2": dict(outgoing=1, incoming=1), "triattn_n33_masked_rows": dict(start=1, end=1),
    "pair_odd_dims": dict(z=5), "single_track_n50": dict(attn_update=1, s=4),
    "stack2_n20": dict(s=4, z=10), "diffusion_block_n24": dict(attn_update=1, a=2),
    "diffusion_stack2_n16": dict(a=4),
}


def excess_err(got: torch.Tensor, ref: torch.Tensor, n_round: int) -> float:
    """max( |got - ref| - n_round * 2^-8 * |ref| )+ / RMS(ref): the error beyond what n_round
    bf16 storage roundings of a perfectly computed value could produce."""
    got, ref = got.double(), ref.double()
    d = ((got - ref).abs() - n_round * 2.0 ** -8 * ref.abs()).clamp_min(0)
    return float(d.max() / ref.pow(2).mean().sqrt())


def record(name, key, raw, excess, rms, ref_raw=None, ref_rms=None):
    """Appends one row of the bf16 parity table when OF3_PARITY_TABLE names a file."""
    import os
    path = os.environ.get("OF3_PARITY_TABLE")
    if path:
        with open(path, "a") as f:
            f.write(f"{name}\t{key}\t{raw:.3e}\t{excess:.3e}\t{rms:.3e}\t"
                    f"{'' if ref_raw is None else f'{ref_raw:.3e}'}\t{'' if ref_rms is None else f'{ref_rms:.3e}'}\n")
