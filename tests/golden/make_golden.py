"""Generates the golden vectors in this directory from the reference implementation itself.

Run where the reference source tree is available:

    python tests/golden/make_golden.py /path/to/openfold-3

It imports the reference's own ``openfold3.core.model`` modules (CPU, fp32, every kernel flag
off, ``eval()``), loads the seeded parameters of ``tests/cases.py`` with ``strict=True`` and
stores the module outputs as ``<case>.pt``. Three small stand-in modules are registered
before the import because the optional packages they replace are not installed
(``ml_collections.ConfigDict`` is only used for attribute access, ``biotite.structure.
AtomArray`` only as an ``isinstance`` target, ``gemmi`` only for its version string); none of
them takes part in the arithmetic. The same script prints how far the CPU oracle is from the
reference outputs (it must be at rounding level).
"""

from __future__ import annotations

import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/openfold-3   (the reference's source tree)")
REF = Path(sys.argv[1])


def install_stubs():
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
    sys.modules["ml_collections"] = ml
    bio, bs = types.ModuleType("biotite"), types.ModuleType("biotite.structure")
    bs.AtomArray = type("AtomArray", (), {})
    bio.structure = bs
    sys.modules["biotite"], sys.modules["biotite.structure"] = bio, bs
    g = types.ModuleType("gemmi")
    g.__version__ = "0.0.0"
    sys.modules["gemmi"] = g
    sys.path.insert(0, str(REF))


def main():
    install_stubs()
    import cases
    from openfold3.core.model.latent.base_blocks import PairBlock
    from openfold3.core.model.latent.pairformer import PairFormerBlock, PairFormerStack
    from openfold3.core.model.layers.diffusion_transformer import DiffusionTransformer, DiffusionTransformerBlock

    torch.manual_seed(0)
    torch.set_grad_enabled(False)

    def load(mod, P):
        mod.load_state_dict(P, strict=True)
        return mod.to(next(iter(P.values())).dtype).eval()

    pf_kw = dict(transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False, inf=1e9)

    def ref_block(P, x, **dims):
        blk = load(PairFormerBlock(**dims, **pf_kw), P)
        s, z = blk(x["s"], x["z"], x["single_mask"], x["pair_mask"])
        return dict(s=s, z=z)

    def ref_pair_taps(P, x):
        blk = load(PairBlock(**cases.PAIR, **pf_kw), P)
        z, m = x["z"], x["pair_mask"]
        out = {}
        z = z + blk.tri_mul_out(z, mask=m)
        out["after_tri_mul_out"] = z
        z = z + blk.tri_mul_in(z, mask=m)
        out["after_tri_mul_in"] = z
        z = z + blk.tri_att_start(z, mask=m)
        out["after_tri_att_start"] = z
        # exactly what PairBlock.tri_att_start_end does around tri_att_end
        zt = z.transpose(-2, -3)
        zt = zt + blk.tri_att_end(zt, mask=m.transpose(-1, -2))
        z = zt.transpose(-2, -3)
        out["after_tri_att_end"] = z
        z = z + blk.pair_transition(z, mask=m)
        out["after_pair_transition"] = z
        # and the block's own forward must agree with the tapped sequence
        z_full = blk(x["z"], m)
        assert torch.allclose(z_full, z, atol=1e-5), float((z_full - z).abs().max())
        # as must its in-place inference path
        z_inpl = blk(x["z"].clone(), m, inplace_safe=True)
        assert torch.allclose(z_inpl, z, atol=1e-4), float((z_inpl - z).abs().max())
        return out

    def ref_trimul(P, x):
        blk = load(PairBlock(**cases.PAIR, **pf_kw), P)
        return dict(outgoing=blk.tri_mul_out(x["z"], mask=x["mask"]), incoming=blk.tri_mul_in(x["z"], mask=x["mask"]))

    def ref_triattn(P, x):
        from openfold3.core.model.layers.triangular_attention import TriangleAttentionEndingNode
        blk = load(PairBlock(**cases.PAIR, **pf_kw), P)
        start = blk.tri_att_start(x["z"], mask=x["mask"])
        end_mod = TriangleAttentionEndingNode(128, 32, 4, inf=1e9)
        end_mod.load_state_dict(blk.tri_att_end.state_dict())
        end = end_mod.eval()(x["z"], mask=x["mask"])
        return dict(start=start, end=end)

    def ref_pair_odd(P, x):
        dims = dict(c_z=20, c_hidden_mul=19, c_hidden_pair_att=14, no_heads_pair=7, transition_n=2)
        blk = load(PairBlock(**dims, **pf_kw), P)
        return dict(z=blk(x["z"], x["pair_mask"]))

    def ref_single(P, x):
        blk = load(PairFormerBlock(**cases.OF3, **pf_kw), P)
        upd = blk.attn_pair_bias(a=x["s"], z=x["z"], s=None, mask=x["single_mask"])
        s = x["s"] + upd
        s2 = s + blk.single_transition(s, mask=x["single_mask"])
        return dict(attn_update=upd, s=s2)

    def ref_stack(P, x):
        st = load(PairFormerStack(**cases.OF3, **pf_kw, no_blocks=2, blocks_per_ckpt=None), P)
        s, z = st(x["s"], x["z"], x["single_mask"], x["pair_mask"])
        return dict(s=s, z=z)

    diff_kw = dict(use_ada_layer_norm=True, n_query=None, n_key=None, inf=1e9)

    def ref_diff_block(P, x):
        blk = load(DiffusionTransformerBlock(**cases.DIFF, **diff_kw), P)
        upd = blk.attention_pair_bias(a=x["a"], z=x["z"], s=x["s"], mask=x["mask"])
        a = blk(x["a"], x["s"], x["z"], mask=x["mask"])
        return dict(attn_update=upd, a=a)

    def ref_diff_stack(P, x):
        st = load(DiffusionTransformer(**cases.DIFF, **diff_kw, no_blocks=2), P)
        return dict(a=st(x["a"], x["s"], x["z"], mask=x["mask"]))

    ref_runs = dict(
        block_n64=lambda P, x: ref_block(P, x, **cases.OF3),
        block_n40_padded=lambda P, x: ref_block(P, x, **cases.OF3),
        pair_taps_n24=ref_pair_taps, trimul_n22_b2=ref_trimul, triattn_n33_masked_rows=ref_triattn,
        pair_odd_dims=ref_pair_odd, single_track_n50=ref_single, stack2_n20=ref_stack,
        diffusion_block_n24=ref_diff_block, diffusion_stack2_n16=ref_diff_stack,
    )
    assert set(ref_runs) == set(cases.CASES)

    bf16_err, bf16_rms = {}, {}
    for name, make in cases.CASES.items():
        P, x, run_oracle = make()
        # the reference's own bf16 path on the same (bf16-rounded) inputs and weights, measured
        # against the fp32 oracle on those rounded values: the yardstick for the bf16 parity bar
        bf = torch.bfloat16
        Pq = {k: v.to(bf) for k, v in P.items()}
        xq = {k: v.to(bf) for k, v in x.items()}
        ref_bf = ref_runs[name](Pq, xq)
        ora_q = run_oracle({k: v.float() for k, v in Pq.items()}, {k: v.float() for k, v in xq.items()})
        bf16_err[name] = {k: cases.rel_err(ref_bf[k].float(), ora_q[k]) for k in ref_bf}
        bf16_rms[name] = {k: cases.rms_err(ref_bf[k].float(), ora_q[k]) for k in ref_bf}
        ref = ref_runs[name](P, x)
        ora = run_oracle(P, x)
        errs = {k: cases.rel_err(ora[k], ref[k]) for k in ref}
        # block_n64's z is the largest tensor: keep every 4th row of it
        store = {k: (v[:, ::4].contiguous() if name == "block_n64" and k == "z" else v.contiguous()).clone()
                 for k, v in ref.items()}
        torch.save(store, HERE / f"{name}.pt")
        size = sum(v.numel() * 4 for v in store.values()) / 1e6
        print(f"{name:28s} {size:6.2f} MB  oracle-vs-reference max|d|/RMS: "
              + ", ".join(f"{k}={e:.2e}" for k, e in errs.items()))
        assert all(e < 2e-5 for e in errs.values()), (name, errs)
        print(" " * 29 + "reference bf16 path vs fp32 oracle: "
              + ", ".join(f"{k}={e:.2e}" for k, e in bf16_err[name].items()))
    # error growth with depth of the reference's own bf16 path (48 blocks, N = 64)
    P, x, run_oracle = cases.depth_curve_n64()
    bf = torch.bfloat16
    Pq = {k: v.to(bf) for k, v in P.items()}
    xq = {k: v.to(bf) for k, v in x.items()}
    st = load(PairFormerStack(**cases.OF3, **pf_kw, no_blocks=max(cases.DEPTHS), blocks_per_ckpt=None), Pq)
    ref_bf = cases.run_depth_curve(st, xq)
    ora_q = run_oracle({k: v.float() for k, v in Pq.items()}, {k: v.float() for k, v in xq.items()})
    valid = dict(s=x["single_mask"][0].bool(), z=x["pair_mask"][0].bool())
    curve = {k: dict(max=cases.rel_err(ref_bf[k].float()[0], ora_q[k][0], valid[k[0]]),
                     rms=cases.rms_err(ref_bf[k].float()[0], ora_q[k][0], valid[k[0]])) for k in ora_q}
    print("reference bf16 path vs fp32 oracle by depth:", curve)
    import json
    (HERE / "reference_bf16_depth_curve.json").write_text(json.dumps(curve, indent=1, sort_keys=True) + "\n")
    (HERE / "reference_bf16_error.json").write_text(json.dumps(bf16_err, indent=1, sort_keys=True) + "\n")
    (HERE / "reference_bf16_rms_error.json").write_text(json.dumps(bf16_rms, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    main()
