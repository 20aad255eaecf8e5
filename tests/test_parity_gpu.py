"""GPU parity: the drop-in modules (calling the C-ABI CUDA library) against the golden vectors
of the reference (fp32 validation mode) and against the CPU oracle evaluated on bf16-rounded
inputs and weights (bf16 mode).

Tolerances (max |got - ref| / RMS(ref)):
  fp32 validation mode  1e-4
  bf16, fp32 accumulate 2e-2 -- or, where the reference's own bf16 path is itself further than
                        that from the fp32 oracle on the same rounded inputs (it is, on every case
                        here: 2.3e-2 .. 1.0e-1, tests/golden/reference_bf16_error.json, measured
                        by tests/golden/make_golden.py), no worse than the reference's bf16 path.
                        The reason is representational: rounding one value x to bf16 moves it by up
                        to 2^-8 |x|, which at the 5-sigma tail of a tensor is already 2e-2 x RMS, and
                        tensor-core operands (LayerNorm output, gated projections) must be bf16.
                        The error in excess of the output's own storage rounding is printed too.
"""

import json

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_BF16 = 2e-2


@pytest.fixture(scope="module")
def dev(pkg):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert pkg.lib.LIB_PATH.exists()
    return torch.device("cuda:0")


@pytest.mark.parametrize("name", list(cases.CASES))
@pytest.mark.parametrize("force_generic", [False, True], ids=["auto", "generic"])
def test_fp32_validation_mode_matches_reference(pkg, dev, name, force_generic):
    P, x, _ = cases.CASES[name]()
    pkg.lib.extra_flags = pkg.lib.FLAG_FORCE_GENERIC if force_generic else 0
    try:
        got = cases.run_dropin(name, P, x, dev, torch.float32)
        torch.cuda.synchronize()
        pkg.lib.check_device_status()
    finally:
        pkg.lib.extra_flags = 0
    ref = cases.golden(name)
    for k, r in ref.items():
        g = cases.golden_view(name, k, got[k].cpu())
        assert torch.isfinite(g).all(), (name, k)
        err = cases.rel_err(g, r)
        assert err < TOL_F32, (name, k, err)
    if name == "pair_taps_n24":
        for k in ("block_forward", "block_forward_inplace"):
            err = cases.rel_err(got[k].cpu(), ref["after_pair_transition"])
            assert err < TOL_F32, (name, k, err)


@pytest.mark.parametrize("name", list(cases.CASES))
@pytest.mark.parametrize("force_generic", [False, True], ids=["auto", "generic"])
def test_bf16_matches_oracle_on_rounded_inputs(pkg, dev, name, force_generic):
    P, x, run_oracle = cases.CASES[name]()
    bf = torch.bfloat16
    Pq = {k: v.to(bf).float() for k, v in P.items()}
    xq = {k: v.to(bf).float() for k, v in x.items()}
    ref = run_oracle(Pq, xq)
    pkg.lib.extra_flags = pkg.lib.FLAG_FORCE_GENERIC if force_generic else 0
    try:
        got = cases.run_dropin(name, P, x, dev, bf)
        torch.cuda.synchronize()
        pkg.lib.check_device_status()
    finally:
        pkg.lib.extra_flags = 0
    ref_bf16 = json.loads((cases.ROOT / "tests" / "golden" / "reference_bf16_error.json").read_text())[name]
    for k, r in ref.items():
        g = got[k].float().cpu()
        assert torch.isfinite(g).all(), (name, k)
        err = cases.rel_err(g, r)
        # the maximum over ~1e5 elements is an extreme-value statistic: allow 25 % scatter around
        # the reference path's own figure
        bar = max(TOL_BF16, 1.25 * ref_bf16[k])
        print(f"{name}.{k}: bf16 max-abs/RMS {err:.3e} (reference bf16 path: {ref_bf16[k]:.3e}; beyond "
              f"storage rounding: {cases.excess_err(g, r, cases.BF16_ROUNDINGS[name][k]):.3e})")
        assert err <= bar, (name, k, err, bar)


def test_contract_kernel_matches_einsum(pkg, dev):
    """The tcgen05 contraction alone, bit-level layout check on ragged sizes."""
    g = torch.Generator(device="cpu").manual_seed(5)
    for batch, M, N, K in ((1, 128, 128, 64), (3, 200, 84, 200), (2, 22, 22, 22), (4, 384, 384, 384)):
        ld = (K + 63) // 64 * 64
        a = torch.zeros(batch, M, ld, dtype=torch.bfloat16, device=dev)
        b = torch.zeros(batch, N, ld, dtype=torch.bfloat16, device=dev)
        a[:, :, :K] = torch.randn(batch, M, K, generator=g).to(dev)
        b[:, :, :K] = torch.randn(batch, N, K, generator=g).to(dev)
        out = torch.zeros(batch, M, (N + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)
        pkg.lib.contract_nt_bf16(a, b, out)
        torch.cuda.synchronize()
        pkg.lib.check_device_status()
        ref = torch.einsum("bik,bjk->bij", a.float(), b.float())
        err = cases.rel_err(out[:, :, :N].float().cpu(), ref.cpu())
        assert err < 2e-2, (batch, M, N, K, err)  # one bf16 rounding of the output


def test_repeatable(pkg, dev):
    """Same inputs twice give bit-identical outputs (no atomics / race-dependent ordering)."""
    P, x, _ = cases.CASES["block_n40_padded"]()
    a = cases.run_dropin("block_n40_padded", P, x, dev, torch.bfloat16)
    b = cases.run_dropin("block_n40_padded", P, x, dev, torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(a["z"], b["z"]) and torch.equal(a["s"], b["s"])
