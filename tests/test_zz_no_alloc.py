"""The allocation-free triangle-update entry point (of3_trimul_forward_static) against the regular
one (of3_trimul_forward with a caller-owned workspace), through the C ABI.

The static variant exists for hosts that must not allocate device memory (fixed memory budget,
code running inside another component's stream-ordered region); its scratch is a 16 MiB array built
into the library. Both entry points run the same shape-generic kernels, so their outputs must
agree to fp32 rounding (1e-6 x RMS; in practice bit for bit). Two calls in a row check that the
shared scratch carries nothing over from one call into the next. This file sorts last so that a
run stopping at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _params(pkg, P, prefix, dtype, dev):
    names = ["layer_norm_in.weight", "layer_norm_in.bias", "linear_a_p.weight", "linear_a_g.weight",
             "linear_b_p.weight", "linear_b_g.weight", "linear_g.weight", "layer_norm_out.weight",
             "layer_norm_out.bias", "linear_z.weight"]
    tensors = [P[prefix + n].to(dev, dtype).contiguous() for n in names]
    return tensors, pkg.lib.TrimulParams(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_static_entry_matches_workspace_entry(pkg, dtype):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = pkg.lib.load()
    dt = pkg.lib.dtype_code(dtype)
    P = pkg.weights.pair_block_params(seed=31, final_std=None)
    stream = torch.cuda.current_stream(dev).cuda_stream
    g = torch.Generator().manual_seed(9)
    # two calls in a row with different sizes, directions and masks
    for call, (B, N, outgoing) in enumerate([(1, 40, True), (2, 24, False)]):
        prefix = "tri_mul_out." if outgoing else "tri_mul_in."
        keep, params = _params(pkg, P, prefix, dtype, dev)
        z = torch.randn(B, N, N, 128, generator=g).to(dev, dtype)
        mask = (torch.rand(B, N, N, generator=g) < 0.8).to(dev, dtype)
        flags = (pkg.lib.FLAG_OUTGOING if outgoing else 0) | pkg.lib.FLAG_ADD_RESIDUAL
        out_static = torch.empty_like(z)
        rc = lib.of3_trimul_forward_static(z.data_ptr(), mask.data_ptr(), out_static.data_ptr(), B, N, 128, 128,
                                           dt, flags, ctypes.byref(params), stream)
        assert rc == 0, lib.of3_last_error_string()
        gflags = flags | pkg.lib.FLAG_FORCE_GENERIC
        nbytes = lib.of3_trimul_workspace_bytes(B, N, 128, 128, dt, gflags)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        out_ws = torch.empty_like(z)
        rc = lib.of3_trimul_forward(z.data_ptr(), mask.data_ptr(), out_ws.data_ptr(), B, N, 128, 128, dt, gflags,
                                    ctypes.byref(params), ws.data_ptr(), ws.numel(), stream)
        assert rc == 0, lib.of3_last_error_string()
        torch.cuda.synchronize()
        assert torch.isfinite(out_static.float()).all()
        err = cases.rel_err(out_static.float().cpu(), out_ws.float().cpu())
        assert err <= 1e-6, (call, err)
        # and it is the right answer, not merely the same one
        Pq = {k: v.to(dtype).float() for k, v in P.items()}
        ref = z.float().cpu() + cases.oracle.triangle_multiplicative_update(
            z.float().cpu(), mask.float().cpu(), Pq, prefix, outgoing)
        if dtype == torch.float32:
            assert cases.rel_err(out_static.float().cpu(), ref) < 1e-4
        else:  # beyond the one bf16 rounding of the stored result
            assert cases.excess_err(out_static.float().cpu(), ref, 1) < 2e-2
        del keep


def test_static_entry_rejects_oversize(pkg):
    lib = pkg.lib.load()
    assert lib.of3_trimul_static_scratch_bytes() == 16 << 20
    params = pkg.lib.TrimulParams(*([1] * 10))  # never dereferenced: the size check comes first
    rc = lib.of3_trimul_forward_static(1, None, 1, 1, 512, 128, 128, 0, 0, ctypes.byref(params), None)
    assert rc == -4
    assert b"built-in array" in lib.of3_last_error_string()
