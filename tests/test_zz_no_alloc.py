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


def _run_both(pkg, lib, P_tensors, params, z, mask, c_h, flags, dt):
    """The static entry point and the workspace entry point on the same inputs -> (rc_static, out_static, out_ws)."""
    dev = z.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    B, N, c_z = z.shape[0], z.shape[1], z.shape[-1]
    mptr = None if mask is None else mask.data_ptr()
    out_static = torch.empty_like(z)
    rc = lib.of3_trimul_forward_static(z.data_ptr(), mptr, out_static.data_ptr(), B, N, c_z, c_h, dt, flags,
                                       ctypes.byref(params), stream)
    if rc != 0:
        return rc, None, None
    gflags = flags | pkg.lib.FLAG_FORCE_GENERIC
    ws = torch.empty(lib.of3_trimul_workspace_bytes(B, N, c_z, c_h, dt, gflags), dtype=torch.uint8, device=dev)
    out_ws = torch.empty_like(z)
    rc2 = lib.of3_trimul_forward(z.data_ptr(), mptr, out_ws.data_ptr(), B, N, c_z, c_h, dt, gflags,
                                 ctypes.byref(params), ws.data_ptr(), ws.numel(), stream)
    assert rc2 == 0, lib.of3_last_error_string()
    torch.cuda.synchronize()
    return rc, out_static, out_ws


def test_static_entry_at_its_size_limit_without_mask_and_with_unequal_widths(pkg):
    """The documented bound: 24 * B * N^2 * max(c_z, c_hidden) bytes must fit the 16 MiB array, i.e. N = 73 is
    the largest accepted size at B = 1, c = 128 and N = 74 the first rejected one. Also a call without a mask,
    and widths c_z != c_hidden (the bound uses the larger of the two)."""
    dev = torch.device("cuda:0")
    lib = pkg.lib.load()
    dt = pkg.lib.dtype_code(torch.float32)
    g = torch.Generator().manual_seed(11)
    P = pkg.weights.pair_block_params(seed=32, final_std=None)
    keep, params = _params(pkg, P, "tri_mul_out.", torch.float32, dev)
    flags = pkg.lib.FLAG_OUTGOING
    z73 = torch.randn(1, 73, 73, 128, generator=g).to(dev)
    rc, a, b = _run_both(pkg, lib, keep, params, z73, None, 128, flags, dt)   # no mask
    assert rc == 0, lib.of3_last_error_string()
    assert cases.rel_err(a.cpu(), b.cpu()) <= 1e-6
    z74 = torch.randn(1, 74, 74, 128, generator=g).to(dev)
    rc, _, _ = _run_both(pkg, lib, keep, params, z74, None, 128, flags, dt)
    assert rc == -4 and b"built-in array" in lib.of3_last_error_string()
    # c_z = 48, c_hidden = 80: the chain holds one buffer of c_z and five of max(c_z, c_hidden) floats per
    # position (1792 B; the documented 24 * max(c) = 1920 B is an upper bound): N = 96 fits, N = 97 does not
    P2 = pkg.weights.pair_block_params(seed=33, final_std=None, c_z=48, c_hidden_mul=80, c_hidden_pair_att=8,
                                       no_heads_pair=2)
    keep2, params2 = _params(pkg, P2, "tri_mul_in.", torch.float32, dev)
    z = torch.randn(1, 96, 96, 48, generator=g).to(dev)
    m = (torch.rand(1, 96, 96, generator=g) < 0.7).to(dev, torch.float32)
    rc, a, b = _run_both(pkg, lib, keep2, params2, z, m, 80, 0, dt)
    assert rc == 0, lib.of3_last_error_string()
    assert cases.rel_err(a.cpu(), b.cpu()) <= 1e-6
    z = torch.randn(1, 97, 97, 48, generator=g).to(dev)
    rc, _, _ = _run_both(pkg, lib, keep2, params2, z, None, 80, 0, dt)
    assert rc == -4
    del keep, keep2


def test_static_entry_leaves_free_device_memory_unchanged(pkg):
    """What the entry point is for: after its first call on the device (which looks the array's address up),
    a call changes neither the driver's free-memory figure nor torch's allocator statistics."""
    dev = torch.device("cuda:0")
    lib = pkg.lib.load()
    dt = pkg.lib.dtype_code(torch.bfloat16)
    P = pkg.weights.pair_block_params(seed=34, final_std=None)
    keep, params = _params(pkg, P, "tri_mul_out.", torch.bfloat16, dev)
    z = torch.randn(1, 48, 48, 128, device=dev).to(torch.bfloat16)
    out = torch.empty_like(z)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call():
        rc = lib.of3_trimul_forward_static(z.data_ptr(), None, out.data_ptr(), 1, 48, 128, 128, dt,
                                           pkg.lib.FLAG_OUTGOING, ctypes.byref(params), stream)
        assert rc == 0, lib.of3_last_error_string()

    call()  # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    alloc0, reserved0 = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0, (free0, free1)
    assert (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)) == (alloc0, reserved0)
    del keep
