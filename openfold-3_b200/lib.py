"""ctypes binding of the C-ABI library and thin tensor-level wrappers.

The wrappers take torch tensors only to read ``data_ptr()``, shapes and the current CUDA
stream; all arithmetic happens inside ``libof3b200.so``. There is no fallback: if the
library is missing or a call fails, a ``RuntimeError`` is raised.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libof3b200.so"

DTYPE_BF16, DTYPE_F32 = 0, 1
FLAG_ADD_RESIDUAL, FLAG_FORCE_GENERIC, FLAG_OUTGOING, FLAG_TRANSPOSED, FLAG_ADA_LN = 1, 2, 4, 8, 16
MODULE_TRIMUL, MODULE_TRIATTN, MODULE_TRANSITION = 1, 2, 3

_lib = None
# Set to FLAG_FORCE_GENERIC to route every call through the shape-generic kernels (tests).
extra_flags = 0


def _struct(name, fields):
    return type(name, (ctypes.Structure,), {"_fields_": [(f, c_void_p) for f in fields]})


TrimulParams = _struct("TrimulParams", ["ln_in_w", "ln_in_b", "w_a_p", "w_a_g", "w_b_p", "w_b_g", "w_g",
                                       "ln_out_w", "ln_out_b", "w_z"])
TriattnParams = _struct("TriattnParams", ["ln_w", "ln_b", "w_bias", "w_q", "w_k", "w_v", "w_g", "w_o"])
TransitionParams = _struct("TransitionParams", ["ln_w", "ln_b", "w_a", "w_b", "w_out"])
AttnPairBiasParams = _struct("AttnPairBiasParams", [
    "ln_a_w", "ln_a_b", "ada_ln_s_w", "ada_w_g", "ada_b_g", "ada_w_s", "w_ada_out", "b_ada_out",
    "ln_z_w", "ln_z_b", "w_z", "w_q", "b_q", "w_k", "w_v", "w_g", "w_o"])
CondTransitionParams = _struct("CondTransitionParams", [
    "ada_ln_s_w", "ada_w_g", "ada_b_g", "ada_w_s", "w_a", "w_b", "w_g", "b_g", "w_out"])

# name -> (restype, argtypes); the same list is checked against include/of3b200.h by the tests
SIGNATURES = {
    "of3_last_error_string": (c_char_p, []),
    "of3_device_status": (c_int, [ctypes.POINTER(c_int)]),
    "of3_device_status_clear": (c_int, []),
    "of3_device_status_async": (c_int, [c_void_p, c_void_p]),
    "of3_profile_enable": (c_int, [c_int]),
    "of3_profile_reset": (c_int, []),
    "of3_profile_read": (c_int, [c_int, ctypes.POINTER(c_longlong), ctypes.POINTER(c_float)]),
    "of3_fast_path_available": (c_int, [c_int] * 6),
    "of3_trimul_workspace_bytes": (c_size_t, [c_int] * 6),
    "of3_trimul_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                   ctypes.POINTER(TrimulParams), c_void_p, c_size_t, c_void_p]),
    "of3_trimul_static_scratch_bytes": (c_size_t, []),
    "of3_trimul_forward_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          ctypes.POINTER(TrimulParams), c_void_p]),
    "of3_triattn_workspace_bytes": (c_size_t, [c_int] * 7),
    "of3_triattn_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                    c_int, c_int, ctypes.POINTER(TriattnParams), c_void_p, c_size_t,
                                    c_void_p]),
    "of3_transition_workspace_bytes": (c_size_t, [c_longlong, c_int, c_int, c_int, c_int]),
    "of3_transition_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                       ctypes.POINTER(TransitionParams), c_void_p, c_size_t, c_void_p]),
    "of3_attn_pair_bias_workspace_bytes": (c_size_t, [c_int] * 10),
    "of3_attn_pair_bias_forward": (c_int, [c_void_p] * 5 + [c_int] * 8 + [c_float, c_int, c_int,
                                           ctypes.POINTER(AttnPairBiasParams), c_void_p, c_size_t,
                                           c_void_p]),
    "of3_cond_transition_workspace_bytes": (c_size_t, [c_longlong, c_int, c_int, c_int, c_int, c_int]),
    "of3_cond_transition_forward": (c_int, [c_void_p] * 4 + [c_longlong, c_int, c_int, c_int, c_int, c_int,
                                            ctypes.POINTER(CondTransitionParams), c_void_p, c_size_t,
                                            c_void_p]),
    "of3_dap_pitch": (c_int, [c_int, c_int]),
    "of3_dap_triattn_image_elems": (c_longlong, [c_int, c_int]),
    "of3_dap_triattn_bias_elems": (c_longlong, [c_int, c_int]),
    "of3_dap_trimul_project": (c_int, [c_void_p] * 3 + [c_int] * 4 + [ctypes.POINTER(TrimulParams), c_void_p]),
    "of3_dap_trimul_contract": (c_int, [c_void_p] * 2 + [c_int] * 3 + [c_void_p]),
    "of3_dap_trimul_output": (c_int, [c_void_p] * 3 + [c_int] * 3 + [ctypes.POINTER(TrimulParams), c_void_p]),
    "of3_copy_rows_3d": (c_int, [c_void_p] * 2 + [c_int] * 3 + [c_longlong] * 6 + [c_int, c_void_p]),
    "of3_attn_pair_bias_rows_workspace_bytes": (c_size_t, [c_int] * 3),
    "of3_attn_pair_bias_forward_rows": (c_int, [c_void_p] * 4 + [c_int] * 6 + [c_float, c_int, c_int,
                                                ctypes.POINTER(AttnPairBiasParams), c_void_p, c_size_t, c_void_p]),
    "of3_dap_triattn_project": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, ctypes.POINTER(TriattnParams), c_void_p]),
    "of3_dap_triattn_finish": (c_int, [c_void_p] * 8 + [c_int, c_int, c_float, c_int,
                                       ctypes.POINTER(TriattnParams), c_void_p]),
    "of3_pair_bias_project": (c_int, [c_void_p] * 5 + [c_longlong, c_int, c_int, c_int, c_void_p]),
    "of3_attn_pair_bias_forward_prebias": (c_int, [c_void_p] * 5 + [c_int] * 7 + [c_float, c_int, c_int,
                                                   ctypes.POINTER(AttnPairBiasParams), c_void_p, c_size_t,
                                                   c_void_p]),
    "of3_pair_bias_tiles_elems": (c_longlong, [c_int]),
    "of3_pair_bias_project_tiles": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_void_p]),
    "of3_attn_pair_bias_forward_pretiles": (c_int, [c_void_p] * 5 + [c_int] * 7 + [c_float, c_int, c_int,
                                                    ctypes.POINTER(AttnPairBiasParams), c_void_p, c_size_t,
                                                    c_void_p]),
    "of3_peer_heap_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "of3_peer_heap_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "of3_peer_heap_close": (c_int, [c_void_p]),
    "of3_peer_heap_free": (c_int, [c_void_p]),
    "of3_peer_barrier": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "of3_peer_barrier_step_entry": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "of3_peer_pull_rows": (c_int, [ctypes.POINTER(c_void_p), c_longlong, c_void_p, c_int, c_int, c_int, c_int]
                           + [c_longlong] * 5 + [c_int, c_void_p]),
    "of3_peer_push_rows": (c_int, [ctypes.POINTER(c_void_p), c_longlong, c_void_p, c_int, c_int, c_int, c_int]
                           + [c_longlong] * 5 + [c_int, c_void_p]),
    "of3_contract_nt_bf16": (c_int, [c_void_p] * 3 + [c_int] * 7 + [c_longlong] * 3 + [c_void_p]),
}


def load():
    """dlopen the library and bind every entry point. Works without a GPU."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it first (python __graft_entry__.py, or "
            "openfold3_b200._build.build()). There is no fallback path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().of3_last_error_string().decode()


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")


def check_device_status():
    """Raises if a kernel's bounded wait ran out since the last clear (synchronises the device)."""
    arr = (c_int * 4)()
    _check(load().of3_device_status(arr), "of3_device_status")
    if arr[0] != 0:
        load().of3_device_status_clear()
        raise RuntimeError(
            f"device-side wait ran out: code {arr[0]}, kernel {arr[1]}, block {arr[2]}, site {arr[3]}"
        )


KERNEL_NAMES = {1: "trimul_contract", 2: "trimul_in", 3: "trimul_out", 4: "transition", 5: "triattn_proj",
                6: "triattn_core", 7: "triattn_out", 8: "single_track", 9: "pair_bias", 10: "single_linear",
                11: "single_attn_core", 20: "generic", 30: "peer_barrier",
                31: "peer_pull"}


def profile_begin(timing: bool = True):
    """Resets the launch counters and (optionally) starts recording an event pair per launch."""
    lib = load()
    _check(lib.of3_profile_reset(), "of3_profile_reset")
    _check(lib.of3_profile_enable(1 if timing else 0), "of3_profile_enable")


def profile_end() -> dict:
    """Stops timing; returns {kernel name: (launches, total device ms)} since profile_begin."""
    lib = load()
    _check(lib.of3_profile_enable(0), "of3_profile_enable")
    out = {}
    for kid, name in KERNEL_NAMES.items():
        n, ms = c_longlong(0), c_float(0)
        _check(lib.of3_profile_read(kid, ctypes.byref(n), ctypes.byref(ms)), "of3_profile_read")
        if n.value:
            out[name] = (int(n.value), float(ms.value))
    return out


def fast_path_available(module_id, dtype, c, c_hidden=0, heads=0, head_dim=0) -> bool:
    return bool(load().of3_fast_path_available(module_id, dtype_code(dtype), c, c_hidden, heads, head_dim))


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    if dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"unsupported activation dtype {dtype}: the kernels take bfloat16 or float32")


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream); owned by torch, handed to the library per call."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = None
        _workspaces.pop(key, None)
        buf = torch.empty(int(nbytes * 1.0) + 1024, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the B200 library has no CPU path")


def trimul_forward(z, mask, out, params, c_h: int, outgoing: bool, add_residual: bool):
    """z/out [B, N, N, c_z] contiguous, mask [B, N, N] or None (same dtype), params tuple of 10."""
    _require_cuda(z, "z")
    lib = load()
    B, N, _, c_z = z.shape
    dt = dtype_code(z.dtype)
    flags = extra_flags | (FLAG_OUTGOING if outgoing else 0) | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_trimul_workspace_bytes(B, N, c_z, c_h, dt, flags)
    ws = workspace(nbytes, z.device)
    p = TrimulParams(*[_ptr(t) for t in params])
    _check(lib.of3_trimul_forward(z.data_ptr(), _ptr(mask), out.data_ptr(), B, N, c_z, c_h, dt, flags,
                                  ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(z.device)),
           "of3_trimul_forward")


def triattn_forward(z, mask, out, params, H: int, d: int, inf: float, transposed: bool, add_residual: bool):
    _require_cuda(z, "z")
    lib = load()
    B, N, _, c_z = z.shape
    dt = dtype_code(z.dtype)
    flags = extra_flags | (FLAG_TRANSPOSED if transposed else 0) | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_triattn_workspace_bytes(B, N, c_z, H, d, dt, flags)
    ws = workspace(nbytes, z.device)
    p = TriattnParams(*[_ptr(t) for t in params])
    _check(lib.of3_triattn_forward(z.data_ptr(), _ptr(mask), out.data_ptr(), B, N, c_z, H, d, float(inf), dt,
                                   flags, ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(z.device)),
           "of3_triattn_forward")


def transition_forward(x, mask, out, params, n: int, add_residual: bool):
    """x/out [rows, c] contiguous, mask [rows] or None."""
    _require_cuda(x, "x")
    lib = load()
    rows, c = x.shape
    dt = dtype_code(x.dtype)
    flags = extra_flags | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_transition_workspace_bytes(rows, c, n, dt, flags)
    ws = workspace(nbytes, x.device)
    p = TransitionParams(*[_ptr(t) for t in params])
    _check(lib.of3_transition_forward(x.data_ptr(), _ptr(mask), out.data_ptr(), rows, c, n, dt, flags,
                                      ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(x.device)),
           "of3_transition_forward")


def attn_pair_bias_forward(a, z, s, mask, out, params, H: int, d: int, inf: float, ada: bool,
                           add_residual: bool):
    """a/out [Ba, N, c_a], z [Bz, N, N, c_z], s [Ba, N, c_s] or None, mask [Ba, N] or None."""
    _require_cuda(a, "a")
    lib = load()
    Ba, N, c_a = a.shape
    Bz, c_z = z.shape[0], z.shape[-1]
    c_s = s.shape[-1] if s is not None else 0
    dt = dtype_code(a.dtype)
    flags = extra_flags | (FLAG_ADA_LN if ada else 0) | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_attn_pair_bias_workspace_bytes(Ba, Bz, N, c_a, c_s, c_z, H, d, dt, flags)
    ws = workspace(nbytes, a.device)
    p = AttnPairBiasParams(*[_ptr(t) for t in params])
    _check(lib.of3_attn_pair_bias_forward(a.data_ptr(), z.data_ptr(), _ptr(s), _ptr(mask), out.data_ptr(),
                                          Ba, Bz, N, c_a, c_s, c_z, H, d, float(inf), dt, flags,
                                          ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(a.device)),
           "of3_attn_pair_bias_forward")


def pair_bias_project(z, ln_w, ln_b, w, out=None):
    """Pair-bias projection of AttentionPairBias for whole pair tensors: z [Bz, N, N, 128], LayerNorm_z weight /
    bias (bias may be None), linear_z.weight [16, 128] -> [Bz, 16, N, N] fp32."""
    _require_cuda(z, "z")
    lib = load()
    Bz, N = z.shape[0], z.shape[1]
    H = w.shape[0]
    if out is None:
        out = torch.empty((Bz, H, N, N), dtype=torch.float32, device=z.device)
    for b in range(Bz):
        _check(lib.of3_pair_bias_project(z[b].data_ptr(), _ptr(ln_w), _ptr(ln_b), w.data_ptr(), out[b].data_ptr(),
                                         N * N, z.shape[-1], H, dtype_code(z.dtype), _stream(z.device)),
               "of3_pair_bias_project")
    return out


def attn_pair_bias_forward_prebias(a, pair_bias, s, mask, out, params, H: int, d: int, inf: float, ada: bool,
                                   add_residual: bool):
    """attn_pair_bias_forward with the pair bias [Bz, H, N, N] (fp32) already projected (c_z = 128)."""
    _require_cuda(a, "a")
    lib = load()
    Ba, N, c_a = a.shape
    Bz = pair_bias.shape[0]
    c_s = s.shape[-1] if s is not None else 0
    dt = dtype_code(a.dtype)
    flags = extra_flags | (FLAG_ADA_LN if ada else 0) | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_attn_pair_bias_workspace_bytes(Ba, Bz, N, c_a, c_s, 128, H, d, dt, flags)
    ws = workspace(nbytes, a.device)
    p = AttnPairBiasParams(*[_ptr(t) for t in params])
    _check(lib.of3_attn_pair_bias_forward_prebias(a.data_ptr(), pair_bias.data_ptr(), _ptr(s), _ptr(mask),
                                                  out.data_ptr(), Ba, Bz, N, c_a, c_s, H, d, float(inf), dt, flags,
                                                  ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(a.device)),
           "of3_attn_pair_bias_forward_prebias")


def pair_bias_project_tiles(z, ln_w, ln_b, w):
    """The pair-bias projection of AttentionPairBias written as the bias tiles of the tensor-core attention kernel:
    z [Bz, N, N, 128] bf16 -> [Bz, 16, ceil(N / 32), N, 32] bf16 (times log2(e), 64-byte swizzled rows). Opaque:
    only ``attn_pair_bias_forward_pretiles`` reads it."""
    _require_cuda(z, "z")
    lib = load()
    Bz, N = z.shape[0], z.shape[1]
    assert z.dtype == torch.bfloat16 and w.shape[0] == 16 and z.shape[-1] == 128
    out = torch.empty((Bz, 16, (N + 31) // 32, N, 32), dtype=torch.bfloat16, device=z.device)
    assert out[0].numel() == lib.of3_pair_bias_tiles_elems(N)
    for b in range(Bz):
        _check(lib.of3_pair_bias_project_tiles(z[b].data_ptr(), _ptr(ln_w), _ptr(ln_b), w.data_ptr(), out[b].data_ptr(),
                                               N, 128, 16, dtype_code(z.dtype), _stream(z.device)),
               "of3_pair_bias_project_tiles")
    return out


def attn_pair_bias_forward_pretiles(a, tiles, s, mask, out, params, H: int, d: int, inf: float, ada: bool,
                                    add_residual: bool):
    """attn_pair_bias_forward with the bias tiles of ``pair_bias_project_tiles`` (bf16 tensor-core path only)."""
    _require_cuda(a, "a")
    lib = load()
    Ba, N, c_a = a.shape
    Bz = tiles.shape[0]
    c_s = s.shape[-1] if s is not None else 0
    dt = dtype_code(a.dtype)
    flags = extra_flags | (FLAG_ADA_LN if ada else 0) | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_attn_pair_bias_workspace_bytes(Ba, Bz, N, c_a, c_s, 128, H, d, dt, flags)
    ws = workspace(nbytes, a.device)
    p = AttnPairBiasParams(*[_ptr(t) for t in params])
    _check(lib.of3_attn_pair_bias_forward_pretiles(a.data_ptr(), tiles.data_ptr(), _ptr(s), _ptr(mask),
                                                   out.data_ptr(), Ba, Bz, N, c_a, c_s, H, d, float(inf), dt, flags,
                                                   ctypes.byref(p), ws.data_ptr(), ws.numel(), _stream(a.device)),
           "of3_attn_pair_bias_forward_pretiles")


def cond_transition_forward(a, s, mask, out, params, n: int, add_residual: bool):
    _require_cuda(a, "a")
    lib = load()
    rows, c_a = a.shape
    c_s = s.shape[-1]
    dt = dtype_code(a.dtype)
    flags = extra_flags | (FLAG_ADD_RESIDUAL if add_residual else 0)
    nbytes = lib.of3_cond_transition_workspace_bytes(rows, c_a, c_s, n, dt, flags)
    ws = workspace(nbytes, a.device)
    p = CondTransitionParams(*[_ptr(t) for t in params])
    _check(lib.of3_cond_transition_forward(a.data_ptr(), s.data_ptr(), _ptr(mask), out.data_ptr(), rows, c_a,
                                           c_s, n, dt, flags, ctypes.byref(p), ws.data_ptr(), ws.numel(),
                                           _stream(a.device)),
           "of3_cond_transition_forward")


def contract_nt_bf16(a, b, out):
    """out[b, i, j] = sum_k a[b, i, k] * b[b, j, k]; 3-D bf16 tensors with contiguous last dim."""
    _require_cuda(a, "a")
    lib = load()
    batch, M, K = a.shape
    N = b.shape[1]
    _check(lib.of3_contract_nt_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, M, N, K,
                                    a.stride(1), b.stride(1), out.stride(1), a.stride(0), b.stride(0),
                                    out.stride(0), _stream(a.device)),
           "of3_contract_nt_bf16")
