"""Row-sharded ("DAP") Pairformer trunk over the GPUs of one node.

The pair tensor z[N, N, C] is split by rows over P ranks (N divisible by P); the single
representation and the masks are replicated. Per block (reference order,
openfold3/core/model/latent/base_blocks.py:453-478 and pairformer.py:177-211):

  tri_mul_out    project local rows -> a, b (channel-major) | ALL-GATHER b | contract + finish
  tri_mul_in     ALL-TO-ALL transpose of z (copy) -> project on the transposed shard
                 (a'[i,k] = a[k,i]) | ALL-GATHER b' | contract + finish on the ORIGINAL rows
  tri_att_start  project q,k,v + local rows of the pair bias | ALL-GATHER bias | attention + finish
  tri_att_end    ALL-TO-ALL transpose of z -> the same on the transposed shard, in place there,
  transition     pointwise, still on the transposed shard | ALL-TO-ALL transpose back
  single track   pair-bias projection of the local rows | ALL-GATHER | (replicated, small) update of s

The reference has no model-parallel path (only data-parallel DDP / ZeRO), so this is new design
judged against the single-GPU result. Collectives go through ``torch.distributed`` (NCCL on GPUs,
gloo in the CPU tests); every remote tile is landed in local memory before a kernel reads it.
``ops`` is the compute backend: ``CudaOps`` (the C-ABI library) or, in the CPU tests, an oracle
backend with the same phase semantics, which lets the exchange logic be checked without a GPU.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import lib


def _pitch(n: int, m: int) -> int:
    return (n + m - 1) // m * m


# ----------------------------------------------------------------------------- collectives
def all_gather_lines(x_loc: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """x_loc [G, R, L] (G groups: channels or heads) -> [G, world * R, L], rank-major along dim 1."""
    if world == 1:
        return x_loc
    G, R, L = x_loc.shape
    buf = torch.empty((world * G, R, L), dtype=x_loc.dtype, device=x_loc.device)
    dist.all_gather_into_tensor(buf, x_loc.contiguous(), group=group)
    return buf.view(world, G, R, L).permute(1, 0, 2, 3).reshape(G, world * R, L).contiguous()


def all_to_all_transpose(x_loc: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Row shard [R, N, C] of X[N, N, C] -> row shard [R, N, C] of X^T (y[i, k] = X[k, r*R + i])."""
    if world == 1:
        return x_loc.transpose(0, 1).contiguous()
    R, N, C = x_loc.shape
    send = x_loc.view(R, world, R, C).permute(1, 0, 2, 3).contiguous()  # [dest][k_loc][i_loc][C]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                    # [src][k_loc][i_loc][C]
    return recv.permute(2, 0, 1, 3).reshape(R, N, C).contiguous()


# ----------------------------------------------------------------------------- CUDA backend
class CudaOps:
    """Phase kernels of ``libof3b200.so`` on bf16 CUDA tensors (c_z = c_hidden = 128, 4 heads x 32)."""

    def __init__(self, device):
        self.device = device
        self.l = lib.load()

    def _st(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def trimul_project(self, z_loc, mask_rows, mod):
        R, N, _ = z_loc.shape
        ld = _pitch(N, 8)
        a_t = torch.empty((128, R, ld), dtype=z_loc.dtype, device=z_loc.device)
        b_t = torch.empty((128, R, ld), dtype=z_loc.dtype, device=z_loc.device)
        p = lib.TrimulParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_trimul_project(z_loc.data_ptr(), lib._ptr(mask_rows), a_t.data_ptr(),
                                                 b_t.data_ptr(), R, N, ctypes.byref(p), self._st()),
                   "of3_dap_trimul_project")
        return a_t, b_t

    def trimul_finish(self, z_loc, a_t, b_all, mod):
        R, N, _ = z_loc.shape
        x = torch.empty_like(a_t)
        p = lib.TrimulParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_trimul_finish(z_loc.data_ptr(), z_loc.data_ptr(), a_t.data_ptr(), b_all.data_ptr(),
                                                x.data_ptr(), R, N, lib.FLAG_ADD_RESIDUAL, ctypes.byref(p),
                                                self._st()), "of3_dap_trimul_finish")

    def triattn_project(self, z_loc, mod):
        R, N, _ = z_loc.shape
        ldn = _pitch(N, 64)
        dt, dev = z_loc.dtype, z_loc.device
        img = int(self.l.of3_dap_triattn_image_elems(R, N))  # opaque pre-swizzled operand tiles
        q = torch.empty(img, dtype=dt, device=dev)
        k = torch.empty(img, dtype=dt, device=dev)
        vt = torch.empty(img, dtype=dt, device=dev)
        tb = torch.empty((4, R, ldn), dtype=dt, device=dev)
        p = lib.TriattnParams(*[t.data_ptr() for t in mod._params(dt, dev)])
        lib._check(self.l.of3_dap_triattn_project(z_loc.data_ptr(), q.data_ptr(), k.data_ptr(), vt.data_ptr(),
                                                  tb.data_ptr(), R, N, ctypes.byref(p), self._st()),
                   "of3_dap_triattn_project")
        return (q, k, vt), tb

    def triattn_finish(self, z_loc, mask_rows, qkv, tb_all, mod):
        R, N, _ = z_loc.shape
        q, k, vt = qkv
        o = torch.empty_like(z_loc)
        p = lib.TriattnParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_triattn_finish(z_loc.data_ptr(), lib._ptr(mask_rows), z_loc.data_ptr(),
                                                 q.data_ptr(), k.data_ptr(), vt.data_ptr(), tb_all.data_ptr(),
                                                 o.data_ptr(), R, N, float(mod.inf), lib.FLAG_ADD_RESIDUAL,
                                                 ctypes.byref(p), self._st()), "of3_dap_triattn_finish")

    def transition(self, x_rows, mask_rows, mod):
        mod._run(x_rows, mask_rows, in_place=True)

    def pair_bias_project(self, z_loc, apb):
        R, N, _ = z_loc.shape
        dt, dev = z_loc.dtype, z_loc.device
        prm = apb._params(dt, dev)
        ln_w, ln_b, w = prm[8], prm[9], prm[10]
        out = torch.empty((16, R, N), dtype=torch.float32, device=dev)
        lib._check(self.l.of3_pair_bias_project(z_loc.data_ptr(), lib._ptr(ln_w), lib._ptr(ln_b), w.data_ptr(),
                                                out.data_ptr(), R * N, 128, 16, lib.dtype_code(dt), self._st()),
                   "of3_pair_bias_project")
        return out

    def single_track(self, s, zb_all, single_mask, block, mask_trans=True):
        """s [1, N, c_s] updated in place with the already projected pair bias [16, N, N] (fp32)."""
        apb = block.attn_pair_bias
        N = s.shape[-2]
        dt, dev = s.dtype, s.device
        a = s.view(1, N, apb.c_q)
        m = None if single_mask is None else single_mask.to(dt).reshape(1, N).contiguous()
        p = lib.AttnPairBiasParams(*[lib._ptr(t) for t in apb._params(dt, dev)])
        flags = lib.FLAG_ADD_RESIDUAL
        nbytes = self.l.of3_attn_pair_bias_workspace_bytes(1, 1, N, apb.c_q, 0, 128, apb.no_heads, apb.c_hidden,
                                                           lib.dtype_code(dt), flags)
        ws = lib.workspace(nbytes, dev)
        lib._check(self.l.of3_attn_pair_bias_forward_prebias(
            a.data_ptr(), zb_all.data_ptr(), None, lib._ptr(m), a.data_ptr(), 1, 1, N, apb.c_q, 0, apb.no_heads,
            apb.c_hidden, float(apb.inf), lib.dtype_code(dt), flags, ctypes.byref(p), ws.data_ptr(), ws.numel(),
            self._st()), "of3_attn_pair_bias_forward_prebias")
        block.single_transition._run(s, single_mask if mask_trans else None, in_place=True)


# ----------------------------------------------------------------------------- orchestration
class DapPairFormerStack:
    """Runs a ``PairFormerStack`` with z row-sharded over ``world`` ranks.

    ``__call__(s, z, single_mask, pair_mask)`` takes the full (replicated) tensors of ONE sample
    ([1, N, C] / [1, N, N, C]) and returns the full updated (s, z) on every rank.
    """

    def __init__(self, stack, world: int, rank: int, group=None, ops=None):
        self.stack, self.world, self.rank, self.group = stack, world, rank, group
        self.ops = ops

    def shard(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        R = t.shape[dim] // self.world
        return t.narrow(dim, self.rank * R, R)

    def pair_block(self, z_loc, mask_rows, maskT_rows, pb, mask_trans=True):
        """One PairBlock on the local row shard (in place); returns the shard."""
        ops, P, g = self.ops, self.world, self.group
        # outgoing
        a_t, b_loc = ops.trimul_project(z_loc, mask_rows, pb.tri_mul_out)
        ops.trimul_finish(z_loc, a_t, all_gather_lines(b_loc, P, g), pb.tri_mul_out)
        # incoming: the projections come from the transposed shard, the update lands on the original rows
        zT = all_to_all_transpose(z_loc, P, g)
        a_t, b_loc = ops.trimul_project(zT, maskT_rows, pb.tri_mul_in)
        ops.trimul_finish(z_loc, a_t, all_gather_lines(b_loc, P, g), pb.tri_mul_in)
        # starting node
        qkv, tb_loc = ops.triattn_project(z_loc, pb.tri_att_start)
        ops.triattn_finish(z_loc, mask_rows, qkv, all_gather_lines(tb_loc, P, g), pb.tri_att_start)
        # ending node and transition on the transposed shard, then back
        zT = all_to_all_transpose(z_loc, P, g)
        qkv, tb_loc = ops.triattn_project(zT, pb.tri_att_end)
        ops.triattn_finish(zT, maskT_rows, qkv, all_gather_lines(tb_loc, P, g), pb.tri_att_end)
        ops.transition(zT, maskT_rows if mask_trans else None, pb.pair_transition)
        z_new = all_to_all_transpose(zT, P, g)
        z_loc.copy_(z_new)
        return z_loc

    def __call__(self, s, z, single_mask, pair_mask, _mask_trans=True):
        assert z.shape[0] == 1 and z.dim() == 4, "DAP runs one sample: z [1, N, N, C]"
        N = z.shape[1]
        assert N % self.world == 0, f"N_token {N} must be divisible by the {self.world} ranks"
        z_loc = self.shard(z[0]).contiguous().clone()
        s = s.clone(memory_format=torch.contiguous_format)
        pm = pair_mask[0].to(z.dtype)
        mask_rows = self.shard(pm, 0).contiguous()
        maskT_rows = self.shard(pm, 1).transpose(0, 1).contiguous()
        sm = None if single_mask is None else single_mask[0]
        for block in self.stack.blocks:
            self.pair_block(z_loc, mask_rows, maskT_rows, block.pair_stack, _mask_trans)
            zb_loc = self.ops.pair_bias_project(z_loc, block.attn_pair_bias)          # [H, R, N]
            zb_all = all_gather_lines(zb_loc, self.world, self.group)                  # [H, N, N]
            self.ops.single_track(s, zb_all, sm, block, _mask_trans)
        if self.world > 1:
            z_full = torch.empty((N,) + tuple(z_loc.shape[1:]), dtype=z_loc.dtype, device=z_loc.device)
            dist.all_gather_into_tensor(z_full, z_loc, group=self.group)
            z_full = z_full.reshape(1, N, N, z_loc.shape[-1])
        else:
            z_full = z_loc.unsqueeze(0)
        return s, z_full
