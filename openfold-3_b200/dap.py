"""Row-sharded ("DAP") Pairformer trunk over the GPUs of one node.

The pair tensor z[N, N, C] is split by rows over P ranks (P in 1, 2, 4, 8; N divisible by P); the
single representation and the masks are replicated. Per block (reference order,
openfold3/core/model/latent/base_blocks.py:453-478 and pairformer.py:177-211):

  tri_mul_out    project local rows -> a, b, channel-major, one group of 128/P channels per rank
                 | ALL-TO-ALL rows -> channels | contract this rank's channels over all rows
                 | ALL-TO-ALL channels -> rows | LayerNorm / linear / gate / residual on the local rows
  tri_mul_in     the same with a transposed walk of the projection kernel over the local rows
                 (a'[i, k] = a[k, i]): no transposed copy of z is needed
  tri_att_start  project q, k, v + local rows of the pair bias | ALL-GATHER bias | attention + finish
  tri_att_end    ALL-TO-ALL transpose of z -> the same on the transposed shard, in place there,
  transition     pointwise, still on the transposed shard | ALL-TO-ALL transpose back
  single track   pair-bias projection of the local rows (main stream), then on a SIDE stream:
                 attention of the local query rows against all keys, single transition on those rows.
                 z never depends on s, so the side stream runs concurrently with the next block's pair
                 stack; the updated rows of s are ALL-GATHERed on the main stream one block later.

Exchanging channel groups (each rank sends/receives ~3 N^2 C / P elements per update) replaces an
all-gather of b (N^2 C elements received by every rank, independent of P).

The reference has no model-parallel path (only data-parallel DDP / ZeRO), so this is new design
judged against the single-GPU result. Collectives go through ``torch.distributed`` (NCCL on GPUs,
gloo in the CPU tests); every remote tile is landed in local memory before a kernel reads it.
``ops`` is the compute backend: ``CudaOps`` (the C-ABI library) or, in the CPU tests, an oracle
backend with the same phase semantics, which lets the exchange logic be checked without a GPU.
"""

from __future__ import annotations

import contextlib
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


def exchange_blocks(x: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """x [world, ...]: block q goes to rank q; returns [world, ...] with block q received from rank q."""
    if world == 1:
        return x
    recv = torch.empty_like(x)
    dist.all_to_all_single(recv, x.contiguous(), group=group)
    return recv


def all_to_all_transpose(x_loc: torch.Tensor, world: int, group=None, ops=None) -> torch.Tensor:
    """Row shard [R, N, C] of X[N, N, C] -> row shard [R, N, C] of X^T (y[i, k] = X[k, r*R + i])."""
    if world == 1:
        return x_loc.transpose(0, 1).contiguous()
    R, N, C = x_loc.shape
    copy = getattr(ops, "copy_rows", None)
    e = x_loc.element_size()
    if copy is None:
        send = x_loc.view(R, world, R, C).permute(1, 0, 2, 3).contiguous()  # [dest][k_loc][i_loc][C]
    else:
        send = torch.empty((world, R, R, C), dtype=x_loc.dtype, device=x_loc.device)
        copy(x_loc, send, (1, world, R), (0, R * C * e, N * C * e), (0, R * R * C * e, R * C * e), R * C * e)
    recv = exchange_blocks(send, world, group)                              # [src][k_loc][i_loc][C]
    if copy is None:
        return recv.permute(2, 0, 1, 3).reshape(R, N, C).contiguous()
    out = torch.empty_like(x_loc)
    copy(recv, out, (world, R, R), (R * R * C * e, R * C * e, C * e), (R * C * e, C * e, N * C * e), C * e)
    return out


def regroup_ab(recv: torch.Tensor, N: int, R: int, incoming: bool, copy=None) -> torch.Tensor:
    """The received blocks of the rows -> channels exchange as the contraction's operands.

    outgoing: recv [P, 2, C, R, ld(N)]  (block = a source rank's R lines)      -> [2, C, N, ld(N)]
    incoming: recv [P, 2, C, N, ld(R)]  (block = a source rank's R positions k) -> [2, C, N, ld(N)]
    """
    P, _, C = recv.shape[:3]
    ldn = _pitch(N, 8)
    if P == 1:
        return recv.view(2, C, N, ldn)
    out = torch.empty((2, C, N, ldn), dtype=recv.dtype, device=recv.device)
    e = recv.element_size()
    if not incoming:
        if copy is None:
            out.view(2 * C, P, R, ldn).copy_(recv.view(P, 2 * C, R, ldn).permute(1, 0, 2, 3))
        else:
            copy(recv, out, (P, 2 * C, R), (2 * C * R * ldn * e, R * ldn * e, ldn * e),
                 (R * ldn * e, N * ldn * e, ldn * e), ldn * e)
    else:
        ldr = recv.shape[-1]
        if copy is None:
            src = recv.view(P, 2 * C, N, ldr)[..., :R].permute(1, 2, 0, 3).reshape(2 * C, N, N)
            out.view(2 * C, N, ldn)[:, :, :N].copy_(src)
        else:
            copy(recv, out, (P, 2 * C, N), (2 * C * N * ldr * e, N * ldr * e, ldr * e),
                 (R * e, N * ldn * e, ldn * e), R * e)
    return out


# ----------------------------------------------------------------------------- CUDA backend
class CudaOps:
    """Phase kernels of ``libof3b200.so`` on bf16 CUDA tensors (c_z = c_hidden = 128, 4 heads x 32)."""

    def __init__(self, device):
        self.device = device
        self.l = lib.load()
        self._side = None

    def _st(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # ---- streams: the single track runs on a side stream, ordered against the main one by events
    @contextlib.contextmanager
    def side(self):
        """Run the body on the side stream, after everything queued so far on the current stream."""
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        self._side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._side):
            yield

    def mark_side(self):
        """An event after everything queued so far on the side stream."""
        ev = torch.cuda.Event()
        ev.record(self._side)
        return ev

    def wait_mark(self, ev):
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    # ---- repack
    def copy_rows(self, src, dst, n, s, t, row_bytes):
        lib._check(self.l.of3_copy_rows_3d(src.data_ptr(), dst.data_ptr(), n[0], n[1], n[2], s[0], s[1], s[2], t[0],
                                           t[1], t[2], row_bytes, self._st()), "of3_copy_rows_3d")

    # ---- triangle update
    def trimul_project(self, z_loc, mask_rows, mod, world, incoming):
        """-> ab [world, 2, 128 / world, lines, ld]; see of3_dap_trimul_project."""
        R, N, _ = z_loc.shape
        lines, positions = (N, R) if incoming else (R, N)
        ld = _pitch(positions, 8)
        ab = torch.empty((world, 2, 128 // world, lines, ld), dtype=z_loc.dtype, device=z_loc.device)
        p = lib.TrimulParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_trimul_project(z_loc.data_ptr(), lib._ptr(mask_rows), ab.data_ptr(), lines,
                                                 positions, 1 if incoming else 0, world, ctypes.byref(p), self._st()),
                   "of3_dap_trimul_project")
        return ab

    def regroup_ab(self, recv, N, R, incoming):
        return regroup_ab(recv, N, R, incoming, copy=self.copy_rows)

    def trimul_contract(self, ab_all, N, R):
        """ab_all [2, C, N, ld] -> x_blocks [N / R, C, R, ld]."""
        C = ab_all.shape[1]
        xb = torch.empty((N // R, C, R, ab_all.shape[-1]), dtype=ab_all.dtype, device=ab_all.device)
        lib._check(self.l.of3_dap_trimul_contract(ab_all.data_ptr(), xb.data_ptr(), N, C, R, self._st()),
                   "of3_dap_trimul_contract")
        return xb

    def trimul_output(self, z_loc, x_t, mod):
        R, N, _ = z_loc.shape
        p = lib.TrimulParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_trimul_output(z_loc.data_ptr(), z_loc.data_ptr(), x_t.data_ptr(), R, N,
                                                lib.FLAG_ADD_RESIDUAL, ctypes.byref(p), self._st()),
                   "of3_dap_trimul_output")

    # ---- triangle attention
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

    # ---- single track
    def pair_bias_project(self, z_loc, apb, out=None):
        R, N, _ = z_loc.shape
        dt, dev = z_loc.dtype, z_loc.device
        prm = apb._params(dt, dev)
        ln_w, ln_b, w = prm[8], prm[9], prm[10]
        if out is None:
            out = torch.empty((16, R, N), dtype=torch.float32, device=dev)
        lib._check(self.l.of3_pair_bias_project(z_loc.data_ptr(), lib._ptr(ln_w), lib._ptr(ln_b), w.data_ptr(),
                                                out.data_ptr(), R * N, 128, 16, lib.dtype_code(dt), self._st()),
                   "of3_pair_bias_project")
        return out

    def single_rows(self, s_full, zb_rows, single_mask, block, row0, R, mask_trans=True):
        """Rows [row0, row0 + R) of the updated single representation: s_full [N, c_s] (all rows, for the
        keys and values), zb_rows [16, R, N] the projected pair bias of those rows (fp32) -> [R, c_s]."""
        apb = block.attn_pair_bias
        N = s_full.shape[0]
        dt, dev = s_full.dtype, s_full.device
        m = None if single_mask is None else single_mask.to(dt).reshape(N).contiguous()
        p = lib.AttnPairBiasParams(*[lib._ptr(t) for t in apb._params(dt, dev)])
        nbytes = self.l.of3_attn_pair_bias_rows_workspace_bytes(N, R, apb.c_q)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        out = torch.empty((R, apb.c_q), dtype=dt, device=dev)
        lib._check(self.l.of3_attn_pair_bias_forward_rows(
            s_full.data_ptr(), zb_rows.data_ptr(), lib._ptr(m), out.data_ptr(), N, row0, R, apb.c_q, apb.no_heads,
            apb.c_hidden, float(apb.inf), lib.dtype_code(dt), lib.FLAG_ADD_RESIDUAL, ctypes.byref(p), ws.data_ptr(),
            ws.numel(), self._st()), "of3_attn_pair_bias_forward_rows")
        mrows = None if (m is None or not mask_trans) else m[row0:row0 + R]
        block.single_transition._run(out, mrows, in_place=True)
        return out


# ----------------------------------------------------------------------------- orchestration
class DapPairFormerStack:
    """Runs a ``PairFormerStack`` with z row-sharded over ``world`` ranks.

    ``__call__(s, z, single_mask, pair_mask)`` takes the full (replicated) tensors of ONE sample
    ([1, N, C] / [1, N, N, C]) and returns the full updated (s, z) on every rank.
    Every collective is issued from the main stream on the one process group, in program order: the
    side stream carries kernels only, so no two communicators ever have to make progress at once (their
    relative order inside a CUDA graph is not ours to fix, and a different order on two ranks deadlocks).
    """

    def __init__(self, stack, world: int, rank: int, group=None, ops=None):
        assert world in (1, 2, 4, 8), "the triangle update splits its 128 channels over 1, 2, 4 or 8 ranks"
        self.stack, self.world, self.rank, self.group = stack, world, rank, group
        self.ops = ops

    def shard(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        R = t.shape[dim] // self.world
        return t.narrow(dim, self.rank * R, R)

    def _trimul(self, z_loc, mask_rows, mod, incoming: bool):
        ops, P, g = self.ops, self.world, self.group
        R, N, _ = z_loc.shape
        ab = ops.trimul_project(z_loc, mask_rows, mod, P, incoming)           # [P, 2, C, lines, ld]
        ab_all = ops.regroup_ab(exchange_blocks(ab, P, g), N, R, incoming)    # [2, C, N, ld]
        xb = ops.trimul_contract(ab_all, N, R)                                # [P, C, R, ld]
        x_t = exchange_blocks(xb, P, g)                                       # = [128, R, ld]
        ops.trimul_output(z_loc, x_t, mod)

    def pair_block(self, z_loc, mask_rows, maskT_rows, pb, mask_trans=True):
        """One PairBlock on the local row shard; returns the updated shard (a new tensor: the result of
        the transpose back; z_loc itself holds an intermediate state afterwards)."""
        ops, P, g = self.ops, self.world, self.group
        self._trimul(z_loc, mask_rows, pb.tri_mul_out, incoming=False)
        self._trimul(z_loc, mask_rows, pb.tri_mul_in, incoming=True)
        # starting node
        qkv, tb_loc = ops.triattn_project(z_loc, pb.tri_att_start)
        ops.triattn_finish(z_loc, mask_rows, qkv, all_gather_lines(tb_loc, P, g), pb.tri_att_start)
        # ending node and transition on the transposed shard, then back
        zT = all_to_all_transpose(z_loc, P, g, ops)
        qkv, tb_loc = ops.triattn_project(zT, pb.tri_att_end)
        ops.triattn_finish(zT, maskT_rows, qkv, all_gather_lines(tb_loc, P, g), pb.tri_att_end)
        ops.transition(zT, maskT_rows if mask_trans else None, pb.pair_transition)
        return all_to_all_transpose(zT, P, g, ops)

    def _gather_rows(self, s_rows):
        if self.world == 1:
            return s_rows
        full = torch.empty((self.world * s_rows.shape[0], s_rows.shape[1]), dtype=s_rows.dtype, device=s_rows.device)
        dist.all_gather_into_tensor(full, s_rows.contiguous(), group=self.group)
        return full

    def __call__(self, s, z, single_mask, pair_mask, _mask_trans=True):
        assert z.shape[0] == 1 and z.dim() == 4, "DAP runs one sample: z [1, N, N, C]"
        N = z.shape[1]
        assert N % self.world == 0, f"N_token {N} must be divisible by the {self.world} ranks"
        ops = self.ops
        R = N // self.world
        z_loc = self.shard(z[0]).contiguous().clone()
        s_full = s[0].clone(memory_format=torch.contiguous_format)
        pm = pair_mask[0].to(z.dtype)
        mask_rows = self.shard(pm, 0).contiguous()
        maskT_rows = self.shard(pm, 1).transpose(0, 1).contiguous()
        sm = None if single_mask is None else single_mask[0]
        side = getattr(ops, "side", contextlib.nullcontext)
        mark = getattr(ops, "mark_side", lambda: None)
        wait = getattr(ops, "wait_mark", lambda ev: None)
        zb_buf, zb_free = [None, None], [None, None]
        pending = None  # (rows of s updated on the side stream, event after them)
        for i, block in enumerate(self.stack.blocks):
            z_loc = self.pair_block(z_loc, mask_rows, maskT_rows, block.pair_stack, _mask_trans)
            slot = i & 1
            wait(zb_free[slot])  # the side stream has finished with this buffer (two blocks ago)
            zb_buf[slot] = ops.pair_bias_project(z_loc, block.attn_pair_bias, out=zb_buf[slot])   # [H, R, N]
            if pending is not None:  # the previous block's rows: long finished; gathered on the main stream
                wait(pending[1])
                s_full = self._gather_rows(pending[0])
            with side():
                s_rows = ops.single_rows(s_full, zb_buf[slot], sm, block, self.rank * R, R, _mask_trans)
                zb_free[slot] = mark()
            pending = (s_rows, zb_free[slot])
        if pending is not None:
            wait(pending[1])
            s_full = self._gather_rows(pending[0])
        if s_full.is_cuda and not torch.cuda.is_current_stream_capturing():
            s_full.record_stream(torch.cuda.current_stream(s_full.device))
        if self.world > 1:
            z_full = torch.empty((N,) + tuple(z_loc.shape[1:]), dtype=z_loc.dtype, device=z_loc.device)
            dist.all_gather_into_tensor(z_full, z_loc, group=self.group)
            z_full = z_full.reshape(1, N, N, z_loc.shape[-1])
        else:
            z_full = z_loc.unsqueeze(0)
        return s_full.unsqueeze(0), z_full


class GraphedDapRunner:
    """A ``DapPairFormerStack`` step captured once into a CUDA graph and replayed.

    A block is ~100 short launches and collectives; issued one by one from Python the host cannot keep
    P >= 2 GPUs busy (the per-rank kernels shrink with P, the host work does not). The graph holds the
    kernels of both streams and the NCCL collectives; replaying it costs one launch. Inputs are copied into the static buffers the graph reads; the returned tensors are the
    graph's static outputs (overwritten by the next replay). Every rank must capture and replay at
    the same points.
    """

    def __init__(self, runner: DapPairFormerStack, s, z, single_mask, pair_mask, warmup: int = 2):
        self.runner = runner
        self.s_in, self.z_in = s.clone(), z.clone()
        self.sm_in = None if single_mask is None else single_mask.clone()
        self.pm_in = pair_mask.clone()
        dev = z.device
        cur = torch.cuda.current_stream(dev)
        st = torch.cuda.Stream(dev)
        st.wait_stream(cur)
        with torch.cuda.stream(st), torch.no_grad():  # communicators, kernel attributes, workspaces: all set up eagerly
            for _ in range(max(1, warmup)):
                runner(self.s_in, self.z_in, self.sm_in, self.pm_in)
        cur.wait_stream(st)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.s_out, self.z_out = runner(self.s_in, self.z_in, self.sm_in, self.pm_in)

    def __call__(self, s, z, single_mask, pair_mask):
        for dst, src in ((self.s_in, s), (self.z_in, z), (self.sm_in, single_mask), (self.pm_in, pair_mask)):
            if dst is not None and src is not None and dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.s_out, self.z_out

    def release(self):
        """Drops the graph (and with it its hold on the communicator) and the static buffers."""
        self.graph.reset()
        self.graph = None
        self.s_out = self.z_out = self.s_in = self.z_in = self.sm_in = self.pm_in = None
