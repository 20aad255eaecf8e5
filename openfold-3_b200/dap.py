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


def triattn_bias_shape(R: int, N: int) -> tuple:
    """Shape (bf16) of the triangle-attention pair-bias image of R query rows and N keys: [4 heads x key
    blocks of 32][R][32] (of3_dap_triattn_bias_elems in the library)."""
    return (4 * ((N + 31) // 32), R, 32)


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
    def trimul_project(self, z_loc, mask_rows, mod, world, incoming, out=None):
        """-> ab [world, 2, 128 / world, lines, ld]; see of3_dap_trimul_project."""
        R, N, _ = z_loc.shape
        lines, positions = (N, R) if incoming else (R, N)
        ld = _pitch(positions, 8)
        shape = (world, 2, 128 // world, lines, ld)
        ab = torch.empty(shape, dtype=z_loc.dtype, device=z_loc.device) if out is None else out.view(shape)
        p = lib.TrimulParams(*[t.data_ptr() for t in mod._params(z_loc.dtype, z_loc.device)])
        lib._check(self.l.of3_dap_trimul_project(z_loc.data_ptr(), lib._ptr(mask_rows), ab.data_ptr(), lines,
                                                 positions, 1 if incoming else 0, world, ctypes.byref(p), self._st()),
                   "of3_dap_trimul_project")
        return ab

    def regroup_ab(self, recv, N, R, incoming):
        return regroup_ab(recv, N, R, incoming, copy=self.copy_rows)

    def trimul_contract(self, ab_all, N, R, out=None):
        """ab_all [2, C, N, ld] -> x_blocks [N / R, C, R, ld]."""
        C = ab_all.shape[1]
        shape = (N // R, C, R, ab_all.shape[-1])
        xb = torch.empty(shape, dtype=ab_all.dtype, device=ab_all.device) if out is None else out.view(shape)
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
    def triattn_project(self, z_loc, mod, out=None, row0=0):
        """row0: index of z_loc's first line among the N lines of the (possibly transposed) pair tensor."""
        R, N, _ = z_loc.shape
        dt, dev = z_loc.dtype, z_loc.device
        img = int(self.l.of3_dap_triattn_image_elems(R, N))  # opaque pre-swizzled operand tiles
        q = torch.empty(img, dtype=dt, device=dev)
        k = torch.empty(img, dtype=dt, device=dev)
        vt = torch.empty(img, dtype=dt, device=dev)
        shape = triattn_bias_shape(R, N)
        assert shape[0] * shape[1] * shape[2] == int(self.l.of3_dap_triattn_bias_elems(R, N))
        tb = torch.empty(shape, dtype=dt, device=dev) if out is None else out.view(shape)
        p = lib.TriattnParams(*[t.data_ptr() for t in mod._params(dt, dev)])
        lib._check(self.l.of3_dap_triattn_project(z_loc.data_ptr(), q.data_ptr(), k.data_ptr(), vt.data_ptr(),
                                                  tb.data_ptr(), R, N, row0, ctypes.byref(p), self._st()),
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

    def single_rows(self, s_full, zb_rows, single_mask, block, row0, R, mask_trans=True, out=None):
        """Rows [row0, row0 + R) of the updated single representation: s_full [N, c_s] (all rows, for the
        keys and values), zb_rows [16, R, N] the projected pair bias of those rows (fp32) -> [R, c_s]."""
        apb = block.attn_pair_bias
        N = s_full.shape[0]
        dt, dev = s_full.dtype, s_full.device
        m = None if single_mask is None else single_mask.to(dt).reshape(N).contiguous()
        p = lib.AttnPairBiasParams(*[lib._ptr(t) for t in apb._params(dt, dev)])
        nbytes = self.l.of3_attn_pair_bias_rows_workspace_bytes(N, R, apb.c_q)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        out = torch.empty((R, apb.c_q), dtype=dt, device=dev) if out is None else out.view(R, apb.c_q)
        lib._check(self.l.of3_attn_pair_bias_forward_rows(
            s_full.data_ptr(), zb_rows.data_ptr(), lib._ptr(m), out.data_ptr(), N, row0, R, apb.c_q, apb.no_heads,
            apb.c_hidden, float(apb.inf), lib.dtype_code(dt), lib.FLAG_ADD_RESIDUAL, ctypes.byref(p), ws.data_ptr(),
            ws.numel(), self._st()), "of3_attn_pair_bias_forward_rows")
        mrows = None if (m is None or not mask_trans) else m[row0:row0 + R]
        block.single_transition._run(out, mrows, in_place=True)
        return out


# ----------------------------------------------------------------------------- exchange strategies
class NcclExchange:
    """The exchanges as torch.distributed collectives (NCCL on GPUs, gloo in the CPU tests)."""

    def __init__(self, world: int, rank: int, group=None, ops=None):
        self.world, self.rank, self.group, self.ops = world, rank, group, ops

    def buf(self, name, shape, dtype, device):
        return None  # producers allocate their own outputs

    def begin(self):
        pass

    def ab_all(self, ab, N, R, incoming):
        return self.ops.regroup_ab(exchange_blocks(ab, self.world, self.group), N, R, incoming)

    def x_rows(self, xb):
        P, C, R, ld = xb.shape
        return exchange_blocks(xb, self.world, self.group).view(P * C, R, ld)

    def transpose(self, z_loc, dst_name, rider=None):
        """``rider``: (rows of s, event after their producer) to gather in the same breath (see PeerExchange)."""
        out = all_to_all_transpose(z_loc, self.world, self.group, self.ops)
        self.rider_result = None
        if rider is not None:
            getattr(self.ops, "wait_mark", lambda ev: None)(rider[1])
            self.rider_result = self.gather_rows(rider[0])
        return out

    def gather_lines(self, x_loc):
        return all_gather_lines(x_loc, self.world, self.group)

    def gather_rows(self, s_rows):
        if self.world == 1:
            return s_rows
        full = torch.empty((self.world * s_rows.shape[0], s_rows.shape[1]), dtype=s_rows.dtype, device=s_rows.device)
        dist.all_gather_into_tensor(full, s_rows.contiguous(), group=self.group)
        return full


class _RawDeviceMemory:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerHeap:
    """This rank's peer heap and the mapped heaps of the other ranks of the node (see csrc/peer.cu).

    ``bases[r]`` is the address, in this process, of rank r's heap. Regions are handed out by a bump
    allocator keyed by name; every rank requests the same names and sizes in the same order, so a name
    has the same offset everywhere.
    """

    def __init__(self, nbytes: int, world: int, rank: int, device, group=None):
        self.l = lib.load()
        self.world, self.rank, self.device, self.nbytes = world, rank, device, int(nbytes)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        lib._check(self.l.of3_peer_heap_alloc(self.nbytes, ctypes.byref(ptr), handle), "of3_peer_heap_alloc")
        self._own = ptr.value
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.bases = []
        for r in range(world):
            if r == rank:
                self.bases.append(self._own)
            else:
                q = ctypes.c_void_p()
                lib._check(self.l.of3_peer_heap_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(q)),
                           "of3_peer_heap_open")
                self.bases.append(q.value)
        self._finish_init()

    def _finish_init(self):
        self.local = torch.as_tensor(_RawDeviceMemory(self.bases[self.rank], self.nbytes), device=self.device)
        self.regions, self.top = {}, 256  # bytes [0, 64) are the barrier's flag block
        self.c_bases = (ctypes.c_void_p * self.world)(*self.bases)

    def region(self, name: str, nbytes: int) -> int:
        if name not in self.regions:
            off = self.top
            self.top = (off + nbytes + 255) // 256 * 256
            if self.top > self.nbytes:
                raise RuntimeError(f"peer heap of {self.nbytes} bytes is too small for region {name!r} ({nbytes} bytes)")
            self.regions[name] = (off, nbytes)
        off, size = self.regions[name]
        if nbytes > size:
            raise RuntimeError(f"peer heap region {name!r} holds {size} bytes, {nbytes} requested")
        return off

    def tensor(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = self.region(name, nbytes)
        return self.local[off:off + nbytes].view(dtype).view(*shape)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.bases[self.rank]
        assert 0 <= off < self.nbytes, "tensor does not live in the peer heap"
        return off

    def close(self):
        for r, b in enumerate(self.bases):
            if r != self.rank and b is not None:
                self.l.of3_peer_heap_close(ctypes.c_void_p(b))
        if getattr(self, "_own", None):
            self.l.of3_peer_heap_free(ctypes.c_void_p(self._own))
            self._own = None
        self.bases = []


class LocalPeerHeaps:
    """P heaps inside ONE process (virtual ranks on one GPU, for tests): ``view(r)`` is rank r's PeerHeap-like
    object. The barrier between production and pulls is the host's program order, not a kernel."""

    def __init__(self, nbytes: int, world: int, device):
        self.store = [torch.zeros(int(nbytes), dtype=torch.uint8, device=device) for _ in range(world)]
        self.world, self.device, self.nbytes = world, device, int(nbytes)

    def view(self, rank: int) -> PeerHeap:
        h = PeerHeap.__new__(PeerHeap)
        h.l = lib.load()
        h.world, h.rank, h.device, h.nbytes = self.world, rank, self.device, self.nbytes
        h.bases = [t.data_ptr() for t in self.store]
        h._own = None
        h._finish_init()
        return h


class PeerExchange:
    """The exchanges as barrier + pull over NVLink peer memory: one kernel moves the data from the peers'
    heaps into the layout the next kernel reads (all-to-all / all-gather and repack fused)."""

    def __init__(self, heap: PeerHeap, ops, barrier: bool = True):
        self.heap, self.ops, self.world, self.rank = heap, ops, heap.world, heap.rank
        self.use_barrier = barrier
        self.l = lib.load()

    def buf(self, name, shape, dtype, device):
        return self.heap.tensor(name, shape, dtype)

    def begin(self):
        """Start of a step: the peers have finished reading the previous step's buffers. The ranks' hosts may
        reach this point far apart (data loading, a first graph replay), so this barrier alone has a long limit."""
        if self.use_barrier and self.world > 1:
            lib._check(self.l.of3_peer_barrier_step_entry(self.heap.c_bases, self.world, self.rank, self.ops._st()),
                       "of3_peer_barrier_step_entry")

    def barrier(self):
        if self.use_barrier and self.world > 1:
            lib._check(self.l.of3_peer_barrier(self.heap.c_bases, self.world, self.rank, self.ops._st()),
                       "of3_peer_barrier")

    def _pull(self, src_off, dst, n1, n2, s1, s2, t0, t1, t2, row_bytes):
        lib._check(self.l.of3_peer_pull_rows(self.heap.c_bases, src_off, dst.data_ptr(), self.world, self.rank, n1, n2,
                                             s1, s2, t0, t1, t2, row_bytes, self.ops._st()), "of3_peer_pull_rows")

    def ab_all(self, ab, N, R, incoming):
        P, _, C, lines, ld = ab.shape
        e = ab.element_size()
        ldn = _pitch(N, 8)
        out = torch.empty((2, C, N, ldn), dtype=ab.dtype, device=ab.device)
        self.barrier()
        off = self.heap.offset_of(ab) + self.rank * (2 * C * lines * ld * e)  # the block each source holds for me
        if not incoming:   # source block [2C][R][ldn] -> out[2C][src*R + r][ldn]
            self._pull(off, out, 2 * C, R, R * ldn * e, ldn * e, R * ldn * e, N * ldn * e, ldn * e, ldn * e)
        else:              # source block [2C][N][ld(R)] -> out[2C][i][src*R + k]
            self._pull(off, out, 2 * C, N, N * ld * e, ld * e, R * e, N * ldn * e, ldn * e, R * e)
        return out

    def x_rows(self, xb):
        P, C, R, ld = xb.shape
        e = xb.element_size()
        out = torch.empty((P * C, R, ld), dtype=xb.dtype, device=xb.device)
        blk = C * R * ld * e
        self.barrier()
        self._pull(self.heap.offset_of(xb) + self.rank * blk, out, 1, 1, 0, 0, blk, 0, 0, blk)
        return out

    def transpose(self, z_loc, dst_name, rider=None):
        """``rider``: (rows of s written by an earlier kernel of another stream, event after it). The main stream
        waits for the event BEFORE this exchange's barrier, so once the barrier has been passed every rank's rows
        are complete and they are pulled without a barrier of their own (one barrier less per block)."""
        R, N, C = z_loc.shape
        e = z_loc.element_size()
        out = self.heap.tensor(dst_name, (R, N, C), z_loc.dtype)
        if rider is not None:
            getattr(self.ops, "wait_mark", lambda ev: None)(rider[1])
        self.barrier()
        # out[i_loc][src*R + k_loc][:] = z_src[k_loc][rank*R + i_loc][:]; rows (src, k_loc, i_loc) of C elements
        self._pull(self.heap.offset_of(z_loc) + self.rank * R * C * e, out, R, R, N * C * e, C * e, R * C * e, C * e,
                   N * C * e, C * e)
        self.rider_result = None
        if rider is not None:
            self.rider_result = self.gather_rows(rider[0], barrier=False)
        return out

    def gather_lines(self, x_loc):
        G, R, L = x_loc.shape
        e = x_loc.element_size()
        out = torch.empty((G, self.world * R, L), dtype=x_loc.dtype, device=x_loc.device)
        self.barrier()
        self._pull(self.heap.offset_of(x_loc), out, G, R, R * L * e, L * e, R * L * e, self.world * R * L * e, L * e,
                   L * e)
        return out

    def gather_rows(self, s_rows, barrier=True):
        R, c = s_rows.shape
        e = s_rows.element_size()
        out = torch.empty((self.world * R, c), dtype=s_rows.dtype, device=s_rows.device)
        if barrier:
            self.barrier()
        self._pull(self.heap.offset_of(s_rows), out, 1, 1, 0, 0, R * c * e, 0, 0, R * c * e)
        return out

    @staticmethod
    def heap_bytes(N: int, world: int, c_s: int = 384) -> int:
        """Bytes of peer heap one rank needs for a Pairformer trunk at N tokens (bf16)."""
        R = N // world
        ld = _pitch(N, 8)
        ab = 2 * 128 * max(R * ld, N * _pitch(R, 8)) * 2
        g, r, w = triattn_bias_shape(R, N)
        return 2 * R * N * 128 * 2 + ab + 128 * R * ld * 2 + g * r * w * 2 + 2 * R * c_s * 2 + 16 * 256 + 4096


# ----------------------------------------------------------------------------- orchestration
class DapPairFormerStack:
    """Runs a ``PairFormerStack`` with z row-sharded over ``world`` ranks.

    ``__call__(s, z, single_mask, pair_mask)`` takes the full (replicated) tensors of ONE sample
    ([1, N, C] / [1, N, N, C]) and returns the full updated (s, z) on every rank.
    ``exchange``: how shards move between ranks -- ``NcclExchange`` (default) or ``PeerExchange``.
    Every exchange is issued from the main stream, in program order: the side stream carries kernels
    only, so no two communicators (or barriers) ever have to make progress at once.
    """

    def __init__(self, stack, world: int, rank: int, group=None, ops=None, exchange=None):
        assert world in (1, 2, 4, 8), "the triangle update splits its 128 channels over 1, 2, 4 or 8 ranks"
        self.stack, self.world, self.rank, self.group = stack, world, rank, group
        self.ops = ops
        self.x = exchange if exchange is not None else NcclExchange(world, rank, group, ops)
        self.check_status = True  # eager steps end with a (synchronising) read of the device status block

    def shard(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        R = t.shape[dim] // self.world
        return t.narrow(dim, self.rank * R, R)

    def _trimul(self, z_loc, mask_rows, mod, incoming: bool):
        ops, P, X = self.ops, self.world, self.x
        R, N, _ = z_loc.shape
        lines, pos = (N, R) if incoming else (R, N)
        C, dt, dev = 128 // P, z_loc.dtype, z_loc.device
        ld = _pitch(pos, 8)
        # one region serves both directions: lines x pitch differs between them
        ab_buf = X.buf("ab", (2 * 128 * max(R * _pitch(N, 8), N * _pitch(R, 8)),), dt, dev)
        ab_out = None if ab_buf is None else ab_buf[:2 * 128 * lines * ld].view(P, 2, C, lines, ld)
        ab = ops.trimul_project(z_loc, mask_rows, mod, P, incoming, out=ab_out)              # [P, 2, C, lines, ld]
        ab_all = X.ab_all(ab, N, R, incoming)                                                # [2, C, N, ld]
        xb = ops.trimul_contract(ab_all, N, R, out=X.buf("xb", (P, C, R, _pitch(N, 8)), dt, dev))  # [P, C, R, ld]
        ops.trimul_output(z_loc, X.x_rows(xb), mod)                                          # x_t [128, R, ld]

    def _triattn(self, z_loc, mask_rows, mod):
        ops, X = self.ops, self.x
        R, N, _ = z_loc.shape
        qkv, tb_loc = ops.triattn_project(z_loc, mod, out=X.buf("tb", triattn_bias_shape(R, N), z_loc.dtype, z_loc.device),
                                          row0=self.rank * R)
        ops.triattn_finish(z_loc, mask_rows, qkv, X.gather_lines(tb_loc), mod)

    def pair_block(self, z_loc, mask_rows, maskT_rows, pb, mask_trans=True, rider=None):
        """One PairBlock on the local row shard; returns the updated shard (the result of the transpose
        back: with collectives a new tensor, z_loc itself then holds an intermediate state). ``rider``: the previous
        block's rows of s, gathered together with the last exchange (result in ``self.x.rider_result``)."""
        self._trimul(z_loc, mask_rows, pb.tri_mul_out, incoming=False)
        self._trimul(z_loc, mask_rows, pb.tri_mul_in, incoming=True)
        self._triattn(z_loc, mask_rows, pb.tri_att_start)
        # ending node and transition on the transposed shard, then back
        zT = self.x.transpose(z_loc, "z1")
        self._triattn(zT, maskT_rows, pb.tri_att_end)
        self.ops.transition(zT, maskT_rows if mask_trans else None, pb.pair_transition)
        if rider is None:
            return self.x.transpose(zT, "z0")
        return self.x.transpose(zT, "z0", rider=rider)

    def __call__(self, s, z, single_mask, pair_mask, _mask_trans=True, sharded: bool = False):
        """Replicated interface (default): z [1, N, N, C] and pair_mask [1, N, N] whole on every rank; returns the
        whole updated (s, z) on every rank.
        ``sharded=True``: z is this rank's rows [1, R, N, C], pair_mask a pair (rows [R, N] of the mask, rows
        [R, N] of its transpose); returns (s, this rank's rows of z [1, R, N, C]) -- nothing of size N^2 is
        replicated or gathered."""
        assert z.shape[0] == 1 and z.dim() == 4, "DAP runs one sample: z [1, N, N, C]"
        N = z.shape[2]
        assert N % self.world == 0, f"N_token {N} must be divisible by the {self.world} ranks"
        ops, X = self.ops, self.x
        R = N // self.world
        assert z.shape[1] == (R if sharded else N)
        X.begin()
        z_in = z[0] if sharded else self.shard(z[0])
        z_loc = X.buf("z0", (R, N, z.shape[-1]), z.dtype, z.device)
        if z_loc is None:
            z_loc = z_in.contiguous().clone()
        else:
            z_loc.copy_(z_in)
        s_full = None if s is None else s[0].clone(memory_format=torch.contiguous_format)
        if sharded:
            mask_rows, maskT_rows = (m.to(z.dtype).contiguous() for m in pair_mask)
        else:
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
            # a PairFormerBlock (pair stack + single track) or a bare PairBlock (pair stack only: s is None)
            pair_stack = getattr(block, "pair_stack", block)
            # the previous block's rows of s (long finished on the side stream) ride on this block's last exchange
            z_loc = self.pair_block(z_loc, mask_rows, maskT_rows, pair_stack, _mask_trans, rider=pending)
            if pending is not None:
                s_full, pending = X.rider_result, None
            if s_full is None or not hasattr(block, "attn_pair_bias"):
                continue
            slot = i & 1
            wait(zb_free[slot])  # the side stream has finished with this buffer (two blocks ago)
            zb_buf[slot] = ops.pair_bias_project(z_loc, block.attn_pair_bias, out=zb_buf[slot])   # [H, R, N]
            with side():
                s_rows = ops.single_rows(s_full, zb_buf[slot], sm, block, self.rank * R, R, _mask_trans,
                                         out=X.buf(f"s{slot}", (R, s.shape[-1]), s.dtype, s.device))
                zb_free[slot] = mark()
            pending = (s_rows, zb_free[slot])
        if pending is not None:
            wait(pending[1])
            s_full = X.gather_rows(pending[0])
        if s_full is not None and s_full.is_cuda and not torch.cuda.is_current_stream_capturing():
            s_full.record_stream(torch.cuda.current_stream(s_full.device))
        if s_full is None:
            if sharded:
                return self._checked(None, z_loc.unsqueeze(0))
            return self._checked(None, X.gather_rows(z_loc.view(R, -1)).view(1, N, N, z_loc.shape[-1]))
        if sharded:
            return self._checked(s_full.unsqueeze(0), z_loc.unsqueeze(0))
        z_full = X.gather_rows(z_loc.view(R, -1)).view(1, N, N, z_loc.shape[-1])
        return self._checked(s_full.unsqueeze(0), z_full)

    def _checked(self, s_out, z_out):
        """End of an eager step on a GPU: a bounded device-side wait that ran out (a peer that never reached a
        barrier, a stalled pipeline) raises here instead of handing back a half-exchanged result. Synchronises;
        a captured step is checked by its replayer (GraphedDapRunner) one step late instead."""
        if z_out.is_cuda and not torch.cuda.is_current_stream_capturing() and self.check_status:
            lib.check_device_status()
        return s_out, z_out


class GraphedDapRunner:
    """A ``DapPairFormerStack`` step captured once into a CUDA graph and replayed.

    A block is ~100 short launches and collectives; issued one by one from Python the host cannot keep
    P >= 2 GPUs busy (the per-rank kernels shrink with P, the host work does not). The graph holds the
    kernels of both streams and the NCCL collectives; replaying it costs one launch. Inputs are copied into the static buffers the graph reads; the returned tensors are the
    graph's static outputs (overwritten by the next replay). Every rank must capture and replay at
    the same points.
    """

    def __init__(self, runner: DapPairFormerStack, s, z, single_mask, pair_mask, warmup: int = 2,
                 sharded: bool = False):
        self.runner, self.sharded = runner, sharded
        self.s_in, self.z_in = (None if s is None else s.clone()), z.clone()
        self.sm_in = None if single_mask is None else single_mask.clone()
        self.pm_in = tuple(m.clone() for m in pair_mask) if sharded else pair_mask.clone()
        dev = z.device
        cur = torch.cuda.current_stream(dev)
        st = torch.cuda.Stream(dev)
        st.wait_stream(cur)
        with torch.cuda.stream(st), torch.no_grad():  # communicators, kernel attributes, workspaces: all set up eagerly
            for _ in range(max(1, warmup)):
                runner(self.s_in, self.z_in, self.sm_in, self.pm_in, sharded=sharded)
        cur.wait_stream(st)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.s_out, self.z_out = runner(self.s_in, self.z_in, self.sm_in, self.pm_in, sharded=sharded)
        # status of each replay, copied stream-ordered into pinned memory and looked at before the next replay
        self._status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._status_ready = None

    def __call__(self, s, z, single_mask, pair_mask):
        pairs = [(self.s_in, s), (self.z_in, z), (self.sm_in, single_mask)]
        pairs += list(zip(self.pm_in, pair_mask)) if self.sharded else [(self.pm_in, pair_mask)]
        for dst, src in pairs:
            if dst is not None and src is not None and dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.check(wait=False)
        self.graph.replay()
        l = lib.load()
        st = torch.cuda.current_stream(self.z_in.device)
        lib._check(l.of3_device_status_async(self._status.data_ptr(), st.cuda_stream), "of3_device_status_async")
        self._status_ready = torch.cuda.Event()
        self._status_ready.record(st)
        return self.s_out, self.z_out

    def check(self, wait: bool = True):
        """Raises if a device-side wait of an earlier replay ran out (e.g. a rank that never reached a barrier):
        the outputs of that replay are not to be used. Called without waiting before every replay, so a failure
        surfaces at most one step late; call it with ``wait=True`` before consuming the last step's result."""
        if self._status_ready is None:
            return
        if wait:
            self._status_ready.synchronize()
        elif not self._status_ready.query():
            return
        self._status_ready = None
        if int(self._status[0]) != 0:
            code = [int(v) for v in self._status]
            lib.load().of3_device_status_clear()
            raise RuntimeError(f"device-side wait ran out during a replayed step: code {code[0]}, kernel {code[1]}, "
                               f"block {code[2]}, site {code[3]}")

    def release(self):
        """Drops the graph (and with it its hold on the communicator) and the static buffers."""
        self.graph.reset()
        self.graph = None
        self.s_out = self.z_out = self.s_in = self.z_in = self.sm_in = self.pm_in = None
