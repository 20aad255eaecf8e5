"""Row-sharded (DAP) orchestration on CPU: two gloo ranks with an oracle compute backend.

The exchange logic of ``openfold3_b200.dap`` (row shards, the rows <-> channels all-to-alls around the
triangle contraction, all-gathers of the attention bias, all-to-all transposes for the ending-node
attention, the query-sharded single track) is backend independent; here the per-phase compute is the CPU oracle, so the test
checks that sharding + collectives reproduce the unsharded oracle bit-for-rounding, without a GPU.
"""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


class OracleOps:
    """The phase semantics of dap.CudaOps restated with the CPU oracle (fp32)."""

    def __init__(self, oracle):
        self.o = oracle

    @staticmethod
    def _P(mod):
        return {k: v.detach() for k, v in mod.state_dict().items()}

    @staticmethod
    def _pad(t, ld):
        return F.pad(t, (0, ld - t.shape[-1]))

    def trimul_project(self, z_loc, mask_rows, mod, world, incoming, out=None):
        P, o = self._P(mod), self.o
        zn = o._ln(z_loc, P, "layer_norm_in.", z_loc.shape[-1])
        m = mask_rows.unsqueeze(-1)
        a = m * torch.sigmoid(o._lin(zn, P, "linear_a_g.")) * o._lin(zn, P, "linear_a_p.")
        b = m * torch.sigmoid(o._lin(zn, P, "linear_b_g.")) * o._lin(zn, P, "linear_b_p.")
        # channel-major planes [c][line][position]; incoming: a line runs along the local rows
        perm = (2, 1, 0) if incoming else (2, 0, 1)
        a, b = a.permute(*perm), b.permute(*perm)
        ld = (a.shape[-1] + 7) // 8 * 8
        ab = torch.stack([self._pad(a, ld), self._pad(b, ld)])                       # [2, 128, lines, ld]
        C = 128 // world
        return ab.view(2, world, C, ab.shape[2], ld).permute(1, 0, 2, 3, 4).contiguous()  # [P, 2, C, lines, ld]

    def regroup_ab(self, recv, N, R, incoming):
        import cases
        return cases.pkg.dap.regroup_ab(recv, N, R, incoming)

    def trimul_contract(self, ab_all, N, R, out=None):
        x = torch.einsum("cik,cjk->cij", ab_all[0][:, :, :N], ab_all[1][:, :, :N])    # [C, N, N]
        x = self._pad(x, ab_all.shape[-1])
        C = x.shape[0]
        return x.view(C, N // R, R, x.shape[-1]).permute(1, 0, 2, 3).contiguous()     # [P, C, R, ld]

    def trimul_output(self, z_loc, x_t, mod):
        P, o = self._P(mod), self.o
        R, N, _ = z_loc.shape
        x = x_t.reshape(128, R, -1)[:, :, :N].permute(1, 2, 0)
        x = o._lin(o._ln(x, P, "layer_norm_out.", x.shape[-1]), P, "linear_z.")
        g = torch.sigmoid(o._lin(o._ln(z_loc, P, "layer_norm_in.", z_loc.shape[-1]), P, "linear_g."))
        z_loc += x * g

    def triattn_project(self, z_loc, mod, out=None, row0=0):
        P, o = self._P(mod), self.o
        N = z_loc.shape[1]
        xn = o._ln(z_loc, P, "layer_norm.", z_loc.shape[-1])
        tb = o._lin(xn, P, "linear_z.").permute(2, 0, 1)
        return (xn,), self._pad(tb, (N + 63) // 64 * 64).contiguous()

    def triattn_finish(self, z_loc, mask_rows, qkv, tb_all, mod):
        P, o = self._P(mod), self.o
        N = z_loc.shape[1]
        (xn,) = qkv
        mask_bias = (mod.inf * (mask_rows - 1))[:, None, None, :]
        tb = tb_all[:, :, :N].unsqueeze(0)
        mha = {k[len("mha."):]: v for k, v in P.items() if k.startswith("mha.")}
        z_loc += o.attention(xn, xn, [mask_bias, tb], mha, "", mod.no_heads)

    def transition(self, x_rows, mask_rows, mod):
        x_rows += self.o.swiglu_transition(x_rows, mask_rows, self._P(mod), "")

    def pair_bias_project(self, z_loc, apb, out=None):
        P, o = self._P(apb), self.o
        return o._lin(o._ln(z_loc, P, "layer_norm_z.", z_loc.shape[-1]), P, "linear_z.").permute(2, 0, 1).contiguous()

    def single_rows(self, s_full, zb_rows, single_mask, block, row0, R, mask_trans=True, out=None):
        apb, o = block.attn_pair_bias, self.o
        P = self._P(apb)
        an = o._ln(s_full, P, "layer_norm_a.", s_full.shape[-1])
        mask_bias = (apb.inf * (single_mask - 1))[None, None, :]
        mha = {k[len("mha."):]: v for k, v in P.items() if k.startswith("mha.")}
        rows = s_full[row0:row0 + R] + o.attention(an[row0:row0 + R], an, [mask_bias, zb_rows], mha, "", apb.no_heads)
        m = single_mask[row0:row0 + R] if mask_trans else None
        return rows + o.swiglu_transition(rows, m, self._P(block.single_transition), "")


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _worker(rank, world, port, n_token, n_blocks, result_file):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cases
        from oracle import pairformer_oracle as oracle

        pkg = cases.pkg
        torch.manual_seed(0)
        g = torch.Generator().manual_seed(5)
        s = torch.randn(1, n_token, 384, generator=g)
        z = torch.randn(1, n_token, n_token, 128, generator=g)
        sm = cases.rand_mask((1, n_token), g)
        pm = cases.rand_mask((1, n_token, n_token), g)  # not an outer product, not symmetric
        P = pkg.weights.pairformer_stack_params(seed=3, no_blocks=n_blocks, final_std=None, **cases.OF3)
        stack = pkg.PairFormerStack(**cases.OF3, no_blocks=n_blocks, transition_type="swiglu", pair_dropout=0.25,
                                    fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
        stack.load_state_dict(P, strict=True)
        stack.eval()
        runner = pkg.dap.DapPairFormerStack(stack, world, rank, ops=OracleOps(oracle))
        with torch.no_grad():
            s_d, z_d = runner(s, z, sm, pm)
            s_r, z_r = oracle.pairformer_stack(s, z, sm, pm, P, "", n_blocks, 4, 16)
            # sharded interface: only this rank's rows go in and come out
            R = n_token // world
            rows = slice(rank * R, (rank + 1) * R)
            s_s, z_s = runner(s, z[:, rows].contiguous(), sm, (pm[0, rows], pm[0][:, rows].t()), sharded=True)
            assert torch.equal(s_s, s_d) and torch.equal(z_s, z_d[:, rows])
        es, ez = cases.rel_err(s_d, s_r), cases.rel_err(z_d, z_r)
        # every rank must hold the same full result
        gathered = [None] * world
        dist.all_gather_object(gathered, (float(es), float(ez), float(z_d.double().sum())))
        if rank == 0:
            torch.save(gathered, result_file)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_token", [(2, 16), (4, 12)])
def test_dap_orchestration_matches_unsharded_oracle(tmp_path, world, n_token):
    result = tmp_path / "res.pt"
    mp.spawn(_worker, args=(world, _free_port(), n_token, 2, str(result)), nprocs=world, join=True)
    gathered = torch.load(result)
    assert len(gathered) == world
    for es, ez, _ in gathered:
        assert es < 1e-4 and ez < 1e-4, gathered
    sums = [g[2] for g in gathered]
    assert max(sums) - min(sums) < 1e-6 * max(1.0, abs(sums[0]))


def test_all_to_all_transpose_single_rank():
    import cases

    dap = cases.pkg.dap
    x = torch.randn(6, 6, 3)
    assert torch.equal(dap.all_to_all_transpose(x, 1), x.transpose(0, 1))
    y = torch.randn(5, 4, 7)
    assert torch.equal(dap.all_gather_lines(y, 1), y)


@pytest.mark.parametrize("world,n_token", [(2, 768), (4, 768), (8, 768), (8, 2048), (2, 66)])
def test_peer_heap_layout_fits_and_is_deterministic(world, n_token):
    """The named regions a step requests (same order on every rank) fit the size PeerExchange.heap_bytes
    promises, do not overlap, and get the same offsets on every rank. No GPU: only the bump allocator."""
    import cases

    dap = cases.pkg.dap
    R = n_token // world
    ld = dap._pitch(n_token, 8)
    tb = dap.triattn_bias_shape(R, n_token)
    requests = [("z0", R * n_token * 128 * 2), ("ab", 2 * 128 * max(R * ld, n_token * dap._pitch(R, 8)) * 2),
                ("xb", 128 * R * ld * 2), ("tb", tb[0] * tb[1] * tb[2] * 2), ("z1", R * n_token * 128 * 2),
                ("s0", R * 384 * 2), ("s1", R * 384 * 2)]
    layouts = []
    for rank in range(world):
        h = dap.PeerHeap.__new__(dap.PeerHeap)
        h.nbytes, h.regions, h.top = dap.PeerExchange.heap_bytes(n_token, world), {}, 256
        offs = [h.region(name, nbytes) for name, nbytes in requests]
        assert [h.region(name, nbytes) for name, nbytes in requests] == offs  # asking again returns the same region
        spans = sorted((o, o + n) for o, (_, n) in zip(offs, requests))
        assert spans[0][0] >= 64 and all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= h.nbytes
        assert all(o % 256 == 0 for o in offs)
        layouts.append(offs)
    assert all(l == layouts[0] for l in layouts)
    h = dap.PeerHeap.__new__(dap.PeerHeap)
    h.nbytes, h.regions, h.top = 4096, {}, 256
    with pytest.raises(RuntimeError, match="too small"):
        h.region("big", 1 << 20)
