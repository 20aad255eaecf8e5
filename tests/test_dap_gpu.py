"""Row-shard phase kernels on one GPU: the DAP orchestration with the CUDA backend, (a) as a single
rank and (b) with P virtual ranks whose exchanges are done by local concatenation, both against the
unsharded drop-in stack (same kernels, whole tensor) and the CPU oracle."""

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _exchange(blocks):
    """all_to_all_single among virtual ranks: blocks[r][q] goes to rank q as its block r."""
    P = len(blocks)
    return [torch.stack([blocks[src][dst] for src in range(P)]) for dst in range(P)]


def _virtual_pair_block(ops, shards, mask, pb, P):
    """dap.DapPairFormerStack.pair_block for P shards held on one device."""
    R, N = shards[0].shape[0], shards[0].shape[1]
    mrow = [mask[r * R:(r + 1) * R].contiguous() for r in range(P)]
    mcol = [mask[:, r * R:(r + 1) * R].t().contiguous() for r in range(P)]

    def transpose_all(sh):
        full = torch.cat(sh, 0).transpose(0, 1).contiguous()
        return [full[r * R:(r + 1) * R].contiguous() for r in range(P)]

    def gather(parts):
        return torch.cat(parts, 1).contiguous()

    for mod, incoming in ((pb.tri_mul_out, False), (pb.tri_mul_in, True)):
        ab = [ops.trimul_project(shards[r], mrow[r], mod, P, incoming) for r in range(P)]
        recv = _exchange(ab) if P > 1 else ab
        xb = [ops.trimul_contract(ops.regroup_ab(recv[r], N, R, incoming), N, R) for r in range(P)]
        x_t = _exchange(xb) if P > 1 else xb
        for r in range(P):
            ops.trimul_output(shards[r], x_t[r], mod)
    proj = [ops.triattn_project(shards[r], pb.tri_att_start, row0=r * R) for r in range(P)]
    tb_all = gather([p[1] for p in proj])
    for r in range(P):
        ops.triattn_finish(shards[r], mrow[r], proj[r][0], tb_all, pb.tri_att_start)
    zT = transpose_all(shards)
    proj = [ops.triattn_project(zT[r], pb.tri_att_end, row0=r * R) for r in range(P)]
    tb_all = gather([p[1] for p in proj])
    for r in range(P):
        ops.triattn_finish(zT[r], mcol[r], proj[r][0], tb_all, pb.tri_att_end)
        ops.transition(zT[r], mcol[r], pb.pair_transition)
    return transpose_all(zT)


@pytest.mark.parametrize("P,N", [(1, 40), (2, 48), (4, 200), (8, 96), (2, 66)])
def test_row_shard_kernels_match_whole_tensor(pkg, P, N):
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(N)
    z = torch.randn(1, N, N, 128, generator=g)
    s = torch.randn(1, N, 384, generator=g)
    pm = cases.rand_mask((1, N, N), g)
    sm = cases.rand_mask((1, N), g)
    Pw = pkg.weights.pairformer_stack_params(seed=4, no_blocks=1, final_std=None, **cases.OF3)
    stack = pkg.PairFormerStack(**cases.OF3, no_blocks=1, transition_type="swiglu", pair_dropout=0.25,
                                fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
    stack.load_state_dict(Pw, strict=True)
    stack = stack.to(dev, bf).eval()
    ops = pkg.dap.CudaOps(dev)
    zd, sd, pmd, smd = z.to(dev, bf), s.to(dev, bf), pm.to(dev, bf), sm.to(dev, bf)
    with torch.no_grad():
        s_ref, z_ref = stack(sd, zd, smd, pmd)
        R = N // P
        shards = [zd[0, r * R:(r + 1) * R].contiguous().clone() for r in range(P)]
        block = stack.blocks[0]
        shards = _virtual_pair_block(ops, shards, pmd[0], block.pair_stack, P)
        rows = [ops.single_rows(sd[0], ops.pair_bias_project(shards[r], block.attn_pair_bias), smd[0], block,
                                r * R, R) for r in range(P)]
        s_dap = torch.cat(rows, 0).unsqueeze(0)
    torch.cuda.synchronize()
    pkg.lib.check_device_status()
    z_dap = torch.cat(shards, 0).unsqueeze(0)
    # same kernels on the same values: only the bf16 rounding of intermediates that are summed in a
    # different tile order may differ
    assert cases.rel_err(z_dap.float().cpu(), z_ref.float().cpu()) < 2e-2
    assert cases.rel_err(s_dap.float().cpu(), s_ref.float().cpu()) < 2e-2
    # and against the fp32 oracle on the rounded inputs
    Pq = {k: v.to(bf).float() for k, v in Pw.items()}
    s_o, z_o = cases.oracle.pairformer_stack(s.to(bf).float(), z.to(bf).float(), sm, pm, Pq, "", 1, 4, 16)
    assert cases.rel_err(z_dap.float().cpu(), z_o) < 6e-2
    assert cases.rel_err(s_dap.float().cpu(), s_o) < 6e-2


def test_single_rank_dap_runner(pkg):
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    N = 64
    g = torch.Generator().manual_seed(1)
    z = torch.randn(1, N, N, 128, generator=g).to(dev, bf)
    s = torch.randn(1, N, 384, generator=g).to(dev, bf)
    pm = cases.rand_mask((1, N, N), g).to(dev, bf)
    sm = cases.rand_mask((1, N), g).to(dev, bf)
    Pw = pkg.weights.pairformer_stack_params(seed=5, no_blocks=2, **cases.OF3)
    stack = pkg.PairFormerStack(**cases.OF3, no_blocks=2, transition_type="swiglu", pair_dropout=0.25,
                                fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
    stack.load_state_dict(Pw, strict=True)
    stack = stack.to(dev, bf).eval()
    runner = pkg.dap.DapPairFormerStack(stack, 1, 0, ops=pkg.dap.CudaOps(dev))
    with torch.no_grad():
        s_ref, z_ref = stack(s, z, sm, pm)
        s_d, z_d = runner(s, z, sm, pm)
    torch.cuda.synchronize()
    pkg.lib.check_device_status()
    assert cases.rel_err(z_d.float().cpu(), z_ref.float().cpu()) < 2e-2
    assert cases.rel_err(s_d.float().cpu(), s_ref.float().cpu()) < 2e-2


def test_copy_rows_3d_matches_torch_permute(pkg):
    """The repack kernel against torch indexing: 16-byte vector path and the 2-byte path."""
    dev = torch.device("cuda:0")
    ops = pkg.dap.CudaOps(dev)
    for P, C, R, ld in ((4, 3, 5, 24), (2, 2, 3, 6)):
        src = torch.randn(P, C, R, ld, device=dev).to(torch.bfloat16)
        dst = torch.zeros(C, P * R, ld, device=dev, dtype=torch.bfloat16)
        e = 2
        ops.copy_rows(src, dst, (P, C, R), (C * R * ld * e, R * ld * e, ld * e), (R * ld * e, P * R * ld * e, ld * e),
                      ld * e)
        torch.cuda.synchronize()
        assert torch.equal(dst, src.permute(1, 0, 2, 3).reshape(C, P * R, ld))


def test_graphed_runner_replays_the_eager_result(pkg):
    """One rank: the captured step (both streams, all phase kernels) equals the eager step, twice."""
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    N = 64
    g = torch.Generator().manual_seed(2)
    z = torch.randn(1, N, N, 128, generator=g).to(dev, bf)
    s = torch.randn(1, N, 384, generator=g).to(dev, bf)
    pm = cases.rand_mask((1, N, N), g).to(dev, bf)
    sm = cases.rand_mask((1, N), g).to(dev, bf)
    Pw = pkg.weights.pairformer_stack_params(seed=6, no_blocks=2, **cases.OF3)
    stack = pkg.PairFormerStack(**cases.OF3, no_blocks=2, transition_type="swiglu", pair_dropout=0.25,
                                fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
    stack.load_state_dict(Pw, strict=True)
    stack = stack.to(dev, bf).eval()
    runner = pkg.dap.DapPairFormerStack(stack, 1, 0, ops=pkg.dap.CudaOps(dev))
    with torch.no_grad():
        s_e, z_e = runner(s, z, sm, pm)
        graphed = pkg.dap.GraphedDapRunner(runner, s, z, sm, pm)
        for _ in range(2):
            s_g, z_g = graphed(s, z, sm, pm)
            torch.cuda.synchronize()
            assert torch.equal(s_g, s_e) and torch.equal(z_g, z_e)
        z2 = (z * 0.5).contiguous()
        s_e2, z_e2 = runner(s, z2, sm, pm)
        s_g, z_g = graphed(s, z2, sm, pm)
        torch.cuda.synchronize()
        assert torch.equal(s_g, s_e2) and torch.equal(z_g, z_e2)
    pkg.lib.check_device_status()


def _virtual_pair_block_peer(ops, X, z, mask, pb, P):
    """The same block with the PeerExchange strategy: P virtual ranks whose heaps live in this process;
    the host's program order (all ranks produce, then all ranks pull) stands in for the barrier kernel."""
    dap = cases.pkg.dap
    R, N = z[0].shape[0], z[0].shape[1]
    C = 128 // P
    bf, dev = z[0].dtype, z[0].device
    mrow = [mask[r * R:(r + 1) * R].contiguous() for r in range(P)]
    mcol = [mask[:, r * R:(r + 1) * R].t().contiguous() for r in range(P)]
    nab = 2 * 128 * max(R * dap._pitch(N, 8), N * dap._pitch(R, 8))
    for mod, incoming in ((pb.tri_mul_out, False), (pb.tri_mul_in, True)):
        lines, pos = (N, R) if incoming else (R, N)
        ld = dap._pitch(pos, 8)
        ab = [ops.trimul_project(z[r], mrow[r], mod, P, incoming,
                                 out=X[r].buf("ab", (nab,), bf, dev)[:2 * 128 * lines * ld].view(P, 2, C, lines, ld))
              for r in range(P)]
        ab_all = [X[r].ab_all(ab[r], N, R, incoming) for r in range(P)]
        xb = [ops.trimul_contract(ab_all[r], N, R, out=X[r].buf("xb", (P, C, R, dap._pitch(N, 8)), bf, dev))
              for r in range(P)]
        x_t = [X[r].x_rows(xb[r]) for r in range(P)]
        for r in range(P):
            ops.trimul_output(z[r], x_t[r], mod)

    def attn(zz, mm, mod):
        proj = [ops.triattn_project(zz[r], mod, out=X[r].buf("tb", dap.triattn_bias_shape(R, N), bf, dev), row0=r * R) for r in range(P)]
        tb_all = [X[r].gather_lines(proj[r][1]) for r in range(P)]
        for r in range(P):
            ops.triattn_finish(zz[r], mm[r], proj[r][0], tb_all[r], mod)

    attn(z, mrow, pb.tri_att_start)
    zT = [X[r].transpose(z[r], "z1") for r in range(P)]
    attn(zT, mcol, pb.tri_att_end)
    for r in range(P):
        ops.transition(zT[r], mcol[r], pb.pair_transition)
    return [X[r].transpose(zT[r], "z0") for r in range(P)]


@pytest.mark.parametrize("P,N", [(2, 48), (4, 200), (8, 96), (2, 66)])
def test_peer_exchange_matches_whole_tensor(pkg, P, N):
    """Pull kernels + heap layout: the block through PeerExchange equals the unsharded drop-in stack."""
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(N + 1)
    z = torch.randn(1, N, N, 128, generator=g)
    s = torch.randn(1, N, 384, generator=g)
    pm = cases.rand_mask((1, N, N), g)
    sm = cases.rand_mask((1, N), g)
    Pw = pkg.weights.pairformer_stack_params(seed=4, no_blocks=1, final_std=None, **cases.OF3)
    stack = pkg.PairFormerStack(**cases.OF3, no_blocks=1, transition_type="swiglu", pair_dropout=0.25,
                                fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
    stack.load_state_dict(Pw, strict=True)
    stack = stack.to(dev, bf).eval()
    ops = pkg.dap.CudaOps(dev)
    zd, sd, pmd, smd = z.to(dev, bf), s.to(dev, bf), pm.to(dev, bf), sm.to(dev, bf)
    R = N // P
    heaps = pkg.dap.LocalPeerHeaps(pkg.dap.PeerExchange.heap_bytes(N, P), P, dev)
    X = [pkg.dap.PeerExchange(heaps.view(r), ops, barrier=False) for r in range(P)]
    with torch.no_grad():
        s_ref, z_ref = stack(sd, zd, smd, pmd)
        shards = []
        for r in range(P):
            t = X[r].buf("z0", (R, N, 128), bf, dev)
            t.copy_(zd[0, r * R:(r + 1) * R])
            shards.append(t)
        block = stack.blocks[0]
        shards = _virtual_pair_block_peer(ops, X, shards, pmd[0], block.pair_stack, P)
        rows = [ops.single_rows(sd[0], ops.pair_bias_project(shards[r], block.attn_pair_bias), smd[0], block, r * R, R,
                                out=X[r].buf("s0", (R, 384), bf, dev)) for r in range(P)]
        s_all = [X[r].gather_rows(rows[r]) for r in range(P)]
        z_all = [X[r].gather_rows(shards[r].view(R, -1)).view(1, N, N, 128) for r in range(P)]
    torch.cuda.synchronize()
    pkg.lib.check_device_status()
    for r in range(P):
        assert torch.equal(s_all[r], s_all[0]) and torch.equal(z_all[r], z_all[0])
    assert cases.rel_err(z_all[0].float().cpu(), z_ref.float().cpu()) < 2e-2
    assert cases.rel_err(s_all[0].unsqueeze(0).float().cpu(), s_ref.float().cpu()) < 2e-2


def test_barrier_whose_peer_never_arrives_poisons_the_step(pkg):
    """Failure detection without a fault: rank 0 of a 2-rank world runs the barrier kernel, nobody plays rank 1,
    so its flag word is never set. The kernel's bounded wait (2 s) runs out, it records a status word and returns;
    the pull queued behind it moves nothing (its destination keeps its contents), later barriers do not wait
    again, and the host's status check raises and clears the block. The context stays usable."""
    import ctypes
    import time

    dev = torch.device("cuda:0")
    l = pkg.lib.load()
    torch.cuda.synchronize()
    pkg.lib.check_device_status()
    heaps = pkg.dap.LocalPeerHeaps(1 << 16, 2, dev)
    h0 = heaps.view(0)
    st = torch.cuda.current_stream(dev).cuda_stream
    src = h0.tensor("src", (2, 64), torch.float32)
    heaps.store[0][:] = 0
    heaps.store[1][:] = 0
    heaps.view(0).tensor("src", (2, 64), torch.float32).fill_(1.0)
    heaps.view(1).tensor("src", (2, 64), torch.float32).fill_(2.0)
    dst = torch.full((2, 2, 64), -7.0, device=dev)
    t0 = time.time()
    assert l.of3_peer_barrier(h0.c_bases, 2, 0, st) == 0
    off = h0.offset_of(src)
    assert l.of3_peer_pull_rows(h0.c_bases, off, dst.data_ptr(), 2, 0, 1, 2, 0, 256, 512, 0, 256, 256, st) == 0
    assert l.of3_peer_barrier(h0.c_bases, 2, 0, st) == 0   # must not wait another two seconds
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.5 < waited < 3.5, waited
    assert torch.all(dst == -7.0), "a pull behind a failed barrier must move nothing"
    with pytest.raises(RuntimeError, match="kernel 30"):
        pkg.lib.check_device_status()
    pkg.lib.check_device_status()  # cleared
    # with the status clear the same pull moves the rows
    assert l.of3_peer_pull_rows(h0.c_bases, off, dst.data_ptr(), 2, 0, 1, 2, 0, 256, 512, 0, 256, 256, st) == 0
    torch.cuda.synchronize()
    assert torch.all(dst[0] == 1.0) and torch.all(dst[1] == 2.0)


def test_large_complex_shape_p8_n2048_row_shards_match_whole_tensor(pkg):
    """The large-complex configuration's shape on one GPU: N = 2048 split into 8 virtual ranks of 256 rows,
    5 % of the tokens padded at random (outer-product pair mask), one PairBlock through the phase kernels with
    the peer-heap exchange (pulls between the virtual ranks' heaps; the host's program order stands in for
    the barrier kernel) against the same block on the whole tensor. N = 2048 is the largest size the attention
    core keeps a mask row for, and the only benchmark shape with 64 key blocks per line."""
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    P, N = 8, 2048
    R = N // P
    g = torch.Generator().manual_seed(2048)
    z = torch.randn(1, N, N, 128, generator=g).to(bf)
    tm = torch.ones(N)
    tm[torch.randperm(N, generator=g)[:102]] = 0
    pm = (tm[:, None] * tm[None, :]).to(bf)
    blk = pkg.PairBlock(**cases.PAIR, transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False,
                        inf=1e9)
    blk.load_state_dict(pkg.weights.pair_block_params(seed=2048, **cases.PAIR), strict=True)
    blk = blk.to(dev, bf).eval()
    ops = pkg.dap.CudaOps(dev)
    heaps = pkg.dap.LocalPeerHeaps(pkg.dap.PeerExchange.heap_bytes(N, P), P, dev)
    X = [pkg.dap.PeerExchange(heaps.view(r), ops, barrier=False) for r in range(P)]
    zd, pmd = z.to(dev), pm.to(dev)
    with torch.no_grad():
        z_ref = blk(zd, pmd[None], inplace_safe=False)
        shards = []
        for r in range(P):
            t = X[r].buf("z0", (R, N, 128), bf, dev)
            t.copy_(zd[0, r * R:(r + 1) * R])
            shards.append(t)
        out = _virtual_pair_block_peer(ops, X, shards, pmd, blk, P)
    torch.cuda.synchronize()
    pkg.lib.check_device_status()
    z_dap = torch.cat([o for o in out], 0)
    valid = (pmd > 0)
    d = (z_dap.float() - z_ref[0].float())[valid]
    rms = z_ref[0].float()[valid].pow(2).mean().sqrt()
    assert torch.isfinite(z_dap.float()).all()
    assert float(d.abs().max() / rms) < 2e-2, float(d.abs().max() / rms)


def test_both_projection_kernels_of_the_triangle_update_give_the_same_bits(pkg):
    """A whole N = 2048 tensor (channel planes of 8 MB: the row-oriented projection kernel) against a 256-row shard of
    it (1 MB planes: the transposed kernel), random pair mask: the a / b planes of the shard's rows must be equal bit
    for bit, or a sharded run could differ from the single-GPU run of the same model."""
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    N, R = 2048, 256
    g = torch.Generator().manual_seed(11)
    z = torch.randn(N, N, 128, generator=g).to(dev, bf)
    m = (torch.rand(N, N, generator=g) > 0.1).to(dev, bf)
    blk = pkg.PairBlock(**cases.PAIR, transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False,
                        inf=1e9)
    blk.load_state_dict(pkg.weights.pair_block_params(seed=12, **cases.PAIR), strict=True)
    blk = blk.to(dev, bf).eval()
    ops = pkg.dap.CudaOps(dev)
    with torch.no_grad():
        for mod, incoming in ((blk.tri_mul_out, False),):
            whole = ops.trimul_project(z, m, mod, 1, incoming)
            shard = ops.trimul_project(z[:R].contiguous(), m[:R].contiguous(), mod, 1, incoming)
            torch.cuda.synchronize()
            pkg.lib.check_device_status()
            assert torch.equal(whole[0, :, :, :R, :], shard[0])
