"""Two real ranks on two GPUs: the peer-memory exchange (CUDA IPC heaps, barrier kernel, pull kernels)
against the NCCL exchange on the same inputs. Skipped on a box with fewer than two GPUs."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _worker(rank, world, port, n_token, result_file):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        import cases

        pkg = cases.pkg
        bf = torch.bfloat16
        g = torch.Generator().manual_seed(11)
        s = torch.randn(1, n_token, 384, generator=g).to(dev, bf)
        z = torch.randn(1, n_token, n_token, 128, generator=g).to(dev, bf)
        sm = cases.rand_mask((1, n_token), g).to(dev, bf)
        pm = cases.rand_mask((1, n_token, n_token), g).to(dev, bf)
        Pw = pkg.weights.pairformer_stack_params(seed=3, no_blocks=2, final_std=None, **cases.OF3)
        stack = pkg.PairFormerStack(**cases.OF3, no_blocks=2, transition_type="swiglu", pair_dropout=0.25,
                                    fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
        stack.load_state_dict(Pw, strict=True)
        stack = stack.to(dev, bf).eval()
        ops = pkg.dap.CudaOps(dev)
        heap = pkg.dap.PeerHeap(pkg.dap.PeerExchange.heap_bytes(n_token, world), world, rank, dev)
        peer = pkg.dap.DapPairFormerStack(stack, world, rank, ops=ops, exchange=pkg.dap.PeerExchange(heap, ops))
        nccl = pkg.dap.DapPairFormerStack(stack, world, rank, ops=ops)
        with torch.no_grad():
            s_n, z_n = nccl(s, z, sm, pm)
            for _ in range(2):  # twice: the second step reuses every heap buffer
                s_p, z_p = peer(s, z, sm, pm)
            graphed = pkg.dap.GraphedDapRunner(peer, s, z, sm, pm, warmup=1)
            s_g, z_g = graphed(s, z, sm, pm)
            torch.cuda.synchronize(dev)
            ok = bool(torch.equal(s_p, s_n) and torch.equal(z_p, z_n) and torch.equal(s_g, s_n)
                      and torch.equal(z_g, z_n))
            graphed.release()
        pkg.lib.check_device_status()
        torch.cuda.synchronize(dev)
        dist.barrier()
        heap.close()
        res = [None] * world
        dist.all_gather_object(res, ok)
        if rank == 0:
            torch.save(res, result_file)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_exchange_equals_nccl_exchange_on_two_gpus(tmp_path):
    result = tmp_path / "res.pt"
    mp.spawn(_worker, args=(2, _free_port(), 64, str(result)), nprocs=2, join=True)
    assert torch.load(result) == [True, True]
