#!/usr/bin/env python
"""Benchmark of the Pairformer hot path: the 48-block trunk at N_token = 768 in bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the whole trunk (48 PairFormerBlocks: pair stack + single track) over
one synthetic input (seeded N(0,1) activations, all-ones masks, seeded random weights with the
reference's zero-initialised matrices re-drawn N(0, 0.02)). Rank 0 prints ONE JSON line:

  value        algorithmic TFLOP/s of the whole job with inputs resident in HBM
  e2e          the same through the public module API with pinned HOST buffers: per step the
               inputs are copied host->device and the results device->host inside the timed region
  roofline     the kernel with the largest share of device time, timed live with CUDA-event pairs
               around each of its launches (library launch accounting), against the measured bf16
               tensor peak of this pool
  cpu_baseline the CPU oracle (a restatement of the reference's stock PyTorch path) on the host
               cores, on a bounded sample (one of the 48 blocks), scaled to the trunk

`--impl reference` times that CPU path alone, with all host threads, one block per step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

C_Z, C_S, H_PAIR, H_SINGLE = 128, 384, 4, 16
OF3 = dict(c_s=C_S, c_z=C_Z, c_hidden_pair_bias=24, no_heads_pair_bias=H_SINGLE, c_hidden_mul=128,
           c_hidden_pair_att=32, no_heads_pair=H_PAIR, transition_n=4)


def flops_pair_block(n: int) -> float:
    """Algorithmic flop of one pair stack: 12 N^3 c + 68 N^2 c^2 + 4 N^2 c H (c = 128, H = 4)."""
    c = C_Z
    return 12.0 * n**3 * c + 68.0 * n**2 * c**2 + 4.0 * n**2 * c * H_PAIR


def flops_single_block(n: int) -> float:
    """Single track of one block: pair-bias projection, q/k/v/g/o projections, attention, transition."""
    return 2.0 * n**2 * C_Z * H_SINGLE + 10.0 * n * C_S**2 + 4.0 * n**2 * C_S + 24.0 * n * C_S**2


def kernel_flops(n: int) -> dict:
    """Algorithmic flop per launch of each tcgen05 kernel (c = 128)."""
    c2 = float(C_Z * C_Z)
    return {
        "trimul_in": 8.0 * n * n * c2,         # four 128x128 projections
        "trimul_contract": 2.0 * n**3 * C_Z,   # the einsum
        "trimul_out": 4.0 * n * n * c2,        # linear_z + linear_g
        "triattn_proj": 6.0 * n * n * c2 + 2.0 * n * n * C_Z * H_PAIR,
        "triattn_core": 4.0 * n**3 * C_Z,      # Q K^T + P V over 4 heads x 32
        "triattn_out": 4.0 * n * n * c2,       # linear_g + linear_o
        "transition": 24.0 * n * n * c2,
    }


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) at N = 768 from the committed ncu
# summaries under profiles/ (captured at N = 768 itself, one block).
KERNEL_DRAM_TRAFFIC = {
    "triattn_core": 593.1e6,
    "trimul_in": 411e6,
    "contract": 417e6,
    "trimul_out": 411e6,
    "triattn_proj": 552e6,
    "triattn_out": 413e6,
    "transition": 268e6,
}


def peaks() -> tuple[float, float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops_sustained"]), float(d["hbm_gbs"]), "measured"
    return 1400.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    PERIOD_S = 0.05

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []   # (host time of arrival, csv line)
        self.t_start = self.t_end = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:  # nvidia-smi needs a moment before its first sample:
                time.sleep(0.02)                               # be sampling before the timed region starts
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def region_start(self):
        self.t_start = time.time()

    def region_end(self):
        self.t_end = time.time()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self.lines
        if self.t_start is not None and self.t_end is not None and lines:
            # samples taken while the timed region ran (a sample is printed up to one period after it was read);
            # a region shorter than the period keeps the sample nearest to it
            inside = [x for x in lines if self.t_start <= x[0] <= self.t_end + self.PERIOD_S]
            mid = 0.5 * (self.t_start + self.t_end)
            lines = inside or [min(lines, key=lambda x: abs(x[0] - mid))]
        for _, line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def oracle_block_seconds(n: int, repeats: int = 1) -> tuple[float, int]:
    """Seconds for one PairFormerBlock of the CPU oracle at N_token = n (fp32, all host threads)."""
    import torch

    from __graft_entry__ import load_package
    from oracle import pairformer_oracle as oracle

    pkg = load_package()
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1)
    s = torch.randn(1, n, C_S, generator=g)
    z = torch.randn(1, n, n, C_Z, generator=g)
    sm, pm = torch.ones(1, n), torch.ones(1, n, n)
    P = pkg.weights.pairformer_block_params(seed=7, **OF3)
    best = float("inf")
    with torch.no_grad():
        for _ in range(repeats):
            t0 = time.perf_counter()
            oracle.pairformer_block(s, z, sm, pm, P, "", H_PAIR, H_SINGLE)
            best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()


def run_reference(args) -> None:
    """The CPU path alone: one block of the trunk per step on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    n, blocks = args.n_token, args.blocks
    for _ in range(args.warmup):
        oracle_block_seconds(n)
    times = [oracle_block_seconds(n)[0] for _ in range(args.steps)]
    t = sum(times) / len(times)
    flop = flops_pair_block(n) + flops_single_block(n)
    value = flop / t / 1e12
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "pairformer_trunk_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Pairformer trunk, {blocks} blocks, N_token={n}, CPU fp32 oracle of the reference's "
                               "PyTorch path; each step = one block (1/%d of the trunk)" % blocks},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"one PairFormerBlock at N_token={n} per step"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        # a collective that cannot complete ends the run with an error after two minutes instead of hanging
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))

    pkg = load_package()
    lib = pkg.lib
    lib.load()
    n, blocks = args.n_token, args.blocks
    bf = torch.bfloat16

    # ---- model and synthetic inputs (identical on every rank)
    stack = pkg.PairFormerStack(**OF3, no_blocks=blocks, transition_type="swiglu", pair_dropout=0.25,
                                fuse_projection_weights=False, blocks_per_ckpt=None, inf=1e9)
    stack.load_state_dict(pkg.weights.pairformer_stack_params(seed=2024, no_blocks=blocks, **OF3), strict=True)
    stack = stack.to(dev, bf).eval()
    g = torch.Generator().manual_seed(768)
    s_host = torch.randn(1, n, C_S, generator=g).to(bf).pin_memory()
    z_host = torch.randn(1, n, n, C_Z, generator=g).to(bf).pin_memory()
    sm_host = torch.ones(1, n, dtype=bf).pin_memory()
    pm_host = torch.ones(1, n, n, dtype=bf).pin_memory()
    s_out_host = torch.empty_like(s_host).pin_memory()
    z_out_host = torch.empty_like(z_host).pin_memory()

    heap = None
    if world > 1:
        ops = pkg.dap.CudaOps(dev)
        xchg = None  # None: torch.distributed collectives (NCCL)
        if args.exchange == "peer":
            try:
                heap = pkg.dap.PeerHeap(pkg.dap.PeerExchange.heap_bytes(n, world), world, rank, dev)
            except Exception as exc:  # e.g. CUDA IPC not permitted between the ranks' processes
                print(f"[bench] rank {rank}: no peer heap ({exc}); falling back to NCCL", file=sys.stderr, flush=True)
                heap = None
            agreed = torch.tensor([1 if heap is not None else 0], device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 1:
                xchg = pkg.dap.PeerExchange(heap, ops)
            else:
                if heap is not None:
                    heap.close()
                    heap = None
                args.exchange = "nccl"
        runner = pkg.dap.DapPairFormerStack(stack, world, rank, ops=ops, exchange=xchg)
    else:
        runner = None

    def stage(msg):  # progress on stderr: a stalled multi-GPU run shows where it stopped
        if rank == 0 and world > 1:
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    graphed = None  # N > 1: the step captured into a CUDA graph (kernels of both streams + collectives)

    def step_resident(s_d, z_d, sm_d, pm_d):
        if graphed is not None:
            return graphed(s_d, z_d, sm_d, pm_d)
        if runner is not None:
            return runner(s_d, z_d, sm_d, pm_d, sharded=True)
        return stack(s_d, z_d, sm_d, pm_d)  # clones the inputs, then updates the clones in place

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    if world > 1:
        # N > 1: the job's input and output are row-sharded -- a rank moves only its R = N / world rows of z and
        # of the pair mask (and of the mask's transpose) between host and device; s and the token mask are whole
        R = n // world
        rows = slice(rank * R, (rank + 1) * R)
        z_host = z_host[:, rows].contiguous().pin_memory()
        pm_host = (pm_host[0, rows].contiguous().pin_memory(), pm_host[0][:, rows].t().contiguous().pin_memory())
        z_out_host = torch.empty_like(z_host).pin_memory()

    def to_dev(t, **kw):
        return tuple(x.to(dev, **kw) for x in t) if isinstance(t, tuple) else t.to(dev, **kw)

    with torch.no_grad():
        s_d, z_d = s_host.to(dev), z_host.to(dev)
        sm_d, pm_d = sm_host.to(dev), to_dev(pm_host)
        for _ in range(args.warmup):
            step_resident(s_d, z_d, sm_d, pm_d)
        sync()
        lib.check_device_status()
        graph_note = "eager launches"
        stage(f"eager warm-up done ({args.warmup} steps)")
        if runner is not None and not args.no_graph:
            graphed = pkg.dap.GraphedDapRunner(runner, s_d, z_d, sm_d, pm_d, warmup=1, sharded=True)
            stage("graph captured")
            graph_note = "one CUDA graph per step (kernels of both streams and the NCCL collectives)"
            for _ in range(args.warmup):
                step_resident(s_d, z_d, sm_d, pm_d)
            sync()

        # ---- device-resident timing (value) with per-kernel event pairs
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            lib.profile_begin(timing=graphed is None)
            sync()
            clocks.region_start()
            e0.record()
            for _ in range(args.steps):
                s_o, z_o = step_resident(s_d, z_d, sm_d, pm_d)
            e1.record()
            sync()
            clocks.region_end()
            prof = lib.profile_end()
        ms_resident = e0.elapsed_time(e1) / args.steps
        stage(f"resident timing done: {ms_resident:.2f} ms per step")
        lib.check_device_status()
        assert torch.isfinite(z_o.float()).all() and torch.isfinite(s_o.float()).all(), "non-finite trunk output"

        # ---- end to end through the public API with host buffers
        def nbytes(*ts):
            return sum(x.numel() * x.element_size() for t in ts for x in (t if isinstance(t, tuple) else (t,)))

        # whole-job bytes per step: every rank copies its own shard (and the small replicated tensors)
        h2d = nbytes(s_host, z_host, sm_host, pm_host) * world
        d2h = nbytes(s_out_host, z_out_host) * world

        def step_e2e():
            s_in = s_host.to(dev, non_blocking=True)
            z_in = z_host.to(dev, non_blocking=True)
            sm_in = sm_host.to(dev, non_blocking=True)
            pm_in = to_dev(pm_host, non_blocking=True)
            if runner is not None:
                s_r, z_r = step_resident(s_in, z_in, sm_in, pm_in)
            else:
                s_r, z_r = stack(s_in, z_in, sm_in, pm_in, inplace_safe=True)
            s_out_host.copy_(s_r, non_blocking=True)
            z_out_host.copy_(z_r, non_blocking=True)

        step_e2e()
        sync()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        for _ in range(args.steps):
            step_e2e()
        e3.record()
        sync()
        ms_e2e = e2.elapsed_time(e3) / args.steps

        launches_in_timed_region = int(sum(l for l, _ in prof.values()))
        if graphed is not None:
            # per-kernel breakdown and launch count of a step: one eager, profiled step outside the timed region
            lib.profile_begin(timing=True)
            runner(s_d, z_d, sm_d, pm_d, sharded=True)
            sync()
            prof = lib.profile_end()
            launches_in_timed_region = int(sum(l for l, _ in prof.values())) * args.steps

    # ---- max over ranks
    if world > 1:
        t = torch.tensor([ms_resident, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_resident, ms_e2e = float(t[0]), float(t[1])

    flop = blocks * (flops_pair_block(n) + flops_single_block(n))
    value = flop / (ms_resident * 1e-3) / 1e12
    e2e_value = flop / (ms_e2e * 1e-3) / 1e12

    if rank == 0:
        tensor_peak, hbm_peak, peak_kind = peaks()
        kf = kernel_flops(n)
        total_kernel_ms = sum(ms for _, ms in prof.values()) or 1.0
        kernels = {}
        for name, (launches, ms) in sorted(prof.items(), key=lambda kv: -kv[1][1]):
            per_launch_ms = ms / max(1, launches)
            entry = {"launches": launches, "total_ms": round(ms, 3), "share": round(ms / total_kernel_ms, 4),
                     "ms_per_launch": round(per_launch_ms, 4)}
            if name in kf and world == 1:
                entry["tflops"] = round(kf[name] / (per_launch_ms * 1e-3) / 1e12, 1)
            kernels[name] = entry
        top = next((k for k in kernels if k in kf), None)
        roofline = None
        if top is not None:
            per_launch_ms = kernels[top]["ms_per_launch"]
            achieved = kf[top] / world / (per_launch_ms * 1e-3) / 1e12
            roofline = {"kernel": top, "bound": "tensor", "achieved": round(achieved, 1), "peak": tensor_peak,
                        "unit": "TFLOP/s", "frac": round(achieved / tensor_peak, 4),
                        "traffic": KERNEL_DRAM_TRAFFIC.get(top) if (n == 768 and world == 1) else None, "peak_kind": f"bf16 sustained, {peak_kind}",
                        "algorithmic_flop_per_launch": kf[top] / world}
            if top == "triattn_core":
                # second ceiling of this kernel: one exp2 per logit on the MUFU pipe (16 per clock and SM)
                exps = 4.0 * n * n * n / world
                sm_hz = (clocks.summary().get("sm_mhz") or 1965.0) * 1e6
                exp_peak = 16.0 * 148 * sm_hz
                roofline["exp_bound"] = {"exps_per_launch": exps, "peak_exps_per_s": exp_peak,
                                         "frac": round(exps / (per_launch_ms * 1e-3) / exp_peak, 4)}
        cpu_s, cores = oracle_block_seconds(n) if world == 1 and not args.no_cpu_baseline else (None, 0)
        cpu_baseline = None
        if cpu_s is not None:
            cpu_baseline = {"value": (flops_pair_block(n) + flops_single_block(n)) / cpu_s / 1e12, "unit": "TFLOP/s",
                            "cores": cores, "kind": "port",
                            "sample": f"one of the {blocks} PairFormerBlocks at N_token={n} on the CPU oracle "
                                      f"({cpu_s:.1f} s); the trunk is {blocks} such blocks"}
        line = {
            "metric": "pairformer_trunk_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_resident, 3),
            "ms_per_block": round(ms_resident / blocks, 4), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"Pairformer trunk, {blocks} blocks, N_token={n}, bf16, all-ones masks, "
                                   "seeded random weights",
                       "parallelism": "single GPU" if world == 1 else f"DAP row-sharded over {world} GPUs",
                       "launch": graph_note,
                       "io": ("whole tensors" if world == 1 else
                              "row-sharded: each rank holds, uploads and downloads its N/world rows of z; s replicated"),
                       "exchange": ("none" if world == 1 else
                                    "barrier + pull kernels over NVLink peer memory" if args.exchange == "peer"
                                    else "NCCL all-to-all / all-gather"),
                       "l2": "inputs and per-layer working set (>1 GB) exceed the 126 MB L2; no explicit flush"},
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_in_timed_region,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "kernels": kernels,
            "frac_of_tensor_peak": round(value / world / tensor_peak, 4),
        }
        print(json.dumps(line))
    if world > 1:
        if graphed is not None:  # a live graph still holds the communicator's captured work
            s_o = z_o = None
            graphed.release()
        torch.cuda.synchronize(dev)
        dist.barrier()
        if heap is not None:
            runner = None
            heap.close()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--blocks", type=int, default=48)
    ap.add_argument("--n-token", type=int, default=768)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how shards move between GPUs")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: launch eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
