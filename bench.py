#!/usr/bin/env python
"""Benchmark of the Pairformer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1|c2|c3|c4]

The headline workload (default, ``--config c2``) is the 48-block Pairformer trunk at N_token = 768 in bf16:
one "step" is one pass of the whole trunk (48 PairFormerBlocks: pair stack + single track) over one synthetic
input (seeded N(0,1) activations, seeded random weights with the reference's zero-initialised matrices
re-drawn N(0, 0.02)). The other configurations of the benchmark description produce their own lines:
  c1  pair stack only, 4 PairBlocks, N = 384, the last 32 tokens padded
  c3  pair stack only, 8 PairBlocks, N = 2048, 5 % of the tokens padded at random (meant for 8 GPUs)
  c4  diffusion token stack, 24 blocks, N = 768, 5 samples sharing one pair tensor (samples split over GPUs)
At N > 1 the pair tensor is row-sharded over the ranks (c1 - c3) or the samples are dealt out (c4).
Rank 0 prints ONE JSON line:

  value        algorithmic TFLOP/s of the whole job with inputs resident in HBM, timed with one CUDA-event pair
               around the K steps (no per-launch instrumentation inside the timed region)
  e2e          the same through the public module API with pinned HOST buffers: per step the inputs are copied
               host->device and the results device->host inside the timed region
  kernels      per-kernel device time of ONE more step, run after the timed region with an event pair around
               every launch (library launch accounting)
  roofline     a list, dominant kernel first: algorithmic flop (or bytes) per launch / that kernel's average launch
               time, against the measured bf16 tensor peak (or copy bandwidth) of this pool; `traffic` = DRAM bytes
               per launch from the committed ncu summary profiles/kernel_dram_traffic_n768.md
  cpu_baseline the CPU oracle (a restatement of the reference's stock PyTorch path) on the host cores, on a bounded
               sample (one block), in the same TFLOP/s
  parity_vs_single_gpu  (N > 1) the row-sharded path against the single-GPU path on the same inputs, outside the
               timed region; the run fails if they disagree

`--impl reference` times that CPU path alone, with all host threads, one block per step.
"""

from __future__ import annotations

import argparse
import json
import os
import re
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
PAIR = dict(c_z=C_Z, c_hidden_mul=128, c_hidden_pair_att=32, no_heads_pair=H_PAIR, transition_n=4)
DIFF = dict(c_a=768, c_s=C_S, c_z=C_Z, c_hidden=48, no_heads=16, n_transition=2)

# kind: "trunk" = PairFormerStack (pair stack + single track), "pair" = PairBlocks only, "diffusion" = token stack
CONFIGS = {
    "c1": dict(kind="pair", n=384, blocks=4, pad=("tail", 32),
               label="pair stack only, 4 PairBlocks, N_token=384, last 32 tokens padded"),
    "c2": dict(kind="trunk", n=768, blocks=48, pad=None,
               label="Pairformer trunk, 48 blocks, N_token=768, all-ones masks"),
    "c3": dict(kind="pair", n=2048, blocks=8, pad=("random", 0.05),
               label="pair stack only, 8 PairBlocks, N_token=2048, 5 % of the tokens padded at random"),
    "c4": dict(kind="diffusion", n=768, blocks=24, samples=5, pad=None,
               label="diffusion token stack, 24 blocks, N_token=768, 5 samples sharing one pair tensor"),
}


def flops_pair_block(n: int) -> float:
    """Algorithmic flop of one pair stack: 12 N^3 c + 68 N^2 c^2 + 4 N^2 c H (c = 128, H = 4)."""
    c = C_Z
    return 12.0 * n**3 * c + 68.0 * n**2 * c**2 + 4.0 * n**2 * c * H_PAIR


def flops_single_block(n: int) -> float:
    """Single track of one block: pair-bias projection, q/k/v/g/o projections, attention, transition."""
    return 2.0 * n**2 * C_Z * H_SINGLE + 10.0 * n * C_S**2 + 4.0 * n**2 * C_S + 24.0 * n * C_S**2


def flops_diffusion_block(n: int, samples: int) -> float:
    """One DiffusionTransformerBlock over `samples` samples that share one pair tensor (c_a = 768, c_s = 384,
    16 heads x 48, transition n = 2). Per sample: q / k / v / g / o projections (10 N c_a^2), the three
    conditioning linears of the attention and the three of the transition (12 N c_s c_a), attention
    (4 N^2 c_a), the three SwiGLU GEMMs of N x c_a x 2 c_a. Once per block: the pair-bias projection
    (2 N^2 c_z H). 24 blocks, 5 samples, N = 768: 1.797e12 flop."""
    c_a, c_s = DIFF["c_a"], DIFF["c_s"]
    per_sample = (10.0 * n * c_a**2 + 12.0 * n * c_s * c_a + 4.0 * n**2 * c_a
                  + 3 * 2.0 * n * c_a * (DIFF["n_transition"] * c_a))
    return samples * per_sample + 2.0 * n**2 * C_Z * DIFF["no_heads"]


def workload_flops(cfg: dict, n: int, blocks: int) -> float:
    if cfg["kind"] == "trunk":
        return blocks * (flops_pair_block(n) + flops_single_block(n))
    if cfg["kind"] == "pair":
        return blocks * flops_pair_block(n)
    return blocks * flops_diffusion_block(n, cfg["samples"])


def kernel_flops(n: int) -> dict:
    """Algorithmic flop per launch of each tcgen05 kernel of the pair stack (c = 128)."""
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


def kernel_min_bytes(n: int) -> dict:
    """Algorithmic HBM bytes per launch of the row-tile kernels (the tensors each one must read and write once)."""
    plane = float(n) * n * C_Z * 2          # one [N, N, 128] bf16 tensor
    return {
        "trimul_in": 3 * plane,             # z in, a_t and b_t out
        "trimul_out": 3 * plane,            # x_t and z in, z out
        "triattn_proj": 4 * plane,          # z in, q, k, v images out
        "triattn_out": 3 * plane,           # z and o in, z out
    }


TENSOR_BOUND = ("triattn_core", "trimul_contract", "transition")


def dram_traffic_table() -> dict:
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) at N = 768, read from the committed
    ncu summary: rows `| kernel | read MB | written MB | ...`."""
    out = {}
    p = ROOT / "profiles" / "kernel_dram_traffic_n768.md"
    if p.exists():
        for line in p.read_text().splitlines():
            m = re.match(r"\|\s*`?(\w+)`?\s*\|\s*([\d.]+)\s*\|\s*([\d.]+)\s*\|", line)
            if m:
                out[m.group(1)] = (float(m.group(2)) + float(m.group(3))) * 1e6
    return out


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


def token_mask(cfg: dict, n: int):
    """The configuration's token mask [n] (float 0/1), seeded."""
    import torch

    m = torch.ones(n)
    if cfg["pad"] is not None:
        how, amount = cfg["pad"]
        if how == "tail":
            m[n - int(amount):] = 0
        else:
            g = torch.Generator().manual_seed(2048)
            m[torch.randperm(n, generator=g)[:int(round(amount * n))]] = 0
    return m


def oracle_sample(cfg: dict, n: int) -> tuple[float, float, int, str]:
    """One bounded sample of the workload on the CPU oracle (fp32, all host threads):
    -> (seconds, algorithmic flop of the sample, threads, description)."""
    import torch

    from __graft_entry__ import load_package
    from oracle import pairformer_oracle as oracle

    pkg = load_package()
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1)
    kind = cfg["kind"]
    with torch.no_grad():
        if kind == "diffusion":
            S = cfg["samples"]
            a = torch.randn(1, S, n, DIFF["c_a"], generator=g)
            s = torch.randn(1, S, n, C_S, generator=g)
            z = torch.randn(1, 1, n, n, C_Z, generator=g)
            mask = torch.ones(1, 1, n)
            P = pkg.weights.diffusion_block_params(seed=7, **DIFF)
            t0 = time.perf_counter()
            oracle.diffusion_transformer_block(a, s, z, mask, P, "", DIFF["no_heads"])
            dt = time.perf_counter() - t0
            return dt, flops_diffusion_block(n, S), torch.get_num_threads(), \
                f"one of the {cfg['blocks']} DiffusionTransformerBlocks ({S} samples, N_token={n})"
        # the oracle materialises the [N, H, N, N] logits: above N = 768 that is more memory than a host has, so the
        # large-N pair stack is sampled at N = 768 (the figure is a rate, TFLOP/s, which grows slowly with N)
        ns = min(n, 768)
        z = torch.randn(1, ns, ns, C_Z, generator=g)
        tm = token_mask(cfg, ns) if cfg["pad"] is not None and ns == n else torch.ones(ns)
        pm = (tm[:, None] * tm[None, :])[None]
        if kind == "pair":
            P = pkg.weights.pair_block_params(seed=7, **PAIR)
            t0 = time.perf_counter()
            oracle.pair_block(z, pm, P, "", H_PAIR)
            dt = time.perf_counter() - t0
            return dt, flops_pair_block(ns), torch.get_num_threads(), \
                f"one PairBlock at N_token={ns} (the workload: {cfg['blocks']} blocks at N_token={n})"
        s = torch.randn(1, ns, C_S, generator=g)
        P = pkg.weights.pairformer_block_params(seed=7, **OF3)
        t0 = time.perf_counter()
        oracle.pairformer_block(s, z, tm[None], pm, P, "", H_PAIR, H_SINGLE)
        dt = time.perf_counter() - t0
        return dt, flops_pair_block(ns) + flops_single_block(ns), torch.get_num_threads(), \
            f"one of the {cfg['blocks']} PairFormerBlocks at N_token={ns}"


def run_reference(args, cfg) -> None:
    """The CPU path alone: one block of the workload per step on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.n_token or cfg["n"]
    for _ in range(args.warmup):
        oracle_sample(cfg, n)
    samples = [oracle_sample(cfg, n) for _ in range(args.steps)]
    t = sum(x[0] for x in samples) / len(samples)
    _, flop, cores, what = samples[0]
    value = flop / t / 1e12
    line = {
        "impl": "reference", "metric": "pairformer_trunk_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.config}: {cfg['label']}; CPU fp32 oracle of the reference's PyTorch path, "
                               f"each step = {what}; the metric is a rate (algorithmic TFLOP/s), so a step of one "
                               "block is comparable with a step of the whole workload",
                   "same_config": False},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": what + " per step"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def build_job(pkg, cfg, n, blocks, dev, world, rank):
    """Model (seeded weights), pinned host inputs / outputs of THIS rank, and the functions that run one step.

    Returns a dict: model, host_in (tuple of pinned tensors or tuples of them), host_out, run(dev_inputs) ->
    tuple of device outputs for the single-GPU path, and for the row-sharded path the pieces DapPairFormerStack needs.
    """
    import torch

    bf = torch.bfloat16
    kind = cfg["kind"]
    kw = dict(transition_type="swiglu", pair_dropout=0.25, fuse_projection_weights=False, inf=1e9)
    g = torch.Generator().manual_seed(768)
    job = {"kind": kind}
    if kind == "diffusion":
        S = cfg["samples"]
        model = pkg.DiffusionTransformer(**DIFF, no_blocks=blocks, use_ada_layer_norm=True, n_query=None, n_key=None,
                                         inf=1e9)
        model.load_state_dict(pkg.weights.diffusion_stack_params(seed=2024, no_blocks=blocks, **DIFF), strict=True)
        a = torch.randn(1, S, n, DIFF["c_a"], generator=g).to(bf)
        s = torch.randn(1, S, n, C_S, generator=g).to(bf)
        z = torch.randn(1, 1, n, n, C_Z, generator=g).to(bf)
        mask = torch.ones(1, 1, n, dtype=bf)
        # samples are independent: rank r takes samples r, r + world, ... (3+2 / 2+1+1+1 / 5 of 8 ranks busy);
        # z, s and the mask of a rank's samples are its inputs, nothing is exchanged between the ranks
        mine = list(range(rank, S, world))
        job["samples_here"] = mine
        if mine:
            a, s = a[:, mine].contiguous(), s[:, mine].contiguous()
            job["host_in"] = tuple(t.pin_memory() for t in (a, s, z, mask))
            job["host_out"] = (torch.empty_like(a).pin_memory(),)
        else:
            job["host_in"], job["host_out"] = (), ()
        model = model.to(dev, bf).eval()
        # the timed step recomputes the 24 pair-bias projections like the reference does (a step whose outputs
        # come out of a cache would not be the workload); the hoisted variant is timed separately
        model.hoist_pair_bias = False
        job["model"] = model
        job["run"] = lambda x: (model(x[0], x[1], x[2], mask=x[3]),) if x else ()
        return job
    tm = token_mask(cfg, n)
    pm = tm[:, None] * tm[None, :]
    z = torch.randn(1, n, n, C_Z, generator=g).to(bf)
    if kind == "trunk":
        model = pkg.PairFormerStack(**OF3, no_blocks=blocks, blocks_per_ckpt=None, **kw)
        model.load_state_dict(pkg.weights.pairformer_stack_params(seed=2024, no_blocks=blocks, **OF3), strict=True)
        s = torch.randn(1, n, C_S, generator=g).to(bf)
    else:
        model = pkg.PairStack(no_blocks=blocks, **PAIR, **kw)
        model.load_state_dict(pkg.weights.pair_stack_params(seed=2024, no_blocks=blocks, **PAIR), strict=True)
        s = None
    model = model.to(dev, bf).eval()
    job["model"] = model
    sm = tm[None].to(bf)
    if world == 1:
        pmh = pm[None].to(bf)
        if kind == "trunk":
            job["host_in"] = tuple(t.pin_memory() for t in (s, z, sm, pmh))
            job["host_out"] = (torch.empty_like(s).pin_memory(), torch.empty_like(z).pin_memory())
            job["run"] = lambda x: model(x[0], x[1], x[2], x[3])   # clones the inputs, then updates the clones in place
            job["run_inplace"] = lambda x: model(x[0], x[1], x[2], x[3], inplace_safe=True)
        else:
            job["host_in"] = tuple(t.pin_memory() for t in (z, pmh))
            job["host_out"] = (torch.empty_like(z).pin_memory(),)
            job["run"] = lambda x: (model(x[0], x[1]),)
            job["run_inplace"] = lambda x: (model(x[0], x[1], inplace_safe=True),)
        return job
    # row-sharded: a rank holds, uploads and downloads only its R = n / world rows of z and of the pair mask (and of
    # the mask's transpose); s and the token mask are whole on every rank
    R = n // world
    rows = slice(rank * R, (rank + 1) * R)
    z_rows = z[:, rows].contiguous().pin_memory()
    pm_rows = (pm[rows].to(bf).contiguous().pin_memory(), pm[:, rows].t().to(bf).contiguous().pin_memory())
    job["whole"] = (s, z, sm, pm[None].to(bf))   # for the parity check against the single-GPU path
    job["rows"] = rows
    if kind == "trunk":
        job["host_in"] = (s.pin_memory(), z_rows, sm.pin_memory(), pm_rows)
        job["host_out"] = (torch.empty_like(s).pin_memory(), torch.empty_like(z_rows).pin_memory())
    else:
        job["host_in"] = (z_rows, pm_rows)
        job["host_out"] = (torch.empty_like(z_rows).pin_memory(),)
    return job


def to_dev(t, dev, **kw):
    return tuple(to_dev(x, dev, **kw) for x in t) if isinstance(t, tuple) else t.to(dev, **kw)


def nbytes(t) -> int:
    return sum(nbytes(x) for x in t) if isinstance(t, tuple) else t.numel() * t.element_size()


def rel_errors(got, ref):
    """(max |got - ref| / RMS(ref), RMS(got - ref) / RMS(ref)) in fp64 on the device."""
    d = got.double() - ref.double()
    rms = ref.double().pow(2).mean().sqrt()
    return float(d.abs().max() / rms), float(d.pow(2).mean().sqrt() / rms)


def run_ours(args, cfg) -> None:
    import datetime
    import types

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
        # a collective that cannot complete ends the run with an error after two minutes instead of hanging
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))

    pkg = load_package()
    lib = pkg.lib
    lib.load()
    n, blocks = args.n_token or cfg["n"], args.blocks or cfg["blocks"]
    kind = cfg["kind"]
    sharded = world > 1 and kind != "diffusion"
    if sharded and n % world:
        raise SystemExit(f"N_token {n} is not divisible by {world} ranks")
    job = build_job(pkg, cfg, n, blocks, dev, world, rank)
    model = job["model"]

    def stage(msg):  # progress on stderr: a stalled multi-GPU run shows where it stopped
        if rank == 0 and world > 1:
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    heap = runner = graphed = None
    parity = None
    if sharded:
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
        runner = pkg.dap.DapPairFormerStack(model, world, rank, ops=ops, exchange=xchg)

        def dap_step(r, x):
            if kind == "trunk":
                return r(x[0], x[1], x[2], x[3], sharded=True)
            return r(None, x[0], None, x[1], sharded=True)[1:]

        # ---- correctness of the sharded path on these GPUs, outside any timed region: the first two blocks
        # through the same runner and exchange against the single-GPU modules on the whole tensors (this rank's
        # rows), and the peer-memory exchange against the NCCL one (bit for bit)
        with torch.no_grad():
            nb = min(2, blocks)
            sub = types.SimpleNamespace(blocks=model.blocks[:nb])
            s_w, z_w, sm_w, pm_w = (None if t is None else t.to(dev) for t in job["whole"])
            z_ref, s_ref = z_w.clone(), (None if s_w is None else s_w.clone())
            for b in sub.blocks:
                if kind == "trunk":
                    s_ref, z_ref = b(s_ref, z_ref, sm_w, pm_w, inplace_safe=True)
                else:
                    z_ref = b(z_ref, pm_w, inplace_safe=True)
            x_dev = to_dev(job["host_in"], dev)
            r2 = pkg.dap.DapPairFormerStack(sub, world, rank, ops=ops, exchange=xchg)
            out2 = [t.clone() for t in dap_step(r2, x_dev)]
            torch.cuda.synchronize(dev)
            zmax, zrms = rel_errors(out2[-1][0], z_ref[0, job["rows"]])
            parity = {"blocks": nb, "z_max": zmax, "z_rms": zrms}
            if kind == "trunk":
                parity["s_max"], parity["s_rms"] = rel_errors(out2[0], s_ref)
            if xchg is not None:
                r3 = pkg.dap.DapPairFormerStack(sub, world, rank, ops=ops, exchange=None)
                out3 = dap_step(r3, x_dev)
                torch.cuda.synchronize(dev)
                parity["peer_equals_nccl"] = bool(all(torch.equal(a, b) for a, b in zip(out2, out3)))
            t = torch.tensor([parity["z_max"], parity["z_rms"], parity.get("s_max", 0.0), parity.get("s_rms", 0.0),
                              0.0 if parity.get("peer_equals_nccl", True) else 1.0], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)   # worst rank
            parity.update(z_max=float(t[0]), z_rms=float(t[1]))
            if kind == "trunk":
                parity.update(s_max=float(t[2]), s_rms=float(t[3]))
            if xchg is not None:
                parity["peer_equals_nccl"] = float(t[4]) == 0.0
            parity["bar_max"] = 2e-2
            del s_w, z_w, z_ref, s_ref, out2, r2
            stage(f"parity vs single GPU over {nb} blocks: {parity}")
            if parity["z_max"] > parity["bar_max"] or parity.get("s_max", 0.0) > parity["bar_max"] or \
                    not parity.get("peer_equals_nccl", True):
                raise SystemExit(f"row-sharded path disagrees with the single-GPU path: {parity}")

    graphed_mod = None   # diffusion stack: one CUDA graph per step of this rank's samples

    def step_resident(x):
        if graphed is not None:
            if kind == "trunk":
                return graphed(x[0], x[1], x[2], x[3])
            return graphed(None, x[0], None, x[1])[1:]
        if runner is not None:
            return dap_step(runner, x)
        if graphed_mod is not None and x:
            res = graphed_mod(*x)
            return res if isinstance(res, tuple) else (res,)
        return job["run"](x)

    def step_eager(x):
        return dap_step(runner, x) if runner is not None else job["run"](x)

    with torch.no_grad():
        x_dev = to_dev(job["host_in"], dev)
        for _ in range(args.warmup):
            step_resident(x_dev)
        sync()
        lib.check_device_status()
        graph_note = "eager launches"
        stage(f"eager warm-up done ({args.warmup} steps)")
        if runner is not None and not args.no_graph:
            runner.check_status = False  # replays are checked one step late by the graph runner
            if kind == "trunk":
                graphed = pkg.dap.GraphedDapRunner(runner, x_dev[0], x_dev[1], x_dev[2], x_dev[3], warmup=1, sharded=True)
            else:
                graphed = pkg.dap.GraphedDapRunner(runner, None, x_dev[0], None, x_dev[1], warmup=1, sharded=True)
            stage("graph captured")
            graph_note = "one CUDA graph per step (kernels of both streams and the exchanges)"
            for _ in range(args.warmup):
                step_resident(x_dev)
            sync()
        if world == 1 and kind != "diffusion" and not args.no_graph:
            # the whole single-GPU step (both streams of PairFormerStack) as one CUDA graph
            if kind == "trunk":
                graphed_mod = pkg.GraphedModule(lambda s_, z_, sm_, pm_: model(s_, z_, sm_, pm_, inplace_safe=True),
                                                *x_dev, warmup=1)
            else:
                graphed_mod = pkg.GraphedModule(lambda z_, pm_: (model(z_, pm_, inplace_safe=True),), *x_dev, warmup=1)
            stage("graph captured")
            graph_note = "one CUDA graph per step"
            for _ in range(args.warmup):
                step_resident(x_dev)
            sync()
        if kind == "diffusion" and not args.no_graph:
            # ~500 launches of a few microseconds per step: replayed from one CUDA graph (openfold-3_b200/graphs.py).
            # Every rank walks through here (sync() is a collective), ranks without a sample capture nothing.
            if job["host_in"]:
                graphed_mod = pkg.GraphedModule(lambda a, s, z, m: model(a, s, z, mask=m), *x_dev, warmup=1)
            stage("graph captured")
            graph_note = "one CUDA graph per step"
            for _ in range(args.warmup):
                step_resident(x_dev)
            sync()

        # ---- device-resident timing (value): one event pair around the K steps, nothing else inside
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            lib.profile_begin(timing=False)
            sync()
            clocks.region_start()
            e0.record()
            for _ in range(args.steps):
                out = step_resident(x_dev)
            e1.record()
            sync()
            clocks.region_end()
            counted = lib.profile_end()
        ms_resident = e0.elapsed_time(e1) / args.steps
        stage(f"resident timing done: {ms_resident:.2f} ms per step")
        lib.check_device_status()
        if graphed is not None:
            graphed.check()
        for t in out:
            assert torch.isfinite(t.float()).all(), "non-finite output"

        # ---- end to end through the public API with host buffers
        h2d = nbytes(job["host_in"])
        d2h = nbytes(job["host_out"])
        if world > 1:
            t = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
            dist.all_reduce(t)   # whole job: every rank copies its own shard (and the small replicated tensors)
            h2d, d2h = int(t[0]), int(t[1])

        def step_e2e():
            if graphed_mod is not None and job["host_in"]:
                res = graphed_mod(*job["host_in"])   # the copy into the graph's input buffers is the upload
                res = res if isinstance(res, tuple) else (res,)
                for dst, src in zip(job["host_out"], res):
                    dst.copy_(src, non_blocking=True)
                return
            x = to_dev(job["host_in"], dev, non_blocking=True)
            if runner is not None:
                res = step_resident(x)
            else:
                res = job.get("run_inplace", job["run"])(x)
            for dst, src in zip(job["host_out"], res):
                dst.copy_(src, non_blocking=True)

        step_e2e()
        sync()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        for _ in range(args.steps):
            step_e2e()
        e3.record()
        sync()
        ms_e2e = e2.elapsed_time(e3) / args.steps

        # ---- per-kernel breakdown and launch count: ONE more step, eager, an event pair around every launch
        if runner is not None:
            runner.check_status = True
        lib.profile_begin(timing=True)
        step_eager(x_dev)
        sync()
        prof = lib.profile_end()
        launches_per_step = int(sum(l for l, _ in prof.values()))
        eager_launches = int(sum(l for l, _ in counted.values()))
        launches_in_timed_region = (eager_launches if graphed is None and graphed_mod is None
                                    else launches_per_step * args.steps)

    ms_hoisted = 0.0
    if kind == "diffusion" and job["host_in"]:
        # the same step inside a rollout: the pair tensor is unchanged from call to call, so the projections of all
        # blocks are computed once and kept (DiffusionTransformer.hoist_pair_bias); reported next to the headline
        with torch.no_grad():
            model.hoist_pair_bias = True
            if graphed_mod is not None:   # the projections captured in this graph are those of the warm-up calls
                graphed_mod = pkg.GraphedModule(lambda a, s, z, m: model(a, s, z, mask=m), *x_dev, warmup=2)
            for _ in range(2):
                step_resident(x_dev)
            torch.cuda.synchronize(dev)
            e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e4.record()
            for _ in range(args.steps):
                step_resident(x_dev)
            e5.record()
            torch.cuda.synchronize(dev)
            ms_hoisted = e4.elapsed_time(e5) / args.steps
            model.hoist_pair_bias = False

    # ---- max over ranks
    if world > 1:
        t = torch.tensor([ms_resident, ms_e2e, ms_hoisted], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_resident, ms_e2e, ms_hoisted = float(t[0]), float(t[1]), float(t[2])

    flop = workload_flops(cfg, n, blocks)
    value = flop / (ms_resident * 1e-3) / 1e12
    e2e_value = flop / (ms_e2e * 1e-3) / 1e12

    if rank == 0:
        tensor_peak, hbm_peak, peak_kind = peaks()
        kf, kb = kernel_flops(n), kernel_min_bytes(n)
        traffic = dram_traffic_table() if (n == 768 and world == 1) else {}
        share_of = 1.0 / world if sharded else 1.0   # a rank's share of a layer's work
        total_kernel_ms = sum(ms for _, ms in prof.values()) or 1.0
        kernels, roofline = {}, []
        clk = clocks.summary()
        for name, (launches, ms) in sorted(prof.items(), key=lambda kv: -kv[1][1]):
            per_launch_ms = ms / max(1, launches)
            entry = {"launches": launches, "total_ms": round(ms, 3), "share": round(ms / total_kernel_ms, 4),
                     "ms_per_launch": round(per_launch_ms, 4)}
            kernels[name] = entry
            if per_launch_ms <= 0:
                continue
            sec = per_launch_ms * 1e-3
            if name == "single_attn_core" and kind != "diffusion":
                continue   # runs on the second stream under the next block's pair stack: its event time includes waiting
            if name == "single_attn_core":
                # Q K^T + P V over 16 heads of 24 (trunk) or 48 (diffusion): 4 N^2 (H d) flop per sample; a
                # row-sharded rank holds 1 / world of the queries, a diffusion rank its share of the samples
                if kind == "diffusion":
                    fl = 4.0 * n * n * DIFF["c_a"] * -(-cfg["samples"] // world)
                else:
                    fl = 4.0 * n * n * 384 * share_of
                ach = fl / sec / 1e12
                entry["tflops"] = round(ach, 1)
                roofline.append({"kernel": name, "bound": "tensor", "achieved": round(ach, 1), "peak": tensor_peak,
                                 "unit": "TFLOP/s", "frac": round(ach / tensor_peak, 4), "traffic": None,
                                 "peak_kind": f"bf16 sustained, {peak_kind}", "algorithmic_flop_per_launch": fl})
                continue
            if kind == "diffusion":
                continue
            if name in TENSOR_BOUND:
                ach = kf[name] * share_of / sec / 1e12
                r = {"kernel": name, "bound": "tensor", "achieved": round(ach, 1), "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": round(ach / tensor_peak, 4), "traffic": traffic.get(name),
                     "peak_kind": f"bf16 sustained, {peak_kind}", "algorithmic_flop_per_launch": kf[name] * share_of}
                if name == "triattn_core":
                    # second ceiling of this kernel: one exp2 per logit on the MUFU pipe (16 per clock and SM)
                    exps = 4.0 * n * n * n * share_of
                    exp_peak = 16.0 * 148 * (clk.get("sm_mhz") or 1965.0) * 1e6
                    r["exp_bound"] = {"exps_per_launch": exps, "peak_exps_per_s": exp_peak,
                                      "frac": round(exps / sec / exp_peak, 4)}
                entry["tflops"] = round(ach, 1)
                roofline.append(r)
            elif name in kb:
                ach = kb[name] * share_of / sec / 1e9
                roofline.append({"kernel": name, "bound": "hbm", "achieved": round(ach, 1), "peak": hbm_peak,
                                 "unit": "GB/s", "frac": round(ach / hbm_peak, 4), "traffic": traffic.get(name),
                                 "peak_kind": f"copy bandwidth, {peak_kind}",
                                 "algorithmic_bytes_per_launch": kb[name] * share_of})
                entry["gbs"] = round(ach, 1)
        if not roofline:  # no per-kernel model of this workload: the whole step against the tensor peak
            roofline.append({"kernel": "whole step", "bound": "tensor", "achieved": round(value / world, 1),
                             "peak": tensor_peak, "unit": "TFLOP/s", "frac": round(value / world / tensor_peak, 4),
                             "traffic": None, "peak_kind": f"bf16 sustained, {peak_kind}"})
        cpu_baseline = None
        if world == 1 and not args.no_cpu_baseline:
            cpu_s, cpu_flop, cores, what = oracle_sample(cfg, n)
            cpu_baseline = {"value": cpu_flop / cpu_s / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                            "sample": f"{what} on the CPU oracle ({cpu_s:.1f} s)"}
        if kind == "diffusion":
            par = "single GPU" if world == 1 else f"samples dealt over {world} GPUs (rank r: samples r, r+{world}, ...)"
            io = "each rank uploads its samples, the pair tensor and the conditioning; downloads its samples"
            exch = "none"
        else:
            par = "single GPU" if world == 1 else f"DAP row-sharded over {world} GPUs"
            io = ("whole tensors" if world == 1 else
                  "row-sharded: each rank holds, uploads and downloads its N/world rows of z; s replicated")
            exch = ("none" if world == 1 else "barrier + pull kernels over NVLink peer memory"
                    if args.exchange == "peer" else "NCCL all-to-all / all-gather")
        line = {
            "metric": "pairformer_trunk_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_resident, 3),
            "ms_per_block": round(ms_resident / blocks, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.config}: {cfg['label'] if (n, blocks) == (cfg['n'], cfg['blocks']) else cfg['kind'] + f' stack, {blocks} blocks, N_token={n}'}"
                                   ", bf16, seeded random weights",
                       "parallelism": par, "launch": graph_note, "io": io, "exchange": exch,
                       "l2": "inputs and per-layer working set exceed the 126 MB L2; no explicit flush"
                             if n >= 768 else "per-layer working set of a few hundred MB exceeds the 126 MB L2; no explicit flush"},
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_in_timed_region,
            "clocks": clk,
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "kernels": kernels,
            "frac_of_tensor_peak": round(value / world / tensor_peak, 4),
        }
        if parity is not None:
            line["parity_vs_single_gpu"] = parity
        if ms_hoisted > 0:
            line["rollout_step_with_hoisted_pair_bias"] = {
                "ms_per_step": round(ms_hoisted, 3), "value": round(flop / (ms_hoisted * 1e-3) / 1e12, 2),
                "note": "same step when the pair tensor is unchanged since the previous call (a diffusion rollout): the "
                        "blocks' pair-bias projections are reused; the flop count still includes them"}
        print(json.dumps(line))
    if world > 1:
        if graphed is not None:  # a live graph still holds the communicator's captured work
            out = None
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
    ap.add_argument("--config", choices=sorted(CONFIGS), default="c2",
                    help="workload; c2 (the 48-block trunk at N_token = 768) is the headline")
    ap.add_argument("--blocks", type=int, default=0, help="override the configuration's depth (profiling runs)")
    ap.add_argument("--n-token", type=int, default=0, help="override the configuration's N_token (profiling runs)")
    ap.add_argument("--samples", type=int, default=0, help="override c4's sample count (test runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how shards move between GPUs")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying one CUDA graph per step")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.samples and "samples" in cfg:
        cfg["samples"] = args.samples
        cfg["label"] = cfg["label"].replace("5 samples", f"{args.samples} samples")
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
