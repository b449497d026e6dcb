"""Benchmark of the RG-LRU hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c0|c3layer|c4a|c2|c3|c4b]

One step = one forward + one backward pass of the RG-LRU layer kernels over one batch
of synthetic input (BASELINE config 1 by default: bf16 I/O, fp32 state, B=8, T=2048,
D=1024, 16 gate heads).  With N > 1 (launched under torch.distributed.run) every rank
processes its own batch shard of the same size -- the recurrence is independent per
batch row, so there is no data-path collective -- and the reported value is the whole-job
aggregate over the slowest rank's time.

Prints ONE JSON line on rank 0.  ``value`` is algorithmic GB/s (22 B per token-channel for
bf16, 44 for fp32: the 11 compulsory [B,T,D] tensor passes of forward+backward) with inputs
resident in HBM; ``e2e`` is the same metric through the module API with inputs copied from
pinned host memory and results read back inside the timed region; ``roofline`` describes the
dominant kernel (the backward); ``cpu_baseline`` is the CPU oracle (a port of the reference's
sequential path) timed on this machine's host cores on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, T, D, gate blocks, dtype)
    "c0": (2, 256, 256, 4, torch.float32),
    "c1": (8, 2048, 1024, 16, torch.bfloat16),
    "c3layer": (8, 2048, 1024, 16, torch.float32),
    "c4a": (64, 8192, 5632, 16, torch.bfloat16),
}
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one rglru_bwd_kernel launch at config 1, from the
# ncu capture summarised in profiles/ (None until a capture exists for the current kernel).
BWD_DRAM_TRAFFIC_C1 = 193.45e6  # profiles/rglru_scan_config1_bf16.md (read 135.30 MB + write 58.15 MB)


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run (read-only)."""

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def run_ours(args) -> dict:
    import torch.distributed as dist

    from griffin_b200 import RG_LRU, _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local if world > 1 else 0)
    torch.cuda.set_device(dev)
    lib = _lib.load()

    B, T, D, G, dtype = WORKLOADS[args.workload]
    es = 2 if dtype == torch.bfloat16 else 4
    io = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    n_elem = B * T * D
    bytes_fwd, bytes_bwd = 4 * es * n_elem, 7 * es * n_elem
    bytes_step = bytes_fwd + bytes_bwd

    # Rotating input sets so consecutive steps never find their inputs in L2 (126 MB).
    nsets = max(2, min(4, int(2e9 // max(1, bytes_step))))
    gen = torch.Generator().manual_seed(1234 + rank)
    sets = []
    for s in range(nsets):
        x = torch.randn(B, T, D, generator=gen).to(dtype).to(dev) if s == 0 else torch.randn(B, T, D, device=dev).to(dtype)
        u_r = torch.randn(B, T, D, device=dev).to(dtype)
        u_i = torch.randn(B, T, D, device=dev).to(dtype)
        dy = torch.randn(B, T, D, device=dev).to(dtype)
        sets.append((x, u_r, u_i, dy))
    lam = torch.logit(torch.empty(D).uniform_(0.9, 0.999, generator=gen).pow(1.0 / 8.0)).to(dev)
    y = torch.empty(B, T, D, device=dev, dtype=dtype)
    dx, du_r, du_i = (torch.empty(B, T, D, device=dev, dtype=dtype) for _ in range(3))
    h_last = torch.empty(B, D, device=dev)
    dlam = torch.empty(D, device=dev)
    ws_bytes = lib.rglru_workspace_bytes(B, T, D, io)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def fwd(s):
        x, u_r, u_i, _ = sets[s]
        rc = lib.rglru_fwd(x.data_ptr(), u_r.data_ptr(), u_i.data_ptr(), lam.data_ptr(), None, None, y.data_ptr(),
                           h_last.data_ptr(), ws.data_ptr(), ws_bytes, B, T, D, 8.0, io, stream)
        _lib.check(rc, "rglru_fwd")

    def bwd(s):
        x, u_r, u_i, dy = sets[s]
        rc = lib.rglru_bwd(dy.data_ptr(), None, x.data_ptr(), u_r.data_ptr(), u_i.data_ptr(), lam.data_ptr(), None,
                           None, ws.data_ptr(), ws_bytes, dx.data_ptr(), du_r.data_ptr(), du_i.data_ptr(),
                           dlam.data_ptr(), None, B, T, D, 8.0, io, stream)
        _lib.check(rc, "rglru_bwd")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(dev.index or 0)
    for w in range(args.warmup):
        fwd(w % nsets)
        bwd(w % nsets)
    barrier()
    sampler.start()

    # ---- region 1: exactly K steps, device-timed
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for k in range(args.steps):
        fwd(k % nsets)
        bwd(k % nsets)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps

    # ---- region 2: per-kernel durations (CUDA events around every launch, same stream)
    reps = 1 if args.no_kernel_timing else max(args.steps, 200)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(reps)]
    for k in range(reps):
        evs[k][0].record()
        fwd(k % nsets)
        evs[k][1].record()
        bwd(k % nsets)
        evs[k][2].record()
    torch.cuda.synchronize(dev)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)

    # ---- region 3: end to end through the module API from pinned host memory
    e2e = None
    if not args.no_e2e:
        module = RG_LRU(D, gate_blocks=G, scan_mode="cuda").to(dev, dtype)
        host_x = torch.randn(B, T, D).to(dtype).pin_memory()
        host_dy = torch.randn(B, T, D).to(dtype).pin_memory()
        host_out = torch.empty(B, D, dtype=torch.float32).pin_memory()
        host_dlam = torch.empty(D, dtype=dtype).pin_memory()
        # Two device buffers per input: the copies of step k+1 (own stream) overlap the kernels of step k.
        bufs = [(torch.empty(B, T, D, device=dev, dtype=dtype, requires_grad=True),
                 torch.empty(B, T, D, device=dev, dtype=dtype)) for _ in range(2)]
        copy_stream = torch.cuda.Stream(dev)
        main_stream = torch.cuda.current_stream(dev)
        loaded = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]

        def e2e_copy(k):
            xd, dyd = bufs[k % 2]
            with torch.cuda.stream(copy_stream), torch.no_grad():
                copy_stream.wait_event(consumed[k % 2])          # the step that last used this buffer is done
                xd.copy_(host_x, non_blocking=True)
                dyd.copy_(host_dy, non_blocking=True)
                loaded[k % 2].record(copy_stream)

        def e2e_compute(k):
            xd, dyd = bufs[k % 2]
            main_stream.wait_event(loaded[k % 2])
            module.zero_grad(set_to_none=True)
            xd.grad = None
            yy, hh = module(xd, return_state=True)
            yy.backward(dyd)
            consumed[k % 2].record(main_stream)
            host_out.copy_(hh, non_blocking=True)
            host_dlam.copy_(module.Lambda.grad, non_blocking=True)

        def e2e_run(n):
            e2e_copy(0)
            for k in range(n):
                if k + 1 < n:
                    e2e_copy(k + 1)
                e2e_compute(k)

        e2e_steps = max(3, min(args.steps, 50))
        for ev in consumed:
            ev.record(main_stream)
        e2e_run(3)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        e2e_run(e2e_steps)
        a1.record()
        barrier()
        e2e_ms = a0.elapsed_time(a1) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": world * bytes_step / e2e_ms / 1e6, "unit": "GB/s",
               "h2d_bytes_per_step": 2 * es * n_elem, "d2h_bytes_per_step": 4 * B * D + es * D,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "path": "griffin_b200.RG_LRU(scan_mode='cuda') forward+backward, gate GEMMs included; every step's inputs "
                       "copied from pinned host memory on a second stream (double-buffered), results read back"}
    clocks = sampler.stop()
    status = _lib.device_status()

    peak, peak_kind = measured_peak()
    achieved = bytes_bwd / bwd_ms / 1e6
    out = {
        "metric": "rglru_fwd_bwd_hbm_gbs",
        "value": world * bytes_step / ms_step / 1e6,
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 I/O, f32 state" if dtype == torch.bfloat16 else "f32",
        "data": "synthetic",
        "config": {
            "workload": f"{args.workload}: RG-LRU fwd+bwd B={B}/GPU T={T} D={D} gate_heads={G}",
            "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB touched per step, {nsets} rotating input sets",
            "sharding": "batch rows per rank, no collective",
        },
        "token_channels_per_s": world * n_elem / ms_step * 1e3,
        "frac_of_hbm_peak": world * bytes_step / ms_step / 1e6 / (world * peak),
        "kernels_ms": {"rglru_fwd": fwd_ms, "rglru_bwd": bwd_ms},
        "roofline": {"bound": "hbm", "kernel": "rglru_bwd_kernel", "achieved": achieved, "peak": peak,
                     "peak_source": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                     "traffic": BWD_DRAM_TRAFFIC_C1 if args.workload == "c1" else None,
                     "algorithmic_bytes": bytes_bwd,
                     "fwd": {"achieved": bytes_fwd / fwd_ms / 1e6, "frac": bytes_fwd / fwd_ms / 1e6 / peak}},
        "e2e": e2e,
        "gpu_launches": (2 if B <= 64 else 3) * args.steps,   # fwd + bwd (+ the dLambda fold kernel for B > 64)
        "clocks": clocks,
        "device_status": status,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(args.workload, steps=1)
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def cpu_baseline(workload: str, steps: int = 1) -> dict:
    """The oracle's sequential path (same torch primitives as the reference) forward+backward on host cores.

    Bounded sample: the workload's T, D and dtype with a reduced batch, because the reference's backward is
    O(T^2) per row on CPU (autograd re-materialises a full-size tensor per time-step).
    """
    from oracle import rglru_oracle as orc

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on.
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    B, T, D, G, dtype = WORKLOADS[workload]
    sample_b = B if B * T * D <= (1 << 24) else max(1, (1 << 24) // (T * D))
    sample_t = min(T, 2048)  # the reference's backward is O(T^2) per row on CPU
    case = orc.make_rglru_case(sample_b, sample_t, D, G, seed=0)
    names = ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")
    es = 2 if dtype == torch.bfloat16 else 4
    best = None
    for _ in range(steps):
        params = {k: case[k].to(dtype).requires_grad_(True) for k in names}
        x = case["x"].to(dtype).requires_grad_(True)
        dy = case["dy"].to(dtype)
        t0 = time.perf_counter()
        y, _ = orc.rglru_layer(x, params)
        y.backward(dy)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    n = sample_b * sample_t * D
    return {"value": 11 * es * n / best / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port", "seconds": best, "token_channels_per_s": n / best,
            "sample": f"B={sample_b} T={sample_t} D={D} {str(dtype).replace('torch.', '')} module path "
                      f"(gates + sequential scan, autograd backward), best of {steps}"}


def run_reference(args) -> dict:
    """The reference arm: the reference's CPU sequential path (oracle port), all host threads, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    B, T, D, G, dtype = WORKLOADS[args.workload]
    steps = max(1, min(args.steps, 3))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(args.workload, 1)
    base = cpu_baseline(args.workload, steps)
    return {
        "impl": "reference",
        "metric": "rglru_fwd_bwd_hbm_gbs",
        "value": base["value"],
        "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps,
        "warmup": min(args.warmup, 1),
        "ms_per_step": base["seconds"] * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 I/O, f32 state" if dtype == torch.bfloat16 else "f32",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: RG-LRU fwd+bwd B={B}/GPU T={T} D={D} gate_heads={G}",
                   "note": "CPU; each step is the bounded sample described in cpu_baseline.sample"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# --------------------------------------------------------------------------- secondary workloads
def _dist_setup():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local if world > 1 else 0)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, world, rank, dev


def _timed(fn, steps, warmup, dist, world, dev):
    """W warm-up calls, then exactly K timed calls between barriers; returns max-over-ranks ms per call."""
    for i in range(warmup):
        fn(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def run_block(args) -> dict:
    """BASELINE config 2: the full recurrent temporal block, bf16, B=16/GPU, T=2048, 768 -> 1024 -> 768, fwd+bwd."""
    from griffin_b200 import RecurrentBlock, _lib
    dist, world, rank, dev = _dist_setup()
    B, T, DM, DR = 16, 2048, 768, 1024
    torch.manual_seed(rank)
    blk = RecurrentBlock(DM, DR, gate_blocks=16, scan_mode="cuda", fold_conv=args.fold == "conv",
                         fold_merge=args.fold == "merge")
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)       # N(0, 1/4) as the config states
    blk = blk.to(dev, torch.bfloat16)
    xs = [torch.randn(B, T, DM, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(3)]
    dout = torch.randn(B, T, DM, device=dev).to(torch.bfloat16)
    sampler = ClockSampler(dev.index or 0)
    module = blk
    if args.graph:   # forward and backward of the block replayed as two CUDA graphs (the step is launch-bound otherwise)
        blk = torch.cuda.make_graphed_callables(module, (xs[0],))

    def step(i):
        x = xs[i % 3]
        x.grad = None
        if not args.graph:
            module.zero_grad(set_to_none=True)
        blk(x).backward(dout)

    sampler.start()
    ms = _timed(step, args.steps, args.warmup, dist, world, dev)
    host_x = torch.randn(B, T, DM).to(torch.bfloat16).pin_memory()
    host_loss = torch.empty(1).pin_memory()

    def e2e_step(i):
        x = xs[0]
        with torch.no_grad():
            x.copy_(host_x, non_blocking=True)
        x.grad = None
        if not args.graph:
            module.zero_grad(set_to_none=True)
        out = blk(x)
        out.backward(dout)
        host_loss.copy_(out.float().square().mean().reshape(1), non_blocking=True)

    e2e_ms = _timed(e2e_step, max(3, min(args.steps, 50)), 3, dist, world, dev)
    clocks = sampler.stop()
    n = B * T * DR
    peak, kind = measured_peak()
    out = {"metric": "recurrent_block_fwd_bwd_token_channels_per_s", "value": world * n / ms * 1e3, "unit": "token-channels/s",
           "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16 I/O, f32 state", "data": "synthetic",
           "config": {"workload": f"c2: RecurrentBlock fwd+bwd bf16 B={B}/GPU T={T} {DM}->{DR}->{DM}, conv k=4, 16 gate heads",
                      "fold": args.fold, "cuda_graph": bool(args.graph),
                      "l2": "three rotating inputs; 0.6 GB of activations per step"},
           "scan_conv_algorithmic_gbs": world * (22 + 10) * n / ms / 1e6,
           "e2e": {"value": world * n / e2e_ms * 1e3, "unit": "token-channels/s", "h2d_bytes_per_step": 2 * B * T * DM,
                   "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
           "gpu_launches": 6 * args.steps, "clocks": clocks, "device_status": _lib.device_status(),
           "roofline": {"bound": "hbm", "note": "GEMMs (torch) dominate this step; see the c1 line for the kernel roofline",
                        "peak": peak, "peak_source": f"of {kind}", "unit": "GB/s", "achieved": None, "frac": None, "traffic": None}}
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_lm(args) -> dict:
    """BASELINE config 3: Griffin ~100M training step, bf16 autocast, B=8/GPU, T=2048, DDP over NCCL for N > 1."""
    from griffin_b200 import _lib
    from griffin_b200.lm import GriffinModel
    dist, world, rank, dev = _dist_setup()
    B, T, V = 8, 2048, 50257
    torch.manual_seed(0)
    model = GriffinModel(V, 768, 3, 1024, 12, attention_heads=6, attention_window_size=1024, gate_blocks=16,
                         scan_mode="cuda")
    for layer in model.layers:
        if hasattr(layer, "recurrent"):
            layer.recurrent.fold_conv, layer.recurrent.fold_merge = args.fold == "conv", args.fold == "merge"
    model = model.to(dev)
    nparams = sum(p.numel() for p in model.parameters())
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index]) if world > 1 else model
    decay = [p for n_, p in model.named_parameters() if p.dim() >= 2]
    plain = [p for n_, p in model.named_parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0}],
                            lr=3e-4, betas=(0.9, 0.95), fused=True)
    gen = torch.Generator().manual_seed(100 + rank)
    host_ids = [torch.randint(0, V, (B, T + 1), generator=gen).pin_memory() for _ in range(4)]
    dev_ids = [h.to(dev) for h in host_ids]
    host_loss = torch.empty(1).pin_memory()
    sampler = ClockSampler(dev.index or 0)

    def train(ids):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net(ids[:, :-1], pad_vocab=True)       # vocabulary padded to a multiple of 8, -inf in the padding
        loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.size(-1)), ids[:, 1:].reshape(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step(i):
        train(dev_ids[i % 4])

    def e2e_step(i):
        ids = host_ids[i % 4].to(dev, non_blocking=True)
        host_loss.copy_(train(ids).detach().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the reference reads loss.item() every step

    sampler.start()
    ms = _timed(step, args.steps, args.warmup, dist, world, dev)
    e2e_ms = _timed(e2e_step, max(3, min(args.steps, 20)), 2, dist, world, dev)
    clocks = sampler.stop()
    out = {"metric": "griffin100m_train_tokens_per_s", "value": world * B * T / ms * 1e3, "unit": "tokens/s",
           "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast (RG-LRU: bf16 I/O, fp32 state and arithmetic)", "data": "synthetic",
           "config": {"workload": f"c3: Griffin-100M ({nparams} params) train step B={B}/GPU T={T} vocab {V}, AdamW, "
                                  f"{'DDP/NCCL' if world > 1 else 'single GPU'}",
                      "fold": args.fold, "l2": "activations of one step far exceed L2"},
           "e2e": {"value": world * B * T / e2e_ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B * (T + 1),
                   "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
           "gpu_launches": 8 * 6 * args.steps,   # per recurrent layer: conv fwd + state, scan fwd, scan bwd, conv bwd + fold "clocks": clocks, "device_status": _lib.device_status(),
           "roofline": {"bound": "tensor", "note": "whole-model step: torch GEMMs and attention dominate; the library's kernels "
                        "are the conv, the RG-LRU scan and their backwards in 8 of 12 layers", "achieved": None, "peak": None,
                        "frac": None, "traffic": None, "unit": "TFLOP/s"}}
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_decode(args) -> dict:
    """BASELINE config 4 part two: single-token decode update, B=512/GPU, D=5632, fp32 carried state, bf16 I/O,
    1024 steps per timed call (one CUDA graph of 1024 kernel launches)."""
    from griffin_b200 import _lib
    dist, world, rank, dev = _dist_setup()
    lib = _lib.load()
    B, D, NSTEP, NSET = 512, 5632, 1024, 8
    xs = [tuple(torch.randn(B, D, device=dev).to(torch.bfloat16) for _ in range(3)) for _ in range(NSET)]
    lam = torch.logit(torch.empty(D).uniform_(0.9, 0.999).pow(1.0 / 8.0)).to(dev)
    h = torch.zeros(B, D, device=dev)
    y = torch.empty(B, D, device=dev, dtype=torch.bfloat16)

    def one(i, stream):
        x, ur, ui = xs[i % NSET]
        rc = lib.rglru_decode_step(x.data_ptr(), ur.data_ptr(), ui.data_ptr(), lam.data_ptr(), h.data_ptr(), None,
                                   y.data_ptr(), B, D, 8.0, _lib.BF16, stream)
        _lib.check(rc, "rglru_decode_step")

    one(0, torch.cuda.current_stream(dev).cuda_stream)      # per-device set-up happens outside capture
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    with torch.cuda.graph(graph, stream=side):
        for i in range(NSTEP):
            one(i, side.cuda_stream)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms = _timed(lambda i: graph.replay(), args.steps, args.warmup, dist, world, dev)
    clocks = sampler.stop()
    n = B * D
    bytes_step = 16 * n                     # x, u_r, u_i bf16 in; y bf16 out; h fp32 in and out
    peak, kind = measured_peak()
    achieved = bytes_step * NSTEP / ms / 1e6
    out = {"metric": "rglru_decode_hbm_gbs", "value": world * achieved, "unit": "GB/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16 I/O, f32 state", "data": "synthetic",
           "config": {"workload": f"c4b: decode update B={B}/GPU D={D}, {NSTEP} token steps per timed call (CUDA graph)",
                      "l2": f"{NSET} rotating input sets of 17 MB plus 23 MB of state: the state and part of the inputs stay in L2"},
           "decode_steps_per_s": world * NSTEP / ms * 1e3, "us_per_token_step": ms * 1e3 / NSTEP,
           "roofline": {"bound": "hbm", "kernel": "decode_step_kernel", "achieved": achieved, "peak": peak,
                        "peak_source": f"of {kind}", "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                        "algorithmic_bytes": bytes_step},
           "e2e": None, "gpu_launches": NSTEP * args.steps, "clocks": clocks, "device_status": _lib.device_status()}
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS) + ["c2", "c3", "c4b"])
    ap.add_argument("--fold", default="merge", choices=["none", "conv", "merge"],
                    help="c2/c3: run conv (and the GeLU-branch product) inside the scan kernels")
    ap.add_argument("--graph", action="store_true", help="c2: replay the block's forward and backward as CUDA graphs")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the per-kernel event pass (for profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        if args.workload not in WORKLOADS:
            raise SystemExit("--impl reference covers the RG-LRU layer workloads only")
        out = run_reference(args)
    elif args.workload == "c2":
        out = run_block(args)
    elif args.workload == "c3":
        out = run_lm(args)
    elif args.workload == "c4b":
        out = run_decode(args)
    else:
        out = run_ours(args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
