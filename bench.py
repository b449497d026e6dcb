"""Benchmark of the RG-LRU hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c4a|c0]

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
BWD_DRAM_TRAFFIC_C1 = 195.28e6  # profiles/rglru_scan_config1_bf16.md (read 135.29 MB + write 59.99 MB)


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
        xd = torch.empty(B, T, D, device=dev, dtype=dtype, requires_grad=True)
        dyd = torch.empty(B, T, D, device=dev, dtype=dtype)

        def e2e_step():
            with torch.no_grad():
                xd.copy_(host_x, non_blocking=True)
                dyd.copy_(host_dy, non_blocking=True)
            module.zero_grad(set_to_none=True)
            xd.grad = None
            yy, hh = module(xd, return_state=True)
            yy.backward(dyd)
            host_out.copy_(hh, non_blocking=True)
            host_dlam.copy_(module.Lambda.grad, non_blocking=True)

        e2e_steps = max(3, min(args.steps, 50))
        for _ in range(3):
            e2e_step()
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(e2e_steps):
            e2e_step()
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
               "path": "griffin_b200.RG_LRU(scan_mode='cuda') forward+backward, gate GEMMs included"}
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
        "gpu_launches": 3 * args.steps,
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the per-kernel event pass (for profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
