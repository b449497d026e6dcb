"""Benchmark of the RG-LRU hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c1|c0|c3layer|c4a|c2|c3|c4b] [--no-extra]

One step = one forward + one backward pass of the RG-LRU layer kernels over one batch of synthetic
input.  The default workload ("c1") is bf16 I/O with fp32 state, B=8, T=2048, D=1024, 16 gate heads.
With N > 1 (launched under torch.distributed.run) every rank processes its own batch shard of the same
size -- the recurrence is independent per batch row, so there is no data-path collective -- and the
reported value is the whole-job aggregate over the slowest rank's time.

Prints ONE JSON line on rank 0.  ``value`` is algorithmic GB/s (22 B per token-channel for bf16, 44 for
fp32: the 11 compulsory [B,T,D] tensor passes of forward+backward) with inputs resident in HBM;
``e2e`` is the same metric through the module API with inputs copied from pinned host memory and
results read back inside the timed region; ``roofline`` describes the dominant kernel (the backward);
``cpu_baseline`` is the reference's sequential path timed on this machine's host cores.  Unless
``--no-extra`` is given, the default line also carries two sub-objects measured in the same run: ``c4a``
(the B=64, T=8192, D=5632 problem batch-sharded over the N ranks) and ``c3`` (the Griffin-100M training
step, data-parallel over NCCL for N > 1).
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


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_name(workload: str) -> str:
    B, T, D, G, dtype = WORKLOADS[workload]
    return f"{workload}: RG-LRU fwd+bwd {'bf16' if dtype == torch.bfloat16 else 'fp32'} B={B}/GPU T={T} D={D} gate_heads={G}"


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
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


class Dist:
    """Process-group plumbing shared by all workloads: one process per GPU, NCCL, barrier + max over ranks."""

    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", local if self.world > 1 else 0)
        torch.cuda.set_device(self.dev)
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1 and self.dist.is_initialized():
            self.dist.destroy_process_group()


class LayerKernels:
    """rglru_fwd / rglru_bwd through the C ABI on rotating sets of device-resident tensors.

    Inputs AND outputs rotate together, so a step neither finds its inputs in the 126 MB L2 nor overwrites
    results that are still dirty there from the step before."""

    def __init__(self, B, T, D, dtype, dev, seed, max_bytes=3e9):
        from griffin_b200 import _lib

        self._lib = _lib
        self.lib = _lib.load()
        self.B, self.T, self.D, self.dev = B, T, D, dev
        self.es = 2 if dtype == torch.bfloat16 else 4
        self.io = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
        self.n_elem = B * T * D
        self.bytes_fwd, self.bytes_bwd = 4 * self.es * self.n_elem, 7 * self.es * self.n_elem
        per_set = 8 * self.es * self.n_elem
        self.nsets = max(2, min(4, int(max_bytes // max(1, per_set))))
        gen = torch.Generator(device=dev).manual_seed(seed)
        mk = lambda: torch.randn(B, T, D, device=dev, generator=gen).to(dtype)
        self.sets = [tuple(mk() for _ in range(4)) for _ in range(self.nsets)]                       # x, u_r, u_i, dy
        self.outs = [tuple(torch.empty(B, T, D, device=dev, dtype=dtype) for _ in range(4))          # y, dx, du_r, du_i
                     for _ in range(self.nsets)]
        cpu_gen = torch.Generator().manual_seed(seed)
        self.lam = torch.logit(torch.empty(D).uniform_(0.9, 0.999, generator=cpu_gen).pow(1.0 / 8.0)).to(dev)
        self.h_last = torch.empty(B, D, device=dev)
        self.dlam = torch.empty(D, device=dev)
        self.ws_bytes = self.lib.rglru_workspace_bytes(B, T, D, self.io)
        # one workspace per set: the backward of a set reads the states its own forward left there
        self.wss = [torch.empty(self.ws_bytes, device=dev, dtype=torch.uint8) for _ in range(self.nsets)]
        self.stream = torch.cuda.current_stream(dev).cuda_stream
        self.calls = 0
        self.kernels_per_step = 2 if B <= 64 else 3      # fwd + bwd (+ the dLambda fold kernel for B > 64)

    def fwd(self, s):
        x, u_r, u_i, _ = self.sets[s % self.nsets]
        y = self.outs[s % self.nsets][0]
        ws = self.wss[s % self.nsets]
        rc = self.lib.rglru_fwd(x.data_ptr(), u_r.data_ptr(), u_i.data_ptr(), self.lam.data_ptr(), None, None,
                                y.data_ptr(), self.h_last.data_ptr(), ws.data_ptr(), self.ws_bytes,
                                self.B, self.T, self.D, 8.0, self.io, self.stream)
        self._lib.check(rc, "rglru_fwd")
        self.calls += 1

    def bwd(self, s):
        x, u_r, u_i, dy = self.sets[s % self.nsets]
        _, dx, du_r, du_i = self.outs[s % self.nsets]
        ws = self.wss[s % self.nsets]
        rc = self.lib.rglru_bwd(dy.data_ptr(), None, x.data_ptr(), u_r.data_ptr(), u_i.data_ptr(), self.lam.data_ptr(),
                                None, None, ws.data_ptr(), self.ws_bytes, dx.data_ptr(), du_r.data_ptr(),
                                du_i.data_ptr(), self.dlam.data_ptr(), None, self.B, self.T, self.D, 8.0, self.io,
                                self.stream)
        self._lib.check(rc, "rglru_bwd")
        self.calls += 1

    def step(self, s):
        self.fwd(s)
        self.bwd(s)


def timed_steps(d: Dist, step, steps: int, repeats: int) -> tuple[float, list[float]]:
    """``repeats`` regions of exactly ``steps`` steps each, CUDA events on the launching stream, barrier on both
    sides; returns (median ms per step over the regions after max over ranks, the per-region values)."""
    per_region = []
    for r in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d.barrier()
        e0.record()
        for k in range(steps):
            step(r * steps + k)
        e1.record()
        d.barrier()
        per_region.append(d.max_over_ranks(e0.elapsed_time(e1)) / steps)
    return statistics.median(per_region), per_region


def run_layer(args, d: Dist) -> dict:
    from griffin_b200 import RG_LRU, _lib

    dev, world, rank = d.dev, d.world, d.rank
    B, T, D, G, dtype = WORKLOADS[args.workload]
    k = LayerKernels(B, T, D, dtype, dev, seed=1234 + rank)
    es, n_elem = k.es, k.n_elem
    bytes_step = k.bytes_fwd + k.bytes_bwd

    sampler = ClockSampler(dev.index or 0)
    for w in range(args.warmup):
        k.step(w)
    d.barrier()
    sampler.start()

    # ---- region 1: exactly K steps per region, device-timed; regions repeated until they span about half a second
    probe, _ = timed_steps(d, k.step, args.steps, 1)
    repeats = 1 if args.no_repeat else max(1, min(400, int(500.0 / max(1e-3, probe * args.steps))))
    k.calls = 0
    ms_step, regions = timed_steps(d, k.step, args.steps, repeats)
    launches = k.calls // 2 * k.kernels_per_step // repeats        # counted calls of one region x kernels per call

    # ---- region 2: per-kernel durations: each kernel launched back to back over the rotating sets, CUDA events
    # on the launching stream around the run (an event between every two launches would keep a kernel's prologue
    # from overlapping the tail of the one before it, which it does in region 1)
    reps = 1 if args.no_kernel_timing else max(args.steps, 200)
    for s_ in range(k.nsets):
        k.fwd(s_)                                   # every set's workspace now holds its forward's states
    torch.cuda.synchronize(dev)
    per_kernel = {}
    for name, launch in (("rglru_fwd", k.fwd), ("rglru_bwd", k.bwd)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            launch(i)
        e1.record()
        torch.cuda.synchronize(dev)
        per_kernel[name] = e0.elapsed_time(e1) / reps
    fwd_ms, bwd_ms = per_kernel["rglru_fwd"], per_kernel["rglru_bwd"]

    # ---- region 3: end to end through the module API from pinned host memory, every result read back
    e2e = None
    if not args.no_e2e:
        module = RG_LRU(D, gate_blocks=G, scan_mode="cuda").to(dev, dtype)
        host_x = torch.randn(B, T, D).to(dtype).pin_memory()
        host_dy = torch.randn(B, T, D).to(dtype).pin_memory()
        host_y = torch.empty(B, T, D, dtype=dtype).pin_memory()
        host_dx = torch.empty(B, T, D, dtype=dtype).pin_memory()
        host_h = torch.empty(B, D, dtype=torch.float32).pin_memory()
        host_dlam = torch.empty(D, dtype=dtype).pin_memory()
        # Two device buffers per tensor: the host-to-device copies of step k+1 and the device-to-host copies of
        # step k-1 (each on a stream of its own) overlap the kernels of step k.
        bufs = [(torch.empty(B, T, D, device=dev, dtype=dtype, requires_grad=True),
                 torch.empty(B, T, D, device=dev, dtype=dtype)) for _ in range(2)]
        res = [None, None]
        in_stream, out_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        main_stream = torch.cuda.current_stream(dev)
        loaded = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        computed = [torch.cuda.Event() for _ in range(2)]
        drained = [torch.cuda.Event() for _ in range(2)]

        def e2e_copy_in(i):
            xd, dyd = bufs[i % 2]
            with torch.cuda.stream(in_stream), torch.no_grad():
                in_stream.wait_event(consumed[i % 2])          # the step that last used this buffer is done
                xd.copy_(host_x, non_blocking=True)
                dyd.copy_(host_dy, non_blocking=True)
                loaded[i % 2].record(in_stream)

        def e2e_compute(i):
            xd, dyd = bufs[i % 2]
            main_stream.wait_event(loaded[i % 2])
            main_stream.wait_event(drained[i % 2])            # the results two steps back have left the device
            module.zero_grad(set_to_none=True)
            xd.grad = None
            yy, hh = module(xd, return_state=True)
            yy.backward(dyd)
            res[i % 2] = (yy.detach(), xd.grad, hh.detach(), module.Lambda.grad)
            consumed[i % 2].record(main_stream)
            computed[i % 2].record(main_stream)

        def e2e_copy_out(i):
            yy, dxx, hh, dl = res[i % 2]
            with torch.cuda.stream(out_stream), torch.no_grad():
                out_stream.wait_event(computed[i % 2])
                host_y.copy_(yy, non_blocking=True)
                host_dx.copy_(dxx, non_blocking=True)
                host_h.copy_(hh, non_blocking=True)
                host_dlam.copy_(dl, non_blocking=True)
                drained[i % 2].record(out_stream)

        def e2e_run(n):
            e2e_copy_in(0)
            for i in range(n):
                if i + 1 < n:
                    e2e_copy_in(i + 1)
                e2e_compute(i)
                e2e_copy_out(i)
            main_stream.wait_stream(out_stream)

        e2e_steps = max(3, min(args.steps, 50))
        for ev in consumed + drained:
            ev.record(main_stream)
        e2e_run(3)
        d.barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        e2e_run(e2e_steps)
        a1.record()
        d.barrier()
        e2e_ms = d.max_over_ranks(a0.elapsed_time(a1) / e2e_steps)
        e2e = {"value": world * bytes_step / e2e_ms / 1e6, "unit": "GB/s",
               "h2d_bytes_per_step": 2 * es * n_elem, "d2h_bytes_per_step": 2 * es * n_elem + 4 * B * D + es * D,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "path": "griffin_b200.RG_LRU(scan_mode='cuda') forward+backward, gate GEMMs included; every step's x and "
                       "dy copied from pinned host memory, y, dx, h_last and dLambda copied back to pinned host memory; "
                       "copies double-buffered on their own streams"}
    clocks = sampler.stop()
    status = _lib.device_status()

    peak, peak_kind = measured_peak()
    achieved = k.bytes_bwd / bwd_ms / 1e6
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
        "config": {"workload": workload_name(args.workload)},
        "timing": {"regions": repeats, "steps_per_region": args.steps, "value_is": "median over regions",
                   "ms_per_step_min": min(regions), "ms_per_step_max": max(regions),
                   "l2": f"inputs larger than L2: {bytes_step / 1e6:.0f} MB touched per step, {k.nsets} rotating sets of "
                         "inputs and outputs",
                   "sharding": "batch rows per rank, no collective"},
        "token_channels_per_s": world * n_elem / ms_step * 1e3,
        "frac_of_hbm_peak": world * bytes_step / ms_step / 1e6 / (world * peak),
        "kernels_ms": {"rglru_fwd": fwd_ms, "rglru_bwd": bwd_ms},
        "roofline": {"bound": "hbm", "kernel": "rglru_bwd_kernel", "achieved": achieved, "peak": peak,
                     "peak_source": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None,     # not measured by this run (an ncu capture is summarised under profiles/)
                     "algorithmic_bytes": k.bytes_bwd,
                     "fwd": {"achieved": k.bytes_fwd / fwd_ms / 1e6, "frac": k.bytes_fwd / fwd_ms / 1e6 / peak}},
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clocks,
        "device_status": status,
    }
    del k
    torch.cuda.empty_cache()
    return out


def run_c4a_shard(args, d: Dist) -> dict:
    """The B=64, T=8192, D=5632 bf16 problem with its batch rows split over the ranks (strong scaling): every
    rank runs rglru_fwd + rglru_bwd on its 64/N rows, no collective; max over ranks."""
    from griffin_b200 import _lib
    from griffin_b200.sharding import batch_shard

    B, T, D, G, dtype = WORKLOADS["c4a"]
    lo, hi = batch_shard(B, d.rank, d.world)
    rows = hi - lo
    k = LayerKernels(rows, T, D, dtype, d.dev, seed=77 + d.rank, max_bytes=2 * 8 * 2 * rows * T * D)
    sampler = ClockSampler(d.dev.index or 0).start()
    steps = max(2, min(args.steps, 5))
    for w in range(3):
        k.step(w)
    ms, regions = timed_steps(d, k.step, steps, 3)
    clocks = sampler.stop()
    peak, kind = measured_peak()
    total = 22 * B * T * D
    gbs = total / ms / 1e6
    out = {"workload": f"c4a: RG-LRU fwd+bwd bf16 B={B} T={T} D={D} batch-sharded over {d.world} rank(s), {rows} rows on this rank",
           "scaling": "strong", "ms_per_step": ms, "steps": steps, "regions": 3, "gbs": gbs,
           "gbs_per_gpu": gbs / d.world, "frac": gbs / d.world / peak, "peak_source": f"of {kind}",
           "token_channels_per_s": B * T * D / ms * 1e3, "clocks": clocks, "device_status": _lib.device_status()}
    del k
    torch.cuda.empty_cache()
    return out


def run_time_shard(args, d: Dist) -> dict:
    """One sequence of B=8, D=1024 (``--width``), bf16, T = 8192 per rank, split along TIME over the ranks: forward + backward
    through ``griffin_b200.time_shard.rglru_time_sharded`` (per direction a carry-only pass, one all-gather of
    [B, D] carries over NCCL, and the full pass); beside it the same rank's slice as an ordinary
    unsplit call, i.e. what the step would cost were there no carry between the slices."""
    from griffin_b200 import _lib, ops
    from griffin_b200.time_shard import rglru_time_sharded

    B, TS, D = 8, 8192, args.width
    dev, world = d.dev, d.world
    if world == 1 and not d.dist.is_initialized():     # the operator wants a process group even for one slice
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        d.dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    g = torch.Generator(device=dev).manual_seed(11 + d.rank)
    sets = []
    for _ in range(3):    # 3 x 4 tensors x 134 MB: a step never finds its inputs in L2
        x = torch.randn(B, TS, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        u_r = torch.randn(B, TS, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        u_i = torch.randn(B, TS, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        dy = torch.randn(B, TS, D, device=dev, generator=g).to(torch.bfloat16)
        sets.append((x, u_r, u_i, dy))
    lam = torch.logit(torch.empty(D, device=dev).uniform_(0.9, 0.999, generator=g).pow(1.0 / 8.0)).requires_grad_(True)

    def clear(x, u_r, u_i):
        x.grad = u_r.grad = u_i.grad = lam.grad = None

    def sharded(i):
        x, u_r, u_i, dy = sets[i % 3]
        clear(x, u_r, u_i)
        y, _ = rglru_time_sharded(x, u_r, u_i, lam, None, None, 8.0, None)
        y.backward(dy)

    def unsplit(i):
        x, u_r, u_i, dy = sets[i % 3]
        clear(x, u_r, u_i)
        y, _ = ops.rglru(x, u_r, u_i, lam, None, None, 8.0)
        y.backward(dy)

    sampler = ClockSampler(dev.index or 0).start()
    steps = max(3, min(args.steps, 50))
    for w in range(max(3, args.warmup)):
        sharded(w)
        unsplit(w)
    ms, regions = timed_steps(d, sharded, steps, 3)
    ms_one, _ = timed_steps(d, unsplit, steps, 3)
    clocks = sampler.stop()
    if world == 1:
        d.dist.destroy_process_group()
    peak, kind = measured_peak()
    total = 22 * B * TS * world * D          # algorithmic bytes of the whole sequence, forward + backward
    return {"metric": "rglru_time_sharded_fwd_bwd_hbm_gbs", "value": total / ms / 1e6, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 I/O, f32 state", "data": "synthetic",
            "config": {"workload": f"time-sharded RG-LRU fwd+bwd bf16 B={B} T={TS * world} ({TS} per rank) D={D}",
                       "l2": f"three rotating input sets of {4 * 2 * B * TS * D / 1e6:.0f} MB each"},
            "timing": {"regions": len(regions), "value_is": "median over regions",
                       "ms_per_step_min": min(regions), "ms_per_step_max": max(regions)},
            "unsplit_slice_ms_per_step": ms_one, "cost_of_the_split": ms / ms_one,
            "exchange_bytes_per_rank_per_step": 3 * B * D * 4,
            "frac_of_hbm_peak_per_gpu": total / world / ms / 1e6 / peak, "peak_source": f"of {kind}",
            "gpu_launches": (4 if world > 1 else 2) * steps, "clocks": clocks, "device_status": _lib.device_status(),
            "roofline": {"bound": "hbm", "note": "algorithmic bytes count the full pass of each direction only; the carry-only passes are the cost of the split",
                         "achieved": total / world / ms / 1e6, "peak": peak, "peak_source": f"of {kind}", "unit": "GB/s",
                         "frac": total / world / ms / 1e6 / peak, "traffic": None}}


def cpu_baseline(workload: str, steps: int = 1) -> dict:
    """The reference's sequential path forward+backward on the host cores.

    When the unmodified reference package has been staged (oracle/make_ref.py) it is what runs:
    ``RG_LRU(..., scan_mode="sequential")`` (griffin/griffin.py:157-306), kind "reference".  Otherwise the
    oracle's restatement of the same lines runs, kind "port".  Bounded sample: the workload's T, D and dtype
    with the batch cut to 2^24 token-channels at most (the reference's backward is O(T^2) per row on CPU:
    autograd re-materialises a full-size tensor per time-step).
    """
    from oracle import rglru_oracle as orc
    from oracle.make_ref import import_reference

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on.
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    B, T, D, G, dtype = WORKLOADS[workload]
    sample_b = B if B * T * D <= (1 << 24) else max(1, (1 << 24) // (T * D))
    sample_t = min(T, 2048)
    case = orc.make_rglru_case(sample_b, sample_t, D, G, seed=0)
    names = ("Lambda", "recurrence_gate.weight", "recurrence_gate.bias", "input_gate.weight", "input_gate.bias")
    es = 2 if dtype == torch.bfloat16 else 4
    reference = import_reference()
    best = None
    for _ in range(steps):
        x = case["x"].to(dtype).requires_grad_(True)
        dy = case["dy"].to(dtype)
        if reference is not None:
            module = reference.RG_LRU(D, gate_blocks=G, scan_mode="sequential")
            module.load_state_dict({k: case[k] for k in names})
            module = module.to(dtype)
            t0 = time.perf_counter()
            y = module(x)
            y.backward(dy)
        else:
            params = {k: case[k].to(dtype).requires_grad_(True) for k in names}
            t0 = time.perf_counter()
            y, _ = orc.rglru_layer(x, params)
            y.backward(dy)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    n = sample_b * sample_t * D
    return {"value": 11 * es * n / best / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "reference" if reference is not None else "port", "seconds": best, "token_channels_per_s": n / best,
            "sample": f"B={sample_b} T={sample_t} D={D} {str(dtype).replace('torch.', '')} module path "
                      f"(gates + sequential scan, autograd backward), best of {steps}"}


def reference_gpu_probe(workload: str, steps: int) -> dict:
    """Opt-in (--ref-gpu): the staged reference's own GPU path (its Triton fused scan when it validates on this
    device, else its associative scan; griffin/griffin.py:259-306) forward+backward at the workload's shape,
    CUDA events.  Context for the CPU arm above, not a substitute for it."""
    from oracle import rglru_oracle as orc
    from oracle.make_ref import import_reference

    reference = import_reference()
    if reference is None:
        return {"unavailable": "the reference package is not staged (oracle/make_ref.py)"}
    B, T, D, G, dtype = WORKLOADS[workload]
    dev = torch.device("cuda", 0)
    try:
        module = reference.RG_LRU(D, gate_blocks=G, scan_mode="auto").to(dev, dtype)
        xs = [torch.randn(B, T, D, device=dev).to(dtype).requires_grad_(True) for _ in range(4)]
        dy = torch.randn(B, T, D, device=dev).to(dtype)

        def step(i):
            x = xs[i % 4]
            x.grad = None
            module.zero_grad(set_to_none=True)
            module(x).backward(dy)

        for i in range(3):
            step(i)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        es = 2 if dtype == torch.bfloat16 else 4
        fused = bool(getattr(reference.griffin, "triton_scan_is_usable", lambda *_: False)(dev))
        return {"ms_per_step": ms, "gbs": 11 * es * B * T * D / ms / 1e6, "steps": steps,
                "path": "reference RG_LRU(scan_mode='auto') on cuda:0, module forward+backward (gate GEMMs included); "
                        + ("Triton fused scan" if fused else "associative scan (its Triton scan did not validate here)")}
    except Exception as exc:      # the reference's GPU path is context only; never let it take the arm down
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


def run_reference(args) -> dict:
    """The reference arm: the reference's CPU sequential path, all host threads, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    B, T, D, G, dtype = WORKLOADS[args.workload]
    steps = max(1, min(args.steps, 3))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(args.workload, 1)
    base = cpu_baseline(args.workload, steps)
    out = {
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
        "config": {"workload": workload_name(args.workload)},
        "timing": {"note": "CPU; each step is the bounded sample described in cpu_baseline.sample"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if args.ref_gpu and torch.cuda.is_available():
        out["reference_gpu"] = reference_gpu_probe(args.workload, max(3, min(args.steps, 20)))
    return out


# --------------------------------------------------------------------------- secondary workloads
def _timed(fn, steps, warmup, d: Dist):
    """W warm-up calls, then exactly K timed calls between barriers; returns max-over-ranks ms per call."""
    for i in range(warmup):
        fn(i)
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    d.barrier()
    return d.max_over_ranks(e0.elapsed_time(e1) / steps)


# Library kernels per forward+backward of one recurrent block on the TMA-staged conv path: conv forward, scan forward,
# scan backward, conv backward and its partial-row fold, and two column-sum kernels for each of the three bias gradients.
BLOCK_LAUNCHES = 11


def run_block(args, d: Dist) -> dict:
    """The full recurrent temporal block, bf16, B=16/GPU, T=2048, 768 -> 1024 -> 768, conv weights ~ N(0, 1/4), fwd+bwd."""
    from griffin_b200 import RecurrentBlock, _lib

    dev, world, rank = d.dev, d.world, d.rank
    B, T, DM, DR = 16, 2048, 768, 1024
    torch.manual_seed(rank)
    blk = RecurrentBlock(DM, DR, gate_blocks=16, scan_mode="cuda", fold_conv=args.fold == "conv",
                         fold_merge=args.fold == "merge")
    with torch.no_grad():
        blk.temporal_conv.weight.normal_(0.0, 0.5)
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
    ms = _timed(step, args.steps, args.warmup, d)
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

    e2e_ms = _timed(e2e_step, max(3, min(args.steps, 50)), 3, d)
    clocks = sampler.stop()
    n = B * T * DR
    peak, kind = measured_peak()
    return {"metric": "recurrent_block_fwd_bwd_token_channels_per_s", "value": world * n / ms * 1e3, "unit": "token-channels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 I/O, f32 state", "data": "synthetic",
            "config": {"workload": f"c2: RecurrentBlock fwd+bwd bf16 B={B}/GPU T={T} {DM}->{DR}->{DM}, conv k=4, 16 gate heads",
                       "fold": args.fold, "cuda_graph": bool(args.graph),
                       "l2": "three rotating inputs; 0.6 GB of activations per step"},
            "scan_conv_algorithmic_gbs": world * (22 + 10) * n / ms / 1e6,
            "e2e": {"value": world * n / e2e_ms * 1e3, "unit": "token-channels/s", "h2d_bytes_per_step": 2 * B * T * DM,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
            "gpu_launches": BLOCK_LAUNCHES * args.steps, "clocks": clocks, "device_status": _lib.device_status(),
            "roofline": {"bound": "hbm", "note": "GEMMs (torch) dominate this step; see the c1 line for the kernel roofline",
                         "peak": peak, "peak_source": f"of {kind}", "unit": "GB/s", "achieved": None, "frac": None, "traffic": None}}


def run_lm(args, d: Dist, steps=None, warmup=None) -> dict:
    """Griffin ~100M training step, bf16 autocast, B=8/GPU, T=2048, AdamW; DDP over NCCL for N > 1."""
    from griffin_b200 import _lib
    from griffin_b200.lm import GriffinModel

    dev, world, rank = d.dev, d.world, d.rank
    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
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

    import contextlib

    def train(ids):
        # --ddp-no-sync: the same step without the gradient all-reduce (what the collective costs, by difference)
        with (net.no_sync() if (world > 1 and args.ddp_no_sync) else contextlib.nullcontext()):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = net(ids[:, :-1], pad_vocab=True)   # vocabulary padded to a multiple of 8, -inf in the padding
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
    ms = _timed(step, steps, warmup, d)
    e2e_ms = _timed(e2e_step, max(3, min(steps, 20)), 2, d)
    clocks = sampler.stop()
    out = {"metric": "griffin100m_train_tokens_per_s", "value": world * B * T / ms * 1e3, "unit": "tokens/s",
           "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None,
           "dtype": "bf16 autocast (RG-LRU: bf16 I/O, fp32 state and arithmetic)", "data": "synthetic",
           "config": {"workload": f"c3: Griffin-100M ({nparams} params) train step B={B}/GPU T={T} vocab {V}, AdamW, "
                                  f"{('DDP/NCCL' + (' WITHOUT all-reduce' if args.ddp_no_sync else '')) if world > 1 else 'single GPU'}",
                      "fold": args.fold, "l2": "activations of one step far exceed L2"},
           "e2e": {"value": world * B * T / e2e_ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B * (T + 1),
                   "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
           # 8 of the 12 layers are recurrent blocks
           "gpu_launches": 8 * BLOCK_LAUNCHES * steps,
           "clocks": clocks,
           "device_status": _lib.device_status(),
           "roofline": {"bound": "tensor", "note": "whole-model step: torch GEMMs and attention dominate; the library's kernels "
                        "are the conv, the RG-LRU scan and their backwards in 8 of 12 layers", "achieved": None, "peak": None,
                        "frac": None, "traffic": None, "unit": "TFLOP/s"}}
    del net, model, opt
    torch.cuda.empty_cache()
    return out


def run_decode(args, d: Dist) -> dict:
    """Single-token decode update, B=512/GPU, D=5632, fp32 carried state, bf16 I/O, 1024 steps per timed call (one
    CUDA graph of 1024 kernel launches).  Two state placements are timed: ONE state that every step updates in
    place (what decoding does; its 23 MB stay in L2), and a ring of states large enough that each step's state
    comes from HBM (the HBM-roofline figure)."""
    from griffin_b200 import _lib

    dev, world = d.dev, d.world
    lib = _lib.load()
    B, D, NSTEP, NSET, NSTATE = 512, 5632, 1024, 8, 16
    xs = [tuple(torch.randn(B, D, device=dev).to(torch.bfloat16) for _ in range(3)) for _ in range(NSET)]
    lam = torch.logit(torch.empty(D).uniform_(0.9, 0.999).pow(1.0 / 8.0)).to(dev)
    states = [torch.zeros(B, D, device=dev) for _ in range(NSTATE)]      # 16 x 11.5 MB = 185 MB > L2
    y = torch.empty(B, D, device=dev, dtype=torch.bfloat16)

    def one(i, stream, ring):
        x, ur, ui = xs[i % NSET]
        h = states[i % NSTATE] if ring else states[0]
        rc = lib.rglru_decode_step(x.data_ptr(), ur.data_ptr(), ui.data_ptr(), lam.data_ptr(), h.data_ptr(), None,
                                   y.data_ptr(), B, D, 8.0, _lib.BF16, stream)
        _lib.check(rc, "rglru_decode_step")

    one(0, torch.cuda.current_stream(dev).cuda_stream, False)      # per-device set-up happens outside capture
    torch.cuda.synchronize(dev)
    graphs = {}
    side = torch.cuda.Stream(dev)
    for ring in (False, True):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(NSTEP):
                one(i, side.cuda_stream, ring)
        graphs[ring] = g
    sampler = ClockSampler(dev.index or 0).start()
    ms = _timed(lambda i: graphs[False].replay(), args.steps, args.warmup, d)
    ms_ring = _timed(lambda i: graphs[True].replay(), args.steps, args.warmup, d)
    clocks = sampler.stop()
    n = B * D
    bytes_step = 16 * n                     # x, u_r, u_i bf16 in; y bf16 out; h fp32 in and out
    peak, kind = measured_peak()
    algorithmic = bytes_step * NSTEP / ms / 1e6
    from_hbm = bytes_step * NSTEP / ms_ring / 1e6
    return {"metric": "rglru_decode_algorithmic_gbs", "value": world * algorithmic, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 I/O, f32 state", "data": "synthetic",
            "config": {"workload": f"c4b: decode update B={B}/GPU D={D}, {NSTEP} token steps per timed call (CUDA graph)",
                       "l2": f"{NSET} rotating input sets of 17 MB; value: one 23 MB state updated in place (L2-resident), "
                             f"roofline: a ring of {NSTATE} states (185 MB) so every step's state comes from HBM"},
            "decode_steps_per_s": world * NSTEP / ms * 1e3, "us_per_token_step": ms * 1e3 / NSTEP,
            "in_place_state": {"algorithmic_gbs": algorithmic, "frac_of_copy_bandwidth_l2_assisted": algorithmic / peak,
                               "note": "the state never leaves L2 in this loop; an ncu capture of one launch shows about "
                                       "29 MB read from DRAM and next to nothing written per step, against 46 MB algorithmic"},
            "roofline": {"bound": "hbm", "kernel": "decode_step_kernel", "achieved": from_hbm, "peak": peak,
                         "peak_source": f"of {kind}", "unit": "GB/s", "frac": from_hbm / peak, "traffic": None,
                         "algorithmic_bytes": bytes_step, "us_per_token_step": ms_ring * 1e3 / NSTEP,
                         "note": "state ring larger than L2: inputs and state stream from HBM"},
            "e2e": None, "gpu_launches": 2 * NSTEP * args.steps, "clocks": clocks, "device_status": _lib.device_status()}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS) + ["c2", "c3", "c4b", "tshard"])
    ap.add_argument("--fold", default="merge", choices=["none", "conv", "merge"],
                    help="c2/c3: run conv (and the GeLU-branch product) inside the scan kernels")
    ap.add_argument("--graph", action="store_true", help="c2: replay the block's forward and backward as CUDA graphs")
    ap.add_argument("--width", type=int, default=1024, help="tshard: channels D of the time-sharded sequence")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="default workload: skip the c4a and c3 sub-objects")
    ap.add_argument("--no-repeat", action="store_true", help="time one region of K steps only (for profiler runs)")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the per-kernel event pass (for profiler runs)")
    ap.add_argument("--ddp-no-sync", action="store_true",
                    help="c3 with N > 1: skip the gradient all-reduce (diagnostic: the step's cost without the collective)")
    ap.add_argument("--ref-gpu", action="store_true",
                    help="--impl reference: also time the staged reference's own GPU path (Triton / associative scan)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        if args.workload not in WORKLOADS:
            raise SystemExit("--impl reference covers the RG-LRU layer workloads only")
        out = run_reference(args)
        if out:
            print(json.dumps(out))
        return
    d = Dist()
    if args.workload == "c2":
        out = run_block(args, d)
    elif args.workload == "c3":
        out = run_lm(args, d)
    elif args.workload == "c4b":
        out = run_decode(args, d)
    elif args.workload == "tshard":
        out = run_time_shard(args, d)
    else:
        out = run_layer(args, d)
        if args.workload == "c1" and not args.no_extra:
            out["c4a"] = run_c4a_shard(args, d)
            out["c3"] = {k: v for k, v in run_lm(args, d, steps=max(3, min(args.steps, 10)), warmup=3).items()
                         if k in ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "config", "e2e", "clocks",
                                  "device_status", "dtype", "gpu_launches")}
            out["c3"]["tokens_per_s"] = out["c3"]["value"]
        if d.rank == 0 and d.world == 1 and not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline(args.workload, steps=1)
    d.close()
    if d.rank == 0 and out:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
