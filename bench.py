#!/usr/bin/env python
"""Benchmark of the fused multi-head-attention training step (forward + backward) at the
BERT-large shape, on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --configs      (kernel times of the named configurations, one line each)

One "step" is one forward and one backward pass of the hot path over one batch of synthetic
input (B=32, H=16, S=512, D=64, fp16, valid lengths uniform in [256,512], Philox dropout 0.1).
With N > 1 (launched under torchrun, one rank per GPU) every rank works on its own shard of the
batch x heads axis; there is no collective on the data path, only a barrier and a MAX of the
per-rank device times.  Rank 0 prints ONE JSON line.

`value` is EXECUTED TFLOP/s of exactly K timed steps with every rank holding a full B=32 batch
("scaling": "weak").  What is counted: (4*ceil64(len) + 10*ceil128(len))*H*S_q*D per batch element,
the key length rounded up to the key steps the kernels actually visit (64 keys in the forward
kernel, 128 in the backward kernel; steps that lie wholly in the padding are skipped, which is
exact).  The dense-equivalent figure (14*B*H*S^2*D over the same time) is reported beside it.

Further legs of the same run, each its own object in the line:
  strong        the FIXED B=32 batch split N ways over batch x heads (what the configurations state), with the
                same batch on one GPU timed in the same run, and the efficiency t1 / (N * tN)
  sustained     the step back to back for >= 2 s: ms per step, SM clock and power under sustained load
  other_configs the other named configurations (BERT-base forward, BERT-large forward, long-sequence training
                shard) on this run's ranks
  roofline / roofline_fwd / kernel_ms, e2e (host buffers in and out through the torch operators), cpu_baseline
  clocks        NVML samples of the SM clock and throttle reasons over all loaded legs (read-only)

`--impl reference` times the reference's own CPU path for the same step: the eager composite of
its test scripts (matmul, scale, mask, softmax, dropout, matmul) plus autograd, on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = "bert_large_train"
B0, H, S, D = 32, 16, 512, 64
LEN_RANGE = (256, 512)
P_DROP = 0.1
METRIC = "fused MHA fwd+bwd TFLOP/s at BERT-large shape (executed flops)"
# ncu capture of fmha_bwd_kernel<64,fp16,dropout> (profiles/bwd_kernel_b16_h16_s512_d64.md): at B=16 of this
# workload dram__bytes_read.sum + dram__bytes_write.sum = 97.62 MB + 22.36 MB per launch; DRAM traffic of
# the kernel is proportional to the batch (every CTA touches only its own head), so B=32 is twice that.
BWD_KERNEL_DRAM_TRAFFIC_B16 = 97.62e6 + 22.36e6


def executed_flops(lens, h, s_q, d, mult, granule=128):
    """mult * h * s_q * (key length rounded up to the kernel's key step) * d summed over the batch.
    The forward kernel walks the keys in 64-key steps at D=64, the backward kernel in 128-key tiles."""
    return float(sum(mult * h * s_q * (math.ceil(int(n) / granule) * granule) * d for n in lens))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), tflops_sustained=float(p.get("bf16_tflops_sustained", 0.0)),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Polls SM clock, power and throttle reasons through NVML (read-only) from construction until stop().

    NVML is initialised in the constructor, i.e. BEFORE any timed region, so that even a region of a few
    milliseconds is covered by samples.  `mark(name)` / `unmark(name)` bracket a leg; summaries can be taken per
    leg or over everything that ran between marks."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self.error = index, [], set(), None, None
        self._stop_evt = threading.Event()
        self._legs = {}
        self._open = {}
        self._nv = None
        self._names = {}
        try:
            import pynvml as nv
            nv.nvmlInit()
            self._h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._h, nv.NVML_CLOCK_SM)
            self._names = {
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
            }
            self._get_reasons = (getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None)
                                 or nv.nvmlDeviceGetCurrentClocksThrottleReasons)
            self._nv = nv
        except Exception as e:  # NVML missing: report that instead of numbers
            self.error = f"nvml_unavailable:{type(e).__name__}"

    def run(self):
        nv = self._nv
        if nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                watts = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                r = self._get_reasons(self._h)
            except Exception as e:
                self.error = f"nvml_error:{type(e).__name__}"
                return
            self.samples.append((time.perf_counter(), mhz, watts, r))
            time.sleep(0.001)

    def mark(self, name):
        self._open[name] = time.perf_counter()

    def unmark(self, name):
        self._legs.setdefault(name, []).append((self._open.pop(name), time.perf_counter()))

    def summary(self, names=None):
        """Median SM MHz, max power and the throttle reasons seen inside the marked legs (all legs if None)."""
        spans = [sp for n, v in self._legs.items() if names is None or n in names for sp in v]
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in spans)]
        reasons = set()
        for s in inside:
            for bit, name in self._names.items():
                if s[3] & bit:
                    reasons.add(name)
        if self.error:
            reasons.add(self.error)
        return dict(sm_mhz=statistics.median(s[1] for s in inside) if inside else None, sm_max_mhz=self.max_mhz,
                    power_w_max=max((s[2] for s in inside), default=None), reasons=sorted(reasons), samples=len(inside))

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(2.0)


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the eager composite + autograd on the host cores
# ------------------------------------------------------------------------------------------
def cpu_composite_step(sample_b: int, seed: int):
    """Builds a closure running one fwd+bwd of the composite on `sample_b` batch elements of the
    workload on the CPU, and the dense flops of that sample."""
    import torch
    from nvfuserexamples_b200 import workloads
    from oracle import composite, philox
    x = workloads.make_inputs(sample_b, H, S, D, torch.float16, LEN_RANGE, seed, with_do=True)
    add = composite.padding_add_mask(x["lens"], S)
    keep = torch.from_numpy(philox.dropout_keep_mask(1, 0, 0, sample_b * H, S, S, P_DROP)).reshape(sample_b, H, S, S).float()
    ks = philox.keep_scale(P_DROP)

    def step():
        return composite.attention_grads_fp32(x["q"], x["k"], x["v"], x["d_o"], add_mask=add, keep=keep, keep_scale=ks)

    return step, 14.0 * sample_b * H * S * S * D


def time_cpu(step, flops, warmup, steps):
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return flops / dt / 1e12, dt


def run_reference(args, rank):
    if rank != 0:
        return
    import torch
    torch.set_num_threads(len(os.sched_getaffinity(0)))  # torchrun pins OMP_NUM_THREADS=1: use every host core we may
    sample_b = 2
    step, flops = cpu_composite_step(sample_b, 1004)
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 3))
    tf, dt = time_cpu(step, flops, warm, steps)
    cores = torch.get_num_threads()
    sample = f"{sample_b} of {B0} batch elements (x{H} heads, S={S}, D={D}), fp32 composite + autograd, {steps} timed steps"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3 * (B0 / sample_b), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 inputs, fp32 math", "data": "synthetic",
        "config": {"workload": WORKLOAD, "B_per_gpu": B0, "global_batch": B0 * args.gpus, "H": H, "S": S, "D": D,
                   "p_drop": P_DROP, "valid_len": list(LEN_RANGE),
                   "flops_counted": "dense 14*B*H*S^2*D of the sample; ms_per_step scaled to the full batch"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def pin_to_gpu_cpus(index: int):
    """Binds THIS process to the host cores NVML reports as local to GPU `index` (its NUMA node), so that the pinned
    host buffers of the end-to-end leg are first touched on the memory that GPU's PCIe root reads: with several ranks
    on a two-socket host, all of them staging through one node's memory is what limits the copies.  Changes only this
    process's own CPU affinity (sched_setaffinity); no GPU setting is touched.  Returns what was done, for the record."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(index)
        n_words = (os.cpu_count() + 63) // 64
        words = nv.nvmlDeviceGetCpuAffinity(h, n_words)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return {"pinned": False, "why": "no local core inside the process's allowed set"}
        os.sched_setaffinity(0, allowed)
        return {"pinned": True, "cores": len(allowed), "first_core": min(allowed), "last_core": max(allowed)}
    except Exception as e:  # NVML or the call missing: run unpinned and say so
        return {"pinned": False, "why": f"{type(e).__name__}: {e}"}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class Plan:
    """Device-resident inputs, outputs and parameter blocks of `n_sets` rotating input sets of one shard: no
    allocation happens inside a timed region."""

    def __init__(self, capi, dev, b_loc, h, s, d, dtype, len_range, p_drop, seeds, bh_offset, status, train=True,
                 device_inputs=False):
        import ctypes as C

        import torch
        from nvfuserexamples_b200 import workloads
        self.C, self.capi, self.lib = C, capi, capi.load()
        self.sets, self.plans = [], []
        for i, seed in enumerate(seeds):
            if device_inputs:   # large shapes: seeded generation on the device (same distributions)
                g = torch.Generator(device=dev).manual_seed(seed)
                x = {n: torch.randn(b_loc, h, s, d, device=dev, generator=g, dtype=torch.float32).to(dtype)
                     for n in (("q", "k", "v", "d_o") if train else ("q", "k", "v"))}
                x["lens"] = torch.randint(len_range[0], len_range[1] + 1, (b_loc,), device=dev, generator=g, dtype=torch.int32)
            else:
                x = {k: v.to(dev) for k, v in workloads.make_inputs(b_loc, h, s, d, dtype, len_range, seed, with_do=train).items()}
            self.sets.append(x)
            o = torch.empty_like(x["q"])
            lse = torch.empty(b_loc, h, s, dtype=torch.float32, device=dev)
            fp = capi.FwdParams()
            fp.struct_bytes = C.sizeof(capi.FwdParams)
            fp.dtype = capi.DTYPE_F16 if dtype == torch.float16 else capi.DTYPE_BF16
            fp.B, fp.H, fp.S_q, fp.S_k, fp.D = b_loc, h, s, s, d
            fp.scale = 1.0 / math.sqrt(d)
            fp.q, fp.k, fp.v, fp.o = (capi._t4(t) for t in (x["q"], x["k"], x["v"], o))
            fp.lse = lse.data_ptr()
            fp.mask_kind, fp.mask = capi.MASK_SEQLEN, x["lens"].data_ptr()
            if p_drop > 0:
                fp.dropout_kind, fp.p_drop = capi.DROPOUT_PHILOX, p_drop
            fp.philox_seed, fp.philox_offset, fp.philox_bh_offset = 0x5EED0004, i, bh_offset
            fp.status = status.data_ptr()
            pl = dict(fp=fp, keep=[o, lse])
            if train:
                dq, dk, dv = (torch.empty_like(x["q"]) for _ in range(3))
                bp = capi.bwd_params(x["d_o"], x["q"], x["k"], x["v"], o, lse, dq, dk, dv, mask_kind=capi.MASK_SEQLEN,
                                     mask=x["lens"], p_drop=p_drop, seed=0x5EED0004, offset=i, bh_offset=bh_offset,
                                     status=status)
                ws = torch.empty(capi.bwd_workspace_bytes(bp), dtype=torch.uint8, device=dev)
                bp.workspace, bp.workspace_bytes = ws.data_ptr(), ws.numel()
                bpm = capi.BwdParams.from_buffer_copy(bp)   # main backward kernel alone
                bpm.flags = capi.FLAG_BWD_SKIP_PREPARE | capi.FLAG_BWD_SKIP_FINISH
                pl.update(bp=bp, bp_main=bpm)
                pl["keep"] += [dq, dk, dv, ws]
            self.plans.append(pl)
        self.lens_host = [x["lens"].cpu().tolist() for x in self.sets]
        self.n = len(self.plans)
        self.h, self.s, self.d, self.train = h, s, d, train

    def fwd(self, i, sp):
        return self.lib.fmha_sm100_fwd(self.C.byref(self.plans[i % self.n]["fp"]), sp)

    def bwd(self, i, sp, which="bp"):
        return self.lib.fmha_sm100_bwd(self.C.byref(self.plans[i % self.n][which]), sp)

    def step(self, i, sp):
        rc = self.fwd(i, sp)
        if self.train:
            rc |= self.bwd(i, sp)
        if rc != 0:
            raise RuntimeError(f"kernel library call failed: {rc} {self.capi.strerror(rc)}")

    def flops(self, fwd_granule):
        """(executed forward, executed backward, dense forward, dense backward) flops of one step, averaged over the sets."""
        ef = sum(executed_flops(l, self.h, self.s, self.d, 4.0, fwd_granule) for l in self.lens_host) / self.n
        eb = sum(executed_flops(l, self.h, self.s, self.d, 10.0, 128) for l in self.lens_host) / self.n if self.train else 0.0
        b = len(self.lens_host[0])
        dense_f = 4.0 * b * self.h * self.s * self.s * self.d
        return ef, eb, dense_f, (2.5 * dense_f if self.train else 0.0)


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from nvfuserexamples_b200 import capi, sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the kernels have no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # before any pinned host buffer is touched; BENCH_NO_PIN=1 leaves the affinity alone (for comparison runs)
    numa = None if os.environ.get("BENCH_NO_PIN") == "1" else pin_to_gpu_cpus(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local_rank)   # NVML is up before anything is timed
    sampler.start()
    stream = torch.cuda.current_stream(dev)
    sp = stream.cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    pk = peaks()

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def all_max(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def all_sum(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.item()

    def timed(fn, n, leg, collective=True):
        """n back-to-back calls of fn(i) between two CUDA events on the launching stream, barrier + synchronize on
        both sides; returns the ms per call, as the MAX over ranks when `collective`."""
        if collective:
            sync_all()
        else:
            torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.mark(leg)
        e0.record(stream)
        for i in range(n):
            fn(i)
        e1.record(stream)
        if collective:
            sync_all()
        else:
            torch.cuda.synchronize(dev)
        sampler.unmark(leg)
        ms = e0.elapsed_time(e1) / n
        return all_max(ms) if collective else ms

    # ---- this rank's shard of the headline workload: every rank owns a full B0 batch (weak scaling) -----------
    if args.profile:
        b_global = args.profile_batch  # reduced batch for profiler captures (still larger than L2)
    else:
        b_global = B0 * world
    shard = sharding.make_shard(b_global, H, world, rank)
    if not shard.whole_batches or shard.bh_count == 0:
        raise SystemExit("bench.py: the batch does not split into whole batch elements per rank")
    b_loc = shard.bh_count // H
    plan = Plan(capi, dev, b_loc, H, S, D, torch.float16, LEN_RANGE, P_DROP, [1004 + 17 * rank + i for i in range(2)],
                shard.bh_offset, status)

    if args.profile:
        # A handful of launches of one kernel for an ncu capture; prints no benchmark line.
        which = {"fwd": lambda i: plan.fwd(i, sp), "bwd": lambda i: plan.bwd(i, sp)}[args.profile]
        plan.step(0, sp)
        for i in range(3):
            which(i)
        torch.cuda.synchronize(dev)
        capi.check_status(status)
        sampler.stop()
        print(json.dumps({"profile": args.profile, "B": b_loc, "launches": 3}), flush=True)
        return

    for i in range(args.warmup):
        plan.step(i, sp)
    capi.check_status(status)

    # ---- timed region: exactly K steps -------------------------------------------------------------------------
    ms_step = timed(lambda i: plan.step(i, sp), args.steps, "timed")
    capi.check_status(status)
    exe_f, exe_b, dense_f, dense_b = plan.flops(64)
    value = all_sum(exe_f + exe_b) / (ms_step * 1e-3) / 1e12
    dense_value = (dense_f + dense_b) * world / (ms_step * 1e-3) / 1e12

    # ---- sustained leg: the same step back to back for >= 2 s --------------------------------------------------
    n_sus = max(args.steps, int(math.ceil(2000.0 / max(ms_step, 1e-3))))
    ms_sus = timed(lambda i: plan.step(i, sp), n_sus, "sustained")
    sus_clk = sampler.summary({"sustained"})
    sustained = {"steps": n_sus, "ms_per_step": ms_sus, "value": all_sum(exe_f + exe_b) / (ms_sus * 1e-3) / 1e12,
                 "unit": "TFLOP/s", "sm_mhz": sus_clk["sm_mhz"], "power_w_max": sus_clk["power_w_max"],
                 "reasons": sus_clk["reasons"], "samples": sus_clk["samples"],
                 "pct_of_measured_bf16_sustained_peak": (100.0 * all_sum(exe_f + exe_b) / (ms_sus * 1e-3) / 1e12 /
                                                         (pk["tflops_sustained"] * world)) if pk["tflops_sustained"] else None}

    # ---- kernel-level numbers -------------------------------------------------------------------------------------
    kn = max(20, min(args.steps, 200))
    for i in range(3):
        plan.step(i, sp)
    fwd_ms = timed(lambda i: plan.fwd(i, sp), kn, "kernels", collective=False)
    bwd_main_ms = timed(lambda i: plan.bwd(i, sp, "bp_main"), kn, "kernels", collective=False)
    bwd_all_ms = timed(lambda i: plan.bwd(i, sp), kn, "kernels", collective=False)
    ach = exe_b / (bwd_main_ms * 1e-3) / 1e12
    roofline = {"kernel": "fmha_bwd_kernel<64,fp16,seqlen,dropout>", "bound": "tensor", "achieved": ach, "peak": pk["tflops"],
                "unit": "TFLOP/s", "frac": ach / pk["tflops"], "traffic": BWD_KERNEL_DRAM_TRAFFIC_B16 * b_loc / 16.0,
                "traffic_unit": "bytes per launch (ncu at B=16, scaled by batch)",
                "peak_source": f"{pk['source']} bf16 burst", "ms_per_launch": bwd_main_ms,
                "algorithmic_flops_per_launch": exe_b}
    ach_f = exe_f / (fwd_ms * 1e-3) / 1e12
    roofline_fwd = {"kernel": "fmha_fwd_fast_kernel<64,fp16,seqlen,dropout>", "bound": "tensor", "achieved": ach_f,
                    "peak": pk["tflops"], "unit": "TFLOP/s", "frac": ach_f / pk["tflops"], "ms_per_launch": fwd_ms,
                    "dense_equiv_frac": dense_f / (fwd_ms * 1e-3) / 1e12 / pk["tflops"]}

    # ---- strong scaling: the FIXED B0 batch split over the ranks, and the same batch on one GPU ----------------
    # At B0/N batch elements per GPU a step is tens of microseconds of device work, less than the host needs to
    # issue its four launches (tensor maps + cudaLaunchKernelEx: ~30 us per step), so this leg replays a CUDA graph of
    # the step (both input sets = two steps per replay); the directly launched figure is reported beside it.
    def step_graph(p):
        gs = torch.cuda.Stream(device=dev)
        g = torch.cuda.CUDAGraph()
        gs.wait_stream(stream)
        with torch.cuda.graph(g, stream=gs):
            for i in range(p.n):
                p.step(i, torch.cuda.current_stream(dev).cuda_stream)
        stream.wait_stream(gs)
        return g

    strong = None
    if world > 1:
        sh = sharding.make_shard(B0, H, world, rank)
        if sh.whole_batches and sh.bh_count > 0:
            sb = sh.bh_count // H
            splan = Plan(capi, dev, sb, H, S, D, torch.float16, LEN_RANGE, P_DROP, [2004 + 31 * rank + i for i in range(2)],
                         sh.bh_offset, status)
            n_st = max(50, min(args.steps, 200))
            for i in range(5):
                splan.step(i, sp)
            torch.cuda.synchronize(dev)
            g_n, g_1 = step_graph(splan), (step_graph(plan) if rank == 0 else None)
            for _ in range(3):
                g_n.replay()
            ms_n_direct = timed(lambda i: splan.step(i, sp), n_st, "strong")
            ms_n = timed(lambda i: g_n.replay(), n_st // 2, "strong") / splan.n
            sf, sbk, _, _ = splan.flops(64)
            exe_all = all_sum(sf + sbk)
            # the whole fixed batch on rank 0 alone (the other ranks wait at the barrier inside timed()): `plan` holds B0
            ms_1 = timed(lambda i: g_1.replay() if rank == 0 else None, n_st // 2, "strong") / plan.n
            capi.check_status(status)
            n_q, n_kv = S // 128, S // 128
            strong = {"global_batch": B0, "batch_per_gpu": sb, "ms_per_step": ms_n, "value": exe_all / (ms_n * 1e-3) / 1e12,
                      "unit": "TFLOP/s", "ms_per_step_1gpu_same_run": ms_1, "efficiency": ms_1 / (world * ms_n),
                      "launch": "CUDA graph replay, two steps per replay", "ms_per_step_direct_launch": ms_n_direct,
                      "steps": (n_st // 2) * splan.n,
                      "work_per_gpu": {"bwd_items": sb * H * n_kv, "bwd_ctas": 148, "fwd_ctas": sb * H * n_q,
                                       "bwd_waves": round(sb * H * n_kv / 148.0, 2)}}
            # The optional output gather (outside the attention path): one NCCL all-gather of the sharded O over
            # NVLink, checked against this rank's own slice and a checksum every rank must agree on.
            o_shard = splan.plans[0]["keep"][0]
            t0g = time.perf_counter()
            full = sharding.gather_outputs(o_shard, sh, B0)
            torch.cuda.synchronize(dev)
            gather_ms = (time.perf_counter() - t0g) * 1e3
            mine_ok = bool(torch.equal(sharding.shard_tensor(full, sh), o_shard))
            csum = full.float().sum().item()
            cmax, cmin = all_max(csum), -all_max(-csum)
            strong["output_gather"] = {"backend": "nccl", "shape": list(full.shape), "own_slice_identical": mine_ok and bool(all_max(0.0 if mine_ok else 1.0) == 0.0),
                                       "checksum_equal_on_all_ranks": cmax == cmin, "first_call_ms_incl_setup": gather_ms}
            del splan, g_n, g_1, full
            torch.cuda.empty_cache()

    # ---- the other named configurations on this run's ranks ----------------------------------------------------
    other = {}
    if not args.no_other_configs:
        for name, cb, ch, cs, cd, cdt, clr, cp, ctrain, split in OTHER_CONFIGS:
            dtype = getattr(torch, cdt)
            if split == "strong":      # the configuration's batch, split over the ranks
                csh = sharding.make_shard(cb, ch, world, rank)
                if not csh.whole_batches or csh.bh_count == 0:
                    continue
                cb_loc, coff = csh.bh_count // ch, csh.bh_offset
            else:                      # the configuration's per-GPU shard on every rank
                cb_loc, coff = cb, rank * cb * ch
            cplan = Plan(capi, dev, cb_loc, ch, cs, cd, dtype, clr, cp, [7 + rank], coff, status, train=ctrain,
                         device_inputs=cs * cd >= 2048 * 128)
            n_c = 30 if cs <= 512 else 5
            for i in range(3):
                cplan.step(i, sp)
            f_ms = timed(lambda i: cplan.fwd(i, sp), n_c, "other")
            ef, eb, df, db = cplan.flops(64 if cd == 64 else 128)
            rec = {"B_per_gpu": cb_loc, "global_batch": int(all_sum(cb_loc)), "H": ch, "S": cs, "D": cd, "dtype": cdt, "p_drop": cp,
                   "fwd_ms": f_ms, "fwd_executed_tflops": all_sum(ef) / f_ms / 1e9, "fwd_dense_tflops": df * world / f_ms / 1e9,
                   "fwd_frac_of_measured_peak": all_sum(ef) / f_ms / 1e9 / (pk["tflops"] * world)}
            if ctrain:
                s_ms = timed(lambda i: cplan.step(i, sp), n_c, "other")
                rec.update({"step_ms": s_ms, "bwd_ms": s_ms - f_ms, "step_executed_tflops": all_sum(ef + eb) / s_ms / 1e9,
                            "step_dense_tflops": (df + db) * world / s_ms / 1e9,
                            "step_frac_of_measured_peak": all_sum(ef + eb) / s_ms / 1e9 / (pk["tflops"] * world)})
            capi.check_status(status)
            other[name] = rec
            del cplan
            torch.cuda.empty_cache()

    # ---- end to end through the operator layer, host buffers in and out --------------------------------------
    import mha_manual  # noqa: F401
    ops = torch.ops.mha_manual
    sets = plan.sets
    host = {k: sets[0][k].cpu().pin_memory() for k in ("q", "k", "v", "d_o")}
    host_lens = sets[0]["lens"].cpu().pin_memory()
    host_out = [[torch.empty_like(host["q"]).pin_memory() for _ in range(4)] for _ in range(2)]   # two steps in flight
    h2d = sum(t.numel() * t.element_size() for t in host.values()) + host_lens.numel() * 4
    d2h = sum(t.numel() * t.element_size() for t in host_out[0])

    # Three stages on three streams, as a host loop that prefetches the next batch would run them: copy-in of step
    # i+1, compute of step i and copy-out of step i-1 overlap (PCIe is full duplex).  Every step still copies its own
    # inputs from pinned host memory and its own results back.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    keep = [None, None]        # device tensors of the two steps in flight
    ev_out = [None, None]      # copy-out of the step that used a slot has finished

    def e2e_step(i):
        slot = i & 1
        with torch.cuda.stream(s_in):
            if ev_out[slot] is not None:
                s_in.wait_event(ev_out[slot])      # the slot's previous tensors are no longer needed
            q, k, v, d_o = (host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "d_o"))
            lens = host_lens.to(dev, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        stream.wait_event(ev_in)
        for t in (q, k, v, d_o, lens):
            t.record_stream(stream)
        o, lse = ops.fmha_fwd(q, k, v, None, lens, P_DROP, 0x5EED0004, 0, None, shard.bh_offset)
        dq, dk, dv = ops.fmha_bwd(d_o, q, k, v, o, lse, None, lens, P_DROP, 0x5EED0004, 0, None, shard.bh_offset)
        ev_cmp = torch.cuda.Event()
        ev_cmp.record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp)
            for dst, src in zip(host_out[slot], (o, dq, dk, dv)):
                src.record_stream(s_out)
                dst.copy_(src, non_blocking=True)
            ev_out[slot] = torch.cuda.Event()
            ev_out[slot].record(s_out)
        keep[slot] = (q, k, v, d_o, lens, o, lse, dq, dk, dv)

    e2e_n = max(3, min(args.steps, 20))
    for i in range(2):
        e2e_step(i)
    sync_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark("e2e")
    s_in.wait_stream(stream)
    a.record(s_in)
    for i in range(e2e_n):
        e2e_step(i)
    s_out.wait_stream(stream)
    b.record(s_out)
    sync_all()
    sampler.unmark("e2e")
    te = all_max(a.elapsed_time(b) / e2e_n)
    exe0 = executed_flops(plan.lens_host[0], H, S, D, 4.0, 64) + executed_flops(plan.lens_host[0], H, S, D, 10.0, 128)
    e2e_value = all_sum(exe0) / (te * 1e-3) / 1e12

    # ---- CPU baseline (N = 1 only, bounded sample) ---------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
        cstep, cflops = cpu_composite_step(2, 1004)
        n = 0
        cstep()
        t0 = time.perf_counter()
        while True:
            cstep()
            n += 1
            if time.perf_counter() - t0 > 10.0 or n >= 40:
                break
        cdt = (time.perf_counter() - t0) / n
        cpu = {"value": cflops / cdt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"2 of {B0} batch elements (x{H} heads, S={S}, D={D}): fp32 eager composite + autograd, "
                         f"{n} iterations, {cdt * 1e3:.1f} ms each; dense flops"}

    sampler.stop()
    clocks = sampler.summary({"timed", "sustained", "kernels", "strong", "other"})
    clocks["timed_region"] = sampler.summary({"timed"})
    clocks["note"] = ("median SM clock over every device-timed leg of this run; the K-step region alone lasts "
                      f"{ms_step * args.steps:.0f} ms")
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "B_per_gpu": b_loc, "global_batch": b_loc * world, "H": H, "S": S, "D": D,
                       "p_drop": P_DROP, "valid_len": list(LEN_RANGE), "parallelism": f"bh-shard x{world}, no collective",
                       "l2": "335 MB touched per step (> 126 MB L2), 2 rotating input sets",
                       "flops_counted": "executed: (4*ceil64(len_b) + 10*ceil128(len_b))*H*S*D per batch element"},
            "dense_equiv_tflops": dense_value,
            "pct_of_measured_bf16_peak": 100.0 * value / (pk["tflops"] * world),
            "ms_per_step_x_sm_mhz": (ms_step * clocks["timed_region"]["sm_mhz"]) if clocks["timed_region"]["sm_mhz"] else
                                    ((ms_step * clocks["sm_mhz"]) if clocks["sm_mhz"] else None),
            "sustained": sustained, "strong": strong, "other_configs": other,
            "roofline": roofline, "roofline_fwd": roofline_fwd,
            "kernel_ms": {"fwd": fwd_ms, "bwd_main": bwd_main_ms, "bwd_all_three": bwd_all_ms},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": te, "api": "torch.ops.mha_manual.fmha_fwd + fmha_bwd on pinned host buffers; copy-in, compute and copy-out of consecutive steps overlap on three streams",
                    "h2d_gb_per_s_per_rank": h2d / (te * 1e-3) / 1e9, "d2h_gb_per_s_per_rank": d2h / (te * 1e-3) / 1e9,
                    "host_cores_of_rank0": numa},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


# The other named configurations: (name, B, H, S, D, dtype, valid lengths, p_drop, train, split).  split = "strong":
# B is the configuration's whole batch and is divided over the ranks; "shard": B is the per-GPU shard of an 8-GPU
# configuration (B=256 over 8 GPUs) and every rank runs one.
OTHER_CONFIGS = [
    ("bert_base_fwd", 32, 12, 512, 64, "float16", (256, 512), 0.1, False, "strong"),
    ("bert_large_fwd", 64, 16, 384, 64, "float16", (128, 384), 0.1, False, "strong"),
    ("long_seq_train_shard_of_8", 32, 16, 2048, 128, "bfloat16", (1024, 2048), 0.0, True, "shard"),
]
NAMED_CONFIGS = [
    ("bert_base_fwd", 32, 12, 512, 64, "float16", (256, 512), 0.1, False),
    ("bert_large_fwd", 64, 16, 384, 64, "float16", (128, 384), 0.1, False),
    ("bert_large_train", 32, 16, 512, 64, "float16", (256, 512), 0.1, True),
    ("long_seq_train_shard_of_8", 32, 16, 2048, 128, "bfloat16", (1024, 2048), 0.0, True),
]


def run_configs(args):
    """Times the forward (and backward) library calls of every named configuration on cuda:0 with CUDA
    events and prints one JSON line per configuration: dense-equivalent and executed TFLOP/s."""
    import ctypes as C

    import torch

    from nvfuserexamples_b200 import capi, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the kernels have no CPU fallback)")
    lib = capi.load()
    sp = torch.cuda.current_stream().cuda_stream

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    for name, b, h, s, d, dt, len_range, p, train in NAMED_CONFIGS:
        if args.only and name != args.only:
            continue
        if args.config_batch:
            b = args.config_batch      # reduced batch, e.g. for a profiler capture of one configuration
        dtype = getattr(torch, dt)
        x = workloads.make_inputs(b, h, s, d, dtype, len_range, 7, with_do=True)
        q, k, v, d_o, lens = (x[n].cuda() for n in ("q", "k", "v", "d_o", "lens"))
        kw = dict(mask_kind=capi.MASK_SEQLEN, mask=lens)
        fkw = dict(kw)
        if p > 0:
            fkw.update(dropout_kind=capi.DROPOUT_PHILOX, p_drop=p, seed=1, offset=0)
            kw.update(p_drop=p, seed=1, offset=0)
        o = torch.empty_like(q)
        res = capi.fwd(q, k, v, out=o, **fkw)
        n = 30 if s <= 512 else 5     # every configuration's tensors exceed the L2 capacity
        step_f = 64 if d == 64 else 128
        if args.which in ("all", "fwd"):
            f_ms = timed(lambda: capi.fwd(q, k, v, out=o, **fkw), n)
        else:
            f_ms = float("nan")
        exe_f = executed_flops(lens.tolist(), h, s, d, 4.0, step_f)
        line = {"config": name, "B": b, "H": h, "S": s, "D": d, "dtype": dt, "p_drop": p, "fwd_ms": round(f_ms, 4),
                "fwd_dense_tflops": round(4.0 * b * h * s * s * d / f_ms / 1e9, 1),
                "fwd_executed_tflops": round(exe_f / f_ms / 1e9, 1)}
        if train and args.which in ("all", "bwd"):
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            bp = capi.bwd_params(d_o, q, k, v, res["o"], res["lse"], dq, dk, dv, **kw)
            ws = torch.empty(capi.bwd_workspace_bytes(bp), dtype=torch.uint8, device="cuda")
            bp.workspace, bp.workspace_bytes = ws.data_ptr(), ws.numel()
            b_ms = timed(lambda: lib.fmha_sm100_bwd(C.byref(bp), sp), n)
            exe_b = executed_flops(lens.tolist(), h, s, d, 10.0, 128)
            line.update({"bwd_ms": round(b_ms, 4), "step_ms": round(f_ms + b_ms, 4),
                         "step_dense_tflops": round(14.0 * b * h * s * s * d / (f_ms + b_ms) / 1e9, 1),
                         "step_executed_tflops": round((exe_f + exe_b) / (f_ms + b_ms) / 1e9, 1)})
        print(json.dumps(line), flush=True)
        del x, q, k, v, d_o, o, res
        torch.cuda.empty_cache()


def run_legacy_profile():
    """The reference's three operators (fmha/fmha_manual.cpp:1218-1238 of shmsong/NvFuserExamples) at its hard-coded shape,
    three calls each with their GPU times (CUDA events): what an ncu capture of the general forward kernel runs."""
    import torch

    import mha_manual  # noqa: F401
    ops = torch.ops.mha_manual
    torch.manual_seed(0)
    bh, s, d = 32 * 16, 128, 64
    q, k, v = (torch.randn(bh, s, d, dtype=torch.half, device="cuda") for _ in range(3))
    amask = torch.empty(bh, s, s, device="cuda").random_(2).half()
    pad = (1 - amask) * -1000
    dm = torch.empty(bh, s, s, device="cuda").random_(2).half()
    calls = {"fmha_nvfuser": lambda: ops.fmha_nvfuser(q, k, v, amask),
             "fmha_train_nvfuser": lambda: ops.fmha_train_nvfuser(q, k, v, pad, dm),
             "fmha_train_saveim_nvfuser": lambda: ops.fmha_train_saveim_nvfuser(q, k, v, pad, dm)}
    out = {name: [] for name in calls}
    for rnd in range(5):   # round-robin: launches 3, 4, 5 of the kernel are one call of each operator after a warm round
        for name, fn in calls.items():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if rnd >= 2:
                out[name].append(a.elapsed_time(b) * 1e3)
    out = {name: {"us_per_call_incl_host": round(min(ts), 1)} for name, ts in out.items()}
    ops.check_status()
    print(json.dumps({"profile": "legacy", "BH": bh, "S": s, "D": d, "calls": out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="accepted for compatibility: `value` is always the weak-scaling figure (B=32 per GPU) and the "
                         "strong split of the fixed batch is always reported as the `strong` object of the same line")
    ap.add_argument("--profile", choices=["fwd", "bwd", "legacy"], default=None,
                    help="run three launches of one kernel path on a reduced batch and exit (for ncu); `legacy`: the three "
                         "reference operators at the reference's own shape (B*H=512, S=128, D=64)")
    ap.add_argument("--profile-batch", type=int, default=16)
    ap.add_argument("--no-other-configs", action="store_true", help="skip the `other_configs` legs")
    ap.add_argument("--configs", action="store_true",
                    help="kernel times of every named configuration on one GPU, one JSON line each (not the benchmark line)")
    ap.add_argument("--only", default=None, help="with --configs: run this named configuration alone")
    ap.add_argument("--which", choices=["all", "fwd", "bwd"], default="all", help="with --configs: time only one direction")
    ap.add_argument("--config-batch", type=int, default=0, help="with --configs: override the batch size")
    args = ap.parse_args()
    if args.configs:
        return run_configs(args)
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("bench.py: --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.profile == "legacy":
        return run_legacy_profile()
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
