#!/usr/bin/env python
"""Benchmark of the attention hot path: causal bf16 FlashAttention forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c3|c2]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one forward + one backward pass over the workload's batch of synthetic tensors.
Default workload: B=4, H=16, S=8192, D=128 bf16 causal (the long-context configuration the
headline metric is quoted on).  With N ranks the 64 (batch x head) slices are split contiguously,
one process per GPU, no data-path collective (total work fixed: strong scaling); torch.distributed
is used only for the barrier and the max-over-ranks of the device times.

Prints ONE JSON line:
  value        whole-job TFLOP/s with inputs resident in HBM (FLOPs: fwd 2*B*H*S^2*D, bwd 5*B*H*S^2*D,
               the causal-halved FlashAttention convention), device time from CUDA events, max over ranks
  e2e          the same metric through the library's host-tensor call (it_host_step_run via ops.HostAttentionStep):
               every step uploads Q,K,V,dO from pinned memory and downloads O,dQ,dK,dV inside the timed
               region, slices in 16 groups on rotating streams so copies and kernels overlap; copy_only_ms
               (the same copies without the kernels) and host_issue_ms beside it
  roofline     the backward main kernel (dominant) against the measured dense-bf16 peak
  cpu_baseline the CPU oracle timed on this box's host cores on a bounded sample (rank 0, N=1 only)
--impl reference times the reference's algorithm on the host cores instead (the CPU oracle: the
reference itself is Metal-only and cannot run here).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, S, D, qk_scale, description)
    "c4": (4, 16, 8192, 128, 0.5, "causal bf16 attention fwd+bwd B4 H16 S8192 D128"),
    "c3": (32, 12, 1024, 64, 1.0, "causal bf16 attention fwd+bwd B32 H12 S1024 D64"),
    "c2": (16, 4, 256, 64, 1.0, "causal bf16 attention fwd+bwd B16 H4 S256 D64"),
}
METRIC = "causal attention fwd+bwd TFLOP/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of fa_bwd_sm100_kernel<128>, from one ncu capture of this
# workload reduced to 32 of its 64 slices (0.405 GB read + 0.222 GB written); traffic grows in proportion to the slices
# a launch processes, so the full launch is twice that.  Re-captured whenever that kernel changes.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"c4": 2 * (404.859648e6 + 222.464256e6)}


def flops_fwd(bh, S, D):
    return 2.0 * bh * S * S * D


def flops_bwd(bh, S, D):
    return 5.0 * bh * S * S * D


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16": p["bf16_tflops"], "bf16_sustained": p.get("bf16_tflops_sustained"), "hbm": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


def bind_host_to_gpu(gpu_index):
    """Runs this process on the CPU cores next to the GPU (NVML's affinity mask for it), so that the
    page-locked host tensors of the end-to-end leg are allocated in that socket's memory and the
    copies do not cross the inter-socket link.  Changes only this process's own affinity; returns a
    description for the JSON line, or why nothing was changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(int(gpu_index))
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (max(allowed) // 64) + 1)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        use = allowed & near
        if not use:
            return "no allowed core next to the GPU: affinity unchanged"
        if use == allowed:
            return f"all {len(allowed)} allowed cores are next to the GPU"
        os.sched_setaffinity(0, use)
        return f"{len(use)} of {len(allowed)} allowed cores (those next to the GPU)"
    except Exception as e:   # NVML missing or refusing: measure with the default placement
        return f"affinity unchanged ({type(e).__name__})"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, gpu_index):
        self.lines = []
        self.t0 = 0.0
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """Samples that arrived before this call are left out (nvidia-smi needs ~0.1 s to start)."""
        self.t0 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.time()     # samples that arrive later belong to the idle time after the region
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, watts, mx, reasons = [], [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, ln in self.lines:
            if t < self.t0 or t > t1 + 0.005:
                continue
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                clk = float(parts[0])
                mx = float(parts[1])
            except ValueError:
                continue
            try:
                w = float(parts[6])
            except (IndexError, ValueError):
                w = None
            sm.append(clk)
            watts.append(w)
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
               "samples": len(sm)}
        known = [w for w in watts if w is not None]
        if known:
            # nvidia-smi's power figure is averaged over about a second, so it lags a timed region of
            # ~0.1 s; "under load" = samples drawing at least 70 % of the highest power seen
            top = max(known)
            loaded = [c for c, w in zip(sm, watts) if w is not None and w >= 0.7 * top]
            out.update({"power_w_max": top, "sm_mhz_under_load": statistics.median(loaded) if loaded else None,
                        "sm_mhz_min": min(sm), "samples_under_load": len(loaded)})
        return out


def cpu_oracle_rate(S, D, qk_scale, n_slices, seed):
    """TFLOP/s of the CPU oracle (forward + composed backward) on `n_slices` head-slices of the workload."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    from irontensor_b200 import synth
    ol.oracle().oracle_set_num_threads(os.cpu_count() or 1)   # torchrun sets OMP_NUM_THREADS=1
    q, k, v, d_o = [t.reshape(1, n_slices, S, D) for t in
                    synth.attention_inputs(seed, 1, n_slices, S, D, bf16=True, qk_scale=qk_scale)]
    ol.fwd(q[:, :1, :256], k[:, :1, :256], v[:, :1, :256])   # load the library, warm the thread pool
    t0 = time.perf_counter()
    ol.fwd(q, k, v, True)
    ol.bwd(q, k, v, d_o, True)
    dt = time.perf_counter() - t0
    cores = ol.oracle().oracle_num_threads()
    return (flops_fwd(n_slices, S, D) + flops_bwd(n_slices, S, D)) / dt / 1e12, dt, cores


def oracle_on_slices(q, k, v, d_o):
    """Runs the CPU oracle (forward + composed backward, all host threads) on host arrays [n, S, D] of
    bf16-representable fp32.  Returns (o, lse, dq, dk, dv, seconds, threads)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    ol.oracle().oracle_set_num_threads(os.cpu_count() or 1)   # torchrun sets OMP_NUM_THREADS=1
    ol.fwd(q[None, :1, :256], k[None, :1, :256], v[None, :1, :256])   # load the library, warm the thread pool
    t0 = time.perf_counter()
    o, lse = ol.fwd(q[None], k[None], v[None], True)
    dq, dk, dv = ol.bwd(q[None], k[None], v[None], d_o[None], True)
    dt = time.perf_counter() - t0
    return o[0], lse[0], dq[0], dk[0], dv[0], dt, ol.oracle().oracle_num_threads()


def parity_against_oracle(slices, dev, S, D):
    """Compares what the device-resident run left in HBM with the CPU oracle on the same inputs, for the listed
    (batch x head) slices.  `dev` = (q, k, v, d_o, o, lse, dq, dk, dv) torch tensors [n, S, D] / [n, S].
    Returns the `parity` dict of the JSON line and the oracle's rate for the `cpu_baseline` dict."""
    import numpy as np
    import torch
    idx = torch.tensor(slices, device=dev[0].device)
    host = [t.index_select(0, idx).float().cpu().numpy() for t in dev]
    q, k, v, d_o, o, lse, dq, dk, dv = host
    ro, rlse, rdq, rdk, rdv, dt, threads = oracle_on_slices(q, k, v, d_o)
    out = {"slices": list(slices), "against": "CPU oracle (oracle/attention_oracle.cpp) on the same inputs, fp32",
           "max_abs": {}, "rel_l2": {}, "lse_max_abs": float(np.abs(lse - rlse).max()),
           "tolerance": {"max_abs": 2e-2, "lse_max_abs": 1e-4,
                         "rel_l2": "1e-3 stated; a bf16-stored result cannot be below 1.48e-3 against an fp32 oracle"}}
    for name, got, want in (("O", o, ro), ("dQ", dq, rdq), ("dK", dk, rdk), ("dV", dv, rdv)):
        g64, w64 = got.astype(np.float64), want.astype(np.float64)
        out["max_abs"][name] = float(np.abs(g64 - w64).max())
        out["rel_l2"][name] = float(np.linalg.norm(g64 - w64) / (np.linalg.norm(w64) + 1e-300))
    out["within_max_abs"] = bool(max(out["max_abs"].values()) <= 2e-2 and out["lse_max_abs"] <= 1e-4)
    n = len(slices)
    rate = (flops_fwd(n, S, D) + flops_bwd(n, S, D)) / dt / 1e12
    return out, rate, dt, threads


def run_reference(args, rank, world):
    """The reference's algorithm on the host cores (the CPU oracle, all threads)."""
    if rank != 0:
        return
    B, H, S, D, qs, desc = WORKLOADS[args.workload]
    # bounded sample per step: head-slices of the workload at full sequence length
    n_slices = 1 if S >= 4096 else min(B * H, 16)
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt, cores = cpu_oracle_rate(S, D, qs, n_slices, 0x1A7E5EED + 4 + i)
        if i >= args.warmup:
            rates.append((r, dt))
    value = statistics.mean(r for r, _ in rates)
    ms = statistics.mean(dt for _, dt in rates) * 1e3
    sample = f"{n_slices} of {B * H} (batch x head) slices at full S={S}, fwd+bwd, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "note": "reference is Metal-only; its algorithm restated in C++ (oracle/) runs on the host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from irontensor_b200 import Precision, Tensor, attention_backward_recompute, context, flash_attention, raw, synth
    from irontensor_b200 import _lib
    from irontensor_b200.sharding import shard_range

    all_cores = os.sched_getaffinity(0)
    host_binding = "off" if args.no_bind else bind_host_to_gpu(
        local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    torch.cuda.set_device(local_rank)
    ctx = context(local_rank)
    B, H, S, D, qs, desc = WORKLOADS[args.workload]
    BH = B * H
    if args.slices:
        BH = min(BH, args.slices)
        desc += f" (reduced to {BH} slices)"
    b0, b1 = shard_range(BH, world, rank)
    nbh = b1 - b0
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- this rank's shard, generated on the device (seeded; same distribution as the parity tests' generator)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + 4 + 1000 * rank)
    n = max(nbh, 1)

    def mk(scale):
        return (torch.randn((n, S, D), generator=gen, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)

    q, k, v, d_o = mk(qs), mk(qs), mk(1.0), mk(1.0)
    o = torch.empty_like(q)
    lse = torch.empty((n, S), dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    ws_bytes = raw.bwd_workspace_bytes(_lib.IT_BF16, 1, n, S, D)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # > 126 MB L2

    def step_device():
        if nbh == 0:
            return
        raw.fwd(_lib.IT_BF16, 1, nbh, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                lse.data_ptr(), ctx=ctx)
        raw.bwd(_lib.IT_BF16, 1, nbh, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                d_o.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws_bytes,
                ctx=ctx)

    ctx.enable_kernel_timing(1)
    use_timers2 = D in (64, 128) and S >= 128     # the tensor-core backward has the prepare and finish passes
    for _ in range(warmup):
        step_device()
    ctx.poll_status()

    # nvidia-smi needs ~0.15 s to deliver its first sample; during that wait the GPU leaves its active power
    # state, so one more untimed step runs right before the timed ones (otherwise the first timed step of a
    # short workload pays for the wake-up: 0.10 ms against 0.05 ms on the TINY shape).
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    sampler.start()
    time.sleep(0.15)
    flush.fill_(0)       # also the first use of the fill kernel: its one-time set-up stays outside the timed steps
    step_device()
    launches0 = ctx.launch_count()
    barrier()
    sampler.mark()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    fwd_ms, bwd_ms, prep_ms, fin_ms = [], [], [], []
    for i in range(steps):
        flush.fill_(i & 0xFF)                 # evict the previous step's tensors from L2 (outside the event pair)
        ev[i][0].record()
        step_device()
        ev[i][1].record()
        if nbh:
            bwd_ms.append(ctx.kernel_ms(1))   # waits for this step's kernels
    barrier()
    launches = ctx.launch_count() - launches0
    ctx.poll_status()
    if nbh:   # the forward kernel and the small passes of the backward, timed in three extra steps outside the timed region
        ctx.enable_kernel_timing(3 if use_timers2 else 2)
        for _ in range(3):
            step_device()
            fwd_ms.append(ctx.kernel_ms(0))
            if use_timers2:
                prep_ms.append(ctx.kernel_ms(2))
                fin_ms.append(ctx.kernel_ms(3))
        ctx.enable_kernel_timing(1)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    my_ms = sum(step_ms) / steps
    ms_per_step = max_over_ranks(my_ms)
    total_flops = flops_fwd(BH, S, D) + flops_bwd(BH, S, D)
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public ops with host tensors
    clocks = sampler.stop()      # samples of the device-resident timed region only
    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                              "warmup": warmup, "ms_per_step": ms_per_step, "config": {"workload": desc},
                              "kernel_ms": {"fwd": statistics.mean(fwd_ms), "bwd": statistics.mean(bwd_ms)},
                              "gpu_launches": int(launches), "clocks": clocks, "note": "profiling run: no e2e / cpu legs"}),
                  flush=True)
        return
    hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, d_o))
    ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
    from irontensor_b200 import HostAttentionStep
    pipe = HostAttentionStep(n, S, D, Precision.BF16, causal=True, chunks=args.e2e_chunks)
    sampler_e2e = ClockSampler(sampler.gpu_index)

    def step_e2e(copies_only=False):
        pipe.run(hq, hk, hv, hdo, ho, hdq, hdk, hdv, copies_only=copies_only)

    e2e_steps = steps
    if nbh:
        for _ in range(2):
            step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler_e2e.start()
    e0.record()
    issue_s = 0.0
    if nbh:
        for _ in range(e2e_steps):
            t_issue = time.perf_counter()
            step_e2e()
            issue_s += time.perf_counter() - t_issue     # host time spent enqueueing (the call does not wait for the GPU)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    clocks_e2e = sampler_e2e.stop()
    ctx.poll_status()
    host_issue_ms = max_over_ranks(issue_s / e2e_steps * 1e3)
    # the same uploads and downloads, same groups, streams and pinned buffers, without the kernels
    ho_keep = ho.clone() if nbh else None
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    if nbh:
        for _ in range(e2e_steps):
            step_e2e(copies_only=True)
    c1.record()
    barrier()
    copy_only_ms = max_over_ranks(c0.elapsed_time(c1) / e2e_steps)
    if nbh:
        ho.copy_(ho_keep)
    e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12
    nbytes = nbh * S * D * 2
    if nbh:
        assert torch.equal(ho.view(torch.int16), o[:nbh].cpu().view(torch.int16)), "e2e forward differs from the device-resident run"

    if rank != 0:
        return
    peaks = measured_peaks()
    bwd_avg_ms = statistics.mean(bwd_ms) if bwd_ms else float("nan")
    fwd_avg_ms = statistics.mean(fwd_ms) if fwd_ms else float("nan")
    ach = flops_bwd(nbh, S, D) / (bwd_avg_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "fa_bwd_sm100_kernel", "achieved": ach, "peak": peaks["bf16"], "unit": "TFLOP/s",
        "frac": ach / peaks["bf16"], "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(args.workload if world == 1 else None),
        "peak_source": peaks["source"] + " (burst)", "avg_launch_ms": bwd_avg_ms,
        "frac_of_sustained_peak": ach / peaks["bf16_sustained"] if peaks["bf16_sustained"] else None,
        "profiler_tag": ctx.kernel_tag(1),
        "other_kernels_ms": {ctx.kernel_tag(2): statistics.mean(prep_ms) if prep_ms else None,
                             ctx.kernel_tag(3): statistics.mean(fin_ms) if fin_ms else None},
        "forward_kernel": {"kernel": "fa_fwd_pp_sm100_kernel" if (D == 128 and S >= 4096) else "fa_fwd_sm100_kernel",
                           "avg_launch_ms": fwd_avg_ms,
                           "achieved": flops_fwd(nbh, S, D) / (fwd_avg_ms * 1e-3) / 1e12,
                           "frac": flops_fwd(nbh, S, D) / (fwd_avg_ms * 1e-3) / 1e12 / peaks["bf16"]},
    }
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "step_ms": {"min": min(step_ms), "median": statistics.median(step_ms),
                                                "first": step_ms[0], "last": step_ms[-1], "note": "rank 0's timed steps"},
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "sharding": f"{BH} (batch x head) slices split contiguously over {world} GPU(s), no collective",
                   "l2": "256 MB buffer written between timed steps; per-GPU tensors exceed L2 at N=1",
                   "tflops_per_gpu": value / world, "frac_of_bf16_peak_per_gpu": value / world / peaks["bf16"]},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": 4 * nbytes,
                "d2h_bytes_per_step": 4 * nbytes, "note": "bytes are rank 0's", "groups": args.e2e_chunks,
                "copy_only_ms": copy_only_ms, "host_issue_ms": host_issue_ms,
                "copy_only_gbs_per_direction": 4 * nbytes / (copy_only_ms * 1e-3) / 1e9 if nbh else None,
                "breakdown_note": "copy_only_ms: the step's uploads and downloads alone on the same streams; host_issue_ms: "
                                  "wall time the host spends enqueueing one step; both max over ranks",
                "host_cores": host_binding, "clocks": clocks_e2e},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
    }
    if world == 1 and not args.no_cpu:
        os.sched_setaffinity(0, all_cores)   # the CPU baseline uses every core the process was given
        # The oracle runs on the very slices the GPU just processed (inputs and results downloaded from HBM): slices either
        # side of a boundary of the backward's CTA-order groups of four (3 | 4), the first and the last (the forward's tail
        # group).  One run gives both the parity figures and the CPU baseline's time.
        want = [0, 3, 4, BH - 1] if S >= 4096 else sorted(set([0, 3, 4, BH // 2, BH - 1] + list(range(8, min(BH, 35)))))
        sl = [b for b in sorted(set(want)) if 0 <= b < nbh]
        step_device()                         # results of the device-resident path (the e2e leg shares no buffers with it)
        ctx.poll_status()
        parity, r, dt, cores = parity_against_oracle(sl, (q, k, v, d_o, o, lse, dq, dk, dv), S, D)
        line["parity"] = parity
        line["cpu_baseline"] = {"value": r, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": f"{len(sl)} of {BH} (batch x head) slices at full S={S} (the slices of `parity`), "
                                          f"fwd+bwd, {dt:.1f} s"}
    if world == 1 and args.workload == "c4" and not args.no_secondary:
        line["secondary"] = secondary_configs(ctx, peaks)
    print(json.dumps(line), flush=True)


def _timed_us(fn, reps, flush):
    """Median and minimum device time of fn() in microseconds (CUDA events); `flush`: a buffer larger than L2
    written before each call, or None to leave L2 warm."""
    import torch
    ts = []
    for i in range(reps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts), min(ts)


def measure_c1(ctx, peaks, flush, steps, warmup):
    """fp32 causal forward B16 H4 S256 D64 (the reference's own benchmark shape), device-resident."""
    import torch
    from irontensor_b200 import _lib, raw
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + 1)
    B, H, S, D = 16, 4, 256, 64
    q, k, v = (torch.randn((B, H, S, D), generator=gen, device="cuda") for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((B, H, S), device="cuda")

    def f():
        raw.fwd(_lib.IT_F32, B, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=ctx)
    for _ in range(max(warmup, 3)):
        f()
    med_cold, min_cold = _timed_us(f, steps, flush)
    med_warm, min_warm = _timed_us(f, steps, None)
    flops, nbytes = 2.0 * B * H * S * S * D, 4 * B * H * S * D * 4 + B * H * S * 4
    return {"metric": "causal attention forward latency", "unit": "us", "value": med_cold, "higher_is_better": False,
            "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "dtype": "f32", "data": "synthetic",
            "config": {"workload": "causal fp32 attention forward B16 H4 S256 D64", "l2": "flushed between calls (value); warm figures alongside"},
            "us_min": min_cold, "us_warm_l2": med_warm, "gbs": nbytes / med_cold / 1e3, "gbs_warm_l2": nbytes / med_warm / 1e3,
            "tflops": flops / med_cold / 1e6, "roofline": {"bound": "hbm", "achieved": nbytes / med_cold / 1e3, "peak": peaks["hbm"],
                                                           "unit": "GB/s", "frac": nbytes / med_cold / 1e3 / peaks["hbm"], "traffic": None}}


def measure_c5(ctx, peaks, steps, warmup):
    """The greedy no-KV-cache pattern: fp32 causal forward B1 H4 D64 at every prefix length 20..119 (100 calls),
    eager, replayed from one CUDA graph, and served from a key/value cache instead."""
    import torch
    from irontensor_b200 import _lib, raw
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + 5)
    H, D = 4, 64
    lens = list(range(20, 120))
    bufs = []
    for S in lens:
        q, k, v = (torch.randn((1, H, S, D), generator=gen, device="cuda") for _ in range(3))
        bufs.append((S, q, k, v, torch.empty_like(q), torch.empty((1, H, S), device="cuda")))

    def seq():
        for S, q, k, v, o, lse in bufs:
            raw.fwd(_lib.IT_F32, 1, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=ctx)
    for _ in range(max(warmup, 3)):
        seq()
    torch.cuda.synchronize()
    med_eager, min_eager = _timed_us(seq, steps, None)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        seq()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            seq()
    torch.cuda.synchronize()
    med_graph, min_graph = _timed_us(graph.replay, steps, None)
    # The same generation served from a key/value cache (it_attention_decode): each step attends one new token
    # against the cached positions instead of recomputing the whole prefix.
    kc = torch.randn((1, 128, H, D), generator=gen, device="cuda")
    vc = torch.randn((1, 128, H, D), generator=gen, device="cuda")
    qd = torch.randn((1, H, D), generator=gen, device="cuda")
    od = torch.empty_like(qd)
    nws = raw.decode_workspace_bytes(1, H, D)
    wsd = torch.empty(nws, dtype=torch.uint8, device="cuda")

    def seq_cached():
        for S in lens:
            raw.decode(_lib.IT_F32, 1, H, H, D, S, 128, qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), od.data_ptr(), None,
                       wsd.data_ptr(), nws, ctx=ctx)
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        seq_cached()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph2, stream=side):
            seq_cached()
    torch.cuda.synchronize()
    med_cached, _ = _timed_us(graph2.replay, steps, None)
    flops = sum(512.0 * S * S for S in lens)
    nbytes = sum(4112.0 * S for S in lens)
    line = {"metric": "greedy no-KV-cache attention forward, per-call latency", "unit": "us", "value": med_graph / len(lens),
            "higher_is_better": False, "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3), "dtype": "f32",
            "data": "synthetic", "config": {"workload": "fp32 causal forward B1 H4 D64 at prefix lengths 20..119 (100 calls)",
                                            "note": "value = one CUDA-graph replay of the 100 calls / 100; tensors stay in L2 (28.6 MB in total)"},
            "us_per_call_eager": med_eager / len(lens), "us_per_call_graph_min": min_graph / len(lens),
            "us_per_call_with_kv_cache": med_cached / len(lens),
            "gbs": nbytes / med_graph / 1e3, "tflops": flops / med_graph / 1e6,
            "roofline": {"bound": "hbm", "achieved": nbytes / med_graph / 1e3, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": nbytes / med_graph / 1e3 / peaks["hbm"], "traffic": None,
                         "note": "launch-latency bound: the HBM time of the longest call is 0.08 us"}}
    return line




def measure_fwd_bwd(ctx, peaks, flush, workload, steps, warmup):
    """bf16 causal forward + backward of one of WORKLOADS, device-resident, one GPU: ms per step and TFLOP/s."""
    import torch
    from irontensor_b200 import _lib, raw
    B, H, S, D, qs, desc = WORKLOADS[workload]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + int(workload[1:]))
    mk = lambda sc: (torch.randn((B * H, S, D), generator=gen, device="cuda") * sc).to(torch.bfloat16)
    q, k, v, d_o = mk(qs), mk(qs), mk(1.0), mk(1.0)
    o, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((B * H, S), device="cuda")
    nws = raw.bwd_workspace_bytes(_lib.IT_BF16, B, H, S, D)
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda")

    def f():
        raw.fwd(_lib.IT_BF16, B, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=ctx)
        raw.bwd(_lib.IT_BF16, B, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
                lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), nws, ctx=ctx)
    for _ in range(max(warmup, 3)):
        f()
    med, mn = _timed_us(f, steps, flush)
    # steps one behind the other, as a training loop issues them, one event pair around all of them and no flush: each
    # kernel is then set up under the tail of the one in front (programmatic dependent launch)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = None
    for _ in range(3):
        e0.record()
        for _ in range(steps):
            f()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / steps
        best = t if best is None else min(best, t)
    flops = flops_fwd(B * H, S, D) + flops_bwd(B * H, S, D)
    return {"workload": desc, "ms_per_step": med / 1e3, "ms_min": mn / 1e3, "tflops": flops / med / 1e6,
            "frac_of_bf16_peak": flops / med / 1e6 / peaks["bf16"], "steps": steps, "l2": "flushed between steps",
            "ms_per_step_back_to_back": best, "back_to_back": f"{steps} steps in a row, no flush, best of 3"}


def secondary_configs(ctx, peaks):
    """Short single-GPU reports on the four configurations that are not the headline one, each with its own clock
    sample: C1 (fp32 forward latency and achieved HBM rate), C2 and C3 (bf16 forward + backward), C5 (per-call
    latency of the 100-call greedy pattern in a CUDA graph)."""
    import torch
    ctx.enable_kernel_timing(0)     # the event records around the main kernels cost microseconds: visible on these shapes
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    gpu = torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else \
        os.environ["CUDA_VISIBLE_DEVICES"].split(",")[torch.cuda.current_device()]
    out = {}

    def sampled(name, fn):
        sm = ClockSampler(gpu)
        sm.start()
        time.sleep(0.15)     # nvidia-smi needs a moment to deliver its first sample
        sm.mark()
        r = fn()             # each measurement warms up by itself; the samples cover its warm-up too
        r["clocks"] = sm.stop()
        out[name] = r

    def c1():
        m = measure_c1(ctx, peaks, flush, 600, 3)   # long enough for a few clock samples to land inside
        return {"workload": m["config"]["workload"], "us": m["value"], "us_warm_l2": m["us_warm_l2"], "gbs": m["gbs"],
                "frac_of_hbm_peak": m["roofline"]["frac"], "tflops": m["tflops"]}

    def c5():
        m = measure_c5(ctx, peaks, 20, 3)
        return {"workload": m["config"]["workload"], "us_per_call_graph": m["value"], "us_per_call_eager": m["us_per_call_eager"],
                "us_per_call_with_kv_cache": m["us_per_call_with_kv_cache"], "gbs": m["gbs"]}
    sampled("c1", c1)
    sampled("c2", lambda: measure_fwd_bwd(ctx, peaks, flush, "c2", 300, 3))
    sampled("c3", lambda: measure_fwd_bwd(ctx, peaks, flush, "c3", 50, 3))
    sampled("c5", c5)
    return out


def run_small(args):
    """Single-GPU reports that are not the headline line: c1, c5 (see measure_c1, measure_c5), decode, linear, layer.
    Device-resident inputs, CUDA events."""
    import torch
    from irontensor_b200 import _lib, context, raw
    torch.cuda.set_device(0)
    ctx = context(0)
    peaks = measured_peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + 9)

    def timed(fn, reps, flush_l2):
        return _timed_us(fn, reps, flush if flush_l2 else None)

    if args.workload == "c1":
        print(json.dumps(measure_c1(ctx, peaks, flush, args.steps, args.warmup)), flush=True)
        return
    if args.workload == "c5":
        print(json.dumps(measure_c5(ctx, peaks, args.steps, args.warmup)), flush=True)
        return
    if args.workload == "decode":
        # One new token per sequence against a bf16 key/value cache (grouped heads): the op reads the cache once.
        B, H, Hkv, D, L = 32, 32, 8, 128, 8192
        dt = torch.bfloat16
        q = torch.randn((B, H, D), generator=gen, device="cuda").to(dt)
        kc = torch.randn((B, L, Hkv, D), generator=gen, device="cuda").to(dt)
        vc = torch.randn((B, L, Hkv, D), generator=gen, device="cuda").to(dt)
        o = torch.empty_like(q)
        lse = torch.empty((B, H), device="cuda")
        nws = raw.decode_workspace_bytes(B, H, D)
        ws = torch.empty(nws, dtype=torch.uint8, device="cuda")

        def f():
            raw.decode(_lib.IT_BF16, B, H, Hkv, D, L, L, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), lse.data_ptr(),
                       ws.data_ptr(), nws, ctx=ctx)
        for _ in range(max(args.warmup, 3)):
            f()
        med, mn = timed(f, args.steps, True)     # the 1.07 GB cache exceeds L2 by itself; flushed anyway
        nbytes = 2.0 * B * L * Hkv * D * 2 + 2.0 * B * H * D * 2
        line = {"metric": "KV-cache decode attention, cache bytes per second", "unit": "GB/s", "value": nbytes / med / 1e3,
                "higher_is_better": True, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bf16",
                "data": "synthetic", "config": {"workload": "decode B32 H32 kv_heads 8 D128, 8192 cached positions, bf16"},
                "us": med, "us_min": mn,
                "roofline": {"bound": "hbm", "achieved": nbytes / med / 1e3, "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": nbytes / med / 1e3 / peaks["hbm"], "traffic": None,
                             "note": "peak is the measured copy bandwidth (read + write); a read-only stream can exceed it"}}
        print(json.dumps(line), flush=True)
        return
    if args.workload == "linear":
        # The projections around attention for the C4 token count: n = B*S = 32768 tokens, hidden 2048,
        # fused QKV width (16 + 2*16 heads of 128) = 6144: y = x W^T, dx = dy W, dW = dy^T x.
        n, k, out = 32768, 2048, 6144
        x = torch.randn((n, k), generator=gen, device="cuda").to(torch.bfloat16)
        w = (torch.randn((out, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)
        dy = torch.randn((n, out), generator=gen, device="cuda").to(torch.bfloat16)
        y = torch.empty((n, out), dtype=torch.bfloat16, device="cuda")
        dx = torch.empty_like(x)
        dw = torch.empty((out, k), device="cuda")

        def f():
            raw.linear_fwd(n, k, out, x.data_ptr(), w.data_ptr(), y.data_ptr(), ctx=ctx)
            raw.linear_bwd(n, k, out, dy.data_ptr(), x.data_ptr(), w.data_ptr(), dx.data_ptr(), dw.data_ptr(), ctx=ctx)

        def lib():   # the same three products through torch (cuBLAS), for the ratio only
            torch.matmul(x, w.t())
            torch.matmul(dy, w)
            torch.matmul(dy.t(), x)
        for _ in range(max(args.warmup, 3)):
            f()
            lib()
        med, mn = timed(f, args.steps, True)
        med_lib, _ = timed(lib, args.steps, True)
        flops = 3 * 2.0 * n * k * out
        line = {"metric": "projection GEMMs fwd+bwd TFLOP/s", "unit": "TFLOP/s", "value": flops / med / 1e6,
                "higher_is_better": True, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bf16",
                "data": "synthetic", "config": {"workload": "linear forward + backward, 32768 tokens, 2048 -> 6144, bf16"},
                "us": med, "us_min": mn, "gpu_launches": 3 * (args.steps + max(args.warmup, 3)),
                "cublas_same_box_tflops": flops / med_lib / 1e6,
                "roofline": {"bound": "tensor", "achieved": flops / med / 1e6, "peak": peaks["bf16"], "unit": "TFLOP/s",
                             "frac": flops / med / 1e6 / peaks["bf16"], "traffic": None}}
        print(json.dumps(line), flush=True)
        return


def run_layer(args, rank, world, local_rank):
    """The whole attention layer of the C4 shape, forward + backward, with the HEADS split over the ranks: every rank
    projects with its rows of [Wq; Wk; Wv] (one GEMM with the rotary epilogue, packed q|k|v layout), attends over its
    heads, multiplies by its columns of Wo -- and the partial outputs are summed by an NCCL all-reduce, the one real
    exchange step around the path (src/train/forward.rs:146 of the reference; backward: the gradient of the layer's
    input, src/train/backward.rs:139-147, is the second sum over ranks).  Rank 0 also runs the unsharded layer and
    compares.  No library GEMM is given a peer's memory; the all-reduce is NCCL's own."""
    import torch
    import torch.distributed as dist
    from irontensor_b200 import (Precision, Tensor, attention_packed, attention_packed_backward, context, linear_backward,
                                 linear_forward, qkv_rope_forward, raw)
    from irontensor_b200.sharding import SummedProjection, head_shard, out_projection_all_reduce, qkv_weight_rows
    torch.cuda.set_device(local_rank)
    ctx = context(local_rank)
    peaks = measured_peaks()
    B, S, hidden, H, Hkv, D = 4, 8192, 2048, 16, 16, 128
    n = B * S
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x1A7E5EED + 6)      # the same seed on every rank: every rank generates the same full tensors
    rnd = lambda shape, sc: (torch.randn(shape, generator=gen, device="cuda") * sc).to(torch.bfloat16)
    x, wq, wk, wv = rnd((B, S, hidden), 1.0), rnd((H * D, hidden), 0.02), rnd((Hkv * D, hidden), 0.02), rnd((Hkv * D, hidden), 0.02)
    wo, dout = rnd((hidden, H * D), 0.02), rnd((n, hidden), 1.0)
    T = lambda t: Tensor(t.contiguous().reshape(-1), list(t.shape), Precision.BF16)

    def make(world_, rank_):
        qb, qe, kb, ke = head_shard(H, Hkv, world_, rank_)
        (q0, q1), (k0, k1), (v0, v1) = qkv_weight_rows(H, Hkv, D, world_, rank_)
        hl, hkvl = qe - qb, ke - kb
        w_l, wo_l = T(torch.cat([wq[q0:q1], wk[k0:k1], wv[v0:v1]], 0)), T(wo[:, q0:q1])
        tx, tdout = T(x), T(dout)
        width = (hl + 2 * hkvl) * D

        chunks = max(args.layer_chunks, 1) if world_ > 1 else 1
        rows = n // chunks
        fused = {}   # result buffers in symmetric memory for the GEMMs that do their own reduce-scatter
        if world_ > 1:
            fused["out"], fused["dx"] = SummedProjection(n, hidden), SummedProjection(n, hidden)

        def step(reduce):
            """reduce: False = no exchange; True = one blocking all-reduce per sum; "overlap" = the two GEMMs whose results
            are summed over ranks run in row chunks, each chunk's all-reduce (NCCL's stream) under the next chunk's GEMM;
            "fused" = those two GEMMs add their row blocks into the owners' buffers over NVLink themselves
            (it_linear_scatter_add), followed by an all-gather."""
            qkv = qkv_rope_forward(tx, w_l, hl, hkvl, D, 10000.0, 0, packed=True)
            attn = attention_packed(qkv, hl, hkvl, D, True)
            pending = []
            if reduce == "fused":
                a2 = attn.torch().view(n, hl * D)
                out = Tensor(fused["out"].run(0, a2.data_ptr(), wo_l.data_ptr(), hl * D, hidden).reshape(-1), [n, hidden], Precision.BF16)
            elif reduce == "overlap":
                out = Tensor.empty([n, hidden], Precision.BF16)
                a2 = attn.torch().view(n, hl * D)
                for c in range(chunks):
                    r0 = c * rows
                    raw.linear_fwd(rows, hl * D, hidden, a2[r0:r0 + rows].data_ptr(), wo_l.data_ptr(), out.torch()[r0:r0 + rows].data_ptr())
                    pending.append(dist.all_reduce(out.torch()[r0:r0 + rows], async_op=True))
            else:
                out = linear_forward(attn.view([n, hl * D]), wo_l)                   # this rank's partial [n, hidden]
                if reduce:
                    out_projection_all_reduce(out.torch())
            d_attn, d_wo = linear_backward(tdout, attn.view([n, hl * D]), wo_l)
            d_qkv = attention_packed_backward(d_attn.view([B, S, hl, D]), qkv, attn, hl, hkvl, D, True, rope_base=10000.0)
            if reduce == "fused":
                d_w = Tensor.empty([width, hidden], Precision.FP32)
                g2, x2 = d_qkv.torch().view(n, width), tx.torch().view(n, hidden)
                raw.linear_bwd(n, hidden, width, g2.data_ptr(), x2.data_ptr(), w_l.data_ptr(), None, d_w.data_ptr())   # no exchange
                d_x = Tensor(fused["dx"].run(1, g2.data_ptr(), w_l.data_ptr(), hidden, width).reshape(-1), [n, hidden], Precision.BF16)
            elif reduce == "overlap":
                d_x, d_w = Tensor.empty([n, hidden], Precision.BF16), Tensor.empty([width, hidden], Precision.FP32)
                g2, x2 = d_qkv.torch().view(n, width), tx.torch().view(n, hidden)
                for c in range(chunks):
                    r0 = c * rows
                    raw.linear_bwd(rows, hidden, width, g2[r0:r0 + rows].data_ptr(), x2[r0:r0 + rows].data_ptr(), w_l.data_ptr(),
                                   d_x.torch()[r0:r0 + rows].data_ptr(), None)
                    pending.append(dist.all_reduce(d_x.torch()[r0:r0 + rows], async_op=True))
                raw.linear_bwd(n, hidden, width, g2.data_ptr(), x2.data_ptr(), w_l.data_ptr(), None, d_w.data_ptr())   # no exchange
                for wk_ in pending:
                    wk_.wait()
            else:
                d_x, d_w = linear_backward(d_qkv.view([n, width]), tx.view([n, hidden]), w_l)
                if reduce:
                    out_projection_all_reduce(d_x.torch())
            return out, d_x, d_wo, d_w
        return step, hl, hkvl

    step, hl, hkvl = make(world, rank)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_interleaved(fns):
        """Mean device time per call of each function, the functions taking turns step by step, so that the drift
        of the clock under the power cap during the run falls on all of them alike.  Max over ranks."""
        for _ in range(warmup):
            for fn in fns:
                fn()
        barrier()
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)] for _ in fns]
        for i in range(steps):
            for j, fn in enumerate(fns):
                flush.fill_(1)
                ev[j][i][0].record()
                fn()
                ev[j][i][1].record()
        barrier()
        ctx.poll_status()
        return [max_over_ranks(sum(a.elapsed_time(b) for a, b in e) / steps) for e in ev]

    l0 = ctx.launch_count()
    step(False)
    launches = ctx.launch_count() - l0
    if world > 1:
        ms_nccl, ms_local, ms_fused = timed_interleaved([lambda: step(True), lambda: step(False), lambda: step("fused")])
        ms = min(ms_nccl, ms_fused)      # the line's value is the faster of the two exchanges; both are reported
    else:
        ms = ms_nccl = ms_local = timed_interleaved([lambda: step(False)])[0]
        ms_fused = None
    ms_overlap = timed_interleaved([lambda: step("overlap")])[0] if (world > 1 and args.layer_chunks > 0) else None
    buf = torch.empty((n, hidden), dtype=torch.bfloat16, device="cuda")
    ms_ar = timed_interleaved([lambda: out_projection_all_reduce(buf)])[0] if world > 1 else 0.0
    # the summed results against the unsharded layer on rank 0 (same seed, same kernels, all heads on one GPU)
    out, d_x, _, _ = step("fused" if world > 1 else False)      # the fused exchange's result is the one checked
    check = None
    if rank == 0:
        full_step, _, _ = make(1, 0)
        f_out, f_dx, _, _ = full_step(False)
        torch.cuda.synchronize()
        rel = lambda a, b: float((a.torch().float() - b.torch().float()).norm() / b.torch().float().norm())
        check = {"against": "the unsharded layer on rank 0, same seed", "out_rel_l2": rel(out, f_out), "dx_rel_l2": rel(d_x, f_dx),
                 "out_max_abs": float((out.torch().float() - f_out.torch().float()).abs().max()),
                 "note": "each rank's partial is rounded to bf16 before the sum"}
        assert check["out_rel_l2"] < 1e-2 and check["dx_rel_l2"] < 1e-2, check
    barrier()
    if rank != 0:
        return
    gemm = 2.0 * n * hidden * ((H + 2 * Hkv) * D + H * D)
    flops = 3 * gemm + 7.0 * B * H * S * S * D
    ar_bytes = n * hidden * 2
    line = {"metric": "attention layer fwd+bwd TFLOP/s (projections + rotary + causal attention), heads split over the GPUs",
            "unit": "TFLOP/s", "value": flops / ms / 1e9, "higher_is_better": True, "n_gpus": world, "steps": steps, "warmup": warmup,
            "dtype": "bf16", "data": "synthetic", "ms_per_step": ms, "scaling": "strong",
            "config": {"workload": "attention layer B4 S8192 hidden 2048, 16 heads of 128, packed q|k|v, bf16",
                       "sharding": f"{hl} of {H} heads per rank; output projection and input gradient are sums over ranks",
                       "flops": {"projections": 3 * gemm, "attention": 7.0 * B * H * S * S * D}},
            "exchange": {"used_for_value": None if world == 1 else ("nccl_all_reduce" if ms_nccl <= ms_fused else "fused_reduce_scatter"),
                         "ms_per_step_nccl_all_reduce": ms_nccl if world > 1 else None,
                         "ms_per_step_fused_reduce_scatter": ms_fused,
                         "fused_reduce_scatter": "the two summed GEMMs add their row blocks into the owners' buffers themselves (TMA "
                                                 "reduce-add over NVLink peer memory in the epilogue), then NCCL all-gather",
                         "ms_per_step_no_exchange": ms_local, "share_of_step": (ms - ms_local) / ms if world > 1 else 0.0,
                         "timing": "the three variants take turns step by step (clock drift under the power cap falls on all alike)"},
            "all_reduce": {"per_step": 2 if world > 1 else 0, "bytes_each": ar_bytes, "ms_each_alone": ms_ar,
                           "bus_gbs_alone": (2 * (world - 1) / world * ar_bytes / (ms_ar * 1e-3) / 1e9) if world > 1 else None,
                           "ms_per_step_without": ms_local, "share_of_step": (ms_nccl - ms_local) / ms_nccl if world > 1 else 0.0,
                           "ms_per_step_chunked_overlap": ms_overlap,
                           "chunked_overlap": (f"{args.layer_chunks} row chunks per summed GEMM, each chunk's all-reduce issued under the "
                                               "next chunk's GEMM; slower than one blocking all-reduce: NCCL's kernel cannot run "
                                               "beside a GEMM that holds every SM") if ms_overlap is not None else None},
            "check": check, "gpu_launches": launches, "gpu_launches_note": "library kernels of one step without exchange",
            "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9 / world, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": flops / ms / 1e9 / world / peaks["bf16"], "traffic": None, "note": "per GPU"}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["c1", "c5", "decode", "linear", "layer"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-tensor end-to-end leg (profiling runs)")
    ap.add_argument("--no-bind", action="store_true", help="leave the process's CPU affinity alone")
    ap.add_argument("--no-secondary", action="store_true", help="skip the short reports on the other four configurations")
    ap.add_argument("--e2e-chunks", type=int, default=16,
                    help="groups the end-to-end leg cuts a rank's slices into (upload, kernels and download of "
                         "different groups overlap)")
    ap.add_argument("--layer-chunks", type=int, default=0,
                    help="--workload layer on several GPUs: also time the variant that runs the two summed GEMMs in this many "
                         "row chunks with each chunk's all-reduce under the next chunk's GEMM (0: skip)")
    ap.add_argument("--slices", type=int, default=0,
                    help="use only this many (batch x head) slices of the workload (small profiling cases)")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torchrun, one rank per GPU
        port = os.environ.get("MASTER_PORT", "29517")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", port, os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))

    if args.workload in ("c1", "c5", "decode", "linear"):
        if rank == 0:
            run_small(args)
        return
    if args.workload == "layer":
        if world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        try:
            run_layer(args, rank, world, local_rank)
        finally:
            if world > 1:
                import torch.distributed as dist
                dist.destroy_process_group()
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
