"""Benchmark of the NVFP4 W4A16 MoE decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c1|c4|c5] [--tokens T]

N = 1: configuration 2 (T=32, H=4096, I=1536, E=128, top-8, all experts on the GPU).
N > 1 (launched by torch.distributed.run, one rank per GPU): configuration 4 (T=128, H=7168, I=2048,
E=256 sharded contiguously + a replicated shared expert), all-gather -> local experts -> reduce-scatter.

A step is one MoE layer call on one batch of seeded synthetic inputs (three routing seeds, rotated).
`value` is the weight-stream rate: the algorithmic bytes of the step (FP4 codes + E4M3 scales of every
touched expert + activations) over the device time of the step, summed over ranks; `ms_per_step`
is the step time.  The touched weights of one step (>= 0.8 GB) are larger than the 126 MB L2, and
a 256 MB buffer is read between timed steps on top of that; timing is CUDA events on the launching
stream, max over ranks.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# dram bytes of one okc_moe_gemm launch under ncu, configuration 2 with 115 touched experts
NCU_TRAFFIC_C2_115 = 1223.3e6 + 6.7e6
SEEDS = (7, 8, 9)
METRIC = "moe_step_weight_stream_bandwidth"
UNIT = "GB/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class NvmlSampler:
    """Reads SM clock and clock-event reasons of one GPU through NVML from a thread of this process
    every few milliseconds (read-only queries).  Same interface as ClockSampler, which it falls back
    to when NVML cannot be loaded: nvidia-smi needs a good part of a second before its first sample,
    more than a short timed region lasts."""
    REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"), (0x40, "hw_thermal_slowdown"))

    def __init__(self, index: int):
        self.index = index
        self.fallback = None
        self.samples: list[tuple[int, int]] = []
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:      # noqa: BLE001 - older torch / NVML: fall back to the ordinal
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml, self.handle = pynvml, handle
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:          # noqa: BLE001
            self.nvml = None
            self.fallback = ClockSampler(index)

    def start(self):
        if self.fallback is not None:
            return self.fallback.start()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except AttributeError:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((int(mhz), int(mask)))
            except Exception:      # noqa: BLE001
                pass
            time.sleep(0.003)

    def mark(self):
        """Samples taken before this call are dropped (call when the timed region starts)."""
        self.samples.clear()

    def stop(self) -> dict:
        if self.fallback is not None:
            return self.fallback.stop()
        self.stop_flag.set()
        self.thread.join(timeout=2)
        sm = [m for m, _ in self.samples]
        reasons = sorted({name for _, mask in self.samples for bit, name in self.REASONS if mask & bit})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(sm), "reasons": reasons}


def _touched(ids: np.ndarray, lo: int, cnt: int) -> int:
    u = np.unique(ids)
    return int(((u >= lo) & (u < lo + cnt)).sum())


# --------------------------------------------------------------------------------------- CPU arm
def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (its eager dequantise-then-matmul, restated in
    oracle/) on the host cores.  Each step times a bounded sample of the step's touched experts and
    scales the time to all of them; rank 0 alone works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from okc_muse_kernels_b200 import synth
    from oracle import moe_torch
    wl = synth.WORKLOADS[args.workload or ("c2" if args.gpus == 1 else "c4")]
    tokens = args.tokens or wl.tokens
    n_sample = 4
    torch.set_num_threads(os.cpu_count() or 1)
    keys = ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")
    cache: dict = {}
    per_step, step_bytes = [], []
    for i in range(args.warmup + args.steps):
        hidden, logits = synth.make_inputs(wl, seed=SEEDS[i % len(SEEDS)], device="cpu", tokens=tokens)
        ids, w = moe_torch.route_softmax_topk(logits, wl.top_k)
        touched = sorted(int(e) for e in torch.unique(ids).tolist())
        sample = touched[:n_sample]
        for e in sample:      # only the sampled experts' weights are generated
            if e not in cache:
                cache[e] = synth.make_weights(wl, device="cpu", n_experts=1, first_expert=e)
        wn = {k: _IndexByExpert({e: cache[e][k][0] for e in sample}, wl.n_experts) for k in keys}
        t0 = time.perf_counter()
        moe_torch.experts(hidden, ids, w, wn, only_experts=set(sample))
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            per_step.append(dt * len(touched) / len(sample))
            step_bytes.append(synth.algorithmic_bytes(wl, len(touched), tokens, shared=False))
    ms = 1e3 * statistics.mean(per_step)
    gbs = statistics.mean(step_bytes) / (ms * 1e-3) / 1e9
    sample_desc = (f"{n_sample} of the step's touched experts per step (dequantise + 2 FP32 matmuls each, torch CPU ops), "
                   "time scaled to all touched experts")
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "us_per_step": 1e3 * ms, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": _workload_name(wl, tokens, args.gpus)},
            "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": sample_desc},
            "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


class _IndexByExpert:
    """weights[key][e] for a sparse set of experts, with the leading dimension the oracle asks for."""

    def __init__(self, by_expert: dict, n_experts: int):
        self.by_expert = by_expert
        first = next(iter(by_expert.values()))
        self.shape = (n_experts,) + tuple(np.shape(first))

    def __getitem__(self, e):
        return self.by_expert[int(e)]


def _workload_name(wl, tokens, gpus):
    s = (f"{wl.name}: T={tokens} H={wl.hidden} I={wl.inter} E={wl.n_experts} top-{wl.top_k} NVFP4 W4A16 MoE decode step"
         + (f" + shared expert I={wl.shared_inter}" if wl.shared_inter else ""))
    if gpus > 1:
        s += f", expert-parallel over {gpus} GPUs (all-gather + reduce-scatter)"
    return s


# --------------------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    import okc_muse_kernels_b200 as okc
    from okc_muse_kernels_b200 import _lib, ep, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    wl = synth.WORKLOADS[args.workload or ("c2" if world == 1 else "c4")]
    tokens = args.tokens or wl.tokens
    peak_gbs, peak_kind = _peaks()

    # ---- state
    if world == 1:
        plan = okc.MoEPlan(hidden=wl.hidden, inter=wl.inter, n_experts=wl.n_experts, top_k=wl.top_k,
                           shared_inter=wl.shared_inter, max_tokens=max(tokens, 16))
        weights = synth.make_weights(wl, device=dev)
        state = okc.prepare(weights, plan)
        layer = None
    else:
        plan = ep.shard_plan(wl.hidden, wl.inter, wl.n_experts, wl.top_k, world, rank, max_tokens=max(tokens, 16),
                             shared_inter=wl.shared_inter)
        weights = synth.make_weights(wl, device=dev, n_experts=plan.local_count, first_expert=plan.local_start)
        # the exchange steps over peer memory with this library's kernels; NCCL collectives if the
        # ranks' buffers cannot be mapped into each other (every rank takes the same branch)
        layer = None
        if args.exchange == "peer":
            try:
                layer = ep.ExpertParallelMoE(plan, tokens, weights=weights, exchange="peer")
            except Exception as exc:      # noqa: BLE001
                print(f"rank {rank}: peer-memory exchange unavailable ({exc}); using NCCL collectives", file=sys.stderr)
        if layer is None:
            layer = ep.ExpertParallelMoE(plan, tokens, weights=weights, exchange="nccl")
        state = layer.state
    del weights
    torch.cuda.empty_cache()

    inputs = [synth.make_inputs(wl, seed=s, device=dev, tokens=tokens) for s in SEEDS]
    t0, t1 = ep.token_block(tokens, world, rank) if world > 1 else (0, tokens)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flush.zero_()
    flush_sink = torch.zeros(1, dtype=torch.int64, device=dev)

    def flush_l2():
        # read (not write) a buffer larger than L2 so no dirty lines are left behind
        flush_sink.add_(flush.view(torch.int64)[::64].sum())

    # --route-from-hidden (N = 1): the router logits are computed from the token rows inside the step
    # (okc.moe_layer_step: hidden . router_w^T in FP32, then softmax top-k) instead of being an input
    router_w = None
    if args.route_from_hidden:
        if world > 1:
            raise SystemExit("--route-from-hidden is a single-GPU option")
        gr = torch.Generator(device=dev).manual_seed(4242)
        router_w = torch.randn((wl.n_experts, wl.hidden), generator=gr, device=dev) * (wl.hidden ** -0.5)

    def one_step(h, lg, o):
        if router_w is not None:
            return okc.moe_layer_step(h, router_w, state, out=o)
        return okc.moe_step(h, lg, state, out=o)

    def do_route(h, lg):
        if router_w is not None:
            return okc.route_hidden(h, router_w, state)
        return okc.route(lg, state, own_tokens=(t0, t1))

    # ---- the step: graph replay at N = 1, eager collectives + kernels at N > 1
    outs = [torch.empty((tokens, wl.hidden), dtype=torch.bfloat16, device=dev) for _ in SEEDS]
    graphs = []
    if world == 1:
        for (h, lg), o in zip(inputs, outs):
            one_step(h, lg, o)                     # eager warm-up (sets kernel attributes)
        torch.cuda.synchronize()
        for (h, lg), o in zip(inputs, outs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step(h, lg, o)
            graphs.append(g)

    exch = "" if world == 1 else ("peer-memory exchange kernels" if layer.exchange == "peer" else "NCCL collectives")
    ep_timing = f"eager launches + {exch} per step"
    if world > 1:
        # the expert-parallel step (two all-gathers, five kernels, a reduce-scatter, a cast) as one CUDA
        # graph per routing seed: at 8 ranks a rank's kernels take about as long as the host needs to
        # launch them one by one.  Every rank captures; if capture is refused the step stays eager.
        own = [(h[t0:t1].contiguous(), lg[t0:t1].contiguous()) for h, lg in inputs]
        for ho, lo in own:
            layer.step(ho, lo)
        torch.cuda.synchronize()
        dist.barrier()
        try:
            if not args.ep_graphs:
                raise RuntimeError("not requested")
            for ho, lo in own:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    layer.step(ho, lo)
                graphs.append(g)
            ep_timing = f"CUDA-graph replay per step (kernels + {exch} captured)"
        except Exception as exc:      # noqa: BLE001 - any capture failure means: run eagerly
            graphs = []
            if args.ep_graphs:
                print(f"rank {rank}: graph capture of the expert-parallel step failed ({exc}); running eagerly", file=sys.stderr)
        ok_flag = torch.tensor([1 if graphs else 0], device=dev)
        dist.all_reduce(ok_flag, op=dist.ReduceOp.MIN)
        if int(ok_flag.item()) == 0:
            graphs = []
            ep_timing = f"eager launches + {exch} per step"

    def step(i):
        j = i % len(SEEDS)
        if graphs:
            graphs[j].replay()
        else:
            h, lg = inputs[j]
            layer.step(h[t0:t1], lg[t0:t1])

    # touched experts per seed (this rank), for the algorithmic bytes
    touched = []
    for h, lg in inputs:
        ids, _ = do_route(h, lg)
        touched.append(_touched(ids.cpu().numpy(), plan.local_start, plan.local_count))
    bytes_per_seed = [synth.algorithmic_bytes(wl, n, tokens if world == 1 else tokens, shared=bool(wl.shared_inter))
                      for n in touched]

    # ---- roofline of the dominant kernel (the grouped-GEMM launch): CUDA events around each kernel of the
    # expert phase, taken before the timed region (right after a long back-to-back run the same kernels
    # were measured up to 5 % slower between their events than they run inside the replayed step)
    phases = {"gather": [], "gemm": [], "combine": [], "total": []}
    prof_out = torch.empty((tokens, wl.hidden), dtype=torch.float32 if world > 1 else torch.bfloat16, device=dev)
    n_prof = 15
    gate_up_bytes = []
    for i in range(n_prof + 2):
        j = i % len(SEEDS)
        h, lg = inputs[j]
        do_route(h, lg)
        flush_l2()
        torch.cuda.synchronize()
        ms = okc.experts_profiled(h, state, prof_out)
        if i >= 2:
            for k in phases:
                phases[k].append(ms[k])
            n_exp = touched[j] + (1 if wl.shared_inter else 0)
            # weight stream of both GEMMs (4 bits + 1/16 scale byte per element) + the gathered token rows
            gate_up_bytes.append(n_exp * 3 * wl.inter * wl.hidden * 9 // 16 + tokens * wl.top_k * wl.hidden * 2)

    # the clock sampler starts before the warm-up; samples from before the timed region are dropped
    # when NVML is read in-process (the nvidia-smi fallback keeps them: it is slow to start, and they
    # too were taken under this workload)
    sampler = NvmlSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    if rank == 0 and sampler.fallback is None:
        sampler.mark()
    for i in range(args.steps):
        flush_l2()
        ev[i][0].record()
        step(i)
        ev[i][1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    times_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = sum(times_ms)
    step_bytes = sum(bytes_per_seed[i % len(SEEDS)] for i in range(args.steps))
    rc, detail = okc.read_status(state)
    if rc != 0:
        raise SystemExit(f"device status {rc} detail {detail:#x}")
    if world > 1 and layer.peer is not None:
        rc, detail = layer.peer.read_status()
        if rc != 0:
            raise SystemExit(f"rank {rank}: exchange status {rc} detail {detail:#x}")

    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        b = torch.tensor([float(step_bytes)], dtype=torch.float64, device=dev)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
        step_bytes = float(b.item())
    ms_per_step = total_ms / args.steps
    value = step_bytes / (total_ms * 1e-3) / 1e9

    # ---- roofline figures from the per-kernel events taken before the timed region
    roof = None
    gu_ms = statistics.median(phases["gemm"])
    achieved = statistics.mean(gate_up_bytes) / (gu_ms * 1e-3) / 1e9
    # DRAM traffic of one launch from the ncu capture summarised under profiles/
    # (dram__bytes_read.sum + dram__bytes_write.sum at 115 touched experts of configuration 2),
    # scaled to this run's touched experts: the traffic is the weight stream, which grows in proportion
    traffic = None
    if wl.name == "c2":
        traffic = NCU_TRAFFIC_C2_115 / 115.0 * statistics.mean(touched)
    roof = {"kernel": "okc_moe_gemm (gate_up + SiLU*mul units, then down units, one launch)", "bound": "hbm", "achieved": achieved, "peak": peak_gbs,
            "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak_gbs, "traffic": traffic,
            "kernel_ms": {k: statistics.median(v) for k, v in phases.items()},
            "step_frac_of_peak": value / (peak_gbs * world)}


    # ---- end to end through the public API with host buffers
    e2e = None
    if router_w is None:      # (the end-to-end leg is the step with logits as a host input)
        # okc.HostStep: pinned host inputs -> device, the step, result -> pinned host memory, captured
        # once per routing seed in a CUDA graph (one launch per step); the host waits for every step
        host_out = torch.empty((t1 - t0, wl.hidden), dtype=torch.bfloat16).pin_memory()
        host_steps = []
        for h, lg in inputs:
            hh, ll = h[t0:t1].cpu().pin_memory(), lg[t0:t1].cpu().pin_memory()
            host_steps.append(okc.HostStep(state, hh, ll, host_out, step=None if world == 1 else layer.step))
            if world > 1:
                dist.barrier()       # every rank has captured this seed's step before the next capture's eager run

        def e2e_step(i):
            host_steps[i % len(SEEDS)].replay()
            torch.cuda.current_stream().synchronize()

        for i in range(max(3, args.warmup)):
            e2e_step(i)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            e2e_step(i)
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        e2e = {"value": step_bytes / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms / args.steps,
               "h2d_bytes_per_step": (t1 - t0) * wl.hidden * 2 + (t1 - t0) * wl.n_experts * 4,
               "d2h_bytes_per_step": (t1 - t0) * wl.hidden * 2}

    # ---- CPU baseline (rank 0, N = 1 only): the oracle on a bounded sample of the same step
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        torch.set_num_threads(os.cpu_count() or 1)
        h, lg = inputs[0]
        n_sample = 8
        from oracle import moe_torch
        hc, lc = h.cpu(), lg.cpu()
        ids_o, w_o = moe_torch.route_softmax_topk(lc, wl.top_k)
        sample = sorted(int(e) for e in torch.unique(ids_o).tolist())[:n_sample]
        keys = ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")
        sub = {e: {k: v.cpu() for k, v in synth.make_weights(wl, device=dev, n_experts=1, first_expert=e).items()}
               for e in sample}
        wn = {k: _IndexByExpert({e: sub[e][k][0] for e in sample}, wl.n_experts) for k in keys}
        moe_torch.experts(hc, ids_o, w_o, wn, only_experts={sample[0]})          # warm-up
        c0 = time.perf_counter()
        moe_torch.experts(hc, ids_o, w_o, wn, only_experts=set(sample))
        dt = time.perf_counter() - c0
        full_s = dt * touched[0] / len(sample)
        cpu = {"value": bytes_per_seed[0] / full_s / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
               "seconds_per_step": full_s,
               "sample": f"{len(sample)} of {touched[0]} touched experts of one step (torch CPU dequantise + 2 FP32 matmuls each), scaled to the step"}

    # kernels of this library per step beyond the single-GPU step's: the token push and, unless the
    # combine is fused with the reduce-scatter, the pull-reduce (peer exchange); the cast (NCCL exchange)
    ep_extra_launches = 0
    if world > 1:
        ep_extra_launches = (1 if layer.fuse_combine else 2) if layer.exchange == "peer" else 1
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "us_per_step": 1e3 * ms_per_step, "higher_is_better": True,
                "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": _workload_name(wl, tokens, world),
                           "l2": "touched weights per step exceed L2 (126 MB) and a 256 MB buffer is read between timed steps",
                           "timing": "CUDA-graph replay per step" if world == 1 else ep_timing,
                           "router": "logits = hidden . router_w^T computed inside the step" if router_w is not None else "logits given",
                           "touched_experts_per_seed": touched, "routing_seeds": list(SEEDS)},
                "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
                "gpu_launches": (_lib.lib().okc_moe_launches_per_step() + ep_extra_launches) * args.steps,
                "step_ms_median": statistics.median(times_ms), "step_ms_min": min(times_ms)}
        print(json.dumps(line), flush=True)
    if world > 1:
        captured = True      # the end-to-end leg always captures the step (okc.HostStep)
        graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        if captured:
            # tearing down a communicator whose collectives were captured in CUDA graphs was seen to
            # block; every rank is past its last collective here, so leave without the teardown
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "c1", "c2", "c4", "c5"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--route-from-hidden", action="store_true",
                    help="N = 1: compute the router logits from the token rows inside the step (okc.moe_layer_step)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the all-gather / reduce-scatter through this library's peer-memory kernels or NCCL")
    ap.add_argument("--ep-graphs", type=int, default=1, choices=[0, 1],
                    help="N > 1: capture the expert-parallel step (kernels + NCCL collectives) in CUDA graphs")
    args = ap.parse_args()
    # a run that stops making progress prints every thread's stack and exits instead of hanging
    faulthandler.dump_traceback_later(int(os.environ.get("OKC_BENCH_WATCHDOG_S", "900")), exit=True)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
