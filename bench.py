"""Benchmark of the NVFP4 W4A16 MoE decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c1|c4|c5] [--tokens T]
    python bench.py --sweep            # configuration 3: one line per batch size T = 1 ... 256
    python bench.py --route-from-hidden [fma|mma]   # the router logits computed from the token rows inside the step

N = 1: configuration 2 (T=32, H=4096, I=1536, E=128, top-8, all experts on the GPU); the line also
carries `c4_n1`, configuration 4 on this one GPU, as the anchor of the 1 -> 8 GPU curve.
N > 1 (launched by torch.distributed.run, one rank per GPU): configuration 4 (T=128, H=7168, I=2048,
E=256 sharded contiguously + a replicated shared expert), all-gather -> local experts -> reduce-scatter.
Every run compares the output of one step with the CPU oracle on a token subset (`parity`) and exits
non-zero when that fails.

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


def _workload_name(wl, tokens, gpus):
    s = (f"{wl.name}: T={tokens} H={wl.hidden} I={wl.inter} E={wl.n_experts} top-{wl.top_k} NVFP4 W4A16 MoE decode step"
         + (f" + shared expert I={wl.shared_inter}" if wl.shared_inter else ""))
    if gpus > 1:
        s += f", expert-parallel over {gpus} GPUs (all-gather + reduce-scatter)"
    return s


def _config(wl, tokens, gpus):
    """The same dictionary in both arms (the driver compares them)."""
    return {"workload": _workload_name(wl, tokens, gpus),
            "l2": "a 256 MB buffer is read between timed steps (cold L2); the touched weights of a step also exceed the "
                  "126 MB L2 in every configuration but c1",
            "routing_seeds": list(SEEDS)}


class _IndexByExpert:
    """weights[key][e] for a sparse set of experts, with the leading dimension the oracle asks for."""

    def __init__(self, by_expert: dict, key: str, n_experts: int):
        self.by_expert, self.key = by_expert, key
        first = next(iter(by_expert.values()))[key]
        self.shape = (n_experts,) + tuple(first.shape)

    def __getitem__(self, e):
        return self.by_expert[int(e)][self.key]


_KEYS = ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")


def _cpu_expert(wl, e, device):
    """One expert's NVFP4 tensors on the CPU (generated on `device` from the expert's own seed)."""
    from okc_muse_kernels_b200 import synth
    one = synth.make_weights(wl, device=device, n_experts=1, first_expert=int(e))
    return {k: one[k][0].cpu() for k in _KEYS}


def _cpu_shared(wl, device):
    from okc_muse_kernels_b200 import synth
    one = synth.make_weights(wl, device=device, n_experts=0)
    return {k[len("shared_"):]: v.cpu() for k, v in one.items() if k.startswith("shared_")}


# --------------------------------------------------------------------------------------- CPU arm
def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (its eager dequantise-then-matmul, restated in
    oracle/moe_torch.py with the torch operators the reference uses) on all host cores, on this arm's
    workload.  A step times every touched expert of the step when the run's time budget allows
    (`sampled_fraction` 1.0: configuration 2); otherwise as many whole experts as fit, the time scaled
    to all touched experts and `sampled_fraction` says how much was timed.  Rank 0 alone works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from okc_muse_kernels_b200 import synth
    from oracle import moe_torch
    wl = synth.WORKLOADS[args.workload or ("c2" if args.gpus == 1 else "c4")]
    tokens = args.tokens or wl.tokens
    torch.set_num_threads(os.cpu_count() or 1)
    budget_s = float(os.environ.get("OKC_REF_BUDGET_S", "150"))
    n_steps = args.warmup + args.steps
    cache: dict = {}

    def expert(e):
        if e not in cache:
            cache[e] = _cpu_expert(wl, e, "cpu")
        return cache[e]

    shared = _cpu_shared(wl, "cpu") if wl.shared_inter else None
    # calibration: one expert, twice (the first call warms the thread pool up)
    hidden, logits = synth.make_inputs(wl, seed=SEEDS[0], device="cpu", tokens=tokens)
    ids, w = moe_torch.route_softmax_topk(logits, wl.top_k)
    e0 = int(ids[0, 0])
    wn = {k: _IndexByExpert({e0: expert(e0)}, k, wl.n_experts) for k in _KEYS}
    moe_torch.experts(hidden, ids, w, wn, only_experts={e0})
    c0 = time.perf_counter()
    moe_torch.experts(hidden, ids, w, wn, only_experts={e0})
    t_expert = time.perf_counter() - c0
    per_step = max(1, int(budget_s / max(n_steps, 1) / max(t_expert, 1e-6)))

    per_step_s, step_bytes, fractions, wall = [], [], [], 0.0
    for i in range(n_steps):
        hidden, logits = synth.make_inputs(wl, seed=SEEDS[i % len(SEEDS)], device="cpu", tokens=tokens)
        ids, w = moe_torch.route_softmax_topk(logits, wl.top_k)
        touched = sorted(int(e) for e in torch.unique(ids).tolist())
        units = len(touched) + (1 if shared is not None else 0)
        sample = touched[:per_step]
        with_shared = shared is not None and len(sample) == len(touched)
        by = {e: expert(e) for e in sample}                     # generated outside the timed region
        wn = {k: _IndexByExpert(by, k, wl.n_experts) for k in _KEYS}
        t0 = time.perf_counter()
        acc = moe_torch.experts(hidden, ids, w, wn, only_experts=set(sample))
        if with_shared:
            acc = acc + moe_torch.shared_expert(hidden, shared)
        acc.to(torch.bfloat16)
        dt = time.perf_counter() - t0
        timed = len(sample) + (1 if with_shared else 0)
        if i >= args.warmup:
            wall += dt
            per_step_s.append(dt * units / timed)
            fractions.append(timed / units)
            step_bytes.append(synth.algorithmic_bytes(wl, len(touched), tokens, shared=shared is not None))
    ms = 1e3 * statistics.mean(per_step_s)
    gbs = statistics.mean(step_bytes) / (ms * 1e-3) / 1e9
    frac = statistics.mean(fractions)
    sample_desc = ("every touched expert of every step (dequantise + 2 FP32 matmuls each, torch CPU operators)" if frac == 1.0 else
                   f"{per_step} of the step's touched experts per step (dequantise + 2 FP32 matmuls each, torch CPU operators), "
                   "time scaled to all touched experts")
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms if frac == 1.0 else 1e3 * wall / args.steps,
            "ms_per_step_whole_workload": ms, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": _config(wl, tokens, args.gpus), "sampled_fraction": frac,
            "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": sample_desc},
            "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU arm
def _parity(wl, hidden, logits, out_rows, row0, ids_gpu, dev, n_tokens):
    """Output rows [row0, row0 + len(out_rows)) of one step against the CPU oracle (the torch statement
    of the reference's eager path) on a token subset, and the routing ids of every token against the
    oracle's stable top-k.  Tolerances of this path: ids bit-exact, rel-L2 <= 1e-2, and max-abs <= 2e-2
    beyond the rounding of the output format itself (at most half a bf16 ulp of the reference value, 2^-8 |ref|:
    a layer output of magnitude 8 or more, as configuration 4's, cannot be written in bf16 within 2e-2
    at all)."""
    import torch
    from oracle import moe_np, moe_torch
    ids_ref, wts_ref = moe_np.route_softmax_topk(logits.cpu().numpy(), wl.top_k)
    ids_exact = bool(np.array_equal(ids_gpu.cpu().numpy(), ids_ref))
    n = out_rows.shape[0]
    pick = sorted({0, n - 1, n // 2, n // 3})[:n_tokens]
    sub = [row0 + i for i in pick]
    by = {int(e): _cpu_expert(wl, e, dev) for e in np.unique(ids_ref[sub])}
    wn = {k: _IndexByExpert(by, k, wl.n_experts) for k in _KEYS}
    h_sub = hidden.cpu()[sub]
    ref = moe_torch.experts(h_sub, torch.from_numpy(ids_ref[sub]).long(), torch.from_numpy(wts_ref[sub]), wn)
    if wl.shared_inter:
        ref = ref + moe_torch.shared_expert(h_sub, _cpu_shared(wl, dev))
    ref = ref.double().numpy()
    got = out_rows[pick].float().cpu().double().numpy()
    max_abs = float(np.abs(got - ref).max())
    beyond = float((np.abs(got - ref) - np.abs(ref) * 2.0 ** -8).max())
    rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-12))
    ok = ids_exact and bool(np.isfinite(got).all()) and beyond <= 2e-2 and rel <= 1e-2
    return {"ok": ok, "ids_exact": ids_exact, "max_abs": max_abs, "max_abs_beyond_bf16_rounding": max(beyond, 0.0),
            "max_ref": float(np.abs(ref).max()), "rel_l2": rel, "tokens": len(sub)}


def measure(wl, tokens, args, dev, world, rank, *, state=None, layer=None, with_e2e=True, with_parity=True,
            with_clocks=True, steps=None, max_tokens=None):
    """Builds the workload on this rank (unless `state` is given), times `steps` steps and returns the
    figures of the JSON line as a dictionary (on every rank)."""
    import torch
    import torch.distributed as dist

    import okc_muse_kernels_b200 as okc
    from okc_muse_kernels_b200 import ep, synth

    steps = steps or args.steps
    peak_gbs, peak_kind = _peaks()
    local_rank = dev.index
    max_tokens = max(max_tokens or tokens, 16)
    if state is None:
        if world == 1:
            plan = okc.MoEPlan(hidden=wl.hidden, inter=wl.inter, n_experts=wl.n_experts, top_k=wl.top_k,
                               shared_inter=wl.shared_inter, max_tokens=max_tokens)
            weights = synth.make_weights(wl, device=dev)
            state = okc.prepare(weights, plan)
        else:
            plan = ep.shard_plan(wl.hidden, wl.inter, wl.n_experts, wl.top_k, world, rank, max_tokens=max_tokens,
                                 shared_inter=wl.shared_inter)
            weights = synth.make_weights(wl, device=dev, n_experts=plan.local_count, first_expert=plan.local_start)
            # --exchange peer: this library's kernels over peer memory.  If the ranks' buffers cannot be mapped
            # into each other the constructor raises on every rank and the run fails: a scaling record must
            # not change its data path silently.
            layer = ep.ExpertParallelMoE(plan, tokens, weights=weights, exchange=args.exchange)
            state = layer.state
        del weights
        torch.cuda.empty_cache()
    plan = state["plan"]

    inputs = [synth.make_inputs(wl, seed=s, device=dev, tokens=tokens) for s in SEEDS]
    t0, t1 = ep.token_block(tokens, world, rank) if world > 1 else (0, tokens)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flush.zero_()
    flush_sink = torch.zeros(1, dtype=torch.int64, device=dev)

    def flush_l2():
        # read (not write) a buffer larger than L2 so no dirty lines are left behind
        flush_sink.add_(flush.view(torch.int64)[::64].sum())

    # --route-from-hidden (N = 1): the router logits are computed from the token rows inside the step
    router_w = None
    if args.route_from_hidden:
        if world > 1:
            raise SystemExit("--route-from-hidden is a single-GPU option")
        gr = torch.Generator(device=dev).manual_seed(4242)
        router_w = torch.randn((wl.n_experts, wl.hidden), generator=gr, device=dev) * (wl.hidden ** -0.5)
        if args.route_from_hidden == "mma":      # bf16 hi + lo rows: the logits on the tensor cores
            router_w = okc.split_router(router_w)

    def one_step(h, lg, o):
        if router_w is not None:
            return okc.moe_layer_step(h, router_w, state, out=o)
        return okc.moe_step(h, lg, state, out=o)

    def do_route(h, lg):
        if router_w is not None:
            return okc.route_hidden(h, router_w, state)
        return okc.route(lg, state, own_tokens=(t0, t1))

    # ---- the step as a CUDA graph per routing seed
    outs = [torch.empty((tokens, wl.hidden), dtype=torch.bfloat16, device=dev) for _ in SEEDS]
    graphs = []
    exch = "" if world == 1 else ("peer-memory exchange kernels" if layer.exchange == "peer" else "NCCL collectives")
    timing = "CUDA-graph replay per step"
    if world == 1:
        for (h, lg), o in zip(inputs, outs):
            one_step(h, lg, o)                     # eager warm-up (sets kernel attributes)
        torch.cuda.synchronize()
        for (h, lg), o in zip(inputs, outs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                one_step(h, lg, o)
            graphs.append(g)
    else:
        own = [(h[t0:t1].contiguous(), lg[t0:t1].contiguous()) for h, lg in inputs]
        for ho, lo in own:
            layer.step(ho, lo)
        torch.cuda.synchronize()
        dist.barrier()
        if args.ep_graphs:
            for ho, lo in own:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    layer.step(ho, lo)
                graphs.append(g)
            timing = f"CUDA-graph replay per step (kernels + {exch} captured)"
        else:
            timing = f"eager launches + {exch} per step"

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
    bytes_per_seed = [synth.algorithmic_bytes(wl, n, tokens, shared=bool(wl.shared_inter)) for n in touched]

    # ---- roofline of the dominant kernel (the grouped-GEMM launch): CUDA events around each kernel of the
    # expert phase, taken before the timed region
    phases = {"gather": [], "gemm": [], "combine": [], "total": []}
    prof_out = torch.empty((tokens, wl.hidden), dtype=torch.float32 if world > 1 else torch.bfloat16, device=dev)
    gemm_bytes = []
    for i in range(15 + 2):
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
            gemm_bytes.append(n_exp * 3 * wl.inter * wl.hidden * 9 // 16 + tokens * wl.top_k * wl.hidden * 2)

    sampler = NvmlSampler(local_rank) if (with_clocks and rank == 0) else None
    if sampler is not None:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    if sampler is not None and sampler.fallback is None:
        sampler.mark()
    for i in range(steps):
        flush_l2()
        ev[i][0].record()
        step(i)
        ev[i][1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler is not None else None
    times_ms = [a.elapsed_time(b) for a, b in ev]
    my_ms = sum(times_ms)
    my_bytes = sum(bytes_per_seed[i % len(SEEDS)] for i in range(steps))
    rc, detail = okc.read_status(state)
    if rc != 0:
        raise SystemExit(f"rank {rank}: device status {rc} detail {detail:#x}")
    if world > 1 and layer.peer is not None:
        rc, detail = layer.peer.read_status()
        if rc != 0:
            raise SystemExit(f"rank {rank}: exchange status {rc} detail {detail:#x}")

    total_ms, step_bytes, per_rank = my_ms, float(my_bytes), None
    if world > 1:
        t = torch.tensor([my_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        b = torch.tensor([float(my_bytes)], dtype=torch.float64, device=dev)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
        step_bytes = float(b.item())
        mine = {"rank": rank, "touched_experts": touched, "bytes_per_step": my_bytes / steps, "step_ms": my_ms / steps,
                "gemm_ms": statistics.median(phases["gemm"])}
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine)
    ms_per_step = total_ms / steps
    value = step_bytes / (total_ms * 1e-3) / 1e9

    gemm_ms = statistics.median(phases["gemm"])
    achieved = statistics.mean(gemm_bytes) / (gemm_ms * 1e-3) / 1e9
    roof = {"kernel": "okc_moe_gemm (gate_up + SiLU*mul units, then down units, one launch)", "bound": "hbm",
            "achieved": achieved, "peak": peak_gbs, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
            "frac": achieved / peak_gbs, "traffic": None,
            "traffic_source": "not captured in this run; the ncu capture of this kernel (dram__bytes_read.sum + "
                              "dram__bytes_write.sum against the algorithmic bytes) is summarised in profiles/moe_gemm_c2.md",
            "kernel_ms": {k: statistics.median(v) for k, v in phases.items()},
            "step_frac_of_peak": value / (peak_gbs * world)}

    # ---- end to end through the public API with host buffers
    e2e = None
    if with_e2e and router_w is None:
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
        for i in range(steps):
            e2e_step(i)
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([e_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        e2e = {"value": step_bytes / (e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e_ms / steps,
               "h2d_bytes_per_step": (t1 - t0) * wl.hidden * 2 + (t1 - t0) * wl.n_experts * 4,
               "d2h_bytes_per_step": (t1 - t0) * wl.hidden * 2}
        del host_steps

    # ---- parity of one step (outside every timed region): this rank's output rows against the oracle
    parity = None
    if with_parity and router_w is None:
        h, lg = inputs[0]
        if world == 1:
            out_rows = okc.moe_step(h, lg, state).clone()
        else:
            dist.barrier()
            out_rows = layer.step(h[t0:t1].contiguous(), lg[t0:t1].contiguous()).clone()
        torch.cuda.synchronize()
        ids_step = state["ids"][:tokens]
        if world > 1 and layer.route_in_gather:      # the router ran inside the gather kernel: its ids are in the exchange buffer
            ids_step = layer.peer.routed_views(wl.top_k)[0]
        parity = _parity(wl, h, lg, out_rows, t0, ids_step, dev, n_tokens=4 if world == 1 else 2)
        if world > 1:
            allp = [None] * world
            dist.all_gather_object(allp, parity)
            parity = {"ok": all(p["ok"] for p in allp), "ids_exact": all(p["ids_exact"] for p in allp),
                      "max_abs": max(p["max_abs"] for p in allp),
                      "max_abs_beyond_bf16_rounding": max(p["max_abs_beyond_bf16_rounding"] for p in allp),
                      "max_ref": max(p["max_ref"] for p in allp), "rel_l2": max(p["rel_l2"] for p in allp),
                      "tokens": sum(p["tokens"] for p in allp)}

    graphs.clear()
    return {"value": value, "ms_per_step": ms_per_step, "step_bytes": step_bytes, "touched": touched, "timing": timing,
            "roofline": roof, "e2e": e2e, "parity": parity, "clocks": clocks, "per_rank": per_rank, "state": state,
            "layer": layer, "times_ms": times_ms, "t0": t0, "t1": t1, "bytes_seed0": bytes_per_seed[0], "inputs0": inputs[0],
            "router": "logits = hidden . router_w^T computed inside the step" if router_w is not None else "logits given"}


def _cpu_baseline(wl, tokens, hidden, logits, step_bytes, dev):
    """The oracle (torch CPU operators, all host cores) on one whole step of the workload: every
    touched expert of routing seed 0, once after a one-expert warm-up."""
    import torch
    from oracle import moe_torch
    torch.set_num_threads(os.cpu_count() or 1)
    hc, lc = hidden.cpu(), logits.cpu()
    ids_o, w_o = moe_torch.route_softmax_topk(lc, wl.top_k)
    touched = sorted(int(e) for e in torch.unique(ids_o).tolist())
    by = {e: _cpu_expert(wl, e, dev) for e in touched}
    wn = {k: _IndexByExpert(by, k, wl.n_experts) for k in _KEYS}
    moe_torch.experts(hc, ids_o, w_o, wn, only_experts={touched[0]})          # warm-up
    c0 = time.perf_counter()
    moe_torch.experts(hc, ids_o, w_o, wn).to(torch.bfloat16)
    dt = time.perf_counter() - c0
    return {"value": step_bytes / dt / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "seconds_per_step": dt,
            "sample": f"one whole step: all {len(touched)} touched experts of routing seed {SEEDS[0]} "
                      "(torch CPU dequantise + 2 FP32 matmuls each), timed once after a warm-up"}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from okc_muse_kernels_b200 import _lib, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    wl = synth.WORKLOADS[args.workload or ("c2" if world == 1 else "c4")]
    tokens = args.tokens or wl.tokens
    m = measure(wl, tokens, args, dev, world, rank, max_tokens=max(synth.C3_TOKENS) if args.sweep else None)
    failed = m["parity"] is not None and not m["parity"]["ok"]

    extra = {}
    if world == 1 and args.workload is None and args.tokens is None and not args.no_c4_anchor and not args.sweep:
        # configuration 4 on this one GPU (all 256 experts + the shared expert local, no exchange): the
        # N = 1 point of the curve whose N = 2, 4, 8 points are the expert-parallel runs
        state = m.pop("state")
        del state
        torch.cuda.empty_cache()
        c4 = synth.WORKLOADS["c4"]
        a = measure(c4, c4.tokens, args, dev, 1, 0, with_e2e=False, with_clocks=False, steps=min(args.steps, 50))
        extra["c4_n1"] = {"workload": _workload_name(c4, c4.tokens, 1), "ms_per_step": a["ms_per_step"], "value": a["value"],
                          "unit": UNIT, "touched_experts_per_seed": a["touched"], "gemm_ms": a["roofline"]["kernel_ms"]["gemm"],
                          "frac_of_peak": a["roofline"]["step_frac_of_peak"], "parity": a["parity"]}
        failed = failed or not a["parity"]["ok"]
    # (the host-core baseline after every GPU measurement of the run: its threads keep the host busy for a while)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        h, lg = m["inputs0"]
        cpu = _cpu_baseline(wl, tokens, h, lg, m["bytes_seed0"], dev)
    if args.sweep:
        # configuration 3: the batch sweep on configuration 2's weights, one entry per T
        rows = []
        for t in synth.C3_TOKENS:
            a = measure(wl, t, args, dev, 1, 0, state=m["state"], with_e2e=False, with_clocks=False, steps=min(args.steps, 50))
            rows.append({"tokens": t, "ms_per_step": a["ms_per_step"], "value": a["value"],
                         "frac_of_peak": a["roofline"]["step_frac_of_peak"], "touched_experts_per_seed": a["touched"],
                         "gemm_ms": a["roofline"]["kernel_ms"]["gemm"], "gemm_frac": a["roofline"]["frac"], "parity": a["parity"]})
            failed = failed or not a["parity"]["ok"]
        extra["sweep"] = rows

    # kernels of this library per step.  One GPU: top-k + sort (one kernel), gather (steps of more than 8 tokens), the
    # GEMM launch, combine, + the router's logits kernel with --route-from-hidden.  Expert parallel, peer
    # exchange: push + router + sort (one kernel; or push, then top-k + sort), gather, GEMMs, combine + reduce-scatter
    # (or combine, then reduce); the NCCL exchange: the single-GPU kernels + the cast.
    layer = m["layer"]
    gather = 0 if tokens <= 8 else 1
    single = 1 + gather + 2 + (1 if args.route_from_hidden else 0)
    if world == 1:
        launches_per_step = single
    elif layer.exchange == "peer":
        launches_per_step = (1 if layer.route_in_gather else 2) + gather + 1 + (1 if layer.fuse_combine else 2)
    else:
        launches_per_step = single + 1
    if rank == 0:
        line = {"metric": METRIC, "value": m["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": m["ms_per_step"], "higher_is_better": True,
                "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": _config(wl, tokens, world),
                "detail": {"timing": m["timing"], "router": m["router"], "touched_experts_per_seed": m["touched"],
                           "us_per_step": 1e3 * m["ms_per_step"], "step_ms_median": statistics.median(m["times_ms"]),
                           "step_ms_min": min(m["times_ms"])},
                "roofline": m["roofline"], "cpu_baseline": cpu, "e2e": m["e2e"], "parity": m["parity"], "clocks": m["clocks"],
                "gpu_launches": launches_per_step * args.steps}
        if m["per_rank"] is not None:
            line["per_rank"] = m["per_rank"]
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        if layer.exchange == "nccl":
            # The graphs of this exchange hold captured NCCL kernels; destroying their communicator while
            # such graphs were alive was seen to block once, and the cause was not found.  Every rank is
            # past its last collective, so this (non-default) path leaves without the teardown.
            os._exit(1 if failed else 0)
        # default path: no collective was captured.  Tear the group down, but never wait for it for long.
        watchdog = threading.Timer(30.0, lambda: os._exit(1 if failed else 0))
        watchdog.daemon = True
        watchdog.start()
        dist.destroy_process_group()
        watchdog.cancel()
    if failed:
        raise SystemExit("parity check against the oracle failed (see the `parity` keys of the line)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "c1", "c2", "c4", "c5"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-c4-anchor", action="store_true", help="N = 1: skip the configuration-4 single-GPU step (`c4_n1`)")
    ap.add_argument("--sweep", action="store_true", help="N = 1: add configuration 3 (T = 1 ... 256) as `sweep`")
    ap.add_argument("--route-from-hidden", nargs="?", const="fma", default=None, choices=["fma", "mma"],
                    help="N = 1: compute the router logits from the token rows inside the step (okc.moe_layer_step): "
                         "FP32 multiply-adds on CUDA cores (fma) or bf16 hi + lo on the tensor cores (mma)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the all-gather / reduce-scatter through this library's peer-memory kernels or NCCL")
    ap.add_argument("--ep-graphs", type=int, default=1, choices=[0, 1],
                    help="N > 1: capture the expert-parallel step (this library's kernels, and the NCCL collectives "
                         "with --exchange nccl) in CUDA graphs")
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
