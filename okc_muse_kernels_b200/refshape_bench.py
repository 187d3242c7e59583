"""Times ``kernel_fn`` on the reference's own problem shape, the way its harness does.

    python -m okc_muse_kernels_b200.refshape_bench [--steps K] [--warmup W]

The shape of muse_moe_w4a16 (reference.py:18-24): H = I = 4096, a shard of 32 local experts of 256, top-8
routing given as ids and weights, post-expert RMSNorm; batch sizes 1, 8, 16, 32, 128 and 256 (the six loads
of muse_moe_w4a16/bench.py:18-19).  Weights have the distribution of the reference's generator
(``synth.make_reference_style_weights``), ids are uniform over the 256 experts with distinct picks per token,
so about an eighth of a token's routes is local, as in the reference's inputs (reference.py:53-70).

Per batch size: ``prepare`` once, then ``kernel_fn`` captured in a CUDA graph (three input sets), replayed with
256 MB read between replays, CUDA events around each replay.  Prints one JSON line: per batch size the median
microseconds per call, the touched local experts and the touched bytes / time against the measured copy
bandwidth.  Parity of this shape against the oracle is the business of tests/test_gpu_parity.py; here every
output is only checked to be finite and the device status to be clean.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

import okc_muse_kernels_b200 as okc
from okc_muse_kernels_b200 import synth

HIDDEN, INTER, N_EXPERTS, LOCAL, TOP_K = 4096, 4096, 256, 32, 8
BATCHES = (1, 8, 16, 32, 128, 256)
SEEDS = (7, 11, 13)


def _peak_gbs() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "of measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "of fallback"


def _inputs(T: int, seed: int, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    hidden = torch.randn((T, HIDDEN), generator=g, device=dev).to(torch.bfloat16)
    scores = torch.rand((T, N_EXPERTS), generator=g, device=dev)
    ids = scores.topk(TOP_K, dim=1).indices.to(torch.int32)
    wts = torch.softmax(torch.randn((T, TOP_K), generator=g, device=dev), dim=1)
    return {"hidden_states": hidden, "topk_ids": ids, "topk_weights": wts.float()}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("refshape_bench needs a GPU")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peak, peak_kind = _peak_gbs()
    weights = synth.make_reference_style_weights(LOCAL, HIDDEN, INTER, seed=2024, device=dev)
    plan = okc.MoEPlan(hidden=HIDDEN, inter=INTER, n_experts=N_EXPERTS, top_k=TOP_K, local_start=0, local_count=LOCAL,
                       max_tokens=max(BATCHES), post_norm=True)
    state = okc.prepare(weights, plan)
    del weights
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    per_expert = 3 * INTER * HIDDEN * 9 // 16
    rows = []
    for T in BATCHES:
        data = [_inputs(T, s, dev) for s in SEEDS]
        touched = [int(torch.unique(d["topk_ids"][d["topk_ids"] < LOCAL]).numel()) for d in data]
        graphs, outs = [], []
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for d in data:
                okc.kernel_fn(d, state)
            stream.synchronize()
            for d in data:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    outs.append(okc.kernel_fn(d, state))
                graphs.append(g)
            times = []
            for i in range(args.warmup + args.steps):
                sink.add_(flush.view(torch.int64)[::64].sum())
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                graphs[i % len(graphs)].replay()
                e1.record(stream)
                stream.synchronize()
                if i >= args.warmup:
                    times.append(e0.elapsed_time(e1) * 1e3)
        rc, detail = okc.read_status(state)
        if rc != 0:
            raise SystemExit(f"device status {rc} detail {detail:#x} at batch {T}")
        if not all(bool(torch.isfinite(o.float()).all()) for o in outs):
            raise SystemExit(f"non-finite output at batch {T}")
        times.sort()
        us = times[len(times) // 2]
        mean_bytes = sum(touched) / len(touched) * per_expert
        rows.append({"batch": T, "us": round(us, 2), "touched_local_experts": touched,
                     "gbs": round(mean_bytes / us / 1e3, 1), "frac_of_peak": round(mean_bytes / us / 1e3 / peak, 3)})
    print(json.dumps({"shape": {"hidden": HIDDEN, "inter": INTER, "n_experts": N_EXPERTS, "local_experts": LOCAL,
                                "top_k": TOP_K, "post_norm": True},
                      "timing": "CUDA-graph replay of kernel_fn, 256 MB read between replays, CUDA events, median",
                      "peak_gbs": peak, "peak_kind": peak_kind, "steps": args.steps, "rows": rows}))


if __name__ == "__main__":
    main()
