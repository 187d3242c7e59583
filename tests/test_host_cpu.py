"""CPU-side checks: the C-ABI library loads and exports every declared symbol, plan validation,
the packed layout's bit permutation, the synthetic-data quantiser against the oracle, and the
oracle's routing / sort helpers."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from okc_muse_kernels_b200 import _lib, layout, synth
from okc_muse_kernels_b200.moe import MoEPlan
from oracle import moe_np, nvfp4_np as fp4

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "okc_moe.h")).read()
    declared = set(re.findall(r"\b(okc_(?:moe|ep)_[a-z0-9_]+)\s*\(", header))
    declared -= {"okc_moe_plan", "okc_moe_sizes", "okc_moe_error", "okc_ep_comm", "okc_ep_buffer_bytes"} - set(_lib.SIGNATURES)
    assert declared, "no declarations found"
    handle = C.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} declared in include/okc_moe.h but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert _lib.lib().okc_moe_version() >= 100


def test_query_and_plan_validation():
    plan = MoEPlan(hidden=4096, inter=1536, n_experts=128, top_k=8, max_tokens=32)
    sz = plan.sizes()
    b13, b2 = layout.packed_bytes(4096, 1536)
    assert sz.packed_w13_bytes == 128 * b13 and sz.packed_w2_bytes == 128 * b2
    # lossless: same bytes as the NVFP4 tensors (4 bits per code + 1 byte per 16 codes)
    assert b13 == 2 * 1536 * 4096 * 9 // 16 and b2 == 4096 * 1536 * 9 // 16
    assert sz.expert_slots == 128 and sz.routes_per_token == 8 and sz.workspace_bytes > 0
    for bad in (dict(hidden=4000), dict(inter=100), dict(top_k=0), dict(n_experts=1024), dict(max_tokens=0),
                dict(shared_inter=512), dict(local_start=120, local_count=16)):
        kw = dict(hidden=4096, inter=1536, n_experts=128, top_k=8, max_tokens=32)
        kw.update(bad)
        s = _lib.Sizes()
        rc = _lib.lib().okc_moe_query(C.byref(MoEPlan(**kw).c_plan()), C.byref(s))
        assert rc == _lib.OKC_ERR_BAD_PLAN, bad
    assert b"wait" in _lib.lib().okc_moe_strerror(_lib.OKC_ERR_TIMEOUT)


def test_null_and_range_arguments_are_rejected_before_any_launch():
    plan = MoEPlan(hidden=1024, inter=512, n_experts=16, top_k=2, max_tokens=8)
    lib = _lib.lib()
    cp = plan.c_plan()
    assert lib.okc_moe_route(C.byref(cp), None, 4, 0, 0, None, None, None, None) == _lib.OKC_ERR_BAD_ARG
    assert lib.okc_moe_sort(C.byref(cp), None, None, 4, 0, 0, None, None) == _lib.OKC_ERR_BAD_ARG
    assert lib.okc_moe_experts(C.byref(cp), None, None, None, None, None, 1024, 4, None, None, None, 0, None) \
        == _lib.OKC_ERR_BAD_ARG
    assert lib.okc_moe_repack(C.byref(cp), None, None, None, None, 0, 1, None, None, None) == _lib.OKC_ERR_BAD_ARG
    assert lib.okc_moe_read_status(None, None, None) == _lib.OKC_ERR_BAD_ARG
    # expert-parallel exchange: sizes, and argument checks that touch no GPU
    assert lib.okc_ep_buffer_bytes(128, 7168, 256) >= 128 * 7168 * 6 + 128 * 256 * 4
    comm = _lib.EpComm(rank=2, world=2, tokens=128, hidden=7168, n_experts=256)
    assert lib.okc_ep_gather_tokens(C.byref(comm), None, 7168, None, None) == _lib.OKC_ERR_BAD_ARG   # rank >= world
    comm = _lib.EpComm(rank=0, world=2, tokens=127, hidden=7168, n_experts=256)
    assert lib.okc_ep_reduce_scatter(C.byref(comm), None, None) == _lib.OKC_ERR_BAD_ARG            # T % world
    assert lib.okc_ep_views(None, None, None, None) == _lib.OKC_ERR_BAD_ARG


def test_bit_permutation_round_trip():
    rng = np.random.default_rng(1)
    codes = rng.integers(0, 16, (4096, 16)).astype(np.uint8)
    vals = layout.regs_to_values(layout.unpack_block_regs(layout.pack_block(codes)))
    expect = np.where(codes & 8, -fp4.E2M1_GRID[codes & 7], fp4.E2M1_GRID[codes & 7])
    assert np.array_equal(vals, expect)
    assert np.array_equal(np.signbit(vals), (codes & 8) != 0)   # -0 stays -0: lossless
    assert len(set(layout.PAIR_SHIFT)) == 64


def test_cuda_bit_table_matches_layout_module():
    src = open(os.path.join(ROOT, "okc_muse_kernels_b200", "csrc", "repack.cu")).read()
    body = src[src.index("kPairShift[64] = {") + len("kPairShift[64] = {"):]
    nums = [int(x) for x in re.findall(r"\d+", body[:body.index("}")])]
    assert nums == layout.PAIR_SHIFT
    fmt = open(os.path.join(ROOT, "okc_muse_kernels_b200", "csrc", "format.cuh")).read()
    assert f"0x{layout.LEFT_MASK:08X}u" in fmt and f"0x{layout.OUT_MASK:08X}u" in fmt


def test_tile_image_layout():
    rng = np.random.default_rng(2)
    packed = rng.integers(0, 256, (128, 128)).astype(np.uint8)
    sf = rng.integers(1, 0x7F, (128, 16)).astype(np.uint8)
    img = layout.pack_tile_stage(packed, sf)
    assert img.shape == (layout.TILE_BYTES,)
    row, chunk = 37, 5
    words = img[:layout.TILE_CODE_BYTES].view(np.uint32).reshape(8, 128, 4)[chunk, row]
    vals = layout.regs_to_values(layout.unpack_block_regs(words.reshape(2, 2))).reshape(32)
    assert np.array_equal(vals, fp4.unpack_e2m1(packed[row, chunk * 16:(chunk + 1) * 16]))
    sc = img[layout.TILE_CODE_BYTES:].reshape(8, 128, 2)[chunk, row]
    assert np.array_equal(sc, layout.SCALE_CODE[sf[row, 2 * chunk:2 * chunk + 2]])


def test_torch_quantiser_matches_oracle_bit_exact():
    g = torch.Generator().manual_seed(3)
    x = torch.randn((64, 256), generator=g) * 0.02
    x[0, :16] = 0
    x[1, 3] = 0.5
    p, sf, gs = synth.quantize_nvfp4(x)
    p2, sf2, gs2 = fp4.quantize(x.numpy())
    assert np.float32(gs.item()).view(np.uint32) == np.float32(gs2).view(np.uint32)
    assert np.array_equal(sf.view(torch.uint8).numpy(), sf2)
    assert np.array_equal(p.numpy(), p2)


def test_softmax_topk_oracle_properties():
    rng = np.random.default_rng(4)
    logits = rng.standard_normal((33, 128)).astype(np.float32)
    logits[3, 10] = logits[3, 90] = logits[3].max() + 1.0       # a tie for first place
    logits[5, :] = 0.25                                          # everything ties
    ids, w = moe_np.route_softmax_topk(logits, 8)
    assert ids[3, 0] == 10 and ids[3, 1] == 90
    assert np.array_equal(ids[5], np.arange(8))
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
    # equals softmax over all experts, top-k, renormalised over the selected (tie-free rows)
    sm = np.exp(logits - logits.max(axis=1, keepdims=True))
    sm /= sm.sum(axis=1, keepdims=True)
    for t in (0, 1, 2, 7, 20):
        top = np.argsort(-sm[t], kind="stable")[:8]
        assert np.array_equal(top, ids[t])
        assert np.allclose(sm[t, top] / sm[t, top].sum(), w[t], rtol=1e-5)


def test_sort_oracle_is_stable_and_chunks_items():
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 16, (300, 4)).astype(np.int32)
    ids[:, 0] = 3                                              # one hot expert: 300+ rows -> a wide step, 64-row items
    s = moe_np.sort_routes(ids, local_start=2, local_count=8, chunk=32)
    assert s["counts"].sum() == ((ids >= 2) & (ids < 10)).sum()
    flat = ids.reshape(-1)
    srt = s["sorted"]
    ex = flat[srt] - 2
    assert np.all(np.diff(ex) >= 0)
    for e in range(8):
        r = srt[ex == e]
        assert np.all(np.diff(r) > 0)                          # route-index order inside an expert
    assert np.array_equal(s["pos"][srt], np.arange(len(srt)))
    assert np.all(s["pos"][(flat < 2) | (flat >= 10)] == -1)
    items = s["items"]
    hot = 300 + int((ids[:, 1:] == 3).sum())                   # expert 3 is local slot 1
    n_hot = -(-hot // 64)
    assert np.all(items[:n_hot, 0] == 1)
    assert list(items[:n_hot, 2]) == [64] * (n_hot - 1) + [hot - 64 * (n_hot - 1)]
    assert list(items[:n_hot, 1]) == [int(s["offsets"][1]) + 64 * i for i in range(n_hot)]
    # the other experts (about 110 rows each) are cut into 64-row items too; in a step without such an
    # expert the same call cuts into runs of `chunk` rows
    assert all(n <= 64 for n in items[:, 2])
    few = moe_np.sort_routes(ids[:20, 1:], local_start=2, local_count=8, chunk=16)
    assert few["counts"].max() <= 32 and all(n <= 16 for n in few["items"][:, 2])
    loads = [s["counts"][e] for e in items[:, 0]]
    assert all(loads[i] >= loads[i + 1] for i in range(len(loads) - 1))


def test_workload_table_matches_baseline_configs():
    w = synth.WORKLOADS
    assert (w["c1"].tokens, w["c1"].hidden, w["c1"].inter, w["c1"].n_experts, w["c1"].top_k) == (4, 1024, 512, 16, 2)
    assert (w["c2"].tokens, w["c2"].hidden, w["c2"].inter, w["c2"].n_experts, w["c2"].top_k) == (32, 4096, 1536, 128, 8)
    assert (w["c4"].hidden, w["c4"].inter, w["c4"].n_experts, w["c4"].shared_inter) == (7168, 2048, 256, 2048)
    assert (w["c5"].tokens, w["c5"].n_experts, w["c5"].top_k, w["c5"].zipf_alpha) == (512, 160, 6, 1.2)
    assert synth.algorithmic_bytes(w["c2"], 1, 0) == 10616832      # 10.617 MB per touched expert


def test_scale_code_is_exact_for_every_e4m3_byte():
    """The stored scale byte, expanded the way the device does it (byte * 16 + 0x7600 as a bf16, over
    2**118), is the E4M3 value for every finite non-zero byte; NaN stays NaN."""
    from okc_muse_kernels_b200 import layout
    from oracle import nvfp4_np as fp4
    b = np.arange(1, 127, dtype=np.uint8)
    want = fp4.e4m3_to_f32(b)
    got = layout.scale_code_value(layout.SCALE_CODE[b])
    assert np.array_equal(got, want)
    assert np.isnan(layout.scale_code_value(layout.SCALE_CODE[127:128]))[0]
    assert layout.SCALE_CODE.max() == 153 and int(layout.SCALE_CODE[1:127].max()) == 142


def test_layout_pack_folds_zero_and_negative_scales_into_codes():
    from okc_muse_kernels_b200 import layout
    rng = np.random.default_rng(3)
    packed = rng.integers(0, 256, (128, 128)).astype(np.uint8)
    sf = rng.integers(1, 0x7F, (128, 16)).astype(np.uint8)
    sf[0, 0] = 0          # zero scale
    sf[1, 1] = 0x80 | 0x38  # -1.0
    img = layout.pack_tile_stage(packed, sf)
    words = img[:layout.TILE_CODE_BYTES].view(np.uint32).reshape(layout.CHUNKS, layout.TILE_ROWS, 2, 2)
    vals = layout.regs_to_values(layout.unpack_block_regs(words))          # chunk, row, block, 16
    from oracle import nvfp4_np as fp4
    want = fp4.unpack_e2m1(packed).reshape(128, 8, 2, 16).transpose(1, 0, 2, 3).copy()
    want[0, 0, 0] = 0.0
    want[0, 1, 1] = -want[0, 1, 1]
    assert np.array_equal(vals, want)
    scales = img[layout.TILE_CODE_BYTES:].reshape(layout.CHUNKS, layout.TILE_ROWS, 2)
    assert scales[0, 1, 1] == layout.SCALE_CODE[0x38]


def test_oracle_layer_router_and_routing_checker():
    """router_scores + route_sigmoid_topk pass the restated checker; a perturbed choice fails it."""
    rng = np.random.default_rng(5)
    T, H, E, k = 12, 256, 64, 8
    hidden = moe_np.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    w = (rng.standard_normal((E, H)) / 16).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.05).astype(np.float32)
    scores, biased, logits = moe_np.router_scores(hidden, w, bias)
    ids, wts = moe_np.route_sigmoid_topk(logits.astype(np.float32), bias, k)
    assert moe_np.check_routing(ids, biased, k) is None
    assert np.allclose(wts.sum(axis=1), 1.0, atol=1e-6)
    bad = ids.copy()
    bad[0, 0] = int(np.argmin(biased[0]))            # the worst expert instead of the best
    assert moe_np.check_routing(bad, biased, k) is not None
    dup = ids.copy()
    dup[1, 1] = dup[1, 0]
    assert "twice" in moe_np.check_routing(dup, biased, k)


def test_reference_arm_of_the_bench_runs_on_host_cores():
    """`bench.py --impl reference` (the oracle on the host cores, no GPU) prints one JSON line with the keys the
    measurement contract names, on the small configuration."""
    import json
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"].startswith("c1")


def test_oracle_router_split_keeps_sixteen_bits_of_the_matrix():
    """w = hi + lo to about 2^-16 relative; the logits of the split router agree with the float64 logits of the
    FP32 matrix far inside the routing checker's tolerance."""
    rng = np.random.default_rng(11)
    T, H, E = 16, 512, 64
    hidden = moe_np.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    w = (rng.standard_normal((E, H)) / 16).astype(np.float32)
    hi, lo = moe_np.router_split(w)
    back = moe_np.bf16_to_f32(hi).astype(np.float64) + moe_np.bf16_to_f32(lo).astype(np.float64)
    assert np.abs(back - w).max() <= np.abs(w).max() * 2.0 ** -15
    _, _, logits = moe_np.router_scores(hidden, w)
    split = moe_np.router_logits_hilo(hidden, hi, lo)
    assert np.abs(split - logits).max() <= 2e-5 * max(1.0, float(np.abs(logits).max()))
