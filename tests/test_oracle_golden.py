"""The numpy oracle against vectors produced by the reference's own modules
(tests/golden/make_golden.py): codec bit-exact, MoE outputs to float32 round-off."""
import os

import numpy as np
import pytest

from oracle import moe_np, nvfp4_np as fp4


@pytest.fixture(scope="module")
def codec(golden_dir):
    return np.load(os.path.join(golden_dir, "codec.npz"))


@pytest.fixture(scope="module")
def moe(golden_dir):
    return np.load(os.path.join(golden_dir, "moe.npz"))


def test_e4m3_decode_all_patterns(codec):
    ours = fp4.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    ref = codec["e4m3_all"]
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(ours[ok].view(np.uint32), ref[ok].view(np.uint32))


def test_e4m3_rounding_sweep(codec):
    ours = fp4.f32_to_e4m3(np.minimum(codec["e4m3_sweep_in"], np.float32(448.0)))
    assert np.array_equal(ours, codec["e4m3_sweep_out"])


def test_e2m1_unpack_all_bytes(codec):
    ours = fp4.unpack_e2m1(np.arange(256, dtype=np.uint8).reshape(32, 8))
    assert np.array_equal(ours, codec["e2m1_all"])


def test_quantize_dynamic_bit_exact(codec):
    p, sf, gs = fp4.quantize(codec["codec_x"])
    assert np.float32(gs).view(np.uint32) == codec["codec_gs"].astype(np.float32).view(np.uint32)
    assert np.array_equal(sf, codec["codec_sf"])
    assert np.array_equal(p, codec["codec_packed"])
    assert np.array_equal(fp4.dequantize(p, sf, gs).view(np.uint32), codec["codec_deq"].view(np.uint32))


def test_quantize_static_bit_exact(codec):
    p, sf, gs = fp4.quantize(codec["codec_x"], codec["codec_static_gs"])
    assert np.array_equal(sf, codec["codec_static_sf"])
    assert np.array_equal(p, codec["codec_static_packed"])
    assert np.array_equal(fp4.dequantize(p, sf, gs).view(np.uint32), codec["codec_static_deq"].view(np.uint32))


def test_midpoints_go_to_smaller_magnitude(codec):
    p, sf, _ = fp4.quantize(codec["mid_x"], 1.0)
    assert np.array_equal(p, codec["mid_packed"])
    assert np.array_equal(sf, codec["mid_sf"])
    vals = fp4.unpack_e2m1(p)[0]
    # 0.25 -> 0, 2.5 -> 2, 5 -> 4, and a value that rounds to zero never keeps its sign
    assert vals[0] == 0 and vals[4] == 2 and vals[6] == 4
    assert not np.signbit(vals[8]) and not np.signbit(vals[15])


@pytest.mark.parametrize("tag", ["rw", "rww"])
def test_dequantize_reference_random_weights(codec, tag):
    ours = fp4.dequantize(codec[f"{tag}_packed"], codec[f"{tag}_sf"], codec[f"{tag}_gs"])
    assert np.array_equal(ours.view(np.uint32), codec[f"{tag}_deq"].view(np.uint32))


def _weights(moe, tag):
    return {k: moe[f"{tag}_{k}"] for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs", "post_norm_w")}


@pytest.mark.parametrize("tag", ["full", "ep", "qn"])
def test_experts_match_ref_kernel(moe, tag):
    bs, hidden, inter, experts, top_k, lo, cnt = (int(v) for v in moe[f"{tag}_cfg"])
    acc = moe_np.experts(moe[f"{tag}_hidden"], moe[f"{tag}_ids"], moe[f"{tag}_wts"], _weights(moe, tag),
                         local_start=lo, local_count=cnt)
    ref = moe_np.bf16_to_f32(moe[f"{tag}_out"])
    assert acc.shape == (bs, hidden)
    # float32 sums in a different BLAS order, then one bf16 rounding: at most one bf16 ulp on few elements
    ours = moe_np.f32_to_bf16(acc)
    ulp = np.abs(ours.astype(np.int32) - moe[f"{tag}_out"].astype(np.int32))
    assert ulp.max() <= 1 and (ulp != 0).mean() < 0.02
    rel = np.linalg.norm(acc - ref) / np.linalg.norm(ref)
    assert rel < 4e-3          # bf16 rounding of the golden output itself
    ok, msg = moe_np.compare(ours, ref, 1.5e-2)
    assert ok, msg
    # rows without a local route are exact zeros
    local = (moe[f"{tag}_ids"] >= lo) & (moe[f"{tag}_ids"] < lo + cnt)
    for t in np.nonzero(~local.any(axis=1))[0]:
        assert not acc[t].any()


def test_sigmoid_router_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "router.npz"))
    ids, w = moe_np.route_sigmoid_topk(g["sig_logits"], g["sig_bias"], g["sig_ids"].shape[1])
    assert np.array_equal(ids, g["sig_ids"])
    assert np.allclose(w, g["sig_w"], rtol=2e-6, atol=0)


def test_bf16_roundtrip():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(10000).astype(np.float32)
    import torch
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(moe_np.f32_to_bf16(x), ref)
    assert np.array_equal(moe_np.bf16_to_f32(ref), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("tag", ["full", "ep", "qn"])
def test_torch_oracle_matches_ref_kernel(moe, tag):
    """The torch-operator restatement used for the timed CPU baseline, against the same vectors."""
    import torch
    from oracle import moe_torch
    bs, hidden, inter, experts, top_k, lo, cnt = (int(v) for v in moe[f"{tag}_cfg"])
    w = {k: torch.from_numpy(moe[f"{tag}_{k}"]) for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs")}
    hid = torch.from_numpy(moe[f"{tag}_hidden"].view(np.int16)).view(torch.bfloat16)
    post = torch.from_numpy(moe[f"{tag}_post_norm_w"].view(np.int16)).view(torch.bfloat16)
    acc = moe_torch.experts(hid, torch.from_numpy(moe[f"{tag}_ids"]).long(), torch.from_numpy(moe[f"{tag}_wts"]), w,
                            local_start=lo, local_count=cnt, post_norm_w=post)
    ref = torch.from_numpy(moe[f"{tag}_out"].view(np.int16)).view(torch.bfloat16)
    assert torch.equal(acc.to(torch.bfloat16), ref)          # same operators, same order: bit-exact


def test_torch_and_numpy_oracles_agree_on_routing():
    import torch
    from oracle import moe_torch
    g = torch.Generator().manual_seed(0)
    logits = torch.randn((40, 128), generator=g)
    logits[3, 7] = logits[3, 99] = 9.0
    ids_t, w_t = moe_torch.route_softmax_topk(logits, 8)
    ids_n, w_n = moe_np.route_softmax_topk(logits.numpy(), 8)
    assert np.array_equal(ids_t.numpy(), ids_n)
    assert np.allclose(w_t.numpy(), w_n, rtol=1e-6)


def test_torch_and_numpy_oracles_agree_on_the_shared_expert():
    """The shared expert is not in the reference; both statements of it (the same dequantise-then-matmul
    arithmetic as a routed expert with weight 1) must agree, on all rows and on a row block."""
    import torch
    from okc_muse_kernels_b200 import synth
    from oracle import moe_torch
    wl = synth.Workload("sh", 8, 512, 256, 8, 2, shared_inter=256)
    w = synth.make_weights(wl, seed=3, device="cpu")
    hidden, _ = synth.make_inputs(wl, seed=4, device="cpu")
    wn = synth.to_numpy_weights(w)
    hb = hidden.view(torch.uint16).numpy()
    for rows in (None, [2, 3, 4]):
        a = moe_np.shared_expert(hb, {k[7:]: v for k, v in wn.items() if k.startswith("shared_")},
                                 rows=None if rows is None else np.asarray(rows))
        b = moe_torch.shared_expert(hidden, {k[7:]: v for k, v in w.items() if k.startswith("shared_")}, rows=rows)
        assert np.allclose(a, b.numpy(), rtol=1e-5, atol=1e-6)
        if rows is not None:
            assert not a[[0, 1, 5, 6, 7]].any() and not b.numpy()[[0, 1, 5, 6, 7]].any()
