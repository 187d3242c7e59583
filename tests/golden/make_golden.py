"""Generates the golden vectors under tests/golden/ by running the reference's own Python
modules (muse_moe_w4a16/{nvfp4,reference,checks}.py) on the CPU.

    python tests/golden/make_golden.py /path/to/reference

The reference hard-codes its shapes as module constants (reference.py:18-22); they are patched to
small sizes here (the narrowest the CUDA kernels accept: multiples of 256) so the fixtures stay small.  Nothing in the test-suite needs the
reference tree at run time: the tests only read the .npz files this script wrote.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy().copy()


def _u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def codec_vectors(nvfp4) -> dict:
    g = torch.Generator(device="cpu").manual_seed(101)
    x = torch.randn((12, 96), generator=g) * 0.02
    # special values: exact grid midpoints (after scaling), zeros, a zero block, saturating values
    x[0, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[1, 16:32] = 0.0
    x[2, :16] = torch.tensor([7.0, -9.0, 1e-9, -1e-9] * 4)
    p, sf, gs = nvfp4.quantize(x)
    p_s, sf_s, gs_s = nvfp4.quantize(x, 0.003)
    out = {
        "codec_x": x.numpy(), "codec_packed": _u8(p), "codec_sf": _u8(sf), "codec_gs": gs.numpy(),
        "codec_deq": nvfp4.dequantize(p, sf, gs).numpy(),
        "codec_static_gs": np.float32(0.003), "codec_static_packed": _u8(p_s), "codec_static_sf": _u8(sf_s),
        "codec_static_deq": nvfp4.dequantize(p_s, sf_s, gs_s).numpy(),
    }
    # x whose scaled values sit exactly on midpoints with gs = 1 and unit block scale
    y = torch.zeros((1, 16))
    y[0] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -0.1])
    py, sfy, gsy = nvfp4.quantize(y, 1.0)
    out.update({"mid_x": y.numpy(), "mid_packed": _u8(py), "mid_sf": _u8(sfy)})
    # every e4m3 bit pattern and every code byte through dequantize
    allsf = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn)
    out["e4m3_all"] = allsf.float().numpy()
    codes = torch.arange(256, dtype=torch.uint8).view(32, 8)
    out["e2m1_all"] = nvfp4.unpack_e2m1(codes).numpy()
    # e4m3 rounding: a dense sweep of float32 values in [0, 448]
    sweep = torch.cat([torch.linspace(0, 448, 4001), torch.logspace(-12, 2.65, 2000, base=10.0)])
    out["e4m3_sweep_in"] = sweep.numpy()
    out["e4m3_sweep_out"] = _u8(sweep.clamp(max=448.0).to(torch.float8_e4m3fn))
    # the reference's random NVFP4 weights (uniform codes, log-normal / wide scales)
    g2 = torch.Generator(device="cpu").manual_seed(7)
    for tag, wide in (("rw", False), ("rww", True)):
        p, sf, gs = nvfp4.random_weights(6, 64, generator=g2, device="cpu", leading=(2,), wide_scales=wide)
        out.update({f"{tag}_packed": _u8(p), f"{tag}_sf": _u8(sf), f"{tag}_gs": gs.numpy(),
                    f"{tag}_deq": nvfp4.dequantize(p, sf, gs).numpy()})
    return out


def moe_vectors(ref, nvfp4, tag: str, *, hidden: int, inter: int, experts: int, top_k: int, local: tuple,
                bs: int, seed: int, dist: str, quantised_normal: bool) -> dict:
    """One ``ref_kernel`` case at patched module constants."""
    ref.D_HIDDEN, ref.D_EXPERT, ref.N_EXPERTS, ref.ROUTED_PER_TOKEN = hidden, inter, experts, top_k
    ref.LOCAL = {"case": local}
    if quantised_normal:
        # weights drawn N(0, 0.02) and quantised with the reference's own quantiser
        g = torch.Generator(device="cpu").manual_seed(seed + 17)
        w13 = [nvfp4.quantize(torch.randn((2 * inter, hidden), generator=g) * 0.02) for _ in range(experts)]
        w2 = [nvfp4.quantize(torch.randn((hidden, inter), generator=g) * 0.02) for _ in range(experts)]
        weights = {
            "w13": torch.stack([w[0] for w in w13]), "w13_sf": torch.stack([w[1] for w in w13]),
            "w13_gs": torch.stack([w[2] for w in w13]),
            "w2": torch.stack([w[0] for w in w2]), "w2_sf": torch.stack([w[1] for w in w2]),
            "w2_gs": torch.stack([w[2] for w in w2]),
            "post_norm_w": (0.1 * torch.randn((hidden,), generator=g)).to(torch.bfloat16),
        }
    else:
        weights = ref.generate_weights(seed + 17, device="cpu")
    data = ref.generate_input(bs, "case", seed, dist=dist, device="cpu")
    out = ref.ref_kernel(data, weights)
    ok, msg = ref.check_implementation(data, out, weights)
    assert ok, msg
    cfg = data["config"]
    return {
        f"{tag}_cfg": np.array([bs, hidden, inter, experts, top_k, cfg["local_start"], cfg["local_count"]], dtype=np.int64),
        f"{tag}_hidden": _u16(data["hidden_states"]), f"{tag}_ids": data["topk_ids"].numpy(),
        f"{tag}_wts": data["topk_weights"].numpy(),
        f"{tag}_w13": _u8(weights["w13"]), f"{tag}_w13_sf": _u8(weights["w13_sf"]), f"{tag}_w13_gs": weights["w13_gs"].numpy(),
        f"{tag}_w2": _u8(weights["w2"]), f"{tag}_w2_sf": _u8(weights["w2_sf"]), f"{tag}_w2_gs": weights["w2_gs"].numpy(),
        f"{tag}_post_norm_w": _u16(weights["post_norm_w"]),
        f"{tag}_out": _u16(out),
    }


def router_vectors(starter_route) -> dict:
    """The reference's sigmoid router (variants/starter.py:177-182) on seeded logits, with ties."""
    g = torch.Generator(device="cpu").manual_seed(33)
    t, e, k, hdim = 9, 32, 4, 16
    h = torch.randn((t, hdim), generator=g)
    router = torch.randn((e, hdim), generator=g)
    bias = 0.05 * torch.randn((e,), generator=g)
    ids, w = starter_route(h, {"router": router, "router_bias": bias}, k)
    return {"sig_logits": (h.float() @ router.T).numpy(), "sig_bias": bias.numpy(),
            "sig_ids": ids.numpy().astype(np.int32), "sig_w": w.numpy()}


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of tech-cosmos/okc-muse-kernels>")
    root = sys.argv[1]
    sys.path.insert(0, os.path.join(root, "muse_moe_w4a16"))
    nvfp4 = importlib.import_module("nvfp4")
    ref = importlib.import_module("reference")
    np.savez_compressed(os.path.join(HERE, "codec.npz"), **codec_vectors(nvfp4))

    cases = {}
    # the reference's own weight distribution (uniform codes, log-normal scales), with post-norm, all local
    cases.update(moe_vectors(ref, nvfp4, "full", hidden=256, inter=256, experts=4, top_k=2, local=(0, 4),
                             bs=5, seed=1000, dist="normal", quantised_normal=False))
    # expert-parallel shard (4 of 8 local, busiest-rank rotation), skewed routing + outlier channels
    cases.update(moe_vectors(ref, nvfp4, "ep", hidden=256, inter=256, experts=4, top_k=3, local=(0, 2),
                             bs=7, seed=1003, dist="skewed", quantised_normal=False))
    # N(0,0.02) weights through the reference's quantiser (the distribution the benchmark configs use)
    cases.update(moe_vectors(ref, nvfp4, "qn", hidden=256, inter=256, experts=2, top_k=2, local=(0, 2),
                             bs=4, seed=1001, dist="normal", quantised_normal=True))
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **cases)

    # the starter's route() is a plain function; load the file without running its CUDA parts
    src = open(os.path.join(root, "muse_decode_layer", "variants", "starter.py")).read()
    start = src.index("def route(")
    end = src.index("\ndef ", start + 1)
    ns: dict = {"torch": torch}
    exec(src[start:end], ns)  # the reference's own function text, executed, not copied
    np.savez_compressed(os.path.join(HERE, "router.npz"), **router_vectors(ns["route"]))
    for f in ("codec.npz", "moe.npz", "router.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
