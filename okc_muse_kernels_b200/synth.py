"""Seeded synthetic weights and inputs with the shapes and value distributions of the benchmark
configurations (they stand in for the contest judge's inputs; no dataset is involved).

Data generation only: nothing here is on the timed path.  The NVFP4 quantiser below is a torch
statement of the format the reference defines (muse_moe_w4a16/nvfp4.py:60-87: global scale
amax / (6 * 448), E4M3 block scale per 16 elements, round to the E2M1 grid through the midpoints
with exact midpoints going to the smaller magnitude, no negative zero); it runs on whichever
device the tensor lives on so that big configurations can be quantised on the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    tokens: int
    hidden: int
    inter: int
    n_experts: int
    top_k: int
    shared_inter: int = 0
    zipf_alpha: float = 0.0


WORKLOADS = {
    "c1": Workload("c1", 4, 1024, 512, 16, 2),
    "c2": Workload("c2", 32, 4096, 1536, 128, 8),
    "c4": Workload("c4", 128, 7168, 2048, 256, 8, shared_inter=2048),
    "c5": Workload("c5", 512, 5120, 1536, 160, 6, zipf_alpha=1.2),
}
C3_TOKENS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def quantize_nvfp4(x: torch.Tensor):
    """float [..., K] -> (codes uint8 [..., K/2], scales float8_e4m3fn [..., K/16], global scale f32 [])."""
    xf = x.float()
    k = xf.shape[-1]
    assert k % 16 == 0
    amax = xf.abs().amax()
    gs = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    blk = xf.reshape(*xf.shape[:-1], k // 16, 16)
    sf = (blk.abs().amax(dim=-1) / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    scale = (sf.float() * gs).unsqueeze(-1)
    q = torch.where(scale > 0, blk / scale, torch.zeros_like(blk)).reshape(xf.shape)
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32, device=x.device)
    mag = torch.bucketize(q.abs().clamp(max=6.0), mids).to(torch.uint8)          # right=False: ties go down
    code = mag | (((q < 0) & (mag > 0)).to(torch.uint8) << 3)
    code = code.reshape(*xf.shape[:-1], k // 2, 2)
    return code[..., 0] | (code[..., 1] << 4), sf, gs


def _expert_generator(seed: int, expert: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed * 1000003 + expert)


def make_weights(w: Workload, seed: int = 5252, device: str | torch.device = "cuda", n_experts: int | None = None,
                 first_expert: int = 0) -> dict:
    """Per expert W13 ~ N(0, 0.02) [2I, H] and W2 ~ N(0, 0.02) [H, I], quantised to NVFP4 with a
    dynamic global scale per expert tensor (+ the shared expert when the workload has one).
    Every expert has its own seed, so a shard [first_expert, first_expert + n_experts) holds the
    same bits as the matching slice of the full layer."""
    n = w.n_experts if n_experts is None else n_experts
    out = {"w13": torch.empty((n, 2 * w.inter, w.hidden // 2), dtype=torch.uint8, device=device),
           "w13_sf": torch.empty((n, 2 * w.inter, w.hidden // 16), dtype=torch.float8_e4m3fn, device=device),
           "w13_gs": torch.empty((n,), dtype=torch.float32, device=device),
           "w2": torch.empty((n, w.hidden, w.inter // 2), dtype=torch.uint8, device=device),
           "w2_sf": torch.empty((n, w.hidden, w.inter // 16), dtype=torch.float8_e4m3fn, device=device),
           "w2_gs": torch.empty((n,), dtype=torch.float32, device=device)}
    for i in range(n):
        g = _expert_generator(seed, first_expert + i, device)
        a = torch.randn((2 * w.inter, w.hidden), generator=g, device=device) * 0.02
        out["w13"][i], out["w13_sf"][i], out["w13_gs"][i] = quantize_nvfp4(a)
        b = torch.randn((w.hidden, w.inter), generator=g, device=device) * 0.02
        out["w2"][i], out["w2_sf"][i], out["w2_gs"][i] = quantize_nvfp4(b)
    if w.shared_inter:
        g = _expert_generator(seed, 1 << 20, device)
        a = torch.randn((2 * w.shared_inter, w.hidden), generator=g, device=device) * 0.02
        out["shared_w13"], out["shared_w13_sf"], out["shared_w13_gs"] = quantize_nvfp4(a)
        b = torch.randn((w.hidden, w.shared_inter), generator=g, device=device) * 0.02
        out["shared_w2"], out["shared_w2_sf"], out["shared_w2_gs"] = quantize_nvfp4(b)
    return out


def make_reference_style_weights(n_experts: int, hidden: int, inter: int, seed: int,
                                 device: str | torch.device = "cuda", wide_scales: bool = False) -> dict:
    """NVFP4 weights with the distribution of the reference's own generator
    (muse_moe_w4a16/nvfp4.py:105-128, reference.py:33-50): codes uniform over all 16 patterns,
    block scales log-normal (log2 ~ N(7, 0.4), clamped to [8, 448]) or, with wide_scales,
    log-uniform over 2^-6 .. 448; one global scale per tensor that normalises dot products to about
    unit variance; a post-expert norm weight 0.1 * N(0, 1)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def tensor(rows: int, k: int):
        codes = torch.randint(0, 256, (n_experts, rows, k // 2), dtype=torch.uint8, generator=g, device=device)
        if wide_scales:
            u = torch.rand((n_experts, rows, k // 16), generator=g, device=device)
            sf = torch.exp2(-6 + u * (8.807354922057604 + 6)).to(torch.float8_e4m3fn)      # log2(448) = 8.807...
            mean_sq = float(sf.float().pow(2).mean())
        else:
            z = torch.randn((n_experts, rows, k // 16), generator=g, device=device)
            sf = torch.exp2(7.0 + 0.4 * z).clamp(8.0, 448.0).to(torch.float8_e4m3fn)
            mean_sq = 4.0 ** 7.0 * 2.718281828459045 ** (2 * (0.6931471805599453 * 0.4) ** 2)
        gs = torch.full((n_experts,), 1.0 / (8.6 * mean_sq * k) ** 0.5, dtype=torch.float32, device=device)
        return codes, sf, gs

    w13, w13_sf, w13_gs = tensor(2 * inter, hidden)
    w2, w2_sf, w2_gs = tensor(hidden, inter)
    post = (0.1 * torch.randn((hidden,), generator=g, device=device)).to(torch.bfloat16)
    return {"w13": w13, "w13_sf": w13_sf, "w13_gs": w13_gs, "w2": w2, "w2_sf": w2_sf, "w2_gs": w2_gs,
            "post_norm_w": post}


def make_inputs(w: Workload, seed: int, device: str | torch.device = "cuda", tokens: int | None = None):
    """hidden ~ N(0,1) bf16 [T, H]; router logits ~ N(0,1) f32 [T, E] (+ log-popularity bias with
    popularity ~ rank^-alpha over a seeded expert permutation when the workload is Zipf)."""
    t = w.tokens if tokens is None else tokens
    g = torch.Generator(device=device).manual_seed(seed)
    hidden = torch.randn((t, w.hidden), generator=g, device=device).to(torch.bfloat16)
    logits = torch.randn((t, w.n_experts), generator=g, device=device)
    if w.zipf_alpha > 0:
        perm = torch.randperm(w.n_experts, generator=g, device=device)
        pop = (torch.arange(1, w.n_experts + 1, device=device, dtype=torch.float32)) ** (-w.zipf_alpha)
        bias = torch.empty(w.n_experts, device=device)
        bias[perm] = torch.log(pop / pop.sum())
        logits = logits + bias
    return hidden, logits.float().contiguous()


def algorithmic_bytes(w: Workload, touched_experts: int, tokens: int, shared: bool = False) -> int:
    """Bytes one step must move: FP4 codes + E4M3 scales of gate, up and down of every touched
    expert (3*I*H*(1/2 + 1/16)), plus activations in and out and the logits."""
    per_expert = 3 * w.inter * w.hidden * 9 // 16
    n = touched_experts + (1 if shared else 0)
    return n * per_expert + tokens * w.hidden * 2 * 2 + tokens * w.n_experts * 4


def to_numpy_weights(weights: dict) -> dict:
    """Device NVFP4 weight dict -> numpy arrays in the layout the CPU oracle takes."""
    out = {}
    for k, v in weights.items():
        v = v.detach().cpu()
        if v.dtype == torch.float8_e4m3fn:
            out[k] = v.view(torch.uint8).numpy()
        elif v.dtype == torch.bfloat16:
            out[k] = v.view(torch.uint16).numpy()
        else:
            out[k] = v.numpy()
    return out
