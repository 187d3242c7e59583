"""CPU oracle (test infrastructure, never shipped): the reference's eager path with torch CPU ops.

The same arithmetic as oracle/moe_np.py, written with the torch operators the reference itself
uses (``dequantize`` muse_moe_w4a16/nvfp4.py:90-97 then FP32 matmuls, ``ref_kernel``
muse_moe_w4a16/reference.py:93-107), so that the timed CPU baseline runs on every host core the
way the reference's own eager path would.  Shapes are parameters; there is no post-norm unless
``post_norm_w`` is given.  Only tests and the CPU-baseline / reference arm of bench.py import it.
"""
from __future__ import annotations

import torch

_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)


def dequantize(packed: torch.Tensor, sf: torch.Tensor, gs) -> torch.Tensor:
    """uint8 [rows, K/2] codes + e4m3 [rows, K/16] scales + global scale -> float32 [rows, K]."""
    p = packed.view(torch.uint8)
    codes = torch.stack((p & 0x0F, p >> 4), dim=-1).flatten(-2)
    mag = _GRID[(codes & 0x7).long()]
    vals = torch.where((codes & 0x8) != 0, -mag, mag)
    k = vals.shape[-1]
    scale = (sf.view(torch.float8_e4m3fn).float() * torch.as_tensor(gs, dtype=torch.float32)).unsqueeze(-1)
    return (vals.view(*vals.shape[:-1], k // 16, 16) * scale).view_as(vals)


def route_softmax_topk(logits: torch.Tensor, k: int):
    """ids int64 [T,k] by descending logit (ties to the lowest index), weights = softmax over the selected."""
    order = torch.sort(logits.double(), dim=-1, descending=True, stable=True).indices[:, :k]
    sel = torch.gather(logits.float(), 1, order)
    return order, torch.softmax(sel, dim=-1)


def experts(hidden: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, weights, local_start: int = 0,
            local_count: int | None = None, only_experts=None, post_norm_w: torch.Tensor | None = None) -> torch.Tensor:
    """float32 [T,H]: sum over each token's local routes of weight * expert(x).  ``weights[key][e]``
    gives expert e's tensors (w13, w13_sf, w13_gs, w2, w2_sf, w2_gs)."""
    x = hidden.float()
    out = torch.zeros(x.shape, dtype=torch.float32)
    n = weights["w13"].shape[0]
    lo, hi = local_start, local_start + (n if local_count is None else local_count)
    for e in torch.unique(ids).tolist():
        if not lo <= e < hi or (only_experts is not None and e not in only_experts):
            continue
        tok, slot = (ids == e).nonzero(as_tuple=True)
        w13 = dequantize(weights["w13"][e], weights["w13_sf"][e], weights["w13_gs"][e])
        inter = w13.shape[0] // 2
        h = x[tok] @ w13.T
        a = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
        y = a @ dequantize(weights["w2"][e], weights["w2_sf"][e], weights["w2_gs"][e]).T
        if post_norm_w is not None:
            y = y * (1.0 + post_norm_w.float())
            y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-8)
        out.index_add_(0, tok, y * wts[tok, slot].unsqueeze(1))
    return out


def shared_expert(hidden: torch.Tensor, shared: dict, rows=None) -> torch.Tensor:
    """The always-on shared expert (weight 1) on rows ``rows`` (default all), float32 [T,H], other rows
    zero.  Not in the reference; the same dequantise-then-matmul arithmetic with every token routed
    to it.  ``shared`` holds w13, w13_sf, w13_gs, w2, w2_sf, w2_gs of the one expert."""
    x = hidden.float()
    out = torch.zeros(x.shape, dtype=torch.float32)
    sel = torch.arange(x.shape[0]) if rows is None else torch.as_tensor(rows, dtype=torch.long)
    if sel.numel() == 0:
        return out
    w13 = dequantize(shared["w13"], shared["w13_sf"], shared["w13_gs"])
    inter = w13.shape[0] // 2
    h = x[sel] @ w13.T
    a = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
    out[sel] = a @ dequantize(shared["w2"], shared["w2_sf"], shared["w2_gs"]).T
    return out
