"""CPU oracle (test infrastructure, never shipped): the MoE step in numpy.

Restates the reference's eager dequantise-then-matmul path with the shapes as
parameters (the reference hard-codes 4096/4096/256/8 as module constants,
muse_moe_w4a16/reference.py:18-22):

* ``experts``            follows ``ref_kernel``            muse_moe_w4a16/reference.py:93-107
* ``post_expert_norm``   follows                           muse_moe_w4a16/reference.py:88-90
* ``route_softmax_topk`` is the router the reference does not have (softmax over the
  experts, top-k, renormalised over the selected); its tie rule (lowest index wins) is
  the reference's routing tie rule                         muse_decode_layer/layer.py:394-406
* ``route_sigmoid_topk`` follows the reference's router    muse_decode_layer/variants/starter.py:177-182
* ``sort_routes``        is the stable (expert, route index) order of
  ``moe_routegather``                                      muse_moe_w4a16/submission.py:2236-2328
  with the heaviest-first active list of ``moe_route``     muse_moe_w4a16/submission.py:324-368
* expert-parallel semantics: a rank computes only ids in [local_start, local_start+local_count)
  and the full answer is the sum of the ranks' partials    muse_moe_w4a16/reference.py:22,98-101

BF16 tensors are carried as uint16 bit patterns.  Only tests, ``__graft_entry__.smoke`` and
the CPU-baseline / reference arm of ``bench.py`` may import this module.  It is pinned
against outputs of the reference's own ``ref_kernel`` (tests/golden/make_golden.py).
"""
from __future__ import annotations

import numpy as np

from . import nvfp4_np as fp4

POST_NORM_EPS = np.float32(1e-8)   # muse_moe_w4a16/reference.py:24


# ---------------------------------------------------------------- bf16 <-> f32
def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    u = np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16
    return u.view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (what ``.to(torch.bfloat16)`` does)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))
    out = (rounded >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


# ---------------------------------------------------------------- routing
def _stable_topk_ids(scores: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest per row, descending, equal values -> lowest index first."""
    order = np.argsort(-scores.astype(np.float64), axis=-1, kind="stable")
    return order[:, :k].astype(np.int32)


def route_softmax_topk(logits: np.ndarray, k: int):
    """ids int32 [T,k] (descending logit, ties -> lowest index) and float32 weights [T,k] that
    are the softmax over the k selected logits (== softmax over all experts, top-k, renormalised
    over the selected)."""
    lg = np.asarray(logits, dtype=np.float32)
    ids = _stable_topk_ids(lg, k)
    sel = np.take_along_axis(lg, ids.astype(np.int64), axis=1)
    ex = np.exp((sel - sel[:, :1]).astype(np.float32)).astype(np.float32)
    w = (ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    return ids, w


def route_sigmoid_topk(logits: np.ndarray, bias: np.ndarray, k: int, multiplier: float = 0.1767766952966369):
    """The reference's own router: sigmoid scores, the bias only chooses, the chosen scores are
    renormalised (muse_decode_layer/variants/starter.py:177-182)."""
    scores = (1.0 / (1.0 + np.exp(-(np.asarray(logits, np.float32) * np.float32(multiplier))))).astype(np.float32)
    ids = _stable_topk_ids(scores + np.asarray(bias, np.float32), k)
    picked = np.take_along_axis(scores, ids.astype(np.int64), axis=1)
    w = (picked / (picked.sum(axis=1, keepdims=True, dtype=np.float32) + np.float32(1e-15))).astype(np.float32)
    return ids, w


def router_scores(hidden_bf16: np.ndarray, router_w: np.ndarray, bias: np.ndarray | None = None,
                  multiplier: float = 0.1767766952966369):
    """The reference layer's router on the token rows (muse_decode_layer/reference.py:419-424): logits in
    float64, (unbiased sigmoid scores, the biased scores that choose the top k), both float32 [T, E].
    Also returns the float64 logits."""
    h = bf16_to_f32(np.asarray(hidden_bf16)).astype(np.float64)
    logits = h @ np.asarray(router_w, np.float64).T
    scores = (1.0 / (1.0 + np.exp(-logits * multiplier))).astype(np.float32)
    biased = scores if bias is None else (scores + np.asarray(bias, np.float32)).astype(np.float32)
    return scores, biased, logits


def router_split(router_w: np.ndarray):
    """The FP32 router matrix as two bf16 matrices (uint16 bit patterns), w ~ hi + lo with hi = bf16(w) and
    lo = bf16(w - hi): what the reference prepares for its tensor-core router (the ``w`` / ``wlo`` operands of
    ``_router_split``, muse_decode_layer/layer.py:325-351)."""
    w = np.asarray(router_w, np.float32)
    hi = f32_to_bf16(w)
    lo = f32_to_bf16(w - bf16_to_f32(hi))
    return hi, lo


def router_logits_hilo(hidden_bf16: np.ndarray, hi: np.ndarray, lo: np.ndarray) -> np.ndarray:
    """Logits of the split router: h . hi^T + h . lo^T with exact bf16 products, summed in float64 (the kernel
    accumulates the same products in FP32)."""
    h = bf16_to_f32(np.asarray(hidden_bf16)).astype(np.float64)
    return h @ bf16_to_f32(hi).astype(np.float64).T + h @ bf16_to_f32(lo).astype(np.float64).T


# tolerances of the reference's routing checker (muse_decode_layer/reference.py:68-76)
ROUTE_TOL = 5e-2
LOCAL_SLACK = (0.08, 4)
DISTINCT_SLACK = (0.15, 2)
KEEP_TOL = (0.03, 0.04)
KEEP_TOKENS = 256


def check_routing(ids: np.ndarray, biased: np.ndarray, k: int, local_start: int = 0, local_count: int | None = None):
    """None if ``ids`` [T, k] are an acceptable top-k under the biased scores, else what is wrong:
    the reference's tolerance-based checker (muse_decode_layer/reference.py:609-637), with the number
    of experts, k and the local range as arguments instead of module constants."""
    ids = np.asarray(ids, np.int64)
    biased = np.asarray(biased, np.float32)
    n_experts = biased.shape[1]
    local_count = n_experts if local_count is None else local_count
    if ids.min() < 0 or ids.max() >= n_experts:
        return "expert id out of range"
    ranked = np.sort(ids, axis=-1)
    if (ranked[:, 1:] == ranked[:, :-1]).any():
        return "a token routed to the same expert twice"
    order = np.argsort(-biased, axis=-1, kind="stable")
    best_idx = order[:, :k]
    best_val = np.take_along_axis(biased, best_idx, axis=1)
    gap = best_val[:, -1:] - np.take_along_axis(biased, ids, axis=1)
    if gap.max() > ROUTE_TOL:
        return f"an expert was chosen whose biased score is {float(gap.max()):.2e} below the k-th best"
    ninth = np.take_along_axis(biased, order[:, k:k + 1], axis=1)
    keep_tol = KEEP_TOL[0] if len(ids) <= KEEP_TOKENS else KEEP_TOL[1]
    kept = (best_idx[:, :, None] == ids[:, None, :]).any(-1)
    local = (best_idx - local_start) % n_experts < local_count
    lost = local & ~kept & (best_val - ninth > keep_tol)
    if lost.any():
        return "a local expert well above the (k+1)-th best was dropped"

    def load(x):
        loc = x[(x - local_start) % n_experts < local_count]
        return int(loc.size), int(np.unique(loc).size)

    routes, distinct = load(ids)
    ref_routes, ref_distinct = load(best_idx)
    if routes < ref_routes * (1 - LOCAL_SLACK[0]) - LOCAL_SLACK[1]:
        return f"{routes} local routes where the reference has {ref_routes}"
    if distinct < ref_distinct * (1 - DISTINCT_SLACK[0]) - DISTINCT_SLACK[1]:
        return f"{distinct} local experts touched where the reference touches {ref_distinct}"
    return None


def sort_routes(ids: np.ndarray, local_start: int, local_count: int, chunk: int = 16, narrow: int = 32,
                wide: int = 64):
    """Token -> expert sort of the local routes.

    Route index i = t*k + slot.  Returns a dict with
      counts   int32 [local_count]   routes per local expert
      offsets  int32 [local_count+1] exclusive scan of counts
      sorted   int32 [n_local]       route indices in (expert, route index) order
      pos      int32 [T*k]           position of each route in ``sorted`` (-1 if not local)
      items    int32 [n_items, 3]    (local expert, first position, rows) work items: experts by
                                     load descending (ties by id), each cut into runs of <= chunk rows;
                                     or ("wide step") an expert with at most 16 rows is one item and
                                     every other one is cut into runs of <= wide rows: when some expert
                                     has more than ``narrow`` rows and that cut has at least a tenth
                                     fewer items
    """
    ids = np.asarray(ids, dtype=np.int64)
    flat = ids.reshape(-1)
    local = flat - local_start
    is_local = (local >= 0) & (local < local_count)
    counts = np.bincount(local[is_local], minlength=local_count).astype(np.int32)
    offsets = np.zeros(local_count + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    route_idx = np.nonzero(is_local)[0]
    order = np.argsort(local[is_local], kind="stable")
    sorted_routes = route_idx[order].astype(np.int32)
    pos = np.full(flat.shape[0], -1, dtype=np.int32)
    pos[sorted_routes] = np.arange(sorted_routes.shape[0], dtype=np.int32)
    active = [e for e in np.argsort(-counts.astype(np.int64), kind="stable") if counts[e] > 0]
    items = []
    cmax = int(counts.max()) if counts.size else 0
    n_narrow = sum(-(-int(counts[e]) // chunk) for e in active)
    n_wide = sum(-(-int(counts[e]) // (16 if int(counts[e]) <= 16 else wide)) for e in active)
    wide_step = cmax > narrow and 11 * n_wide <= 10 * n_narrow
    for e in active:
        per = chunk if not wide_step else (16 if int(counts[e]) <= 16 else wide)
        for c0 in range(0, int(counts[e]), per):
            items.append((int(e), int(offsets[e]) + c0, min(per, int(counts[e]) - c0)))
    return {"counts": counts, "offsets": offsets, "sorted": sorted_routes, "pos": pos,
            "items": np.asarray(items, dtype=np.int32).reshape(-1, 3)}


# ---------------------------------------------------------------- experts
def silu(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


def post_expert_norm(y: np.ndarray, w_bf16: np.ndarray) -> np.ndarray:
    """Scale by (1 + w), then RMSNorm with eps 1e-8 (muse_moe_w4a16/reference.py:88-90)."""
    y = y.astype(np.float32) * (np.float32(1.0) + bf16_to_f32(w_bf16))
    ms = np.mean(y * y, axis=-1, keepdims=True, dtype=np.float32)
    return (y * (np.float32(1.0) / np.sqrt(ms + POST_NORM_EPS))).astype(np.float32)


def pre_expert_norm(hidden, gain: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """The layer's pre-expert RMSNorm as the experts see it: bf16 bits of x * rsqrt(mean(x^2) + eps) * gain,
    x being the token rows (bf16 bits, or float32 rounded to bf16 first).  Follows ``p = _rms(p) * (1 +
    pre_expert_norm)`` (muse_decode_layer/reference.py:189-191,465) with the rounding points of the
    reference's fused gather (muse_decode_layer/layer.py:1700-1745)."""
    h = np.asarray(hidden)
    x = bf16_to_f32(h) if h.dtype == np.uint16 else bf16_to_f32(f32_to_bf16(h.astype(np.float32)))
    ms = np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    r = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    return f32_to_bf16((x * r * np.asarray(gain, np.float32)).astype(np.float32))


def expert_mlp(x: np.ndarray, w13, w13_sf, w13_gs, w2, w2_sf, w2_gs) -> np.ndarray:
    """One expert on rows x (float32 [n,H]) -> float32 [n,H]: h = x W13^T, silu(gate)*up, @ W2^T
    (muse_moe_w4a16/reference.py:103-105)."""
    inter_dim = w13.shape[0] // 2
    h = x @ fp4.dequantize(w13, w13_sf, w13_gs).T
    inter = silu(h[:, :inter_dim]) * h[:, inter_dim:]
    return (inter @ fp4.dequantize(w2, w2_sf, w2_gs).T).astype(np.float32)


def experts(hidden_bf16: np.ndarray, ids: np.ndarray, wts: np.ndarray, weights: dict,
            local_start: int = 0, local_count: int | None = None, only_experts=None) -> np.ndarray:
    """The routed experts' weighted sum per token, float32 [T,H] (``ref_kernel`` before its final
    cast, muse_moe_w4a16/reference.py:93-107).  Tokens without a local route stay zero.
    ``weights`` holds w13 u8 [E,2I,H/2], w13_sf u8 [E,2I,H/16], w13_gs f32 [E], w2 u8 [E,H,I/2],
    w2_sf u8 [E,H,I/16], w2_gs f32 [E] and optionally post_norm_w (bf16 bits [H]).
    ``only_experts`` limits the loop to a subset (bounded CPU-baseline samples)."""
    x = bf16_to_f32(hidden_bf16)
    n_experts = weights["w13"].shape[0]
    if local_count is None:
        local_count = n_experts
    out = np.zeros(x.shape, dtype=np.float32)
    ids = np.asarray(ids, dtype=np.int64)
    lo, hi = local_start, local_start + local_count
    post = weights.get("post_norm_w")
    for e in np.unique(ids).tolist():
        if not lo <= e < hi:
            continue
        if only_experts is not None and e not in only_experts:
            continue
        tok, slot = np.nonzero(ids == e)
        y = expert_mlp(x[tok], weights["w13"][e], weights["w13_sf"][e], weights["w13_gs"][e],
                       weights["w2"][e], weights["w2_sf"][e], weights["w2_gs"][e])
        if post is not None:
            y = post_expert_norm(y, post)
        np.add.at(out, tok, y * np.asarray(wts, np.float32)[tok, slot][:, None])
    return out


def shared_expert(hidden_bf16: np.ndarray, shared: dict, rows=None) -> np.ndarray:
    """The always-on shared expert (weight 1) on rows ``rows`` (default all), float32 [T,H] with
    the other rows zero.  Not in the reference; same dequantise-then-matmul arithmetic as
    ``expert_mlp`` with every token routed to it."""
    x = bf16_to_f32(hidden_bf16)
    out = np.zeros(x.shape, dtype=np.float32)
    sel = np.arange(x.shape[0]) if rows is None else np.asarray(rows)
    out[sel] = expert_mlp(x[sel], shared["w13"], shared["w13_sf"], shared["w13_gs"],
                          shared["w2"], shared["w2_sf"], shared["w2_gs"])
    return out


def moe_step(hidden_bf16: np.ndarray, logits: np.ndarray, weights: dict, k: int,
             shared: dict | None = None):
    """Whole single-GPU step: route, experts, (+ shared expert), cast.  Returns
    (out bf16 bits [T,H], out float32 [T,H], ids, weights)."""
    ids, w = route_softmax_topk(logits, k)
    acc = experts(hidden_bf16, ids, w, weights)
    if shared is not None:
        acc = acc + shared_expert(hidden_bf16, shared)
    return f32_to_bf16(acc), acc, ids, w


def moe_step_ep(hidden_bf16: np.ndarray, logits: np.ndarray, weights: dict, k: int, world: int,
                shared: dict | None = None):
    """Expert-parallel step emulated on one host: rank r holds experts [r*E/world, (r+1)*E/world),
    computes its partial for all T tokens plus the shared expert for its own token block; the
    partials are summed in rank order (the reduce-scatter) and cast.  Returns (bf16 bits, float32,
    list of per-rank partials)."""
    n_experts = weights["w13"].shape[0]
    per = n_experts // world
    t = hidden_bf16.shape[0]
    tb = t // world
    ids, w = route_softmax_topk(logits, k)
    partials = []
    for r in range(world):
        p = experts(hidden_bf16, ids, w, weights, local_start=r * per, local_count=per)
        if shared is not None:
            p = p + shared_expert(hidden_bf16, shared, rows=np.arange(r * tb, (r + 1) * tb))
        partials.append(p)
    acc = np.zeros_like(partials[0])
    for p in partials:
        acc = acc + p
    return f32_to_bf16(acc), acc, partials


# ---------------------------------------------------------------- checker
def compare(out_bf16: np.ndarray, ref_f32: np.ndarray, tol: float, row_factor: float = 5.0,
            row_norm_floor: float = 0.1):
    """The reference's acceptance test (muse_moe_w4a16/checks.py:31-55): whole-tensor relative L2
    <= tol and every row <= row_factor*tol against max(row norm, floor * mean row norm)."""
    out = bf16_to_f32(out_bf16).astype(np.float64)
    ref = np.asarray(ref_f32, dtype=np.float64)
    if out.shape != ref.shape:
        return False, f"shape {out.shape} != {ref.shape}"
    if not np.isfinite(out).all():
        return False, "output contains NaN or Inf"
    diff = out - ref
    err = float(np.linalg.norm(diff) / max(np.linalg.norm(ref), 1e-12))
    if err > tol:
        return False, f"relative L2 error {err:.3e} > {tol:g}"
    rows_diff = np.linalg.norm(diff.reshape(-1, ref.shape[-1]), axis=-1)
    rows_ref = np.linalg.norm(ref.reshape(-1, ref.shape[-1]), axis=-1)
    floor = max(row_norm_floor * rows_ref.mean(), 1e-12)
    row_err = rows_diff / np.maximum(rows_ref, floor)
    worst = float(row_err.max())
    if worst > row_factor * tol:
        return False, f"relative L2 error {err:.3e}, but row {int(row_err.argmax())} is off by {worst:.3e}"
    return True, f"relative L2 error {err:.3e} (worst row {worst:.3e})"
