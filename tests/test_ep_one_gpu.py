"""The exchange kernels of the expert-parallel step on ONE GPU, through the C ABI.

Kernels that wait for one another must never run as separate launches on one device (nothing
guarantees that they run at the same time), so the ranks of a step are emulated here one after the
other: every rank has its own exchange buffer and its own shard state on the same GPU, the rank that
runs first is told through ``okc_ep_mark_arrived`` that the later rank's part is in place (for the
reduce it then really is: the later rank's partial sums were computed before), and the rank that
runs second sees the first rank's real flags.  What this covers: the data movement of the push
all-gather, the pull reduce-scatter and the fused combine + reduce, their flag / step-count
bookkeeping over several steps, and a wait that runs out.  What it cannot cover, kernels of several
ranks in flight at once, is what tests/test_ep_gpu.py does on two or more GPUs."""
import numpy as np
import pytest
import torch

import okc_muse_kernels_b200 as okc
from okc_muse_kernels_b200 import _lib, ep, synth
from oracle import moe_np

pytestmark = pytest.mark.gpu


def _dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.uint16).numpy()


def _ranks(world, wl, tokens, dev, wait_limit_ms=0, seed=21):
    """world emulated ranks on one device: (exchange, shard state, own token block) each."""
    nbytes = ep.PeerExchange.buffer_bytes(tokens, wl.hidden, wl.n_experts)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    out = []
    for r in range(world):
        plan = ep.shard_plan(wl.hidden, wl.inter, wl.n_experts, wl.top_k, world, r, max_tokens=max(tokens, 16),
                             shared_inter=wl.shared_inter)
        w = synth.make_weights(wl, seed=seed, device=dev, n_experts=plan.local_count, first_expert=plan.local_start)
        ex = ep.PeerExchange.from_buffers(r, world, tokens, wl.hidden, wl.n_experts, bufs[r], ptrs,
                                          wait_limit_ms=wait_limit_ms)
        out.append((ex, okc.prepare(w, plan), ep.token_block(tokens, world, r)))
    return out


def _full_layer(wl, tokens, dev, seed=21):
    w = synth.make_weights(wl, seed=seed, device=dev)
    plan = okc.MoEPlan(hidden=wl.hidden, inter=wl.inter, n_experts=wl.n_experts, top_k=wl.top_k,
                       shared_inter=wl.shared_inter, max_tokens=max(tokens, 16))
    return w, okc.prepare(w, plan)


def _status_ok(ex, state):
    rc, detail = ex.read_status()
    assert rc == 0, f"exchange status {rc} detail {detail:#x}"
    rc, detail = okc.read_status(state)
    assert rc == 0, f"device status {rc} detail {detail:#x}"


def test_single_rank_exchange_equals_the_plain_step():
    """world = 1: the push, the fused combine + reduce and the pull reduce degenerate to copies of
    the rank's own rows; the result must equal okc.moe_step bit for bit, over several steps."""
    dev = _dev()
    wl = synth.Workload("ep1", 24, 512, 256, 16, 4, shared_inter=256)
    (ex, state, own), = _ranks(1, wl, wl.tokens, dev)
    _, full = _full_layer(wl, wl.tokens, dev)
    out = torch.empty((wl.tokens, wl.hidden), dtype=torch.bfloat16, device=dev)
    for step in range(3):
        hidden, logits = synth.make_inputs(wl, seed=200 + step, device=dev)
        want = okc.moe_step(hidden, logits, full)
        ex.gather_tokens(hidden, logits)
        assert torch.equal(ex.hidden_all, hidden) and torch.equal(ex.logits_all, logits)
        okc.route(ex.logits_all, state, own_tokens=own)
        okc.experts_ep(ex.hidden_all, state, ex.comm, out)          # fused combine + reduce
        _status_ok(ex, state)
        assert torch.equal(out, want), f"step {step}: fused"
        ex.gather_tokens(hidden, logits)
        okc.moe_step(ex.hidden_all, ex.logits_all, state, out_f32=True, own_tokens=own, out=ex.partial)
        out.zero_()
        ex.reduce_scatter(out)                                       # pull reduce
        _status_ok(ex, state)
        assert torch.equal(out, want), f"step {step}: unfused"


def test_routed_gather_single_rank_and_two_emulated_ranks():
    """The gather kernel with the router in it (top-k of the own tokens, ids + weights sent instead of
    logits, sort of the whole step by the CTA that saw every flag).  world = 1: equal to the plain step bit
    for bit.  Two emulated ranks: a first pass moves everybody's rows and routing into both buffers (the
    rank that runs first sorts before the other's routing has arrived, its tables are thrown away), a
    second pass over the same inputs then sorts complete data on both ranks."""
    dev = _dev()
    wl = synth.Workload("ep5", 24, 512, 256, 16, 4, shared_inter=256)
    (ex, state, own), = _ranks(1, wl, wl.tokens, dev)
    _, full = _full_layer(wl, wl.tokens, dev)
    out = torch.empty((wl.tokens, wl.hidden), dtype=torch.bfloat16, device=dev)
    for step in range(3):
        hidden, logits = synth.make_inputs(wl, seed=600 + step, device=dev)
        want = okc.moe_step(hidden, logits, full)
        ids, wts = ex.route_gather(state, hidden, logits)
        okc.experts_ep(ex.hidden_all, state, ex.comm, out)
        _status_ok(ex, state)
        assert torch.equal(ids, full["ids"][:wl.tokens]) and torch.equal(wts, full["wts"][:wl.tokens])
        assert torch.equal(out, want), f"step {step}"
        ref = moe_np.sort_routes(ids.cpu().numpy(), 0, wl.n_experts)
        s = okc.sorted_routes(state, wl.tokens)
        assert np.array_equal(s["counts"].cpu().numpy()[:wl.n_experts], ref["counts"])
    # two emulated ranks
    wl = synth.Workload("ep6", 16, 512, 256, 16, 4, shared_inter=256)
    (ex0, st0, own0), (ex1, st1, own1) = _ranks(2, wl, wl.tokens, dev)
    w_full, full = _full_layer(wl, wl.tokens, dev)
    tb = wl.tokens // 2
    out0 = torch.empty((tb, wl.hidden), dtype=torch.bfloat16, device=dev)
    out1 = torch.empty_like(out0)
    for step in range(2):
        hidden, logits = synth.make_inputs(wl, seed=700 + step, device=dev)
        h0, l0 = hidden[own0[0]:own0[1]], logits[own0[0]:own0[1]].contiguous()
        h1, l1 = hidden[own1[0]:own1[1]], logits[own1[0]:own1[1]].contiguous()
        for _ in range(2):
            ex0.mark_arrived("tokens", 1)
            ex0.route_gather(st0, h0, l0)
            ids1, _ = ex1.route_gather(st1, h1, l1)
        ids_ref, _ = moe_np.route_softmax_topk(logits.cpu().numpy(), wl.top_k)
        assert np.array_equal(ids1.cpu().numpy(), ids_ref) and np.array_equal(ex0.routed_views(wl.top_k)[0].cpu().numpy(), ids_ref)
        okc.moe._experts(ex1.hidden_all, ex1.hidden_all.stride(0), wl.tokens, st1, ex1.partial, True)
        ex0.mark_arrived("partial", 1)
        okc.experts_ep(ex0.hidden_all, st0, ex0.comm, out0)
        ex1.reduce_scatter(out1)
        _status_ok(ex0, st0)
        _status_ok(ex1, st1)
        want = okc.moe_step(hidden, logits, full)
        assert torch.allclose(torch.cat([out0, out1]).float(), want.float(), rtol=2 ** -7, atol=1e-5), f"step {step}"


@pytest.mark.parametrize("fused_first_rank", [False, True])
def test_two_emulated_ranks_one_after_the_other(fused_first_rank):
    dev = _dev()
    wl = synth.Workload("ep2", 16, 512, 256, 16, 4, shared_inter=256)
    ranks = _ranks(2, wl, wl.tokens, dev)
    w_full, full = _full_layer(wl, wl.tokens, dev)
    wn = synth.to_numpy_weights(w_full)
    shared = {k[len("shared_"):]: v for k, v in wn.items() if k.startswith("shared_")}
    (ex0, st0, own0), (ex1, st1, own1) = ranks
    tb = wl.tokens // 2
    out0 = torch.empty((tb, wl.hidden), dtype=torch.bfloat16, device=dev)
    out1 = torch.empty_like(out0)
    for step in range(3):
        hidden, logits = synth.make_inputs(wl, seed=300 + step, device=dev)
        # all-gather: rank 0 first (told that rank 1 has arrived), then rank 1 (sees rank 0's real flag)
        ex0.mark_arrived("tokens", 1)
        ex0.gather_tokens(hidden[own0[0]:own0[1]], logits[own0[0]:own0[1]].contiguous())
        ex1.gather_tokens(hidden[own1[0]:own1[1]], logits[own1[0]:own1[1]].contiguous())
        for ex in (ex0, ex1):
            assert torch.equal(ex.hidden_all, hidden) and torch.equal(ex.logits_all, logits)
        # rank 1's partial sums, complete before rank 0 reduces
        okc.moe_step(ex1.hidden_all, ex1.logits_all, st1, out_f32=True, own_tokens=own1, out=ex1.partial)
        ex0.mark_arrived("partial", 1)
        if fused_first_rank:
            okc.route(ex0.logits_all, st0, own_tokens=own0)
            okc.experts_ep(ex0.hidden_all, st0, ex0.comm, out0)      # publishes rank 1's rows, reduces its own
        else:
            okc.moe_step(ex0.hidden_all, ex0.logits_all, st0, out_f32=True, own_tokens=own0, out=ex0.partial)
            ex0.reduce_scatter(out0)
        ex1.reduce_scatter(out1)                                     # waits for rank 0's real flag
        _status_ok(ex0, st0)
        _status_ok(ex1, st1)
        got = torch.cat([out0, out1])
        # two addends per element in another association than the one-GPU sum: a bf16 ulp of slack
        want = okc.moe_step(hidden, logits, full)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-5), f"step {step}"
        _, ref, _, _ = moe_np.moe_step(_bits(hidden), logits.cpu().numpy(), wn, wl.top_k, shared=shared)
        ok, msg = moe_np.compare(_bits(got), ref, 1.5e-2)
        assert ok, f"step {step}: {msg}"


def test_exchange_wait_runs_out_and_the_next_step_is_correct():
    """Failure detection without a GPU fault: rank 0 of two pushes its tokens while rank 1 never
    shows up (nothing raises its flag).  The wait gives up after its 20 ms limit, the kernel returns,
    the status says OKC_ERR_TIMEOUT with the code of the wait and of the missing rank, the context
    stays usable, and after a reset of the buffers a whole step gives the right answer."""
    dev = _dev()
    wl = synth.Workload("ep3", 16, 512, 256, 16, 4)
    ranks = _ranks(2, wl, wl.tokens, dev, wait_limit_ms=20)
    (ex0, st0, own0), (ex1, st1, own1) = ranks
    hidden, logits = synth.make_inputs(wl, seed=400, device=dev)
    ex0.gather_tokens(hidden[own0[0]:own0[1]], logits[own0[0]:own0[1]].contiguous())
    rc, detail = ex0.read_status()
    assert rc == _lib.OKC_ERR_TIMEOUT and detail == 0x100 + 1
    rc, detail = ex0.read_status()
    assert rc == 0, "reading the status clears it"
    # the reduce side: rank 0 waits for partial sums of rank 1 that never come
    out0 = torch.empty((wl.tokens // 2, wl.hidden), dtype=torch.bfloat16, device=dev)
    ex0.reduce_scatter(out0)
    rc, detail = ex0.read_status()
    assert rc == _lib.OKC_ERR_TIMEOUT and detail == 0x200 + 1
    okc.route(logits, st0, own_tokens=own0)
    okc.experts_ep(hidden, st0, ex0.comm, out0)
    rc, detail = ex0.read_status()
    assert rc == _lib.OKC_ERR_TIMEOUT and detail == 0x300 + 1
    # recovery: the ranks' step counts now differ; both reset, then a whole step
    ex0.reset()
    ex1.reset()
    out1 = torch.empty_like(out0)
    ex0.mark_arrived("tokens", 1)
    ex0.gather_tokens(hidden[own0[0]:own0[1]], logits[own0[0]:own0[1]].contiguous())
    ex1.gather_tokens(hidden[own1[0]:own1[1]], logits[own1[0]:own1[1]].contiguous())
    okc.moe_step(ex1.hidden_all, ex1.logits_all, st1, out_f32=True, own_tokens=own1, out=ex1.partial)
    ex0.mark_arrived("partial", 1)
    okc.route(ex0.logits_all, st0, own_tokens=own0)
    okc.experts_ep(ex0.hidden_all, st0, ex0.comm, out0)
    ex1.reduce_scatter(out1)
    _status_ok(ex0, st0)
    _status_ok(ex1, st1)
    w_full, full = _full_layer(wl, wl.tokens, dev)
    want = okc.moe_step(hidden, logits, full)
    assert torch.allclose(torch.cat([out0, out1]).float(), want.float(), rtol=2 ** -7, atol=1e-5)


def test_fused_reduce_with_more_own_row_ctas_than_fit_the_gpu():
    """The fused combine + reduce must not need all of its CTAs resident at once: 768 own rows of
    width 7168 are 5376 CTAs, several times what a B200 holds."""
    dev = _dev()
    wl = synth.Workload("ep4", 768, 7168, 256, 8, 2)
    (ex, state, own), = _ranks(1, wl, wl.tokens, dev)
    hidden, logits = synth.make_inputs(wl, seed=500, device=dev)
    ex.gather_tokens(hidden, logits)
    okc.route(ex.logits_all, state, own_tokens=own)
    out = torch.empty((wl.tokens, wl.hidden), dtype=torch.bfloat16, device=dev)
    okc.experts_ep(ex.hidden_all, state, ex.comm, out)
    _status_ok(ex, state)
    want = okc.moe_step(hidden, logits, state)
    assert torch.equal(out, want)
    sub = [0, 383, 767]
    wn = synth.to_numpy_weights(synth.make_weights(wl, seed=21, device=dev))
    _, ref, _, _ = moe_np.moe_step(_bits(hidden)[sub], logits.cpu().numpy()[sub], wn, wl.top_k)
    ok, msg = moe_np.compare(_bits(out[sub]), ref, 1.5e-2)
    assert ok, msg
