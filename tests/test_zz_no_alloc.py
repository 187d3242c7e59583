"""The workspace-free step, okc_moe_step_static_scratch, against okc_moe_step.

Some callers of this library cannot allocate device memory while they run (a server that gave all
of it to its own pool, a plugin inside one), so they have no workspace to pass; for them the step
keeps its scratch in an array inside the library.  Both entry points run the same kernels in the
same order, so the outputs must be identical bit for bit.  Two calls are made back to back with
different token counts: the second one finds the first one's leftovers in the array.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes on its own in a fresh process as well."""
import ctypes as C

import pytest
import torch

import okc_muse_kernels_b200 as okc
from okc_muse_kernels_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _step(fn_name, state, hidden, logits, with_workspace):
    plan = state["plan"]
    T = hidden.shape[0]
    dev = hidden.device
    ids = torch.zeros((T, plan.top_k), dtype=torch.int32, device=dev)
    wts = torch.zeros((T, plan.top_k), dtype=torch.float32, device=dev)
    out = torch.empty((T, plan.hidden), dtype=torch.bfloat16, device=dev)
    args = [C.byref(plan.c_plan()), state["packed_w13"].data_ptr(), state["packed_w2"].data_ptr(),
            state["gs13"].data_ptr(), state["gs2"].data_ptr(), hidden.data_ptr(), hidden.stride(0),
            logits.data_ptr(), T, 0, 0, None, ids.data_ptr(), wts.data_ptr()]
    if with_workspace:
        args.append(state["workspace"].data_ptr())
    args += [out.data_ptr(), 0, torch.cuda.current_stream().cuda_stream]
    rc = getattr(_lib.lib(), fn_name)(*args)
    assert rc == 0, _lib.lib().okc_moe_strerror(rc)
    torch.cuda.synchronize()
    return out, ids, wts


def test_static_scratch_step_equals_workspace_step_twice_in_a_row():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    wl = synth.WORKLOADS["c1"]
    weights = synth.make_weights(wl, seed=77, device=dev)
    state = okc.prepare(weights, okc.MoEPlan(hidden=wl.hidden, inter=wl.inter, n_experts=wl.n_experts,
                                             top_k=wl.top_k, max_tokens=64))
    assert state["plan"].sizes().workspace_bytes <= 32 << 20
    for call, tokens in enumerate((33, 4)):           # the second call is smaller: stale rows stay behind it
        hidden, logits = synth.make_inputs(wl, seed=300 + call, device=dev, tokens=tokens)
        ref, ref_ids, ref_w = _step("okc_moe_step", state, hidden, logits, True)
        got, ids, w = _step("okc_moe_step_static_scratch", state, hidden, logits, False)
        assert torch.equal(ids, ref_ids) and torch.equal(w, ref_w), f"call {call}: routing differs"
        assert torch.equal(got, ref), f"call {call}: output differs from okc_moe_step"
        assert got.float().abs().max() > 0
        detail = C.c_int32(-1)
        rc = _lib.lib().okc_moe_read_status_static(torch.cuda.current_stream().cuda_stream, C.byref(detail))
        assert (rc, detail.value) == (0, 0), "no bounded wait ran out"


def test_static_scratch_rejects_plans_that_do_not_fit():
    assert torch.cuda.is_available()
    big = okc.MoEPlan(hidden=4096, inter=1536, n_experts=128, top_k=8, max_tokens=256)
    assert big.sizes().workspace_bytes > 32 << 20
    rc = _lib.lib().okc_moe_step_static_scratch(C.byref(big.c_plan()), None, None, None, None, None, 4096, None, 4, 0,
                                                0, None, None, None, None, 0, None)
    assert rc == _lib.OKC_ERR_TOO_LARGE
    assert b"capacity" in _lib.lib().okc_moe_strerror(rc)
