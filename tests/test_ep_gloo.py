"""Expert-parallel host logic on CPU ranks (gloo, world_size 2 and 4): sharding of experts and
token blocks, the all-gather / reduce-scatter plumbing, and identical routing on every rank.  The
local compute is the numpy oracle injected into the harness seam of ExpertParallelMoE (the CUDA
step itself is covered by the -m gpu tests)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from okc_muse_kernels_b200 import ep, synth
from oracle import moe_np

WL = synth.Workload("ep", 8, 256, 256, 8, 2, shared_inter=256)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        weights = synth.to_numpy_weights(synth.make_weights(WL, seed=3, device="cpu"))
        shared = {k[len("shared_"):]: v for k, v in weights.items() if k.startswith("shared_")}
        hidden, logits = synth.make_inputs(WL, seed=4, device="cpu")
        plan = ep.shard_plan(WL.hidden, WL.inter, WL.n_experts, WL.top_k, world, rank, max_tokens=16,
                             shared_inter=WL.shared_inter)
        seen = {}

        def local_step(hidden_all, logits_all, own, out_f32):
            hb = hidden_all.view(torch.uint16).numpy()
            ids, w = moe_np.route_softmax_topk(logits_all.numpy(), WL.top_k)
            seen["ids"] = ids
            part = moe_np.experts(hb, ids, w, weights, local_start=plan.local_start, local_count=plan.local_count)
            part = part + moe_np.shared_expert(hb, shared, rows=np.arange(own[0], own[1]))
            out_f32.copy_(torch.from_numpy(part))

        def cast(src, dst):
            dst.copy_(src.to(torch.bfloat16))

        layer = ep.ExpertParallelMoE(plan, WL.tokens, group=None, local_step=local_step, cast=cast)
        t0, t1 = ep.token_block(WL.tokens, world, rank)
        assert (t0, t1) == layer.own
        out = layer.step(hidden[t0:t1], logits[t0:t1])
        # every rank saw all tokens and routed them identically
        all_ids = [None] * world
        dist.all_gather_object(all_ids, seen["ids"].tolist())
        assert all(a == all_ids[0] for a in all_ids)
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.view(torch.uint16).numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_plumbing_on_cpu_ranks(world, tmp_path):
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    weights = synth.to_numpy_weights(synth.make_weights(WL, seed=3, device="cpu"))
    shared = {k[len("shared_"):]: v for k, v in weights.items() if k.startswith("shared_")}
    hidden, logits = synth.make_inputs(WL, seed=4, device="cpu")
    ref_bits, ref, _ = moe_np.moe_step_ep(hidden.view(torch.uint16).numpy(), logits.numpy(), weights, WL.top_k, world, shared)
    gotf = moe_np.bf16_to_f32(got)
    # float32 sums in another order, then one bf16 rounding: a bf16 ulp (2^-8 relative) of slack
    assert np.allclose(gotf, moe_np.bf16_to_f32(ref_bits), rtol=2 ** -7, atol=1e-5), \
        "rank outputs, concatenated, differ from the single-host sum"
    # and the sharded answer equals the unsharded layer
    full_bits, full, _, _ = moe_np.moe_step(hidden.view(torch.uint16).numpy(), logits.numpy(), weights, WL.top_k, shared)
    assert np.allclose(gotf, moe_np.bf16_to_f32(full_bits), rtol=2 ** -7, atol=1e-5)


def test_shard_plan_and_token_block_errors():
    with pytest.raises(ValueError):
        ep.shard_plan(256, 256, 10, 2, 4, 0, 16)
    with pytest.raises(ValueError):
        ep.token_block(10, 4, 0)
    p = ep.shard_plan(7168, 2048, 256, 8, 8, 3, 128, shared_inter=2048)
    assert (p.local_start, p.local_count) == (96, 32)
    assert ep.token_block(128, 8, 3) == (48, 64)


# ------------------------------------------------------------------------------------------------
# Host-side failure detection (ep.StepGuard): a rank that leaves between steps, and a rank that is
# late.  Nothing here touches a GPU; the failures are made on the host.
def _guard_main(rank, world, port, store_port, out_dir, scenario):
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0))
    guard = ep.StepGuard(store, rank, world, deadline_s=1.5)
    plan = ep.shard_plan(WL.hidden, WL.inter, 9, 3, world, rank, max_tokens=16)
    tokens = 6

    def local_step(hidden_all, logits_all, own, out_f32):
        out_f32.copy_(hidden_all.float() * (rank + 1))

    def cast(src, dst):
        dst.copy_(src.to(torch.bfloat16))

    layer = ep.ExpertParallelMoE(plan, tokens, group=None, local_step=local_step, cast=cast, guard=guard)
    t0, t1 = ep.token_block(tokens, world, rank)
    hidden = torch.ones((tokens, WL.hidden), dtype=torch.bfloat16)
    logits = torch.zeros((tokens, 9))
    result = {"rank": rank}
    out = layer.step(hidden[t0:t1], logits[t0:t1])            # step 0: everybody is there
    result["step0"] = float(out.float().mean())               # 1 * (1 + 2 + 3)
    if scenario == "leave" and rank == 2:
        guard.leave()                                         # between steps, nothing in flight
        result["left"] = True
    else:
        if scenario == "late" and rank == 1:
            time.sleep(4.0)
        begin = time.perf_counter()
        try:
            layer.step(hidden[t0:t1], logits[t0:t1])
            result["step1"] = "ran"
        except ep.PeerLost as exc:
            result["step1"] = f"PeerLost: {exc}"
        result["seconds"] = time.perf_counter() - begin
    import json
    with open(os.path.join(out_dir, f"r{rank}.json.tmp"), "w") as f:
        json.dump(result, f)
    os.replace(os.path.join(out_dir, f"r{rank}.json.tmp"), os.path.join(out_dir, f"r{rank}.json"))
    if rank == 0:    # rank 0 hosts the store: it stays until every rank has reported
        t_end = time.monotonic() + 20
        while time.monotonic() < t_end and not all(os.path.exists(os.path.join(out_dir, f"r{r}.json")) for r in range(world)):
            time.sleep(0.05)
    os._exit(0)      # no teardown handshake with ranks that may be gone


@pytest.mark.parametrize("scenario", ["leave", "late"])
def test_a_rank_that_leaves_or_is_late_stops_the_others_on_the_host(scenario, tmp_path):
    import json
    world = 3
    mp.spawn(_guard_main, args=(world, _free_port(), _free_port(), str(tmp_path), scenario), nprocs=world, join=True)
    res = [json.load(open(tmp_path / f"r{r}.json")) for r in range(world)]
    assert all(abs(r["step0"] - 6.0) < 1e-6 for r in res)
    if scenario == "leave":
        assert res[2].get("left")
        for r in res[:2]:
            assert r["step1"].startswith("PeerLost") and "rank 2 left" in r["step1"], r["step1"]
            assert r["seconds"] < 1.0, "a rank known to have left is noticed without waiting for the deadline"
    else:
        for r in (res[0], res[2]):
            assert r["step1"].startswith("PeerLost") and "within" in r["step1"]
            assert 1.0 < r["seconds"] < 3.5
        # the late rank finds that the others gave up on the step and does not launch alone
        assert res[1]["step1"].startswith("PeerLost") and "gave up on step 1" in res[1]["step1"]
