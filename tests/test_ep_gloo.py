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
