"""Worker of tests/test_ep_gpu.py: one process per GPU (torchrun), expert-parallel steps with the
peer-memory exchange against the NCCL exchange and the numpy oracle.  Prints "EP-PEER-OK"
on rank 0 when every check passed on every rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import okc_muse_kernels_b200 as okc  # noqa: E402
from okc_muse_kernels_b200 import ep, synth  # noqa: E402
from oracle import moe_np  # noqa: E402


def wide_rows(rank, world, dev):
    """A step whose own-row part of the fused combine + reduce has several times more CTAs than the
    GPU can hold at once (384 own rows x 7 column slices per rank): the kernel must not need them
    resident together.  Status 0, bit-equal to the unfused exchange, oracle parity on three tokens."""
    T, H, I, E, K = 384 * world, 7168, 256, 4 * world, 2
    wl = synth.Workload("wide", T, H, I, E, K)
    plan = ep.shard_plan(H, I, E, K, world, rank, max_tokens=T)
    mine = synth.make_weights(wl, seed=23, device=dev, n_experts=plan.local_count, first_expert=plan.local_start)
    fused = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="peer")
    split = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="peer", fuse_combine=False)
    t0, t1 = fused.own
    hidden, logits = synth.make_inputs(wl, seed=123, device=dev)
    ok = True
    for _ in range(2):
        a = fused.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        c = split.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        for layer in (fused, split):
            rc, _ = layer.peer.read_status()
            ok &= rc == 0
        ok &= bool(torch.equal(a, c))
    wn = synth.to_numpy_weights(synth.make_weights(wl, seed=23, device=dev))
    sub = [t0, (t0 + t1) // 2, t1 - 1]
    _, ref, _, _ = moe_np.moe_step(hidden.cpu().view(torch.uint16).numpy()[sub], logits.cpu().numpy()[sub], wn, K)
    good, msg = moe_np.compare(a.cpu().view(torch.uint16).numpy()[[s - t0 for s in sub]], ref, 1.5e-2)
    if not good:
        print(f"rank {rank} wide rows: {msg}", file=sys.stderr)
    return ok and good


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    T, H, I, E, K = 8 * world, 512, 256, 8 * world, 4
    wl = synth.Workload("ep", T, H, I, E, K, shared_inter=I)
    w = synth.make_weights(wl, seed=21, device=dev)             # the whole layer, the same bits on every rank
    plan = ep.shard_plan(H, I, E, K, world, rank, max_tokens=max(T, 16), shared_inter=I)
    mine = synth.make_weights(wl, seed=21, device=dev, n_experts=plan.local_count, first_expert=plan.local_start)
    peer = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="peer")                # fused combine + reduce
    split = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="peer", fuse_combine=False)
    plain = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="peer", route_in_gather=False)     # router as its own kernels
    nccl = ep.ExpertParallelMoE(plan, T, weights=mine, exchange="nccl")
    assert peer.route_in_gather and not plain.route_in_gather
    t0, t1 = peer.own
    wn = synth.to_numpy_weights(w)
    shared = {k[len("shared_"):]: v for k, v in wn.items() if k.startswith("shared_")}
    ok = True
    outs = []
    for step in range(4):
        hidden, logits = synth.make_inputs(wl, seed=100 + step, device=dev)
        a = peer.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        b = nccl.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        c = split.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        d = plain.step(hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()).clone()
        for layer in (peer, split, plain):
            rc, detail = layer.peer.read_status()
            ok &= rc == 0
        ok &= bool(torch.equal(a, c))                           # same sums in the same order
        ok &= bool(torch.equal(a, d))                           # the router inside the gather kernel routes the same
        ids_ref, _ = moe_np.route_softmax_topk(logits.cpu().numpy(), K)
        ok &= bool(np.array_equal(peer.peer.routed_views(K)[0].cpu().numpy(), ids_ref))
        if world == 2:
            ok &= bool(torch.equal(a, b))                       # two addends: the order cannot matter
        ok &= bool(torch.allclose(a.float(), b.float(), rtol=2 ** -7, atol=1e-5))
        _, ref, _, _ = moe_np.moe_step(hidden.cpu().view(torch.uint16).numpy(), logits.cpu().numpy(), wn, K,
                                       shared=shared)
        good, msg = moe_np.compare(a.cpu().view(torch.uint16).numpy(), ref[t0:t1], 1.5e-2)
        ok &= good
        if not good:
            print(f"rank {rank} step {step}: {msg}", file=sys.stderr)
        outs.append((hidden, logits, a))
    # the same steps replayed from a CUDA graph
    hidden, logits, want = outs[-1]
    ho, lo_ = hidden[t0:t1].contiguous(), logits[t0:t1].contiguous()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        peer.step(ho, lo_)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ok &= bool(torch.equal(peer.out, want))
    rc, detail = peer.peer.read_status()
    ok &= rc == 0
    ok &= wide_rows(rank, world, dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("EP-PEER-OK", flush=True)
    dist.barrier()
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
