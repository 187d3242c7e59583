"""Expert-parallel MoE step over the GPUs of one box: one process per GPU, NCCL over NVLink.

Sharding follows the reference's expert-parallel semantics (muse_moe_w4a16/reference.py:22,98-101:
a GPU computes only the routes whose expert id lies in its contiguous local range, and the layer
output is the sum of the GPUs' partial results); the reference never runs that sum ("the expert
all-reduce is not run", muse_moe_w4a16/baseline.py:8), so the exchange steps here are new:

    1. all-gather of the ranks' token blocks: hidden bf16 [T/world, H] and router logits f32 [T/world, E]
    2. every rank routes all T tokens identically and runs its local experts on them, plus the
       replicated shared expert on its own token block only -> FP32 partial sums [T, H]
    3. reduce-scatter of the partial sums (FP32, so the cross-GPU sum adds no bf16 rounding)
    4. cast of the rank's own rows to bf16

Rank r holds experts [r*E/world, (r+1)*E/world) and owns token rows [r*T/world, (r+1)*T/world).

Two implementations of steps 1 and 3 + 4:

  * ``exchange="peer"``: this library's own kernels over peer memory (``PeerExchange``): every rank
    maps every rank's exchange buffer; one kernel stores the rank's token block into all buffers and
    waits for the others' (step 1), one kernel pulls the rank's rows of all partial sums, adds them
    in rank order and rounds once (steps 3 + 4) -- by default fused with the per-token combine of the
    local experts' outputs (``fuse_combine``).  Two launches instead of three collectives and a cast.
  * ``exchange="nccl"``: ``all_gather_into_tensor`` x 2, ``reduce_scatter_tensor``, the cast kernel.
    Also what the CPU test harness (gloo) runs.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib
from .moe import MoEPlan, cast_bf16, experts_ep, moe_step, prepare, route


def shard_plan(hidden: int, inter: int, n_experts: int, top_k: int, world: int, rank: int, max_tokens: int,
               shared_inter: int = 0) -> MoEPlan:
    """The plan of rank `rank`'s shard: experts cut contiguously, E/world per rank."""
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not divide over {world} ranks")
    per = n_experts // world
    return MoEPlan(hidden=hidden, inter=inter, n_experts=n_experts, top_k=top_k, local_start=rank * per,
                   local_count=per, shared_inter=shared_inter, max_tokens=max_tokens)


def token_block(tokens: int, world: int, rank: int) -> tuple[int, int]:
    if tokens % world:
        raise ValueError(f"{tokens} tokens do not divide over {world} ranks")
    tb = tokens // world
    return rank * tb, (rank + 1) * tb


def _reduce_scatter_rows(own: torch.Tensor, full: torch.Tensor, group) -> None:
    """own[tb, H] = sum over ranks of full[rank block].  NCCL has the collective; gloo (the CPU
    test harness) does not, there the sum is an all-reduce followed by a slice."""
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(own, full, group=group)
    else:
        dist.all_reduce(full, group=group)
        r = dist.get_rank(group)
        own.copy_(full[r * own.shape[0]:(r + 1) * own.shape[0]])


def _map_with_symmetric_memory(nbytes: int, group, device):
    """One zeroed buffer per rank from torch's symmetric-memory allocator, mapped by all ranks.
    NVLink multicast is not used by the exchange kernels and is kept off."""
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm_mem
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
    ptrs = [int(x) for x in handle.buffer_ptrs]
    return buf, ptrs, handle


class PeerExchange:
    """The ranks' exchange buffers, each mapped into every rank (torch's symmetric-memory allocator:
    cuMemCreate + cuMemMap with access for every GPU of the group), and the two exchange kernels.
    Raises RuntimeError on every rank if the buffers cannot be mapped."""

    def __init__(self, tokens: int, hidden: int, n_experts: int, group=None, device=None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _lib.EP_MAX_RANKS:
            raise ValueError(f"at most {_lib.EP_MAX_RANKS} ranks")
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        nbytes = int(_lib.lib().okc_ep_buffer_bytes(tokens, hidden, n_experts))
        ok, why = 1, ""
        try:
            self.buf, ptrs, self._keep = _map_with_symmetric_memory(nbytes, group, device)
        except Exception as exc:   # noqa: BLE001 - whatever went wrong, every rank must learn of it
            ok, why = 0, str(exc)
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) != 1:
            raise RuntimeError(f"the ranks' exchange buffers could not be mapped into each other ({why or 'another rank failed'})")
        self.comm = _lib.EpComm(rank=self.rank, world=self.world, tokens=tokens, hidden=hidden, n_experts=n_experts)
        for r, ptr in enumerate(ptrs):
            self.comm.peer[r] = ptr
        views = [C.c_void_p() for _ in range(3)]
        _lib.check(_lib.lib().okc_ep_views(C.byref(self.comm), *[C.byref(v) for v in views]), "okc_ep_views")
        base = self.buf.data_ptr()

        def view(ptr, nelem, dtype, shape):
            off = ptr.value - base
            return self.buf[off:off + nelem * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

        self.hidden_all = view(views[0], tokens * hidden, torch.bfloat16, (tokens, hidden))
        self.logits_all = view(views[1], tokens * n_experts, torch.float32, (tokens, n_experts))
        self.partial = view(views[2], tokens * hidden, torch.float32, (tokens, hidden))
        torch.cuda.synchronize(device)
        dist.barrier(group=group)     # every buffer is zeroed and mapped before anybody's first step

    def gather_tokens(self, hidden_own: torch.Tensor, logits_own: torch.Tensor) -> None:
        if hidden_own.stride(-1) != 1 or not logits_own.is_contiguous():
            raise ValueError("token rows must be contiguous")
        _lib.check(_lib.lib().okc_ep_gather_tokens(
            C.byref(self.comm), hidden_own.data_ptr(), hidden_own.stride(0), logits_own.data_ptr(),
            torch.cuda.current_stream().cuda_stream), "okc_ep_gather_tokens")

    def reduce_scatter(self, out: torch.Tensor) -> None:
        _lib.check(_lib.lib().okc_ep_reduce_scatter(C.byref(self.comm), out.data_ptr(),
                                                   torch.cuda.current_stream().cuda_stream), "okc_ep_reduce_scatter")

    def read_status(self) -> tuple[int, int]:
        detail = C.c_int32(0)
        rc = _lib.lib().okc_ep_read_status(C.byref(self.comm), torch.cuda.current_stream().cuda_stream, C.byref(detail))
        return rc, detail.value


class ExpertParallelMoE:
    """One rank's end of the expert-parallel step.

    ``local_step(hidden_all, logits_all, own_tokens, out_f32)`` computes the rank's FP32 partial sums;
    by default it is this library's CUDA step on the state prepared from ``weights`` (the rank's
    local experts, or the whole layer from which the local range is taken).  A test harness may
    inject ``local_step`` and ``cast`` (both or neither) to exercise the sharding and the collectives
    on CPU ranks; nothing in this module computes on the CPU by itself.
    """

    def __init__(self, plan: MoEPlan, tokens: int, weights: dict | None = None, group=None,
                 local_step: Callable | None = None, cast: Callable | None = None,
                 device: torch.device | str | None = None, exchange: str = "nccl", fuse_combine: bool = True):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.plan = plan
        self.tokens = tokens
        self.own = token_block(tokens, self.world, self.rank)
        tb = tokens // self.world
        if local_step is None:
            if weights is None:
                raise ValueError("weights are required for the CUDA path")
            self.state = prepare(weights, plan)
            device = self.state["workspace"].device
            self._local_step = self._cuda_step
            self._cast = cast_bf16
        else:
            if cast is None:
                raise ValueError("a harness that injects local_step must inject cast too")
            self.state = None
            self._local_step = local_step
            self._cast = cast
            device = torch.device(device or "cpu")
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange is 'nccl' or 'peer'")
        if exchange == "peer" and local_step is not None:
            raise ValueError("the peer-memory exchange runs on GPUs only")
        self.exchange = exchange
        # peer exchange: the combine and the reduce-scatter as one kernel (not with the post-expert
        # norm, which needs whole rows before the sum)
        self.fuse_combine = bool(fuse_combine and exchange == "peer" and not plan.post_norm)
        self.peer = None
        if exchange == "peer":
            self.peer = PeerExchange(tokens, plan.hidden, plan.n_experts, group=group, device=device)
            self.hidden_all, self.logits_all, self.partial = self.peer.hidden_all, self.peer.logits_all, self.peer.partial
        else:
            self.hidden_all = torch.empty((tokens, plan.hidden), dtype=torch.bfloat16, device=device)
            self.logits_all = torch.empty((tokens, plan.n_experts), dtype=torch.float32, device=device)
            self.partial = torch.empty((tokens, plan.hidden), dtype=torch.float32, device=device)
        self.own_f32 = torch.empty((tb, plan.hidden), dtype=torch.float32, device=device)
        self.out = torch.empty((tb, plan.hidden), dtype=torch.bfloat16, device=device)

    def _cuda_step(self, hidden_all, logits_all, own_tokens, out_f32):
        return moe_step(hidden_all, logits_all, self.state, out_f32=True, own_tokens=own_tokens, out=out_f32)

    def step(self, hidden_own: torch.Tensor, logits_own: torch.Tensor) -> torch.Tensor:
        """hidden_own bf16 [T/world, H], logits_own f32 [T/world, E] -> bf16 [T/world, H] (this rank's rows
        of the layer output).  The returned tensor is reused by the next call."""
        if self.peer is not None:
            self.peer.gather_tokens(hidden_own, logits_own)
            if self.fuse_combine:
                route(self.logits_all, self.state, own_tokens=self.own)
                experts_ep(self.hidden_all, self.state, self.peer.comm, self.out)
            else:
                self._local_step(self.hidden_all, self.logits_all, self.own, self.partial)
                self.peer.reduce_scatter(self.out)
            return self.out
        dist.all_gather_into_tensor(self.hidden_all, hidden_own.contiguous(), group=self.group)
        dist.all_gather_into_tensor(self.logits_all, logits_own.contiguous(), group=self.group)
        self._local_step(self.hidden_all, self.logits_all, self.own, self.partial)
        _reduce_scatter_rows(self.own_f32, self.partial, self.group)
        self._cast(self.own_f32, self.out)
        return self.out
