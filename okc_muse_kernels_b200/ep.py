"""Expert-parallel MoE step over the GPUs of one box: one process per GPU, NCCL over NVLink.

Sharding follows the reference's expert-parallel semantics (muse_moe_w4a16/reference.py:22,98-101:
a GPU computes only the routes whose expert id lies in its contiguous local range, and the layer
output is the sum of the GPUs' partial results); the reference never runs that sum ("the expert
all-reduce is not run", muse_moe_w4a16/baseline.py:8), so the exchange steps here are new:

    1. all-gather of the ranks' token blocks: hidden bf16 [T/world, H] and router logits f32 [T/world, E]
       (or, with the router inside the gather kernel, the ids and weights of the rank's own tokens)
    2. every rank routes all T tokens identically (or sorts the gathered routing) and runs its local experts
       on them, plus the replicated shared expert on its own token block only -> FP32 partial sums [T, H]
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
import datetime
import os
import time
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
    """The ranks' exchange buffers, each mapped into every rank, and the exchange kernels.

    The default constructor takes the buffers from torch's symmetric-memory allocator (cuMemCreate +
    cuMemMap with access for every GPU of the group) and raises RuntimeError on every rank if they
    cannot be mapped.  ``from_buffers`` takes addresses the caller already has (any peer mapping; or
    several buffers on one device, for a harness that runs the ranks one after the other).
    ``wait_limit_ms`` bounds every wait on another rank (0: five seconds)."""

    def __init__(self, tokens: int, hidden: int, n_experts: int, group=None, device=None, wait_limit_ms: int = 0):
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > _lib.EP_MAX_RANKS:
            raise ValueError(f"at most {_lib.EP_MAX_RANKS} ranks")
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        nbytes = self.buffer_bytes(tokens, hidden, n_experts)
        ok, why = 1, ""
        buf, ptrs = None, []
        try:
            buf, ptrs, self._keep = _map_with_symmetric_memory(nbytes, group, device)
        except Exception as exc:   # noqa: BLE001 - whatever went wrong, every rank must learn of it
            ok, why = 0, str(exc)
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) != 1:
            raise RuntimeError(f"the ranks' exchange buffers could not be mapped into each other ({why or 'another rank failed'})")
        self._setup(rank, world, tokens, hidden, n_experts, buf, ptrs, wait_limit_ms)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)     # every buffer is zeroed and mapped before anybody's first step

    @staticmethod
    def buffer_bytes(tokens: int, hidden: int, n_experts: int) -> int:
        n = int(_lib.lib().okc_ep_buffer_bytes(tokens, hidden, n_experts))
        if n == 0:
            raise ValueError("bad exchange-buffer shape")
        return n

    @classmethod
    def from_buffers(cls, rank: int, world: int, tokens: int, hidden: int, n_experts: int, own: torch.Tensor,
                     ptrs: list[int], wait_limit_ms: int = 0) -> "PeerExchange":
        """``own``: this rank's zeroed uint8 buffer of ``buffer_bytes`` bytes; ``ptrs[r]``: the address
        under which this process reaches rank r's buffer (``ptrs[rank] == own.data_ptr()``)."""
        self = cls.__new__(cls)
        self.group = None
        self._setup(rank, world, tokens, hidden, n_experts, own, ptrs, wait_limit_ms)
        return self

    def _setup(self, rank, world, tokens, hidden, n_experts, buf, ptrs, wait_limit_ms):
        if len(ptrs) != world or ptrs[rank] != buf.data_ptr():
            raise ValueError("ptrs must hold one address per rank, the rank's own buffer at its own index")
        self.world, self.rank, self.buf = world, rank, buf
        self.comm = _lib.EpComm(rank=rank, world=world, tokens=tokens, hidden=hidden, n_experts=n_experts,
                                wait_limit_ms=int(wait_limit_ms))
        for r, ptr in enumerate(ptrs):
            self.comm.peer[r] = ptr
        views = [C.c_void_p() for _ in range(3)]
        _lib.check(_lib.lib().okc_ep_views(C.byref(self.comm), *[C.byref(v) for v in views]), "okc_ep_views")
        base = buf.data_ptr()

        def view(ptr, nelem, dtype, shape):
            off = ptr.value - base
            return buf[off:off + nelem * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

        self.hidden_all = view(views[0], tokens * hidden, torch.bfloat16, (tokens, hidden))
        self.logits_all = view(views[1], tokens * n_experts, torch.float32, (tokens, n_experts))
        self.partial = view(views[2], tokens * hidden, torch.float32, (tokens, hidden))

    def gather_tokens(self, hidden_own: torch.Tensor, logits_own: torch.Tensor) -> None:
        if hidden_own.stride(-1) != 1 or not logits_own.is_contiguous():
            raise ValueError("token rows must be contiguous")
        _lib.check(_lib.lib().okc_ep_gather_tokens(
            C.byref(self.comm), hidden_own.data_ptr(), hidden_own.stride(0), logits_own.data_ptr(),
            torch.cuda.current_stream().cuda_stream), "okc_ep_gather_tokens")

    def route_gather(self, state: dict, hidden_own: torch.Tensor, logits_own: torch.Tensor):
        """The token all-gather with the router in it (one kernel): routes this rank's own token block, sends
        rows + ids + weights to every rank, waits for every rank's, sorts the whole step's routes into the
        state's workspace.  Returns views (ids int32 [T, k], weights f32 [T, k]) of all tokens' routing in this
        rank's buffer; go on with ``experts_ep`` (or ``moe._experts`` + ``reduce_scatter``)."""
        plan = state["plan"]
        if hidden_own.stride(-1) != 1 or not logits_own.is_contiguous():
            raise ValueError("token rows must be contiguous")
        _lib.check(_lib.lib().okc_ep_route_gather(
            C.byref(plan.c_plan()), C.byref(self.comm), hidden_own.data_ptr(), hidden_own.stride(0), logits_own.data_ptr(),
            state["workspace"].data_ptr(), torch.cuda.current_stream().cuda_stream), "okc_ep_route_gather")
        return self.routed_views(plan.top_k)

    def routed_views(self, top_k: int):
        if getattr(self, "_routed", None) is None or self._routed[0] != top_k:
            a, b = C.c_void_p(), C.c_void_p()
            _lib.check(_lib.lib().okc_ep_routed_views(C.byref(self.comm), top_k, C.byref(a), C.byref(b)), "okc_ep_routed_views")
            base, T = self.buf.data_ptr(), self.comm.tokens
            n = T * top_k * 4
            ids = self.buf[a.value - base:a.value - base + n].view(torch.int32).view(T, top_k)
            wts = self.buf[b.value - base:b.value - base + n].view(torch.float32).view(T, top_k)
            self._routed = (top_k, ids, wts)
        return self._routed[1], self._routed[2]

    def reduce_scatter(self, out: torch.Tensor) -> None:
        _lib.check(_lib.lib().okc_ep_reduce_scatter(C.byref(self.comm), out.data_ptr(),
                                                   torch.cuda.current_stream().cuda_stream), "okc_ep_reduce_scatter")

    def mark_arrived(self, which: str, from_rank: int) -> None:
        """Raises, in this rank's own buffer, the flag rank ``from_rank`` raises when its token rows
        (``which="tokens"``) or its partial sums (``"partial"``) of the coming exchange are in place.
        For a harness that runs the ranks of a step one after the other on one device: there the data
        of the rank that runs later is put in place by other means, and no kernel may wait for a
        kernel launched after it."""
        _lib.check(_lib.lib().okc_ep_mark_arrived(C.byref(self.comm), {"tokens": 0, "partial": 1}[which], int(from_rank),
                                                 torch.cuda.current_stream().cuda_stream), "okc_ep_mark_arrived")

    def read_status(self) -> tuple[int, int]:
        detail = C.c_int32(0)
        rc = _lib.lib().okc_ep_read_status(C.byref(self.comm), torch.cuda.current_stream().cuda_stream, C.byref(detail))
        return rc, detail.value

    def reset(self) -> None:
        """Zeroes this rank's buffer (step counts, flags, status).  After a wait that ran out the ranks'
        step counts may differ: every rank resets, with a host-side barrier before and after, between
        steps."""
        self.buf.zero_()
        torch.cuda.synchronize(self.buf.device)
        if self.group is not None or (dist.is_available() and dist.is_initialized() and self.world > 1):
            dist.barrier(group=self.group)


class PeerLost(RuntimeError):
    """A rank of the expert-parallel group left, or did not reach the step within the deadline."""


class StepGuard:
    """Host-side failure detection for the expert-parallel step: before a rank launches step n it
    checks in through the process group's key-value store and waits, up to ``deadline_s``, until
    every rank has checked in for step n.  A rank that leaves (``leave()``, between steps, nothing
    in flight) or that is late makes the others raise ``PeerLost`` on the host before they launch
    anything, so that no kernel or collective is left waiting for a rank that will not come.

    The device-side waits of the exchange kernels are bounded as well, but a wait that runs out there
    costs the step; this check costs a store round trip and keeps the GPU out of it."""

    def __init__(self, store, rank: int, world: int, deadline_s: float = 5.0, prefix: str = "okc_ep"):
        self.store, self.rank, self.world = store, rank, world
        self.deadline = datetime.timedelta(seconds=deadline_s)
        self.prefix = prefix
        self.n = 0

    def _key(self, kind: str, n, rank: int) -> str:
        return f"{self.prefix}/{kind}/{n}/{rank}"

    def check_in(self) -> int:
        """Call before launching a step.  Returns the step number; raises PeerLost (and then counts
        as gone itself, so that a rank that arrives late does not launch alone)."""
        n = self.n
        self.store.set(self._key("step", n, self.rank), "1")
        others = [r for r in range(self.world) if r != self.rank]
        keys = [self._key("step", n, r) for r in others]
        t_end = time.monotonic() + self.deadline.total_seconds()
        while True:
            self._raise_if_gone(others, n)     # a rank that went is noticed at once, not at the deadline
            try:
                if not keys or self.store.check(keys):
                    break
            except Exception:      # noqa: BLE001 - a store that cannot answer: the deadline decides
                pass
            if time.monotonic() >= t_end:
                msg = f"not every rank reached step {n} within {self.deadline.total_seconds():.1f} s"
                self.leave(f"gave up on step {n}: {msg}")
                raise PeerLost(msg)
            time.sleep(0.002)
        self.n = n + 1
        return n

    def _gone(self, r: int) -> str | None:
        """What rank r said when it went (None: it is still there)."""
        key = self._key("gone", "x", r)
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:          # noqa: BLE001 - a store that cannot answer: the deadline decides
            return None

    def _raise_if_gone(self, others, n) -> None:
        for r in others:
            why = self._gone(r)
            if why is not None:
                msg = f"rank {r} {why}"
                self.leave(f"gave up on step {n}: {msg}")
                raise PeerLost(msg)

    def leave(self, why: str = "left") -> None:
        """Call between steps, with none of this rank's kernels or collectives in flight."""
        self.store.set(self._key("gone", "x", self.rank), why)


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
                 device: torch.device | str | None = None, exchange: str = "nccl", fuse_combine: bool = True,
                 guard: "StepGuard | None" = None, wait_limit_ms: int = 0, route_in_gather: bool = True):
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
        self.guard = guard
        # peer exchange: the combine and the reduce-scatter as one kernel (not with the post-expert
        # norm, which needs whole rows before the sum)
        self.fuse_combine = bool(fuse_combine and exchange == "peer" and not plan.post_norm)
        # peer exchange: the router and the sort inside the token all-gather kernel (needs 2 k <= E)
        self.route_in_gather = bool(route_in_gather and exchange == "peer" and 2 * plan.top_k <= plan.n_experts)
        self.peer = None
        if exchange == "peer":
            self.peer = PeerExchange(tokens, plan.hidden, plan.n_experts, group=group, device=device,
                                     wait_limit_ms=wait_limit_ms)
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
        of the layer output).  The returned tensor is reused by the next call.  With a ``guard`` the
        rank first checks in on the host and raises ``PeerLost`` instead of launching when a rank left
        or is late (not while the step is being captured into a CUDA graph: replays do not pass here)."""
        if self.guard is not None:
            self.guard.check_in()
        if self.peer is not None:
            if self.route_in_gather:
                self.peer.route_gather(self.state, hidden_own, logits_own)
                if self.fuse_combine:
                    experts_ep(self.hidden_all, self.state, self.peer.comm, self.out)
                else:
                    from .moe import _check_hidden, _experts
                    hidden, stride = _check_hidden(self.hidden_all, self.plan)
                    _experts(hidden, stride, self.tokens, self.state, self.partial, True)
                    self.peer.reduce_scatter(self.out)
                return self.out
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
