"""B200-native (sm_100a) NVFP4 W4A16 MoE decode step behind the reference's callable surface.

    state = prepare(weights, MoEPlan(...))          # once: lossless repack of the NVFP4 experts
    out = moe_step(hidden_bf16, router_logits, state)   # router + experts, bf16 [T, H]
    out = kernel_fn(data, state)                    # the reference's entry: routing given

The CUDA kernels live in csrc/ and are reached through the C ABI of include/okc_moe.h
(libokc_moe_b200.so, built by ``python -m okc_muse_kernels_b200.build``).
"""
from .moe import HostStep, MoEPlan, OkcError, cast_bf16, experts_ep, experts_profiled, kernel_fn, moe_layer_step, moe_step, prepare, read_status, route, route_hidden, sorted_routes, split_router, unpack_bf16

__all__ = ["HostStep", "MoEPlan", "OkcError", "cast_bf16", "experts_ep", "experts_profiled", "kernel_fn", "moe_layer_step", "moe_step", "prepare", "read_status", "route", "route_hidden", "sorted_routes",
           "split_router", "unpack_bf16"]
