// Grouped NVFP4 x BF16 GEMMs of the MoE step on tcgen05 tensor cores, swap-AB:
//   D[128 weight rows, N tokens] += A[128, 16] * B[N, 16]^T     (tcgen05.mma kind::f16, FP32 in TMEM)
//
//   MODE 0  gate_up: unit = (expert, 128 gate rows + the matching 128 up rows); epilogue
//           inter = SiLU(gate * gs) * (up * gs) -> bf16, in expert order
//   MODE 1  down:    unit = (expert, two adjacent 128-row tiles of w2); epilogue
//           y[route] = acc * gs * routing weight -> f32, un-permuted to (token, slot) order
//
// One persistent CTA per SM, 24 warps:
//   warp 0        producer: one bulk copy of the 36 KB FP4 stage image + 2-D TMA tiles of the
//                 token operand (128-byte swizzle) per stage, mbarrier ring
//   warp 1        MMA issuer (one thread) and owner of the TMEM allocation
//   warps 4..19   dequantisers: thread = one weight row; FP4 + E4M3 from shared memory ->
//                 bf16x2 registers -> tcgen05.st into a 4-slot ring of A operands in TMEM
//   warps 20..23  epilogue: tcgen05.ld of the accumulators, scale, activation, store
//
// The reference computes the same products with mma.sync / wgmma on Hopper
// (muse_moe_w4a16/submission.py:3828-4014 `tk2f_consume`, :1909-2072 `tw_item`); nothing is shared
// with that code beyond the arithmetic (weights as the M operand, FP32 accumulation, the
// global scale and a power of two applied once in the epilogue, submission.py:3855,3983-3987).
#include <cuda_bf16.h>

#include "params.cuh"

namespace okc {

constexpr int kGemmThreads = 768;
constexpr int kDequantWarp0 = 4;
constexpr int kDequantWarps = 16;
constexpr int kEpilogueWarp0 = 20;
constexpr int kASlots = 4;            // ring of A operands in TMEM, 64 columns each (K = 64, two tiles)
constexpr int kASlotCols = 64;
constexpr int kAccCol0 = 256;         // accumulators live in TMEM columns [256, 512)
constexpr int kTmemCols = 512;
constexpr int kMaxStages = 6;

// Codes written to the status word when a wait gives up: role * 16 + barrier kind.
enum WaitCode { kWaitProducerEmpty = 0x11, kWaitMmaAccEmpty = 0x21, kWaitMmaFull = 0x22, kWaitMmaAFull = 0x23,
                kWaitDqFull = 0x31, kWaitDqAEmpty = 0x32, kWaitEpiAccFull = 0x41 };


struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t a_full[kASlots];
  uint64_t a_empty[kASlots];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_code;
};

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) okc_grouped_gemm(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem0 - smem_u32(smem_raw));
  const uint32_t stage_bytes = kStageBytes + static_cast<uint32_t>(p.ncap) * 512u;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_gen + static_cast<size_t>(p.n_stages) * stage_bytes);
  volatile int* abort_flag = &ctrl->abort_code;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int NS = p.n_stages;
  const int nbuf = (p.ncap <= 64) ? 2 : 1;

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&ctrl->full[i]), 1);
      mbar_init(smem_u32(&ctrl->empty[i]), kDequantWarps + 1);
    }
    for (int i = 0; i < kASlots; ++i) {
      mbar_init(smem_u32(&ctrl->a_full[i]), kDequantWarps);
      mbar_init(smem_u32(&ctrl->a_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctrl->acc_full[i]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[i]), 4);
    }
    ctrl->abort_code = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctrl->tmem_base;

  const int n_items = p.meta[kMetaItems];
  const int total_units = n_items * p.pairs;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      for (int i = 0; i < 4; ++i) tma_prefetch_desc(&p.bmap[i]);
      const uint64_t pol = policy_evict_first();
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < total_units; u += gridDim.x) {
        const int item = u / p.pairs, pair = u - item * p.pairs;
        const int4 wi = p.items[item];
        const int npad = wi.w;
        const int mi = (npad == 16) ? 0 : (npad == 32) ? 1 : (npad == 64) ? 2 : 3;
        const uint8_t* src = p.wpacked + static_cast<size_t>(wi.x) * p.expert_bytes +
                             static_cast<size_t>(pair) * p.stages * kStageBytes;
        for (int s = 0; s < p.stages; ++s, ++it) {
          const int st = it % NS;
          if (!mbar_wait(smem_u32(&ctrl->empty[st]), ((it / NS) & 1) ^ 1, abort_flag, kWaitProducerEmpty)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ctrl->full[st]);
          const uint32_t dst = smem0 + st * stage_bytes;
          mbar_expect_tx(bar, kStageBytes + npad * 512);
          bulk_g2s_hint(dst, src + static_cast<size_t>(s) * kStageBytes, kStageBytes, bar, pol);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tma_2d_g2s(dst + kStageBytes + kb * npad * 128, &p.bmap[mi], s * kStageK + kb * 64, wi.y, bar);
        }
      }
      if (!ok) {
        // give copies already issued a bounded chance to land before the CTA retires
        const int first = it > NS ? it - NS : 0;
        for (int j = first; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try(smem_u32(&ctrl->full[j % NS]), (j / NS) & 1) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it = 0, slot_it = 0, unit_it = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < total_units; u += gridDim.x, ++unit_it) {
        const int item = u / p.pairs;
        const int npad = p.items[item].w;
        const int buf = (nbuf == 2) ? (unit_it & 1) : 0;
        if (!mbar_wait(smem_u32(&ctrl->acc_empty[buf]), ((unit_it / nbuf) & 1) ^ 1, abort_flag, kWaitMmaAccEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t idesc = idesc_bf16_m128(npad);
        const uint32_t d0 = tmem + kAccCol0 + buf * 128;
        const uint32_t d1 = d0 + (nbuf == 2 ? 64 : 128);
        uint32_t acc = 0;
        for (int s = 0; ok && s < p.stages; ++s, ++it) {
          const int st = it % NS;
          if (!mbar_wait(smem_u32(&ctrl->full[st]), (it / NS) & 1, abort_flag, kWaitMmaFull)) { ok = false; break; }
          const uint32_t bsm = smem0 + st * stage_bytes + kStageBytes;
          for (int kb = 0; kb < 4; ++kb, ++slot_it) {
            const int sl = slot_it % kASlots;
            if (!mbar_wait(smem_u32(&ctrl->a_full[sl]), (slot_it / kASlots) & 1, abort_flag, kWaitMmaAFull)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a0 = tmem + sl * kASlotCols;
            const uint64_t bd = smem_desc_sw128(bsm + kb * npad * 128);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint64_t bdk = bd + static_cast<uint64_t>((k4 * 32) >> 4);
              mma_ts(d0, a0 + k4 * 8, bdk, idesc, acc);
              mma_ts(d1, a0 + 32 + k4 * 8, bdk, idesc, acc);
              acc = 1;
            }
            mma_commit(smem_u32(&ctrl->a_empty[sl]));
          }
          if (ok) mma_commit(smem_u32(&ctrl->empty[st]));
        }
        if (ok) mma_commit(smem_u32(&ctrl->acc_full[buf]));
      }
    }
  } else if (warp >= kDequantWarp0 && warp < kDequantWarp0 + kDequantWarps) {
    // ------------------------------------------------------------ dequantisers
    const int dw = warp - kDequantWarp0;
    const int q = warp & 3;               // TMEM lane quarter this warp may touch
    const int tile = (dw >> 2) & 1;       // first or second tile of the pair
    const int half = dw >> 3;             // which 32-element chunk of a 64-element slot
    const int row = q * 32 + lane;
    const uint32_t trow = tmem + (static_cast<uint32_t>(q * 32) << 16) + tile * 32 + half * 16;
    int it = 0, slot_it = 0;
    bool ok = true;
    for (int u = blockIdx.x; ok && u < total_units; u += gridDim.x) {
      for (int s = 0; ok && s < p.stages; ++s, ++it) {
        const int st = it % NS;
        if (!mbar_wait(smem_u32(&ctrl->full[st]), (it / NS) & 1, abort_flag, kWaitDqFull)) { ok = false; break; }
        const uint8_t* img = smem_gen + static_cast<size_t>(st) * stage_bytes + tile * kTileBytes;
        uint4 w[4];
        uint32_t sc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int chunk = 2 * j + half;
          w[j] = *reinterpret_cast<const uint4*>(img + chunk * (kTileRows * 16) + row * 16);
          sc[j] = *reinterpret_cast<const uint16_t*>(img + kTileCodeBytes + chunk * (kTileRows * 2) + row * 2);
        }
        // the stage's bytes are in registers: hand the shared-memory slot back
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->empty[st]));
#pragma unroll
        for (int j = 0; j < 4; ++j, ++slot_it) {
          const int sl = slot_it % kASlots;
          uint32_t regs[16];
          dequant_chunk(w[j], sc[j], regs);
          if (!mbar_wait(smem_u32(&ctrl->a_empty[sl]), ((slot_it / kASlots) & 1) ^ 1, abort_flag, kWaitDqAEmpty)) ok = false;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          tmem_st16(trow + sl * kASlotCols, regs);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctrl->a_full[sl]));
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    int unit_it = 0;
    bool ok = true;
    for (int u = blockIdx.x; ok && u < total_units; u += gridDim.x, ++unit_it) {
      const int item = u / p.pairs, pair = u - item * p.pairs;
      const int4 wi = p.items[item];
      const int n_rows = wi.z, npad = wi.w;
      const int buf = (nbuf == 2) ? (unit_it & 1) : 0;
      const float sc = p.gs[wi.x] * 256.0f;
      if (!mbar_wait(smem_u32(&ctrl->acc_full[buf]), (unit_it / nbuf) & 1, abort_flag, kWaitEpiAccFull)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d0 = tmem + lane_off + kAccCol0 + buf * 128;
      const uint32_t d1 = d0 + (nbuf == 2 ? 64 : 128);
      for (int c0 = 0; c0 < npad; c0 += 16) {
        uint32_t a[16], b[16];
        tmem_ld16(d0 + c0, a);
        tmem_ld16(d1 + c0, b);
        tmem_wait_ld();
        if (c0 + 16 >= npad) {
          // last read of this accumulator: the MMA warp may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[buf]));
        }
        if (c0 < n_rows) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = c0 + j;
            if (n < n_rows) {
              const float va = __uint_as_float(a[j]) * sc;
              const float vb = __uint_as_float(b[j]) * sc;
              if (MODE == 0) {
                const float act = va / (1.0f + __expf(-va)) * vb;
                p.inter[static_cast<size_t>(wi.y + n) * p.I + pair * kTileRows + row] =
                    __bfloat16_as_ushort(__float2bfloat16_rn(act));
              } else {
                const int route = p.sorted[wi.y + n];
                const float wgt = p.weighted ? p.wsorted[wi.y + n] : 1.0f;
                float* dst = p.y + static_cast<size_t>(route) * p.H + pair * 2 * kTileRows + row;
                dst[0] = va * wgt;
                dst[kTileRows] = vb * wgt;
              }
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctrl->abort_code != 0) {
    atomicCAS(const_cast<int32_t*>(&p.meta[kMetaStatus]), 0, OKC_ERR_TIMEOUT);
    atomicCAS(const_cast<int32_t*>(&p.meta[kMetaDetail]), 0, (MODE << 8) | ctrl->abort_code);
  }
}

// Per-token combine: out[t] = sum over the token's local routes (slot order) of y[t*kk + slot],
// optionally through the reference's post-expert norm (scale by 1 + w, RMSNorm eps 1e-8, then the
// routing weight; muse_moe_w4a16/reference.py:88-90,106).  Rows with no local route become zero.

constexpr int kCombineThreads = 256;
constexpr int kCombineMaxPer = 8;   // float4 per thread: H <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kCombineThreads) okc_combine(const CombineParams p) {
  const int t = blockIdx.x, tid = threadIdx.x;
  const int nvec = p.H / 4;
  float4 acc[kCombineMaxPer];
#pragma unroll
  for (int i = 0; i < kCombineMaxPer; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  __shared__ float red[kCombineThreads / 32];
  for (int s = 0; s < p.kk; ++s) {
    const int q = p.pos[t * p.kk + s];
    if (q < 0) continue;   // uniform over the block
    const float4* yr = reinterpret_cast<const float4*>(p.y + static_cast<size_t>(t * p.kk + s) * p.H);
    if (p.post_w == nullptr) {
#pragma unroll
      for (int i = 0; i < kCombineMaxPer; ++i) {
        const int v = tid + i * kCombineThreads;
        if (v < nvec) {
          const float4 a = yr[v];
          acc[i].x += a.x; acc[i].y += a.y; acc[i].z += a.z; acc[i].w += a.w;
        }
      }
    } else {
      float4 tmp[kCombineMaxPer];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kCombineMaxPer; ++i) {
        const int v = tid + i * kCombineThreads;
        if (v < nvec) {
          float4 a = yr[v];
          const uint2 wb = *reinterpret_cast<const uint2*>(p.post_w + v * 4);
          a.x *= 1.0f + __uint_as_float(wb.x << 16);
          a.y *= 1.0f + __uint_as_float(wb.x & 0xFFFF0000u);
          a.z *= 1.0f + __uint_as_float(wb.y << 16);
          a.w *= 1.0f + __uint_as_float(wb.y & 0xFFFF0000u);
          tmp[i] = a;
          ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      __syncthreads();
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kCombineThreads / 32; ++i) tot += red[i];
      const float scale = p.wsorted[q] * rsqrtf(tot / static_cast<float>(p.H) + 1e-8f);
#pragma unroll
      for (int i = 0; i < kCombineMaxPer; ++i) {
        const int v = tid + i * kCombineThreads;
        if (v < nvec) {
          acc[i].x += tmp[i].x * scale; acc[i].y += tmp[i].y * scale;
          acc[i].z += tmp[i].z * scale; acc[i].w += tmp[i].w * scale;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kCombineMaxPer; ++i) {
    const int v = tid + i * kCombineThreads;
    if (v < nvec) {
      if (p.out_f32) {
        reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<size_t>(t) * p.H)[v] = acc[i];
      } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i].x, acc[i].y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i].z, acc[i].w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + static_cast<size_t>(t) * p.H)[v] = o;
      }
    }
  }
}

// f32 -> bf16 (round to nearest even), four elements per thread: the last step of the
// expert-parallel path, after the reduce-scatter of the FP32 partial sums.
__global__ void __launch_bounds__(256) okc_cast_bf16(const float4* __restrict__ in, uint2* __restrict__ out, int64_t nvec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const float4 a = in[i];
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(a.z, a.w);
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&lo);
  o.y = *reinterpret_cast<const uint32_t*>(&hi);
  out[i] = o;
}

cudaError_t launch_cast(const float* in, void* out_bf16, int64_t n, cudaStream_t stream) {
  const int64_t nvec = n / 4;
  okc_cast_bf16<<<static_cast<unsigned>((nvec + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(in), static_cast<uint2*>(out_bf16), nvec);
  return cudaGetLastError();
}

size_t gemm_smem_bytes(int n_stages, int ncap) {
  return 1024 + static_cast<size_t>(n_stages) * (kStageBytes + static_cast<size_t>(ncap) * 512) + sizeof(Ctrl);
}

int gemm_stages_for(int ncap) {
  // 227 KB of shared memory per CTA
  const size_t budget = 232448 - 1024 - sizeof(Ctrl);
  int n = static_cast<int>(budget / (kStageBytes + static_cast<size_t>(ncap) * 512));
  return n > kMaxStages ? kMaxStages : n;
}

cudaError_t launch_gemm(int mode, const GemmParams& p, int grid, cudaStream_t stream) {
  const size_t smem = gemm_smem_bytes(p.n_stages, p.ncap);
  cudaError_t e;
  if (mode == 0) {
    e = cudaFuncSetAttribute(okc_grouped_gemm<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    okc_grouped_gemm<0><<<grid, kGemmThreads, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(okc_grouped_gemm<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    okc_grouped_gemm<1><<<grid, kGemmThreads, smem, stream>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t launch_combine(const CombineParams& p, int T, cudaStream_t stream) {
  okc_combine<<<T, kCombineThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace okc
