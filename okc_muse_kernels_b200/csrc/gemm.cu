// Grouped NVFP4 x BF16 GEMMs of the MoE step on tcgen05 tensor cores, swap-AB:
//   D[128 weight rows, N tokens] += A[128, 16] * B[N, 16]^T     (tcgen05.mma kind::f16, FP32 in TMEM)
//
//   MODE 0  gate_up: unit = (expert, 128 gate rows + the matching 128 up rows); epilogue
//           inter = SiLU(gate * gs) * (up * gs) -> bf16, in expert order
//   MODE 1  down:    unit = (expert, two adjacent 128-row tiles of w2); epilogue
//           y[route] = acc * gs * routing weight -> f32, un-permuted to (token, slot) order
//
// One persistent CTA per SM, 29 warps:
//   warp 28       producer: one bulk copy of the 36 KB FP4 stage image + 2-D TMA tiles of the
//                 token operand (128-byte swizzle) per stage, mbarrier ring.  The whole warp runs
//                 the loop; lane 0 takes the units and starts the weight copies, the token copies
//                 of a stage start from as many lanes at once (steps of up to 8 tokens: a copy per
//                 row straight from the caller's array, no gathered copy of the rows)
//   warps 0..7    MMA issuers, whole warps running the loops, one elected lane issuing.  A thread needs 100+ cycles to issue one
//                 tcgen05.mma whatever its N (more when its warp competes for issue slots), and
//                 issue from several warps overlaps, so the 32 MMAs of a narrow item's stage are
//                 spread over eight issuers: (tile of the pair) x (64-wide K block of the stage).
//                 Each issuer adds into its own accumulator, which keeps the order of additions
//                 fixed; the epilogue adds the four K-block partials in a fixed order.  For a wide
//                 item the two issuers of K block 0 issue all MMAs of their tile in K order, the
//                 others only keep the barriers' books.  Warp 0 owns the TMEM allocation
//   warps 8..23   dequantisers in two groups of 8 that take alternate A slots: thread = one weight
//                 row of one tile; FP4 + E4M3 from shared memory -> bf16x2 registers -> tcgen05.st
//                 into the 4-slot ring of A operands in TMEM (slot = one 64-wide K block)
//   warps 24..27  epilogue: tcgen05.ld of the accumulators (sum of the partials), scale,
//                 activation, store
//
// Work items are "narrow" (N = 16 or 32: the K blocks of a stage spread over eight issuers with a
// partial accumulator each) or, in a step that the sort kernel made a wide one because experts with
// many rows dominate it, "wide" (N = 32 or 64, one issuer and one accumulator per tile, so that an
// expert with hundreds of rows is streamed and dequantised once per 64 rows).  The geometry of a launch (ring slot size and depth, accumulator
// buffers) follows the widest item of the step, which the sort kernel leaves in the workspace.
//
// The reference computes the same products with mma.sync / wgmma on Hopper
// (muse_moe_w4a16/submission.py:3828-4014 `tk2f_consume`, :1909-2072 `tw_item`); nothing is shared
// with that code beyond the arithmetic (weights as the M operand, FP32 accumulation, the
// global scale and a power of two applied once in the epilogue, submission.py:3855,3983-3987).
#include <cuda_bf16.h>

#include <type_traits>

#include "combine_device.cuh"
#include "params.cuh"

namespace okc {

constexpr int kGemmThreads = 928;      // 29 warps
constexpr int kIssuers = 8;           // warps 0..7: MMA-issuing threads, (tile of the pair) x (K block of the stage)
constexpr int kDequantWarp0 = 8;
constexpr int kDequantWarps = 16;
constexpr int kEpilogueWarp0 = 24;
constexpr int kProducerWarp = 28;
constexpr int kASlots = 4;            // ring of A operands in TMEM, 64 columns each (K = 64, two tiles)
constexpr int kASlotCols = 64;
constexpr int kAccCol0 = 256;         // accumulators live in TMEM columns [256, 512)
constexpr int kWideAccCols = 64;      // a wide item's accumulator: one block of 64 columns per tile
constexpr int kTmemCols = 512;

// Codes written to the status word when a wait gives up: role * 16 + barrier kind.
enum WaitCode { kWaitProducerEmpty = 0x11, kWaitProducerUnit = 0x12, kWaitProducerDone = 0x13,
                kWaitMmaAccEmpty = 0x21, kWaitMmaFull = 0x22, kWaitMmaAFull = 0x23, kWaitMmaUnit = 0x24,
                kWaitDqFull = 0x31, kWaitDqAEmpty = 0x32, kWaitDqUnit = 0x33, kWaitEpiAccFull = 0x41, kWaitEpiUnit = 0x42 };


// Optional wait profile (compile with -DOKC_WAIT_PROFILE): per CTA, cycles each role spent in
// each kind of wait, kept in a device array and read back by okc_moe_debug_wait_profile.  The
// role the reference's TWM_TL timeline plays (muse_moe_w4a16/submission.py:2657-2659).
#ifdef OKC_WAIT_PROFILE
constexpr int kProfCtas = 256;
constexpr int kProfSlots = 16;
__device__ long long g_wait_prof[kProfCtas][kProfSlots];
#define OKC_PROF_DECL long long prof_acc[kProfSlots] = {0}; const long long prof_t0 = clock64();
#define OKC_PROF_WAIT(idx, expr) ([&] { const long long _t = clock64(); const bool _r = (expr); prof_acc[idx] += clock64() - _t; return _r; }())
#define OKC_PROF_VOID(idx, stmt) { const long long _t = clock64(); stmt; prof_acc[idx] += clock64() - _t; }
#define OKC_PROF_STORE(idx_total, lo, hi) { prof_acc[idx_total] = clock64() - prof_t0; if (blockIdx.x < kProfCtas) for (int _i = lo; _i <= hi; ++_i) g_wait_prof[blockIdx.x][_i] = prof_acc[_i]; }
#else
#define OKC_PROF_DECL
#define OKC_PROF_WAIT(idx, expr) (expr)
#define OKC_PROF_VOID(idx, stmt) { stmt; }
#define OKC_PROF_STORE(idx_total, lo, hi)
#endif

constexpr int kURing = 4;             // units the producer may run ahead of the other roles
constexpr int kUnitConsumers = kIssuers + kDequantWarps + 4;   // warps that read every unit descriptor

// A unit of work as the producer publishes it to the other roles of the CTA.
struct UnitDesc {
  int phase;      // 0 gate_up, 1 down; -1 = no more units
  int slot;       // expert slot (weights, global scale)
  int pos0;       // first row of the item in the sorted route order
  int rows;       // token rows of the item
  int npad;       // rows padded to 16, 32 or 64 (N of the MMAs)
  int pair;       // tile pair within the expert
  int item;       // work item index
  int stages;     // K / 256 of this phase
};

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t a_full[2 * kASlots];     // [slot][tile]: the four dequantiser warps of one tile filled the slot (narrow unit)
  uint64_t a_full_w[2 * kASlots];   // the same for wide units.  A barrier of its own per kind of unit, because
                                    // a parity wait only tells phases one apart: every barrier needs to have one
                                    // waiter, the thread whose MMAs let the next phase begin.  A thread that only
                                    // looked on while another one issued would miss phases.
  uint64_t a_empty[2 * kASlots];    // [slot][tile]: that tile's MMAs on the slot completed
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t u_full[kURing];          // unit descriptor published
  uint64_t u_empty[kURing];         // every consumer warp has read it
  uint64_t dummy;                   // arrived on, never waited on
  uint64_t drain[kIssuers];         // an issuer that gives up waits here for the MMAs it has in flight
  UnitDesc units[kURing];
  uint32_t tmem_base;
  int abort_code;
};

// Next unit descriptor for a consumer role: waits until the producer published ring entry
// (n mod kURing), copies it, and frees the entry for this warp.  kWholeWarp: all 32 lanes call it
// (lane 0 frees the entry once every lane has its copy); otherwise one lane alone does.
template <bool kWholeWarp>
__device__ __forceinline__ bool next_unit(Ctrl* ctrl, uint32_t bar_ufull, uint32_t bar_uempty, uint32_t n, bool lane0,
                                          volatile int* abort_flag, int code, UnitDesc& u) {
  const uint32_t k = n % kURing;
  if (!mbar_wait(bar_ufull + 8 * k, (n / kURing) & 1, abort_flag, code)) return false;
  u = ctrl->units[k];
  if (kWholeWarp) __syncwarp();
  mbar_arrive_if(bar_uempty + 8 * k, lane0);
  return u.phase >= 0;
}

__global__ void __launch_bounds__(kGemmThreads, 1) okc_moe_gemm(const __grid_constant__ MoeGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the ring first, 1024-byte aligned; the control block behind the largest ring any step can ask for,
  // so that its place does not depend on the step (with the barriers in front of the ring the kernel
  // was measured 3 % slower)
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem0 - smem_u32(smem_raw));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_gen + (kSmemBudget - kGemmCtrlReserve - 1024));
  volatile int* abort_flag = &ctrl->abort_code;

  const int tid = threadIdx.x, lane = tid & 31;
  // the warp index through a shuffle: the compiler then knows it is the same in every lane and keeps
  // what is derived from it (roles, barrier addresses, TMEM columns) in uniform registers
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const bool lane0 = lane == 0;
  // shared-memory addresses of the barrier arrays (element i is 8 bytes further)
  const uint32_t bar_full = smem_u32(&ctrl->full[0]), bar_empty = smem_u32(&ctrl->empty[0]);
  const uint32_t bar_afull = smem_u32(&ctrl->a_full[0]), bar_aempty = smem_u32(&ctrl->a_empty[0]);
  const uint32_t bar_afullw = smem_u32(&ctrl->a_full_w[0]);
  const uint32_t bar_accfull = smem_u32(&ctrl->acc_full[0]), bar_accempty = smem_u32(&ctrl->acc_empty[0]);
  const uint32_t bar_ufull = smem_u32(&ctrl->u_full[0]), bar_uempty = smem_u32(&ctrl->u_empty[0]);

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, kDequantWarps + kIssuers);
    }
    for (int i = 0; i < 2 * kASlots; ++i) {
      mbar_init(bar_afull + 8 * i, 4);             // the four lane quarters of one tile
      mbar_init(bar_afullw + 8 * i, 4);
      mbar_init(bar_aempty + 8 * i, 1);            // that tile's issuer for this K block
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_accfull + 8 * i, kIssuers);
      mbar_init(bar_accempty + 8 * i, 4);
    }
    for (int i = 0; i < kURing; ++i) {
      mbar_init(bar_ufull + 8 * i, 1);
      mbar_init(bar_uempty + 8 * i, kUnitConsumers);
    }
    mbar_init(smem_u32(&ctrl->dummy), 1);
    for (int i = 0; i < kIssuers; ++i) mbar_init(smem_u32(&ctrl->drain[i]), 1);
    ctrl->abort_code = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctrl->tmem_base;

  // everything above overlapped the tail of the kernel before; its outputs are read from here on
  griddep_wait();
  griddep_launch_dependents();

  // Geometry of this launch from the widest item of the step (16, 32, 64 or 128 rows; written by the
  // sort kernel): a stage holds the 36 KB weight image and wcap token rows of 256 K elements.
  // (through a shuffle, like the warp index: what is derived from it then lives in uniform registers and
  // costs the dequantisers' loop no integer-pipe instructions)
  const int wcap = __shfl_sync(0xffffffffu, min(max(p.meta[kMetaWcap], 16), kChunkRows), 0);
  // A ring slot holds a whole stage (256 K elements: the 36 KB weight image + wcap token rows) while
  // every item is narrow.  A step with wide items runs on half stages (128 K elements: half of each
  // tile's codes and scales + wcap token rows of 128 elements): six slots instead of three, so that
  // more copies are in flight while a slot is being consumed.
  const bool half = wcap > kNarrowRows;
  const int sps = half ? 2 : 1;                                  // ring slots per stage
  const uint32_t slot_bytes = gemm_slot_bytes(wcap);
  const int NS = gemm_slots_for(wcap);
  // Accumulators in TMEM columns [256, 512).  Narrow items: per buffer eight blocks of acols columns,
  // block (tile * 4 + K block of the stage).  Wide items: per buffer one block of 64 columns per tile.
  // Two buffers of 128 columns, except in a step of narrow items of up to 32 rows (one of 256).
  const int nbuf = (wcap == kNarrowRows) ? 1 : 2;
  const int acols = (wcap == kNarrowRows) ? 32 : 16;
  const uint32_t acc_buf_stride = 8u * acols;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ producer
    // The whole warp runs the loop (the waits and the decisions are the same in every lane); lane 0 takes the
    // units, publishes them and starts the weight copies, and the token copies of a ring slot are spread over
    // the lanes: a thread that starts a dozen copies per stage one after the other is slower than the stage.
    // (The outcome of every wait is made the same in all lanes by a vote, so that the shuffles below always
    // find the whole warp.)
    {
      if (lane == 0) {
        for (int ph = 0; ph < 2; ++ph)
          for (int i = 0; i < 5; ++i) tma_prefetch_desc(&p.ph[ph].bmap[i]);
        if (p.direct_rows) tma_prefetch_desc(&p.hmap);
      }
      const uint64_t pol = policy_evict_first();
      const int n_items = p.meta[kMetaItems];
      const int units0 = n_items * p.ph[0].pairs, units1 = n_items * p.ph[1].pairs;
      const int first = (p.phase_lo == 0) ? 0 : units0;
      const int last = (p.phase_hi == 1) ? units0 + units1 : units0;
      const int nkb = half ? 2 : 4;                                // 64-element blocks of token rows per ring slot
      const uint32_t tok_off = half ? kHalfStageBytes : kStageBytes;
      int st = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      OKC_PROF_DECL
      for (uint32_t n = 0; ok; ++n) {
        const uint32_t k = n % kURing;
        if (!__all_sync(0xffffffffu, mbar_wait<200>(bar_uempty + 8 * k, ((n / kURing) & 1) ^ 1, abort_flag, kWaitProducerUnit))) { ok = false; break; }
        // the first unit of a CTA is the one of its own number (no trip to the counter before the first copy starts);
        // the counter hands out the units behind those
        int g0 = static_cast<int>(blockIdx.x);
        if (n > 0) {
          if (lane == 0) g0 = static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
          g0 = __shfl_sync(0xffffffffu, g0, 0);
        }
        const int g = first + g0;
        UnitDesc u;
        if (g >= last) {
          u.phase = -1; u.slot = 0; u.pos0 = 0; u.rows = 0; u.npad = 16; u.pair = 0; u.item = 0; u.stages = 0;
          if (lane == 0) {
            ctrl->units[k] = u;
            mbar_arrive(bar_ufull + 8 * k);
          }
          break;
        }
        u.phase = (g < units0) ? 0 : 1;
        const PhaseParams& pp = p.ph[u.phase];
        const int gl = (u.phase == 0) ? g : g - units0;
        u.item = gl / pp.pairs;
        u.pair = gl - u.item * pp.pairs;
        const int4 wi = p.items[u.item];
        u.slot = wi.x; u.pos0 = wi.y; u.rows = wi.z; u.npad = wi.w; u.stages = pp.stages;
        // Only the item's own rows are copied (in boxes of 4 ... 64 rows): the MMAs run over npad rows of
        // the slot, what lies behind the copied ones is left over from earlier stages and only reaches
        // accumulator columns that the epilogue never reads.  At a few rows per expert the padding would
        // otherwise be a sixth of all bytes the SM takes in.
        const int mi = (u.rows <= 4) ? 0 : (u.rows <= 8) ? 1 : (u.rows <= 16) ? 2 : (u.rows <= 32) ? 3 : 4;
        const int brows = 4 << mi;                               // token rows copied per stage
        if (lane == 0) {
          ctrl->units[k] = u;
          mbar_arrive(bar_ufull + 8 * k);
        }
        const uint8_t* src = pp.wpacked + static_cast<size_t>(u.slot) * pp.expert_bytes +
                             static_cast<size_t>(u.pair) * pp.stages * kStageBytes;
        const int steps = pp.stages * sps;                       // ring slots this unit goes through
        // gate_up units of a small step take their rows from the caller's array, row by row: lane j knows
        // the token of row j
        const bool direct = p.direct_rows != 0 && u.phase == 0;
        int my_tok = 0;
        if (direct && lane < u.rows) my_tok = p.sorted[u.pos0 + lane] / p.kk;
        const int crows = direct ? u.rows : brows;               // token rows that arrive per ring slot
        const int n_ops = crows * nkb;                           // direct: row copies per ring slot
        const uint32_t tx_bytes = tok_off + crows * nkb * 128;
        // weights of ring step r of the unit -> slot at dst (lane 0)
        auto send_weights = [&](int r, uint32_t dst, uint32_t bar) {
          if (lane == 0) bulk_g2s_hint(dst, src + static_cast<size_t>(r) * tok_off, tok_off, bar, pol);
        };
        // token rows of ring step r -> behind the weights of the slot (all lanes)
        auto send_tokens = [&](int r, uint32_t dst, uint32_t bar) {
          const int k0 = half ? (r >> 1) * kStageK + (r & 1) * 128 : r * kStageK;
          const uint32_t base = dst + tok_off;
          if (direct) {
            // (the 128-byte swizzle is a function of the shared-memory address, so single rows land where a box
            // of rows would have put them)
            for (int o0 = 0; o0 < n_ops; o0 += 32) {
              const int o = o0 + lane;
              const int row = half ? (o >> 1) : (o >> 2), kb = half ? (o & 1) : (o & 3);
              const int t = __shfl_sync(0xffffffffu, my_tok, row & 31);
              if (o < n_ops) tma_2d_g2s(base + kb * u.npad * 128 + row * 128, &p.hmap, k0 + kb * 64, t, bar);
            }
          } else if (lane < nkb) {
            tma_2d_g2s(base + lane * u.npad * 128, &pp.bmap[mi], k0 + lane * 64, u.pos0, bar);
          }
        };
        int r_begin = 0;
        if (u.phase == 1) {
          // The token operand of a down unit is the gate_up output of its work item: all four
          // epilogue warps of each of the item's gate_up units must have stored and published it.
          const int target = 4 * p.ph[0].pairs;
          if (ld_acquire_gpu(p.done + u.item) < target) {
            // Not yet.  The weights do not depend on it: start their copies for as many slots as the
            // ring holds, wait, then send the token tiles after them (a slot's barrier completes
            // when both parts have arrived).
            const int pre = steps < NS ? steps : NS;
            int st2 = st, sent = 0;
            uint32_t ph2 = ph;
            for (int r = 0; r < pre; ++r) {
              if (!__all_sync(0xffffffffu, OKC_PROF_WAIT(1, mbar_wait<500>(bar_empty + 8 * st2, ph2 ^ 1, abort_flag, kWaitProducerEmpty)))) { ok = false; break; }
              if (lane == 0) mbar_expect_tx(bar_full + 8 * st2, tx_bytes);
              send_weights(r, smem0 + st2 * slot_bytes, bar_full + 8 * st2);
              ++sent;
              if (++st2 == NS) { st2 = 0; ph2 ^= 1; }
            }
            uint32_t spins = 0;
            while (ok && ld_acquire_gpu(p.done + u.item) < target) {
              __nanosleep(100);
              if ((++spins & 255u) == 0) {
                if (*abort_flag != 0) { ok = false; break; }
                if (spins >= (1u << 22)) { atomicCAS(const_cast<int*>(abort_flag), 0, kWaitProducerDone); ok = false; break; }
              }
            }
            ok = __all_sync(0xffffffffu, ok);
            fence_proxy_async();   // those stores were generic-proxy writes; the loads below are TMA
            // (also when giving up: the slots whose weights are in flight get their token tiles, so
            // that their barriers complete and the CTA can wait for its copies before it retires)
            for (int r = 0; r < sent; ++r) {
              send_tokens(r, smem0 + st * slot_bytes, bar_full + 8 * st);
              ++issued;
              if (++st == NS) { st = 0; ph ^= 1; }
            }
            if (!ok) break;
            r_begin = pre;
          } else {
            fence_proxy_async();
          }
        }
        for (int r = r_begin; r < steps; ++r) {
          if (!__all_sync(0xffffffffu, OKC_PROF_WAIT(1, mbar_wait<500>(bar_empty + 8 * st, ph ^ 1, abort_flag, kWaitProducerEmpty)))) { ok = false; break; }
          const uint32_t bar = bar_full + 8 * st;
          const uint32_t dst = smem0 + st * slot_bytes;
          if (lane == 0) mbar_expect_tx(bar, tx_bytes);
          send_weights(r, dst, bar);
          send_tokens(r, dst, bar);
          ++issued;
          if (++st == NS) { st = 0; ph ^= 1; }
        }
      }
      if (lane == 0) { OKC_PROF_STORE(0, 0, 1) }
      if (!ok && lane == 0) {
        // give copies already issued a bounded chance to land before the CTA retires
        const int n = issued < NS ? issued : NS;
        for (int j = 0; j < n; ++j) {
          st = (st == 0) ? NS - 1 : st - 1;
          if (st == NS - 1) ph ^= 1;
          const long long t0 = clock64();
          while (!mbar_try(bar_full + 8 * st, ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp < kIssuers) {
    // ------------------------------------------------------------ MMA issuers
    // The whole warp runs the loops and the waits (a poll costs one warp instruction however many lanes
    // take part); one elected lane issues the MMAs and their commits.  Control flow that is the same in
    // all lanes lets the compiler keep descriptors, barrier addresses and counters in uniform registers,
    // where tcgen05.mma takes them from: from a single-lane branch every operand of every MMA has to be
    // moved there first.
    {
      // (a generic lambda with a compile-time flag: the loops of the whole-stage ring stay as lean as
      // they were before half stages existed)
      auto issue = [&](auto half_tag) {
        constexpr bool kHalf = decltype(half_tag)::value;
        const int tile = warp & 1, kb = warp >> 1;
        const uint32_t my_afull = bar_afull + 16 * kb + 8 * tile, my_aempty = bar_aempty + 16 * kb + 8 * tile;
        const uint32_t a0 = tmem + kb * kASlotCols + tile * 32;
        const uint32_t b_off = kHalf ? kHalfStageBytes : kStageBytes;    // token rows behind the weights of a slot
        int st = 0;
        uint32_t ph = 0;              // ring phase
        uint32_t sph = 0, sphw = 0;   // A-slot phases: narrow units' barriers, wide units' barriers (flip once per stage of that kind)
        OKC_PROF_DECL
        const uint32_t desc_hi = static_cast<uint32_t>(smem_desc_sw128(0) >> 32);
        const uint32_t desc_lo_const = static_cast<uint32_t>(smem_desc_sw128(0));
        UnitDesc u;
        for (uint32_t unit_it = 0; next_unit<true>(ctrl, bar_ufull, bar_uempty, unit_it, lane0, abort_flag, kWaitMmaUnit, u); ++unit_it) {
          const uint32_t npad = static_cast<uint32_t>(u.npad);
          const int buf = (nbuf == 2) ? (unit_it & 1) : 0;
          if (!OKC_PROF_WAIT(2, mbar_wait<500>(bar_accempty + 8 * buf, ((unit_it / nbuf) & 1) ^ 1, abort_flag, kWaitMmaAccEmpty))) goto issuer_done;
          tc_fence_after();
          const uint32_t idesc = idesc_bf16_m128(npad);
          const uint32_t kb_step = (npad * 128u) >> 4;           // descriptor units from one K block's rows to the next
          if (!kHalf || npad <= 16) {
            // narrow item: this issuer's K block of every stage into its own partial accumulator
            const uint32_t d = tmem + kAccCol0 + buf * acc_buf_stride + (tile * 4 + kb) * acols;
            uint32_t acc = 0;
            for (int s = 0; s < u.stages; ++s) {
#pragma unroll
              for (int hh = 0; hh < (kHalf ? 2 : 1); ++hh) {
                if (!OKC_PROF_WAIT(3, mbar_wait(bar_full + 8 * st, ph, abort_flag, kWaitMmaFull))) goto issuer_done;
                if (!kHalf || hh == (kb >> 1)) {
                  const uint32_t lo = (desc_lo_const | (((smem0 + st * slot_bytes + b_off) & 0x3FFFFu) >> 4)) +
                                      (kHalf ? (kb & 1) : kb) * kb_step;
                  if (!OKC_PROF_WAIT(4, mbar_wait(my_afull, sph, abort_flag, kWaitMmaAFull))) goto issuer_done;
                  tc_fence_after();
                  if (elect_one()) {
                    mma_ts2(d, a0, lo, desc_hi, idesc, acc);
                    mma_ts2(d, a0 + 8, lo + 2, desc_hi, idesc, 1);
                    mma_ts2(d, a0 + 16, lo + 4, desc_hi, idesc, 1);
                    mma_ts2(d, a0 + 24, lo + 6, desc_hi, idesc, 1);
                    mma_commit(my_aempty);
                    mma_commit(bar_empty + 8 * st);
                  }
                  __syncwarp();
                  acc = 1;
                } else {
                  mbar_arrive_if(bar_empty + 8 * st, lane0);     // the other half of the stage: not this issuer's K block
                }
                if (++st == NS) { st = 0; ph ^= 1; }
              }
              sph ^= 1;
            }
            if (elect_one()) mma_commit(bar_accfull + 8 * buf);
            __syncwarp();
          } else if (kb == 0) {
            // wide item: all K blocks of this tile, in K order, into the tile's one accumulator
            const uint32_t d = tmem + kAccCol0 + buf * acc_buf_stride + tile * kWideAccCols;
            const uint32_t a_tile = tmem + tile * 32;
            uint32_t acc = 0;
            for (int s = 0; s < u.stages; ++s) {
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                if (!OKC_PROF_WAIT(3, mbar_wait(bar_full + 8 * st, ph, abort_flag, kWaitMmaFull))) goto issuer_done;
                uint32_t lo = desc_lo_const | (((smem0 + st * slot_bytes + b_off) & 0x3FFFFu) >> 4);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int k4 = 2 * hh + j;
                  if (!OKC_PROF_WAIT(4, mbar_wait(bar_afullw + 16 * k4 + 8 * tile, sphw, abort_flag, kWaitMmaAFull))) goto issuer_done;
                  tc_fence_after();
                  const uint32_t a = a_tile + k4 * kASlotCols;
                  if (elect_one()) {
                    mma_ts2(d, a, lo, desc_hi, idesc, acc);
                    mma_ts2(d, a + 8, lo + 2, desc_hi, idesc, 1);
                    mma_ts2(d, a + 16, lo + 4, desc_hi, idesc, 1);
                    mma_ts2(d, a + 24, lo + 6, desc_hi, idesc, 1);
                    mma_commit(bar_aempty + 16 * k4 + 8 * tile);
                    if (j == 1) mma_commit(bar_empty + 8 * st);
                  }
                  __syncwarp();
                  acc = 1;
                  lo += kb_step;
                }
                if (++st == NS) { st = 0; ph ^= 1; }
              }
              sphw ^= 1;
            }
            if (elect_one()) mma_commit(bar_accfull + 8 * buf);
            __syncwarp();
          } else {
            // wide item, an issuer without MMAs of its own: keeps the ring's and the accumulator's barrier counts
            for (int r = 0; r < 2 * u.stages; ++r) {
              if (!OKC_PROF_WAIT(3, mbar_wait<200>(bar_full + 8 * st, ph, abort_flag, kWaitMmaFull))) goto issuer_done;
              mbar_arrive_if(bar_empty + 8 * st, lane0);
              if (++st == NS) { st = 0; ph ^= 1; }
            }
            mbar_arrive_if(bar_accfull + 8 * buf, lane0);
          }
        }
      issuer_done:
        if (*abort_flag != 0 && lane0) {
          // giving up: the MMAs already issued still read the A ring and write the accumulators, so
          // tensor memory may only be freed once they have retired (bounded, like the producer's drain)
          const uint32_t bar = smem_u32(&ctrl->drain[warp]);
          mma_commit(bar);
          const long long t0 = clock64();
          while (!mbar_try(bar, 0) && clock64() - t0 < kWaitLimitCycles) {}
        }
        if (warp == 0 && lane0) { OKC_PROF_STORE(5, 2, 5) }
      };
      if (half) issue(std::true_type{});
      else issue(std::false_type{});
    }
  } else if (warp >= kDequantWarp0 && warp < kDequantWarp0 + kDequantWarps) {
    // ------------------------------------------------------------ dequantisers
    // Two groups of 8 warps; group g fills the A slots kb = g and g + 2 of every stage.  Inside a
    // group a warp is (TMEM lane quarter, tile); a thread dequantises its row's 64 K elements.
    const int dw = warp - kDequantWarp0;
    const int q = warp & 3;               // TMEM lane quarter this warp may touch
    const int tile = (dw >> 2) & 1;       // first or second tile of the pair
    const int grp = dw >> 3;
    const int row = q * 32 + lane;
    const uint32_t trow = tmem + (static_cast<uint32_t>(q * 32) << 16) + tile * 32;
    auto dequantise = [&](auto half_tag) {
      constexpr bool kHalf = decltype(half_tag)::value;
      // this thread's row in its tile's part of a half stage: codes [4 chunks][128 rows][16 B], then
      // scales [4 chunks][128 rows][2 B]; its group's K block is chunks 2 grp, 2 grp + 1 of the half
      const uint32_t code_off = tile * kHalfTileBytes + (2 * grp) * (kTileRows * 16) + row * 16;
      const uint32_t scale_off = tile * kHalfTileBytes + kHalfTileCodeBytes + (2 * grp) * (kTileRows * 2) + row * 2;
      const uint32_t my_aempty = bar_aempty + 8 * tile;
      int st = 0;
      // barrier of the A slot stored to but not yet handed over; a barrier nobody waits on stands in
      // before the first slot, so the hand-over below needs no "is anything pending" test
      uint32_t pend_bar = smem_u32(&ctrl->dummy);
      uint32_t ph = 0, sph = 0;
      OKC_PROF_DECL
      UnitDesc u;
      for (uint32_t unit_it = 0; next_unit<true>(ctrl, bar_ufull, bar_uempty, unit_it, lane0, abort_flag, kWaitDqUnit, u); ++unit_it) {
        // the slots of a wide unit are handed to the tile's one issuer through barriers of their own
        const uint32_t my_afull = ((kHalf && u.npad > 16) ? bar_afullw : bar_afull) + 8 * tile;
        for (int s = 0; s < u.stages; ++s) {
#pragma unroll
          for (int hh = 0; hh < (kHalf ? 2 : 1); ++hh) {
            if (!OKC_PROF_WAIT(6, mbar_wait(bar_full + 8 * st, ph, abort_flag, kWaitDqFull))) goto dq_done;
            {
              const uint8_t* img = smem_gen + static_cast<size_t>(st) * slot_bytes;
              const uint32_t simg = smem0 + st * slot_bytes + scale_off;
#pragma unroll
              for (int h = 0; h < (kHalf ? 1 : 2); ++h) {
                // this group's K block of half h of the stage (whole-stage slots) or of this half (half-stage slots)
                const int kb = 2 * (kHalf ? hh : h) + grp;
                const uint32_t hoff = kHalf ? 0u : h * kHalfStageBytes;
                // this thread's 64 K elements of the slot: two chunks of 16 code bytes + 2 scale bytes
                const uint4 w0 = *reinterpret_cast<const uint4*>(img + hoff + code_off);
                const uint4 w1 = *reinterpret_cast<const uint4*>(img + hoff + code_off + kTileRows * 16);
                const uint32_t sp0 = simg + hoff;
                const uint32_t sp1 = sp0 + kTileRows * 2;
                const uint32_t s00 = lds_u8(sp0), s01 = lds_u8(sp0 + 1), s10 = lds_u8(sp1), s11 = lds_u8(sp1 + 1);
                uint32_t r[16];
                dequant_chunk(w0, s00, s01, r);
                // the stores of the previous slot completed while this chunk was being dequantised:
                // only now wait for them and hand that slot to its MMA issuer
                OKC_PROF_VOID(8, tmem_wait_st())
                tc_fence_before();
                mbar_arrive_if(pend_bar, lane0);
                // every lane polls the same barrier in the same instruction, so the outcome is the same
                // in all of them and the warp stays converged for the tensor-memory stores below
                if (!OKC_PROF_WAIT(7, mbar_wait(my_aempty + 16 * kb, sph ^ 1, abort_flag, kWaitDqAEmpty))) goto dq_done;
                tc_fence_after();
                tmem_st16(trow + kb * kASlotCols, r);
                dequant_chunk(w1, s10, s11, r);
                tmem_st16(trow + kb * kASlotCols + 16, r);
                pend_bar = my_afull + 16 * kb;
              }
            }
            // the slot's bytes have been consumed (the loads fed the arithmetic above): hand the
            // shared-memory slot back
            mbar_arrive_if(bar_empty + 8 * st, lane0);
            if (++st == NS) { st = 0; ph ^= 1; }
          }
          sph ^= 1;
        }
        // The unit's last slot is normally handed over while the first chunk of the next unit is
        // being dequantised.  If that chunk has not arrived, hand the slot over now: the producer may
        // be holding the next unit back until another CTA's -- or this CTA's -- gate_up epilogue has
        // run, and this unit's epilogue cannot run before its last MMAs have their operand.
        if (!__all_sync(0xffffffffu, mbar_test(bar_full + 8 * st, ph))) {
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive_if(pend_bar, lane0);
          pend_bar = smem_u32(&ctrl->dummy);
        }
      }
    dq_done:
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_if(pend_bar, lane0);
#ifdef OKC_WAIT_PROFILE
      if (lane == 0 && blockIdx.x < kProfCtas && (warp == kDequantWarp0 || warp == kDequantWarp0 + kDequantWarps - 1)) {
        const int base = (warp == kDequantWarp0) ? 6 : 10;   // first and last dequantiser warp
        for (int i = 0; i < 3; ++i) g_wait_prof[blockIdx.x][base + i] = prof_acc[6 + i];
        g_wait_prof[blockIdx.x][base + 3] = clock64() - prof_t0;
      }
#endif
    };
    if (half) dequantise(std::true_type{});
    else dequantise(std::false_type{});
  } else if (warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + 4) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    UnitDesc u;
    for (uint32_t unit_it = 0; next_unit<true>(ctrl, bar_ufull, bar_uempty, unit_it, lane0, abort_flag, kWaitEpiUnit, u); ++unit_it) {
      const int n_rows = u.rows, npad = u.npad;
      const int buf = (nbuf == 2) ? (unit_it & 1) : 0;
      const float sc = p.ph[u.phase].gs[u.slot] * 256.0f;
      // down units: the routes and routing weights of 32 of the item's rows at a time, one row per
      // lane, broadcast by shuffles below.  The first 32 are loaded before the accumulators are waited
      // for, the next 32 while the current ones are stored: a load per row inside the store loop
      // would put a round trip to L2 between every two rows' stores.
      int cur_rt = -1, nxt_rt = -1;
      float cur_rw = 1.0f, nxt_rw = 1.0f;
      if (u.phase == 1 && lane < n_rows) {
        cur_rt = p.sorted[u.pos0 + lane];
        if (p.weighted) cur_rw = p.wsorted[u.pos0 + lane];
      }
      if (!mbar_wait<2000>(bar_accfull + 8 * buf, (unit_it / nbuf) & 1, abort_flag, kWaitEpiAccFull)) break;
      tc_fence_after();
      const bool wide = half && npad > 16;
      // narrow: tile 0 / tile 1, K block 0 (the other K blocks acols columns further each); wide: the tiles' accumulators
      const uint32_t d0 = tmem + lane_off + kAccCol0 + buf * acc_buf_stride;
      const uint32_t d1 = d0 + (wide ? kWideAccCols : 4 * acols);
      for (int c0 = 0; c0 < npad; c0 += 16) {
        uint32_t a[16], b[16];
        tmem_ld16(d0 + c0, a);
        tmem_ld16(d1 + c0, b);
        if (wide) {
          tmem_wait_ld();
        } else {
          // ((K block 0 + 1) + 2) + 3 for each tile: the same order for every narrow shape
          uint32_t t[16];
#pragma unroll
          for (int part = 1; part < 4; ++part) {
            tmem_ld16(d0 + part * acols + c0, t);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) a[j] = __float_as_uint(__uint_as_float(a[j]) + __uint_as_float(t[j]));
            tmem_ld16(d1 + part * acols + c0, t);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) b[j] = __float_as_uint(__uint_as_float(b[j]) + __uint_as_float(t[j]));
          }
        }
        if (c0 + 16 >= npad) {
          // last read of this accumulator: the MMA warps may overwrite it
          tc_fence_before();
          mbar_arrive_if(bar_accempty + 8 * buf, lane0);
        }
        if (c0 < n_rows) {
          if (u.phase == 0) {
            uint16_t* dst = p.inter + static_cast<size_t>(u.pos0 + c0) * p.I + u.pair * kTileRows + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c0 + j < n_rows) {
                const float va = __uint_as_float(a[j]) * sc;
                const float vb = __uint_as_float(b[j]) * sc;
                const float act = va / (1.0f + __expf(-va)) * vb;
                dst[static_cast<size_t>(j) * p.I] = __bfloat16_as_ushort(__float2bfloat16_rn(act));
              }
            }
          } else {
            if ((c0 & 16) == 0) {
              nxt_rt = -1;
              nxt_rw = 1.0f;
              if (c0 + 32 + lane < n_rows) {
                nxt_rt = p.sorted[u.pos0 + c0 + 32 + lane];
                if (p.weighted) nxt_rw = p.wsorted[u.pos0 + c0 + 32 + lane];
              }
            }
            float* ybase = p.y + u.pair * 2 * kTileRows + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int route = __shfl_sync(0xffffffffu, cur_rt, (c0 & 16) + j);     // -1 beyond the item's rows
              const float wgt = __shfl_sync(0xffffffffu, cur_rw, (c0 & 16) + j);
              if (route >= 0) {
                float* dst = ybase + static_cast<size_t>(route) * p.H;
                dst[0] = __uint_as_float(a[j]) * sc * wgt;
                dst[kTileRows] = __uint_as_float(b[j]) * sc * wgt;
              }
            }
            if (c0 & 16) {
              cur_rt = nxt_rt;
              cur_rw = nxt_rw;
            }
          }
        }
      }
      if (u.phase == 0) {
        // publish this warp's part of the gate_up output to the producers (of any CTA) that will
        // stream it as the token operand of the item's down units through TMA
        __threadfence();
        fence_proxy_async();
        __syncwarp();
        if (lane0) {
          __threadfence();
          atomicAdd(p.done + u.item, 1);
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctrl->abort_code != 0) {
    atomicCAS(const_cast<int32_t*>(&p.meta[kMetaStatus]), 0, OKC_ERR_TIMEOUT);
    atomicCAS(const_cast<int32_t*>(&p.meta[kMetaDetail]), 0, ((p.phase_lo * 2 + p.phase_hi) << 8) | ctrl->abort_code);
  }
}

// Per-token combine: out[t] = sum over the token's local routes (slot order) of y[t*kk + slot],
// optionally through the reference's post-expert norm (scale by 1 + w, RMSNorm eps 1e-8, then the
// routing weight; muse_moe_w4a16/reference.py:88-90,106).  Rows with no local route become zero.

constexpr int kCombineThreads = 256;
constexpr int kCombineMaxPer = 8;   // float4 per thread: H <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kCombineThreads) okc_combine(const CombineParams p) {
  griddep_wait();
  clear_call_state(p);
  const int t = blockIdx.x, tid = threadIdx.x;
  const int nvec = p.H / 4;
  float4 acc[kCombineMaxPer];
#pragma unroll
  for (int i = 0; i < kCombineMaxPer; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  // (only launched with the post-expert norm; without it okc_combine_sliced runs)
  // Eight slots at a time, in two passes: the sums of squares of all eight rows first (their loads are all in
  // flight together and one block-wide reduction serves the eight), then the rows again (from L1 / L2) scaled and
  // added in slot order.  Slot by slot, every slot cost a trip to L2 and a block-wide reduction of its own.  The
  // operations on every element, and their order, are the same either way.
  __shared__ float red[8][kCombineThreads / 32];
  auto scaled = [&](const float4* yr, int v) {
    float4 a = yr[v];
    const uint2 wb = *reinterpret_cast<const uint2*>(p.post_w + v * 4);
    a.x *= 1.0f + __uint_as_float(wb.x << 16);
    a.y *= 1.0f + __uint_as_float(wb.x & 0xFFFF0000u);
    a.z *= 1.0f + __uint_as_float(wb.y << 16);
    a.w *= 1.0f + __uint_as_float(wb.y & 0xFFFF0000u);
    return a;
  };
  for (int s0 = 0; s0 < p.kk; s0 += 8) {
    int q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = (s0 + j < p.kk) ? p.pos[t * p.kk + s0 + j] : -1;   // uniform over the block
    float ss[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ss[j] = 0.f;
      if (q[j] < 0) continue;
      const float4* yr = reinterpret_cast<const float4*>(p.y + static_cast<size_t>(t * p.kk + s0 + j) * p.H);
#pragma unroll
      for (int i = 0; i < kCombineMaxPer; ++i) {
        const int v = tid + i * kCombineThreads;
        if (v < nvec) {
          const float4 a = scaled(yr, v);
          ss[j] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[j] += __shfl_xor_sync(0xffffffffu, ss[j], o);
    }
    __syncthreads();
    if ((tid & 31) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) red[j][tid >> 5] = ss[j];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (q[j] < 0) continue;
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kCombineThreads / 32; ++i) tot += red[j][i];
      const float scale = p.wsorted[q[j]] * rsqrtf(tot / static_cast<float>(p.H) + 1e-8f);
      const float4* yr = reinterpret_cast<const float4*>(p.y + static_cast<size_t>(t * p.kk + s0 + j) * p.H);
#pragma unroll
      for (int i = 0; i < kCombineMaxPer; ++i) {
        const int v = tid + i * kCombineThreads;
        if (v < nvec) {
          const float4 a = scaled(yr, v);
          acc[i].x += a.x * scale; acc[i].y += a.y * scale;
          acc[i].z += a.z * scale; acc[i].w += a.w * scale;
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

#ifdef OKC_WAIT_PROFILE
// host_out: long long [256][16] = per CTA of the last launch:
// 0 producer total, 1 producer wait-empty, 2 mma wait acc-empty, 3 mma wait full, 4 mma wait a-full, 5 mma total,
// 6..9 first dequantiser warp: wait full, wait a-empty, wait tcgen05.st, total; 10..13 the same for the last one.
extern "C" int okc_moe_debug_stuck(int* host_out, int clear) {
  if (cudaMemcpyFromSymbol(host_out, g_stuck, sizeof(g_stuck)) != cudaSuccess) return -3;
  if (clear) {
    void* dptr = nullptr;
    if (cudaGetSymbolAddress(&dptr, g_stuck) != cudaSuccess || cudaMemset(dptr, 0, sizeof(g_stuck)) != cudaSuccess) return -3;
  }
  return 0;
}
extern "C" int okc_moe_debug_wait_profile(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_wait_prof, sizeof(g_wait_prof)) == cudaSuccess ? 0 : -3;
}
#endif

static_assert(sizeof(Ctrl) <= kGemmCtrlReserve, "the control block outgrew its reserve");

cudaError_t launch_gemm(const MoeGemmParams& p, int grid, cudaStream_t stream) {
  // always the whole 227 KB: how the ring divides it is decided on the device from the step's widest item
  cudaError_t e = cudaFuncSetAttribute(okc_moe_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
  if (e != cudaSuccess) return e;
  return launch_kernel(okc_moe_gemm, dim3(grid), dim3(kGemmThreads), kSmemBudget, stream, true, p);
}

// The combine without the post-expert norm needs no row-wide reduction, so a token's row is cut
// into 1024-column slices over blockIdx.y: four times as many CTAs as tokens keep the small launch
// from being latency-bound.  Same sums in the same (slot) order as okc_combine.
__global__ void __launch_bounds__(kCombineThreads) okc_combine_sliced(const CombineParams p) {
  griddep_wait();
  clear_call_state(p);
  const int t = blockIdx.x;
  const int v = blockIdx.y * kCombineThreads + threadIdx.x;   // float4 index within the row
  if (v >= p.H / 4) return;
  const float4 acc = sum_token_routes(p.y, p.pos, t, p.kk, p.H, v * 4);
  if (p.out_f32) {
    reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<size_t>(t) * p.H)[v] = acc;
  } else {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + static_cast<size_t>(t) * p.H)[v] = o;
  }
}

cudaError_t launch_combine(const CombineParams& p, int T, cudaStream_t stream) {
  if (p.post_w == nullptr) {
    const dim3 grid(T, (p.H / 4 + kCombineThreads - 1) / kCombineThreads);
    return launch_kernel(okc_combine_sliced, grid, dim3(kCombineThreads), 0, stream, true, p);
  }
  return launch_kernel(okc_combine, dim3(T), dim3(kCombineThreads), 0, stream, true, p);
  return cudaGetLastError();
}

}  // namespace okc
