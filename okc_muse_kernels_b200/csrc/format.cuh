// Geometry of the packed weight format, the workspace layout derived from a plan, and the
// device-side FP4 -> BF16 dequantisation shared by the GEMM kernel and the unpack utility.
#pragma once
#include <cstddef>
#include <cstdint>

#include "../../include/okc_moe.h"
#include "ptx.cuh"

namespace okc {

constexpr int kTileRows = 128;                 // rows of one weight tile = M of one tcgen05.mma
constexpr int kStageK = 256;                   // K elements per shared-memory stage
constexpr int kChunkK = 32;                    // K elements one thread dequantises per tcgen05.st
constexpr int kChunks = kStageK / kChunkK;     // 8
// A stage image is two halves of 128 K elements; a half holds, for each of the two tiles (gate + up, or
// two row tiles of w2), the codes of its four chunks and then their scales.  A whole stage is one
// contiguous copy, and so is half a stage (the unit of the ring in a step with wide items).
constexpr int kHalfChunks = kChunks / 2;                          // 4
constexpr int kHalfTileCodeBytes = kHalfChunks * kTileRows * 16;  // 8192
constexpr int kHalfTileScaleBytes = kHalfChunks * kTileRows * 2;  // 1024
constexpr int kHalfTileBytes = kHalfTileCodeBytes + kHalfTileScaleBytes;   // 9216
constexpr int kHalfStageBytes = 2 * kHalfTileBytes;               // 18432
constexpr int kStageBytes = 2 * kHalfStageBytes;                  // 36864
// byte offset of (tile, chunk, row) inside a stage image: codes (16 B) and scales (2 B)
__host__ __device__ inline int stage_code_offset(int tile, int chunk, int row) {
  return (chunk / kHalfChunks) * kHalfStageBytes + tile * kHalfTileBytes + (chunk % kHalfChunks) * (kTileRows * 16) + row * 16;
}
__host__ __device__ inline int stage_scale_offset(int tile, int chunk, int row) {
  return (chunk / kHalfChunks) * kHalfStageBytes + tile * kHalfTileBytes + kHalfTileCodeBytes +
         (chunk % kHalfChunks) * (kTileRows * 2) + row * 2;
}
constexpr int kNarrowRows = 32;                // most rows (tokens) of a narrow work item
constexpr int kChunkRows = 64;                 // most rows of any work item (a wide one)
// Work items.  Normally every expert becomes narrow items of at most chunk_rows_for() rows: 16 while the
// step is decode-sized or an expert gets 8 rows or fewer on average (the accumulators of eight issuers then
// fit TMEM twice, so the epilogue overlaps the next unit, and the stage ring is a stage deeper); 32 beyond,
// where 16-row items would stream and dequantise most experts' weights twice.
// A step can instead be a wide step: an expert is cut into items of 64 rows, what is left over at its end
// being one more item; items of up to 16 rows are narrow ones, all others wide ones padded to 32 or 64
// rows (one accumulator per tile: two wide items' accumulators, or two 16-row items' partial sums, fit
// TMEM side by side, so the epilogue always overlaps the next unit).  A wide step runs on half-stage ring
// slots, which costs its narrow items a few per cent; the sort kernel makes a step a wide one when some
// expert has more than 32 rows and the wide cut has at least a tenth fewer items than the narrow one
// (wide_step_pays).
__host__ __device__ inline int chunk_rows_for(int T, int k, int E) {
  return (T <= 64 || static_cast<long long>(T) * k <= 8LL * E) ? 16 : kNarrowRows;
}
__host__ __device__ inline int item_pad(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : 64; }
// rows per item of an expert with c rows; chunk = chunk_rows_for()
__host__ __device__ inline int item_rows(int c, bool wide_step, int chunk) {
  if (!wide_step) return chunk;
  return c <= 16 ? 16 : kChunkRows;
}
__host__ __device__ inline bool wide_step_pays(int cmax, long long items_narrow, long long items_wide) {
  return cmax > kNarrowRows && 11 * items_wide <= 10 * items_narrow;
}

// Shared memory of the grouped-GEMM kernel: a reserve for its control block and the 1024-byte alignment
// of the ring, then as many ring slots as fit 227 KB.  wcap = rows of the widest item of the step.
// Up to 32 rows a slot is a whole stage (the 36 KB weight image + wcap token rows of 256 K elements);
// beyond, half a stage (18 KB of weights + wcap token rows of 128 K elements).
constexpr int kSmemBudget = 232448;
constexpr int kGemmCtrlReserve = 2048;
// Steps of up to this many tokens read their token rows straight from the caller's array (an item then has at most
// this many rows: a token sends at most one route to an expert).
constexpr int kDirectRowsMaxTokens = 8;
constexpr int kMaxStages = 6;
__host__ __device__ inline int gemm_slot_bytes(int wcap) {
  return wcap > kNarrowRows ? 36864 / 2 + wcap * 256 : 36864 + wcap * 512;
}
__host__ __device__ inline int gemm_slots_for(int wcap) {
  const int n = (kSmemBudget - kGemmCtrlReserve - 1024) / gemm_slot_bytes(wcap);
  return n > kMaxStages ? kMaxStages : n;
}
constexpr int kMaxSlots = 513;                 // 512 experts + shared
constexpr int kMaxRoutes = 16384;              // routes (tokens x routes per token) one step may hold

constexpr uint32_t kOutMask = 0x81C081C0u;     // sign + 3 magnitude bits of both bf16 halves
constexpr uint32_t kLeftMask = 0x60306030u;    // bits of w0 its three rotations leave over

// meta words at the start of the workspace
enum MetaWord { kMetaItems = 0, kMetaLocalRoutes = 1, kMetaStatus = 2, kMetaDetail = 3, kMetaTokens = 4,
                kMetaWcap = 5,       // rows of the step's widest work item, padded: 16, 32 or 64 (64: a wide step)
                kMetaRouterStatus = 6,   // set by the router-logits kernel when one of its waits ran out; the sort takes it over
                kMetaRouteTicket = 7,    // CTAs of the routing kernel that are done; the last one sorts and puts it back to zero
                kMetaWorkFused = 8, kMetaWorkPhase0 = 9, kMetaWorkPhase1 = 10,   // unit counters of the GEMM launches
                kMetaWords = 64 };

struct Geometry {
  int H, I, slots, kk, T, R, Rpad;
  int pairs13, stages13, pairs2, stages2;
  size_t w13_expert_bytes, w2_expert_bytes;
  int max_items;
  // workspace byte offsets
  size_t off_meta, off_counts, off_items, off_done, off_sorted, off_pos, off_wsorted, off_xg, off_inter, off_y, total;
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Fills g from a plan.  Returns false if the plan is outside the supported shapes.
inline bool make_geometry(const okc_moe_plan& p, Geometry& g) {
  if (p.hidden <= 0 || p.inter <= 0 || p.hidden % 256 || p.inter % 256) return false;
  if (p.n_experts <= 0 || p.n_experts > 512 || p.top_k <= 0 || p.top_k > 16 || p.top_k > p.n_experts) return false;
  if (p.local_start < 0 || p.local_count <= 0 || p.local_start + p.local_count > p.n_experts) return false;
  if (p.shared_inter != 0 && p.shared_inter != p.inter) return false;
  if (p.max_tokens <= 0 || p.max_tokens > 4096) return false;
  if (p.post_norm != 0 && p.post_norm != 1) return false;
  for (int i = 0; i < 7; ++i)
    if (p.reserved[i] != 0) return false;
  g.H = p.hidden;
  g.I = p.inter;
  g.slots = p.local_count + (p.shared_inter ? 1 : 0);
  g.kk = p.top_k + (p.shared_inter ? 1 : 0);
  g.T = p.max_tokens;
  g.R = g.T * g.kk;
  if (g.R > kMaxRoutes) return false;
  g.Rpad = g.R + kChunkRows;
  g.pairs13 = g.I / kTileRows;
  g.stages13 = g.H / kStageK;
  g.pairs2 = g.H / (2 * kTileRows);
  g.stages2 = g.I / kStageK;
  g.w13_expert_bytes = static_cast<size_t>(g.pairs13) * g.stages13 * kStageBytes;
  g.w2_expert_bytes = static_cast<size_t>(g.pairs2) * g.stages2 * kStageBytes;
  g.max_items = g.slots + g.R / 16 + 1;
  size_t o = 0;
  g.off_meta = o;     o = align_up(o + kMetaWords * 4, 256);
  g.off_counts = o;   o = align_up(o + static_cast<size_t>(g.slots + 1) * 4, 256);
  g.off_items = o;    o = align_up(o + static_cast<size_t>(g.max_items) * 16, 256);
  g.off_done = o;     o = align_up(o + static_cast<size_t>(g.max_items) * 4, 256);
  g.off_sorted = o;   o = align_up(o + static_cast<size_t>(g.R) * 4, 256);
  g.off_pos = o;      o = align_up(o + static_cast<size_t>(g.R) * 4, 256);
  g.off_wsorted = o;  o = align_up(o + static_cast<size_t>(g.R) * 4, 256);
  g.off_xg = o;       o = align_up(o + static_cast<size_t>(g.Rpad) * g.H * 2, 1024);
  g.off_inter = o;    o = align_up(o + static_cast<size_t>(g.Rpad) * g.I * 2, 1024);
  g.off_y = o;        o = align_up(o + static_cast<size_t>(g.R) * g.H * 4, 1024);
  g.total = o;
  return true;
}

// Exchange buffer of the expert-parallel step (one per rank, the same layout on every rank, mapped
// by every rank): control words used by the owner alone, two flag arrays written by the peers, then
// the gathered token rows, the gathered router logits and this rank's FP32 partial sums.
constexpr int kEpMaxRanks = OKC_EP_MAX_RANKS;
constexpr size_t kEpOffFlagsIn = 256, kEpOffFlagsRs = 512, kEpOffData = 1024;
enum EpCtrlWord { kEpCtrlSeqIn = 0, kEpCtrlSeqRs = 1, kEpCtrlDoneIn = 2, kEpCtrlDoneRs = 3, kEpCtrlStatus = 4, kEpCtrlDetail = 5,
                  kEpCtrlDoneAll = 6 };
struct EpLayout {
  size_t off_hidden, off_logits, off_partial, total;
};
inline EpLayout ep_layout(int tokens, int H, int E) {
  EpLayout l;
  size_t o = kEpOffData;
  l.off_hidden = o;   o = align_up(o + static_cast<size_t>(tokens) * H * 2, 1024);
  l.off_logits = o;   o = align_up(o + static_cast<size_t>(tokens) * E * 4, 1024);
  l.off_partial = o;  o = align_up(o + static_cast<size_t>(tokens) * H * 4, 1024);
  l.total = o;
  return l;
}

#ifdef __CUDACC__
// One stored scale byte -> bf16x2 {scale, scale} * 2^118, with one integer multiply-add (issued to
// the FMA pipe, which has room; the mask / rotate work saturates the integer pipe).
// The stage image does not keep the E4M3 byte itself but `scale_code` of it (below): 16 + 8 * (E + 7)
// + m for the value 2^E * (1 + m/8), with the E4M3 subnormals normalised.  Shifted left by 4 that is
// the exponent and top mantissa bits of a bf16; the added constant rebiases the exponent by 2^118
// (<= 448 * 2^118, finite in bf16).
__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t stored) {
  uint32_t d;
  asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(stored), "n"(0x00100010u), "n"(0x76007600u));
  return d;
}
#endif

// E4M3 magnitude bits (0..127) of a block scale -> the byte kept in the stage image.
//   normal (b >= 8):      value 2^(b/8 - 7) * (1 + (b%8)/8)        -> b + 16
//   subnormal (b = 1..7): value b * 2^-9 = 2^E * (1 + m/8)         -> 16 + 8 * (E + 7) + m  (0, 8, 12, 16, 18, 20, 22)
//   NaN (0x7F):           a byte whose bf16 is a NaN                -> 153
//   zero:                 the repack clears the block's codes instead; any finite scale will do -> 16
__host__ __device__ inline uint32_t scale_code(uint32_t b) {
  if (b == 0x7Fu) return 153u;
  if (b >= 8u) return b + 16u;
  // b:        0   1  2   3   4   5   6   7
  // code:    16   0  8  12  16  18  20  22
  return (0x161412100C080010ull >> (8u * b)) & 0xFFu;
}

#ifdef __CUDACC__
// x << k written as a multiply so that it is issued to the FMA pipe.
template <int K>
__device__ __forceinline__ uint32_t shl_mul(uint32_t x) {
  uint32_t d;
  asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(x), "n"(1u << K));
  return d;
}

// One 16-code block (w0, w1) and its scale (bf16 broadcast to both halves) -> eight bf16x2
// registers holding code * scale * 2^-8, K-ordered (register i = elements 2i, 2i+1).
__device__ __forceinline__ void dequant_block(uint32_t w0, uint32_t w1, uint32_t sc, uint32_t* out) {
  const uint32_t u = (w0 & kLeftMask) | (w1 & ~kLeftMask);
  out[0] = mul_bf16x2(w0 & kOutMask, sc);
  out[1] = mul_bf16x2(rotr32(w0, 4) & kOutMask, sc);
  out[2] = mul_bf16x2(shl_mul<6>(w0) & kOutMask, sc);
  out[3] = mul_bf16x2(rotr32(w1, 2) & kOutMask, sc);
  out[4] = mul_bf16x2(rotr32(w1, 6) & kOutMask, sc);
  out[5] = mul_bf16x2(shl_mul<4>(w1) & kOutMask, sc);
  out[6] = mul_bf16x2(rotr32(u, 8) & kOutMask, sc);
  out[7] = mul_bf16x2(shl_mul<2>(u) & kOutMask, sc);
}

// One 32-code chunk (four words, the two blocks' scale bytes) -> sixteen bf16x2 registers.
__device__ __forceinline__ void dequant_chunk(const uint4& w, uint32_t scale0, uint32_t scale1, uint32_t (&out)[16]) {
  dequant_block(w.x, w.y, scale_bf16x2(scale0), out);
  dequant_block(w.z, w.w, scale_bf16x2(scale1), out + 8);
}
#endif

}  // namespace okc
