// Prepare-time lossless repack of NVFP4 tensors into stage images, and its inverse on CUDA cores.
// Takes the place of the reference's torch repackers `_pack_weight`, `_pack_scales`, `_sq_pack`
// (muse_moe_w4a16/submission.py:5916-5952); the image layout is this library's own.
#include "params.cuh"

namespace okc {

// Destination bit (word * 32 + bit, inside a two-word block) of bit b of code j: entry j*4 + b.
// Generated from the plan {w0: as is, rotr 4, shl 6; w1: rotr 2, rotr 6, shl 4; merged leftovers: rotr 8, shl 2}.
__constant__ uint8_t kPairShift[64] = {
    6, 7, 8, 15, 22, 23, 24, 31, 10, 11, 12, 19, 26, 27, 28, 3, 0, 1, 2, 9, 16, 17, 18, 25, 40, 41,
    42, 49, 56, 57, 58, 33, 44, 45, 46, 53, 60, 61, 62, 37, 34, 35, 36, 43, 50, 51, 52, 59, 14, 47,
    48, 55, 30, 63, 32, 39, 4, 5, 38, 13, 20, 21, 54, 29};


// One thread per (expert, pair, stage, tile, chunk, row): 16 source bytes + 2 scale bytes.
__global__ void __launch_bounds__(256) okc_repack(const RepackParams p) {
  const size_t per_expert = static_cast<size_t>(p.pairs) * p.stages * 2 * kChunks * kTileRows;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= per_expert * p.count) return;
  const int ex = static_cast<int>(gid / per_expert);
  size_t r = gid - static_cast<size_t>(ex) * per_expert;
  const int row = static_cast<int>(r % kTileRows); r /= kTileRows;
  const int chunk = static_cast<int>(r % kChunks); r /= kChunks;
  const int tile = static_cast<int>(r % 2); r /= 2;
  const int stage = static_cast<int>(r % p.stages); r /= p.stages;
  const int pair = static_cast<int>(r);

  const int src_row = p.is_w13 ? (tile * p.inter + pair * kTileRows + row) : (pair * 2 * kTileRows + tile * kTileRows + row);
  const int k0 = stage * kStageK + chunk * kChunkK;
  const uint8_t* src = p.w + (static_cast<size_t>(ex) * p.rows + src_row) * (p.K / 2) + k0 / 2;
  const uint8_t* ssf = p.sf + (static_cast<size_t>(ex) * p.rows + src_row) * (p.K / 16) + k0 / 16;
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t outw[4];
  uint32_t stored[2];
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    // The scale goes into the image as scale_code(magnitude bits).  What that code cannot say is
    // said through the codes, without changing any product: a zero scale clears the block's codes,
    // a negative scale flips their signs.
    const uint32_t sb = ssf[blk];
    stored[blk] = scale_code(sb & 0x7Fu);
    if ((sb & 0x7Fu) == 0u) { words[2 * blk] = 0u; words[2 * blk + 1] = 0u; }
    if (sb & 0x80u) { words[2 * blk] ^= 0x88888888u; words[2 * blk + 1] ^= 0x88888888u; }
    const uint64_t codes = static_cast<uint64_t>(words[2 * blk]) | (static_cast<uint64_t>(words[2 * blk + 1]) << 32);
    uint64_t o = 0;
    for (int j = 0; j < 16; ++j)
#pragma unroll
      for (int b = 0; b < 4; ++b) o |= ((codes >> (4 * j + b)) & 1ull) << kPairShift[j * 4 + b];
    outw[2 * blk] = static_cast<uint32_t>(o);
    outw[2 * blk + 1] = static_cast<uint32_t>(o >> 32);
  }
  uint8_t* img = p.out + static_cast<size_t>(p.first_slot + ex) * p.expert_bytes +
                 (static_cast<size_t>(pair) * p.stages + stage) * kStageBytes;
  *reinterpret_cast<uint4*>(img + stage_code_offset(tile, chunk, row)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
  *reinterpret_cast<uint16_t*>(img + stage_scale_offset(tile, chunk, row)) =
      static_cast<uint16_t>(stored[0]) | (static_cast<uint16_t>(stored[1]) << 8);
}


__global__ void __launch_bounds__(256) okc_unpack(const UnpackParams p) {
  const size_t total = static_cast<size_t>(p.pairs) * p.stages * 2 * kChunks * kTileRows;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= total) return;
  size_t r = gid;
  const int row = static_cast<int>(r % kTileRows); r /= kTileRows;
  const int chunk = static_cast<int>(r % kChunks); r /= kChunks;
  const int tile = static_cast<int>(r % 2); r /= 2;
  const int stage = static_cast<int>(r % p.stages); r /= p.stages;
  const int pair = static_cast<int>(r);
  const uint8_t* img = p.packed + (static_cast<size_t>(pair) * p.stages + stage) * kStageBytes;
  const uint4 w = *reinterpret_cast<const uint4*>(img + stage_code_offset(tile, chunk, row));
  const uint8_t* sc = img + stage_scale_offset(tile, chunk, row);
  uint32_t regs[16];
  dequant_chunk(w, sc[0], sc[1], regs);
  const int dst_row = p.is_w13 ? (tile * p.inter + pair * kTileRows + row) : (pair * 2 * kTileRows + tile * kTileRows + row);
  uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + static_cast<size_t>(dst_row) * p.K + stage * kStageK + chunk * kChunkK);
#pragma unroll
  for (int i = 0; i < 16; ++i) dst[i] = regs[i];
}

cudaError_t launch_repack(const RepackParams& p, cudaStream_t stream) {
  const size_t total = static_cast<size_t>(p.pairs) * p.stages * 2 * kChunks * kTileRows * p.count;
  const size_t blocks = (total + 255) / 256;
  if (blocks == 0) return cudaSuccess;
  okc_repack<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_unpack(const UnpackParams& p, cudaStream_t stream) {
  const size_t total = static_cast<size_t>(p.pairs) * p.stages * 2 * kChunks * kTileRows;
  okc_unpack<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace okc
