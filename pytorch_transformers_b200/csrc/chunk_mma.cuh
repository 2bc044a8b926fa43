// Pieces shared by the chunked recurrences on the tensor cores (linear attention with a fixed decay, the matrix memory
// with exponential gates): the chunk's size, the split of a float32 operand into two bfloat16 terms, and the staging
// of a chunk's projection rows into swizzled shared tiles.
#pragma once
#include "mma_common.cuh"

namespace {

constexpr int CH = 64;   // tokens of a chunk: ptb_linear_attention_chunk_tokens()

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// hi + lo of two float32 values as packed bfloat16 pairs
__device__ __forceinline__ void split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  const __nv_bfloat162 h = __halves2bfloat162(xh, yh);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - __bfloat162float(xh), y - __bfloat162float(yh));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// 8 values of a projection row (one 16-byte word) activated: float32 values rounded to bfloat16
__device__ __forceinline__ void act8(const uint4& w, int act_silu, float (&f)[8]) {
  unpack_bf16x8(w, f);
  if (act_silu) {
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = round_bf16(silu_f(f[e]));
  }
}

// The 16-byte words of rows [0, CH) x D columns of a projection that thread `tid` of NT stages: all loads are issued
// before the first is used (rows >= n read as zero, which silu keeps).
template <int D, int NT>
struct StagedWords {
  static constexpr int CHUNKS = D / 8, PER = CH * CHUNKS / NT;
  uint4 w[PER];
  __device__ __forceinline__ void load(const __nv_bfloat16* first_row, int stride, int n, int tid) {
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = tid + u * NT, row = i / CHUNKS, c = i % CHUNKS;
      w[u] = row < n ? *reinterpret_cast<const uint4*>(first_row + size_t(row) * stride + c * 8) : make_uint4(0, 0, 0, 0);
    }
  }
  // activated, into a swizzled [CH][D] tile
  __device__ __forceinline__ void store(unsigned char* tile, int act_silu, int tid) const {
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = tid + u * NT, row = i / CHUNKS, c = i % CHUNKS;
      float f[8];
      act8(w[u], act_silu, f);
      *reinterpret_cast<uint4*>(tile + swz<D>(row, c)) = pack_bf16x8(f);
    }
  }
};

}  // namespace
