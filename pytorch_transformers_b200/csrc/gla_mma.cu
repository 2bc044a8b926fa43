// Gated linear attention, pass 1 of the chunked form on the tensor cores (bfloat16 projections, mma.m16n8k16 with
// float32 sums): a chunk's own sum from a zero state.
//
// A chunk holds n <= 64 tokens j = 0..n-1 with the logarithms l_j [dim] of their decays (float32). Token j's outer
// product k_j v_j^T reaches the chunk's end decayed by the tokens after it, channel by channel:
//     B = sum_j diag(w_j) k_j v_j^T,      w_j[c] = exp(l_(j+1)[c] + .. + l_(n-1)[c])  (<= 1: no factor can grow),
//     total[c] = l_0[c] + .. + l_(n-1)[c]                  the chunk's total decay, for the join
// so B = Kw^T V with Kw[j][c] = w_j[c] k_j[c], a product of [dim, n] by [n, v_dim]. Kw is float32 (the decays and what
// they meet are 32-bit): it enters the product split into two bfloat16 terms, hi + lo; V is a rounded projection.
// The result has the layout of the walk's pass 1 (csrc/gla.cu): sums [chunks][heads][dim][v_dim], chunk_decay
// [chunks][heads][dim].
#include "chunk_mma.cuh"

namespace {

// One block = one chunk x one head; DK / 16 warps, warp w owns rows 16 w .. 16 w + 15 of B [DK, DV].
template <int DK, int DV>
__global__ void __launch_bounds__(DK * 2)
gla_chunk_sum_mma_kernel(const __nv_bfloat16* __restrict__ proj, int stride, const float* __restrict__ log_decay, StepBatch sb,
                         const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0, float* __restrict__ sums,
                         float* __restrict__ chunk_decay, int heads) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* k_hi = sm;                       // [CH][DK] weighted keys, hi
  unsigned char* k_lo = k_hi + CH * DK * 2;       // lo
  unsigned char* v_s = k_lo + CH * DK * 2;        // [CH][DV]
  float* w_s = reinterpret_cast<float*>(v_s + CH * DV * 2);   // [CH][DK]: the logarithms, then the weights w_j[c]
  constexpr int NT = DK * 2;
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  const __nv_bfloat16* row0 = proj + size_t(start) * stride;
  StagedWords<DK, NT> kw;
  StagedWords<DV, NT> vw;
  kw.load(row0 + heads * DK + h * DK, stride, n, tid);
  vw.load(row0 + 2 * heads * DK + h * DV, stride, n, tid);
  {   // the chunk's logarithms, four channels a load (rows from n on: zero)
    constexpr int QUADS = DK / 4, PER = CH * QUADS / NT;
    const float* l0 = log_decay + size_t(start) * heads * DK + h * DK;
    float4 l[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = tid + u * NT, row = i / QUADS, q = i % QUADS;
      l[u] = row < n ? *reinterpret_cast<const float4*>(l0 + size_t(row) * heads * DK + q * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = tid + u * NT, row = i / QUADS, q = i % QUADS;
      *reinterpret_cast<float4*>(w_s + row * DK + q * 4) = l[u];
    }
  }
  __syncthreads();
  if (tid < DK) {     // channel tid from the chunk's last token to its first: what comes after token j, then with it
    float after = 0.f;
#pragma unroll 8
    for (int j = CH - 1; j >= 0; --j) {
      const float l = w_s[j * DK + tid];
      w_s[j * DK + tid] = expf(after);
      after += l;
    }
    chunk_decay[(size_t(c) * heads + h) * DK + tid] = after;
  }
  __syncthreads();
  {
    constexpr int CHUNKS = DK / 8;
#pragma unroll
    for (int u = 0; u < kw.PER; ++u) {
      const int i = tid + u * NT, row = i / CHUNKS, cc = i % CHUNKS;
      float f[8];
      unpack_bf16x8(kw.w[u], f);      // rows from n on were loaded as zeros and their weights are exp(0)
      const float4 wa = *reinterpret_cast<const float4*>(w_s + row * DK + cc * 8);
      const float4 wb = *reinterpret_cast<const float4*>(w_s + row * DK + cc * 8 + 4);
      uint4 hi, lo;
      split_pack(f[0] * wa.x, f[1] * wa.y, hi.x, lo.x);
      split_pack(f[2] * wa.z, f[3] * wa.w, hi.y, lo.y);
      split_pack(f[4] * wb.x, f[5] * wb.y, hi.z, lo.z);
      split_pack(f[6] * wb.z, f[7] * wb.w, hi.w, lo.w);
      *reinterpret_cast<uint4*>(k_hi + swz<DK>(row, cc)) = hi;
      *reinterpret_cast<uint4*>(k_lo + swz<DK>(row, cc)) = lo;
    }
  }
  vw.store(v_s, 0, tid);
  __syncthreads();

  float acc[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const uint32_t khi = smem_u32(k_hi), klo = smem_u32(k_lo), vs = smem_u32(v_s);
  const int m = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < CH / 16; ++kk) {
    // A[m = d][k = s] from the [s][d] tiles: transposed 8x8 matrices (d 0-7 | 8-15) x (s 0-7 | 8-15)
    uint32_t ah[4], al[4];
    const uint32_t off = swz<DK>(kk * 16 + (m >> 1) * 8 + (lane & 7), warp * 2 + (m & 1));
    ldmatrix_x4_trans(ah[0], ah[1], ah[2], ah[3], khi + off);
    ldmatrix_x4_trans(al[0], al[1], al[2], al[3], klo + off);
#pragma unroll
    for (int j = 0; j < DV / 8; j += 2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vs + swz<DV>(kk * 16 + (m & 1) * 8 + (lane & 7), j + (m >> 1)));
      mma_bf16(acc[j], ah, b0, b1);
      mma_bf16(acc[j], al, b0, b1);
      mma_bf16(acc[j + 1], ah, b2, b3);
      mma_bf16(acc[j + 1], al, b2, b3);
    }
  }
  float* dst = sums + (size_t(c) * heads + h) * DK * DV;
  const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) {
    *reinterpret_cast<float2*>(dst + size_t(warp * 16 + g4) * DV + j * 8 + t4 * 2) = make_float2(acc[j][0], acc[j][1]);
    *reinterpret_cast<float2*>(dst + size_t(warp * 16 + g4 + 8) * DV + j * 8 + t4 * 2) = make_float2(acc[j][2], acc[j][3]);
  }
}

template <int DK, int DV>
int launch_sum(const void* proj, int stride, const float* log_decay, const StepBatch& sb, const int* chunk_seq,
               const int* chunk_q0, int n_chunks, float* sums, float* chunk_decay, int heads, cudaStream_t stream) {
  const size_t smem = size_t(2) * CH * DK * 2 + size_t(CH) * DV * 2 + size_t(CH) * DK * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gla_chunk_sum_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  gla_chunk_sum_mma_kernel<DK, DV><<<dim3(n_chunks, heads), DK * 2, smem, stream>>>((const __nv_bfloat16*)proj, stride, log_decay, sb,
                                                                                   chunk_seq, chunk_q0, sums, chunk_decay, heads);
  return launch_status();
}

}  // namespace

// Sizes and layouts that this pass takes: bfloat16 projections, keys and values of 64 or 128 entries, rows that start
// at whole 16-byte words (then q, k, v and the logarithms' rows do too).
PTB_API int ptb_gla_chunk_sum_mma_supports(int dtype, const void* proj, int stride, const float* log_decay, int dim, int v_dim) {
  return (dtype == PTB_BF16 && (dim == 64 || dim == 128) && (v_dim == 64 || v_dim == 128) && stride % 8 == 0 &&
          reinterpret_cast<size_t>(proj) % 16 == 0 && reinterpret_cast<size_t>(log_decay) % 16 == 0) ? 1 : 0;
}

// Every chunk's own sum and total decay (the caller has checked ptb_gla_chunk_sum_mma_supports and the sizes).
PTB_API int ptb_gla_chunk_sum_mma(const void* proj, int stride, const float* log_decay, const StepBatch* sb, const int* chunk_seq,
                                  const int* chunk_q0, int n_chunks, float* sums, float* chunk_decay, int heads, int dim,
                                  int v_dim, cudaStream_t stream) {
  if (n_chunks <= 0) return PTB_OK;
#define PTB_GLA_SUM(DK, DV) \
  return launch_sum<DK, DV>(proj, stride, log_decay, *sb, chunk_seq, chunk_q0, n_chunks, sums, chunk_decay, heads, stream)
  if (dim == 64 && v_dim == 64) PTB_GLA_SUM(64, 64);
  if (dim == 64 && v_dim == 128) PTB_GLA_SUM(64, 128);
  if (dim == 128 && v_dim == 64) PTB_GLA_SUM(128, 64);
  if (dim == 128 && v_dim == 128) PTB_GLA_SUM(128, 128);
#undef PTB_GLA_SUM
  return PTB_ERR_SIZE;
}
