// The chunked form of linear attention with a fixed decay per head on the tensor cores (bfloat16 projections,
// mma.m16n8k16 with float32 sums). With b the head's decay, a chunk's tokens i = 0..n-1 (n <= 64), S0 [DK, DV] the
// state before the chunk and q, k, v the activated projections rounded to bfloat16:
//     pass 1 (sum):   B = sum_s (b^(n-1-s) k_s) v_s^T                                     per chunk, parallel
//     pass 2 (join):  S0 of every chunk, in order (csrc/linear_attention.cu)                elementwise float32
//     pass 3 (out):   o_i = b^(i+1) (q_i^T S0) + sum_{s<=i} (b^(i-s) q_i . k_s) v_s           per chunk, parallel
// Everything that is not a rounded projection stays in 32-bit: a float32 operand of a product (decayed keys, decayed
// scores, the state) is split into two bfloat16 values hi + lo (hi the rounded value, lo the rounded rest, together
// 16 bits of mantissa) and multiplied in two instructions whose float32 sums add up.
#include "chunk_mma.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ pass 1
// One block = one chunk x one head; DK / 16 warps, warp w owns rows 16 w .. 16 w + 15 of B [DK, DV].
template <int DK, int DV>
__global__ void __launch_bounds__(DK * 2)
la_chunk_sum_mma_kernel(const __nv_bfloat16* __restrict__ proj, int stride, StepBatch sb,
                        const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0,
                        const float* __restrict__ decay, float* __restrict__ sums, int heads, int act_silu) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* k_hi = sm;                       // [CH][DK] decayed keys, hi
  unsigned char* k_lo = k_hi + CH * DK * 2;       // lo
  unsigned char* v_s = k_lo + CH * DK * 2;        // [CH][DV]
  float* pw = reinterpret_cast<float*>(v_s + CH * DV * 2);   // b^0 .. b^CH
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  if (tid == 0) {
    const float a = decay[h];
    float p = 1.f;
    for (int i = 0; i <= CH; ++i) {
      pw[i] = p;
      p *= a;
    }
  }
  const __nv_bfloat16* row0 = proj + size_t(start) * stride;
  StagedWords<DK, DK * 2> kw;
  StagedWords<DV, DK * 2> vw;
  kw.load(row0 + heads * DK + h * DK, stride, n, tid);
  vw.load(row0 + 2 * heads * DK + h * DV, stride, n, tid);
  __syncthreads();
  {
    constexpr int CHUNKS = DK / 8;
#pragma unroll
    for (int u = 0; u < kw.PER; ++u) {
      const int i = tid + u * DK * 2, row = i / CHUNKS, cc = i % CHUNKS;
      float f[8];
      act8(kw.w[u], act_silu, f);
      const float w = row < n ? pw[n - 1 - row] : 0.f;
      uint4 hi, lo;
      split_pack(f[0] * w, f[1] * w, hi.x, lo.x);
      split_pack(f[2] * w, f[3] * w, hi.y, lo.y);
      split_pack(f[4] * w, f[5] * w, hi.z, lo.z);
      split_pack(f[6] * w, f[7] * w, hi.w, lo.w);
      *reinterpret_cast<uint4*>(k_hi + swz<DK>(row, cc)) = hi;
      *reinterpret_cast<uint4*>(k_lo + swz<DK>(row, cc)) = lo;
    }
  }
  vw.store(v_s, act_silu, tid);
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

// ------------------------------------------------------------------------------------------------ pass 3
// One block = one chunk x one head; 8 warps: warp w owns the chunk's tokens 16 (w % 4) .. + 15 and half w / 4 of the
// value columns (both halves form the same scores; the staging of the tiles has twice the threads).
template <int DK, int DV>
__global__ void __launch_bounds__(256)
la_chunk_out_mma_kernel(const __nv_bfloat16* __restrict__ proj, int stride, StepBatch sb,
                        const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0,
                        const float* __restrict__ decay, const float* __restrict__ before, float* __restrict__ out,
                        int heads, int act_silu) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* q_s = sm;                          // [CH][DK]
  unsigned char* k_s = q_s + CH * DK * 2;           // [CH][DK]
  unsigned char* v_s = k_s + CH * DK * 2;           // [CH][DV]
  unsigned char* s_hi = v_s + CH * DV * 2;          // [DK][DV] the state before the chunk, hi
  unsigned char* s_lo = s_hi + DK * DV * 2;         // lo
  float* pw = reinterpret_cast<float*>(s_lo + DK * DV * 2);
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3, half = tid >> 7;
  constexpr int NT = DV / 16;       // n-tiles of 8 value columns that a warp owns
  const int j0 = half * NT;         // its first
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  if (tid == 0) {
    const float a = decay[h];
    float p = 1.f;
    for (int i = 0; i <= CH; ++i) {
      pw[i] = p;
      p *= a;
    }
  }
  const __nv_bfloat16* row0 = proj + size_t(start) * stride;
  {
    StagedWords<DK, 256> qw, kw;
    StagedWords<DV, 256> vw;
    qw.load(row0 + h * DK, stride, n, tid);
    kw.load(row0 + heads * DK + h * DK, stride, n, tid);
    vw.load(row0 + 2 * heads * DK + h * DV, stride, n, tid);
    qw.store(q_s, act_silu, tid);
    kw.store(k_s, act_silu, tid);
    vw.store(v_s, act_silu, tid);
  }
  {
    const float* S0 = before + (size_t(c) * heads + h) * DK * DV;
    constexpr int CHUNKS = DV / 8, PER = DK * CHUNKS / 256, BATCH = PER < 4 ? PER : 4;
    static_assert(PER % BATCH == 0, "the state's words divide among the threads in whole batches");
#pragma unroll
    for (int u0 = 0; u0 < PER; u0 += BATCH) {
      float4 x[BATCH], y[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = tid + (u0 + u) * 256, row = i / CHUNKS, cc = i % CHUNKS;
        x[u] = *reinterpret_cast<const float4*>(S0 + size_t(row) * DV + cc * 8);
        y[u] = *reinterpret_cast<const float4*>(S0 + size_t(row) * DV + cc * 8 + 4);
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = tid + (u0 + u) * 256, row = i / CHUNKS, cc = i % CHUNKS;
        uint4 hi, lo;
        split_pack(x[u].x, x[u].y, hi.x, lo.x);
        split_pack(x[u].z, x[u].w, hi.y, lo.y);
        split_pack(y[u].x, y[u].y, hi.z, lo.z);
        split_pack(y[u].z, y[u].w, hi.w, lo.w);
        *reinterpret_cast<uint4*>(s_hi + swz<DV>(row, cc)) = hi;
        *reinterpret_cast<uint4*>(s_lo + swz<DV>(row, cc)) = lo;
      }
    }
  }
  __syncthreads();
  const uint32_t qs = smem_u32(q_s), ks = smem_u32(k_s), vs = smem_u32(v_s), shi = smem_u32(s_hi), slo = smem_u32(s_lo);
  const int g4 = lane >> 2, t4 = lane & 3, m = lane >> 3;

  // the warp's queries as A fragments
  uint32_t qa[DK / 16][4];
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk)
    ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], qs + swz<DK>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));

  // o = b^(i+1) q_i^T S0
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b0, b1, b2, b3;
      const uint32_t off = swz<DV>(kk * 16 + (m & 1) * 8 + (lane & 7), j0 + j + (m >> 1));
      ldmatrix_x4_trans(b0, b1, b2, b3, shi + off);
      mma_bf16(o[j], qa[kk], b0, b1);
      mma_bf16(o[j + 1], qa[kk], b2, b3);
      ldmatrix_x4_trans(b0, b1, b2, b3, slo + off);
      mma_bf16(o[j], qa[kk], b0, b1);
      mma_bf16(o[j + 1], qa[kk], b2, b3);
    }
  }
  const int r_lo = warp * 16 + g4, r_hi = r_lo + 8;      // this thread's two tokens of the chunk
  {
    const float f_lo = pw[r_lo + 1], f_hi = pw[r_hi + 1];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= f_lo; o[j][1] *= f_lo;
      o[j][2] *= f_hi; o[j][3] *= f_hi;
    }
  }
  // scores of the chunk, decayed and cut at the diagonal, then times the values: only key blocks up to the warp's own
#pragma unroll
  for (int kb = 0; kb < CH / 16; ++kb) {
    if (kb > warp) break;
    float s[2][4];
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      s[jj][0] = s[jj][1] = s[jj][2] = s[jj][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; kk += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + swz<DK>(kb * 16 + jj * 8 + (lane & 7), 2 * kk + (lane >> 3)));
        mma_bf16(s[jj], qa[kk], b0, b1);
        mma_bf16(s[jj], qa[kk + 1], b2, b3);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (e >> 1) ? r_hi : r_lo, col = kb * 16 + jj * 8 + t4 * 2 + (e & 1);
        s[jj][e] = col <= row ? s[jj][e] * pw[row - col] : 0.f;
      }
    }
    uint32_t ph[4], pl[4];
    split_pack(s[0][0], s[0][1], ph[0], pl[0]);
    split_pack(s[0][2], s[0][3], ph[1], pl[1]);
    split_pack(s[1][0], s[1][1], ph[2], pl[2]);
    split_pack(s[1][2], s[1][3], ph[3], pl[3]);
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vs + swz<DV>(kb * 16 + (m & 1) * 8 + (lane & 7), j0 + j + (m >> 1)));
      mma_bf16(o[j], ph, b0, b1);
      mma_bf16(o[j], pl, b0, b1);
      mma_bf16(o[j + 1], ph, b2, b3);
      mma_bf16(o[j + 1], pl, b2, b3);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = i ? r_hi : r_lo;
    if (r >= n) continue;
    float* dst = out + (size_t(start + r) * heads + h) * DV + j0 * 8 + t4 * 2;
#pragma unroll
    for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][2 * i], o[j][2 * i + 1]);
  }
}

template <int DK, int DV>
int launch_sum(const void* proj, int stride, const StepBatch& sb, const int* chunk_seq, const int* chunk_q0, int n_chunks,
               const float* decay, float* sums, int heads, int act, cudaStream_t stream) {
  const size_t smem = size_t(2) * CH * DK * 2 + size_t(CH) * DV * 2 + (CH + 1) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(la_chunk_sum_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  la_chunk_sum_mma_kernel<DK, DV><<<dim3(n_chunks, heads), DK * 2, smem, stream>>>((const __nv_bfloat16*)proj, stride, sb, chunk_seq,
                                                                                  chunk_q0, decay, sums, heads, act);
  return launch_status();
}

template <int DK, int DV>
int launch_out(const void* proj, int stride, const StepBatch& sb, const int* chunk_seq, const int* chunk_q0, int n_chunks,
               const float* decay, const float* before, float* out, int heads, int act, cudaStream_t stream) {
  const size_t smem = size_t(2) * CH * DK * 2 + size_t(CH) * DV * 2 + size_t(2) * DK * DV * 2 + (CH + 1) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(la_chunk_out_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  la_chunk_out_mma_kernel<DK, DV><<<dim3(n_chunks, heads), 256, smem, stream>>>((const __nv_bfloat16*)proj, stride, sb, chunk_seq,
                                                                               chunk_q0, decay, before, out, heads, act);
  return launch_status();
}

}  // namespace

// Sizes and alignment that the tensor-core passes take: keys and values of 64 or 128 entries, projection rows
// whose q, k and v parts start at whole 16-byte words.
PTB_API int ptb_linear_attention_mma_supports(int dim, int v_dim) {
  return ((dim == 64 || dim == 128) && (v_dim == 64 || v_dim == 128)) ? 1 : 0;
}

// pass 1 (which = 0): sums [n_chunks, heads, dim, v_dim] <- every chunk's own sum; pass 3 (which = 1): `sums` holds the
// state before every chunk, out float32 [tokens, heads * v_dim]. bfloat16 projections only.
PTB_API int ptb_linear_attention_chunks_mma(int which, const void* proj, int stride, const StepBatch* sb, const int* chunk_seq,
                                            const int* chunk_q0, int n_chunks, const float* decay, float* sums, float* out,
                                            int heads, int dim, int v_dim, int act, cudaStream_t stream) {
  if (sb->n_tokens <= 0 || n_chunks <= 0) return PTB_OK;
  if (!ptb_linear_attention_mma_supports(dim, v_dim) || heads <= 0 || heads > 65535 || stride < 2 * heads * dim + heads * v_dim)
    return PTB_ERR_SIZE;
  if (!aligned16(proj) || stride % 8 != 0) return PTB_ERR_ALIGN;
#define PTB_LA(DK, DV)                                                                                                         \
  return which == 0 ? launch_sum<DK, DV>(proj, stride, *sb, chunk_seq, chunk_q0, n_chunks, decay, sums, heads, act, stream)    \
                    : launch_out<DK, DV>(proj, stride, *sb, chunk_seq, chunk_q0, n_chunks, decay, sums, out, heads, act, stream)
  if (dim == 64 && v_dim == 64) PTB_LA(64, 64);
  if (dim == 64 && v_dim == 128) PTB_LA(64, 128);
  if (dim == 128 && v_dim == 64) PTB_LA(128, 64);
  PTB_LA(128, 128);
#undef PTB_LA
}
