// The chunked form of the matrix memory with exponential gates (mLSTM) on the tensor cores (bfloat16 projections,
// mma.m16n8k16 with float32 sums). A chunk holds n <= 64 tokens j = 0..n-1 with the gates' logarithms i_j and f_j;
// (S0, n0, m0) is the state before the chunk. With b_j = f_0 + .. + f_j, c_j = i_j - b_j and M_t = max_{j<=t} c_j:
//     m_t = b_t + max(m0, M_t)                           the running maximum that the token-by-token form carries
//     pass 1 (sum):   B = sum_j exp(c_j - M_(n-1)) k_j v_j^T, the same sum of k_j alone, g = b_(n-1), M_(n-1)
//     pass 2 (join):  m1 = max(g + m0, g + M); S1 = exp(g + m0 - m1) S0 + exp(g + M - m1) B; n likewise; in order
//     pass 3 (out):   with mm_t = max(m0, M_t), e_t = exp(m0 - mm_t), D_tj = exp(c_j - mm_t) for j <= t:
//                     num_t = e_t q_t^T S0 + sum_j D_tj (q_t . k_j) v_j,   den_t = e_t q_t . n0 + sum_j D_tj (q_t . k_j)
//                     o_t = num_t / (max(|den_t|, exp(-m_t)) + 1e-6)
// q carries the factor q_scale, which multiplies the float32 sums. Everything that is not a rounded projection is
// 32-bit: a float32 operand of a product (weighted keys, weighted scores, the state) is split into two bfloat16 terms.
// The state area's layout is the token-by-token kernel's (csrc/mlstm.cu): S [heads][dim][v_dim], then for every head
// and every stretch of 32 value columns a copy of n [dim] and m [1].
#include "chunk_mma.cuh"

namespace {

constexpr int VB = 32;   // value columns per copy of n and m in the state area, as in csrc/mlstm.cu

// Warp 0 of a block: b, c and the prefix maxima M of a chunk's gates into shared arrays of CH entries. Tokens from
// n on have f = 0 and i = -inf, so that entry CH - 1 holds the chunk's totals.
__device__ __forceinline__ void chunk_gates(const float* __restrict__ gates, int start, int n, int h, int heads, int lane,
                                            float* b_s, float* c_s, float* M_s) {
  const unsigned full = 0xffffffffu;
  const int j0 = 2 * lane, j1 = j0 + 1;
  const float f0 = j0 < n ? gates[size_t(start + j0) * 2 * heads + heads + h] : 0.f;
  const float f1 = j1 < n ? gates[size_t(start + j1) * 2 * heads + heads + h] : 0.f;
  const float i0 = j0 < n ? gates[size_t(start + j0) * 2 * heads + h] : -INFINITY;
  const float i1 = j1 < n ? gates[size_t(start + j1) * 2 * heads + h] : -INFINITY;
  float s = f0 + f1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(full, s, o);
    if (lane >= o) s += t;
  }
  float before = __shfl_up_sync(full, s, 1);
  if (lane == 0) before = 0.f;
  const float b0 = before + f0, b1 = b0 + f1;
  const float c0 = i0 - b0, c1 = i1 - b1;
  float mx = fmaxf(c0, c1);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(full, mx, o);
    if (lane >= o) mx = fmaxf(mx, t);
  }
  float mb = __shfl_up_sync(full, mx, 1);
  if (lane == 0) mb = -INFINITY;
  const float M0 = fmaxf(mb, c0), M1 = fmaxf(M0, c1);
  b_s[j0] = b0; b_s[j1] = b1;
  c_s[j0] = c0; c_s[j1] = c1;
  M_s[j0] = M0; M_s[j1] = M1;
}

// ------------------------------------------------------------------------------------------------ pass 1
// One block = one chunk x one head; DK / 16 warps, warp w owns rows 16 w .. 16 w + 15 of B [DK, DV].
template <int DK, int DV>
__global__ void __launch_bounds__(DK * 2)
mlstm_chunk_sum_kernel(const __nv_bfloat16* __restrict__ proj, int stride, const float* __restrict__ gates, StepBatch sb,
                       const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0, float* __restrict__ sums,
                       float* __restrict__ nsums, float* __restrict__ meta, int heads) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* k_hi = sm;                       // [CH][DK] weighted keys, hi
  unsigned char* k_lo = k_hi + CH * DK * 2;       // lo
  unsigned char* v_s = k_lo + CH * DK * 2;        // [CH][DV]
  float* b_s = reinterpret_cast<float*>(v_s + CH * DV * 2);
  float* c_s = b_s + CH;
  float* M_s = c_s + CH;
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  const __nv_bfloat16* row0 = proj + size_t(start) * stride;
  StagedWords<DK, DK * 2> kw;
  StagedWords<DV, DK * 2> vw;
  kw.load(row0 + heads * DK + h * DK, stride, n, tid);
  vw.load(row0 + 2 * heads * DK + h * DV, stride, n, tid);
  if (warp == 0) chunk_gates(gates, start, n, h, heads, lane, b_s, c_s, M_s);
  __syncthreads();
  const float M_all = M_s[CH - 1];
  {
    constexpr int CHUNKS = DK / 8;
#pragma unroll
    for (int u = 0; u < kw.PER; ++u) {
      const int i = tid + u * DK * 2, row = i / CHUNKS, cc = i % CHUNKS;
      float f[8];
      unpack_bf16x8(kw.w[u], f);
      const float w = row < n ? expf(c_s[row] - M_all) : 0.f;
      uint4 hi, lo;
      split_pack(f[0] * w, f[1] * w, hi.x, lo.x);
      split_pack(f[2] * w, f[3] * w, hi.y, lo.y);
      split_pack(f[4] * w, f[5] * w, hi.z, lo.z);
      split_pack(f[6] * w, f[7] * w, hi.w, lo.w);
      *reinterpret_cast<uint4*>(k_hi + swz<DK>(row, cc)) = hi;
      *reinterpret_cast<uint4*>(k_lo + swz<DK>(row, cc)) = lo;
    }
  }
  vw.store(v_s, 0, tid);
  __syncthreads();

  if (tid < DK) {     // the weighted keys' own sum, entry tid
    float acc = 0.f;
    const uint32_t in_word = (tid & 7) * 2;
    for (int row = 0; row < n; ++row) {
      const uint32_t off = swz<DK>(row, tid >> 3) + in_word;
      acc += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(k_hi + off)) +
             __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(k_lo + off));
    }
    nsums[(size_t(c) * heads + h) * DK + tid] = acc;
  }
  if (tid == 0) {
    meta[(size_t(c) * heads + h) * 2] = b_s[CH - 1];
    meta[(size_t(c) * heads + h) * 2 + 1] = M_all;
  }

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

// ------------------------------------------------------------------------------------------------ pass 2
// First the heads' chains of maxima, which are two numbers a chunk: a warp per (sequence, head) reads 32 chunks' totals
// and maxima at a time, follows m_new = max(g + m, g + M) in order (the sums that the token-by-token form makes), and
// leaves for every chunk the maximum before it (m_before) and, in place of (g, M), the two factors of its join:
// exp(g + m - m_new) on the state so far and exp(g + M - m_new) on the chunk's own sums. m_after [sequences][heads]
// receives the maximum after the sequence's last chunk. The state area is only read here.
__global__ void mlstm_chunk_decay_kernel(float* __restrict__ meta, float* __restrict__ m_before, float* __restrict__ m_after,
                                         const float* __restrict__ state, int state_stride, const int* __restrict__ slots,
                                         StepBatch sb, const int* __restrict__ seq_chunk0, int heads, int dim, int v_dim) {
  const unsigned full = 0xffffffffu;
  const int seq = blockIdx.y, lane = threadIdx.x & 31;
  const int h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (h >= heads) return;
  const size_t per_S = size_t(dim) * v_dim;
  const int copies = (v_dim + VB - 1) / VB;
  const int n_new = sb.seq_new[seq], c0 = seq_chunk0[seq];
  const int n_chunks = (n_new + CH - 1) / CH;
  const float* st = state + size_t(slots[seq]) * state_stride;
  float m = st[size_t(heads) * per_S + size_t(h) * copies * (dim + 1) + dim];
  for (int g0 = 0; g0 < n_chunks; g0 += 32) {
    const int c = g0 + lane;
    const bool ok = c < n_chunks;
    float* mt = meta + (size_t(c0 + c) * heads + h) * 2;
    const float tot = ok ? mt[0] : 0.f, mx = ok ? mt[1] : 0.f;
    float m_prev = 0.f, m_mine = 0.f;
    const int n_here = min(32, n_chunks - g0);
    for (int i = 0; i < n_here; ++i) {
      const float t = __shfl_sync(full, tot, i), x = __shfl_sync(full, mx, i);
      const float m_new = fmaxf(t + m, t + x);
      if (lane == i) {
        m_prev = m;
        m_mine = m_new;
      }
      m = m_new;
    }
    if (ok) {
      m_before[size_t(c0 + c) * heads + h] = m_prev;
      mt[0] = expf(tot + m_prev - m_mine);
      mt[1] = expf(tot + mx - m_mine);
    }
  }
  if (lane == 0) m_after[size_t(seq) * heads + h] = m;
}

// Then the join itself, elementwise: a thread owns four neighbouring elements of one head's S or n and walks the
// sequence's chunks in order: sums[c] and nsums[c] become the state BEFORE chunk c, and the state area receives the
// state after the last chunk (with m_after in every copy of m). Eight chunks' own sums are loaded ahead of the chain.
__global__ void __launch_bounds__(128)
mlstm_chunk_join_kernel(float* __restrict__ sums, float* __restrict__ nsums, const float* __restrict__ factors,
                        const float* __restrict__ m_after, float* __restrict__ state, int state_stride,
                        const int* __restrict__ slots, StepBatch sb, const int* __restrict__ seq_chunk0, int heads, int dim,
                        int v_dim) {
  const int seq = blockIdx.y;
  const size_t per_S = size_t(dim) * v_dim, per_head = per_S + dim;      // both multiples of 4
  const size_t e = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (e >= per_head * heads) return;
  const int h = int(e / per_head);
  const size_t r = e % per_head;
  const bool is_n = r >= per_S;
  const int copies = (v_dim + VB - 1) / VB;
  const int n_new = sb.seq_new[seq], c0 = seq_chunk0[seq];
  const int n_chunks = (n_new + CH - 1) / CH;
  float* st = state + size_t(slots[seq]) * state_stride;
  float* n_area = st + size_t(heads) * per_S + size_t(h) * copies * (dim + 1);     // the head's copies of n and m
  float* mine = is_n ? n_area + (r - per_S) : st + size_t(h) * per_S + r;          // at no whole 16-byte word in general
  float* chunked = is_n ? nsums + size_t(h) * dim + (r - per_S) : sums + size_t(h) * per_S + r;
  const size_t chunk_stride = is_n ? size_t(heads) * dim : size_t(heads) * per_S;
  float4 s = make_float4(mine[0], mine[1], mine[2], mine[3]);
  constexpr int AHEAD = 8;
  for (int g0 = 0; g0 < n_chunks; g0 += AHEAD) {
    float4 own[AHEAD];
    float keep[AHEAD], add[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      const bool ok = g0 + i < n_chunks;
      own[i] = ok ? *reinterpret_cast<const float4*>(chunked + size_t(c0 + g0 + i) * chunk_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
      keep[i] = ok ? factors[(size_t(c0 + g0 + i) * heads + h) * 2] : 0.f;
      add[i] = ok ? factors[(size_t(c0 + g0 + i) * heads + h) * 2 + 1] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (g0 + i >= n_chunks) break;
      *reinterpret_cast<float4*>(chunked + size_t(c0 + g0 + i) * chunk_stride) = s;
      s.x = fmaf(keep[i], s.x, add[i] * own[i].x);
      s.y = fmaf(keep[i], s.y, add[i] * own[i].y);
      s.z = fmaf(keep[i], s.z, add[i] * own[i].z);
      s.w = fmaf(keep[i], s.w, add[i] * own[i].w);
    }
  }
  if (is_n) {
    const float m = m_after[size_t(seq) * heads + h];
    for (int z = 0; z < copies; ++z) {
      float* dst = n_area + size_t(z) * (dim + 1);
      dst[r - per_S] = s.x;
      dst[r - per_S + 1] = s.y;
      dst[r - per_S + 2] = s.z;
      dst[r - per_S + 3] = s.w;
      if (r == per_S) dst[dim] = m;
    }
  } else {
    mine[0] = s.x;
    mine[1] = s.y;
    mine[2] = s.z;
    mine[3] = s.w;
  }
}

// ------------------------------------------------------------------------------------------------ pass 3
// One block = one chunk x one head; 8 warps: warp w owns the chunk's tokens 16 (w % 4) .. + 15 and half w / 4 of the
// value columns (both halves form the same scores and the same denominators).
template <int DK, int DV>
__global__ void __launch_bounds__(256)
mlstm_chunk_out_kernel(const __nv_bfloat16* __restrict__ proj, int stride, const float* __restrict__ gates, StepBatch sb,
                       const int* __restrict__ chunk_seq, const int* __restrict__ chunk_q0, const float* __restrict__ before,
                       const float* __restrict__ n_before, const float* __restrict__ m_before, float* __restrict__ out,
                       int heads, float q_scale) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* q_s = sm;                          // [CH][DK]
  unsigned char* k_s = q_s + CH * DK * 2;           // [CH][DK]
  unsigned char* v_s = k_s + CH * DK * 2;           // [CH][DV]
  unsigned char* s_hi = v_s + CH * DV * 2;          // [DK][DV] the state before the chunk, hi
  unsigned char* s_lo = s_hi + DK * DV * 2;         // lo
  float* b_s = reinterpret_cast<float*>(s_lo + DK * DV * 2);
  float* c_s = b_s + CH;
  float* M_s = c_s + CH;
  float* qn_s = M_s + CH;                           // [CH] q_t . n0
  float* n0_s = qn_s + CH;                          // [DK]
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3, half = tid >> 7;
  constexpr int NT = DV / 16;       // n-tiles of 8 value columns that a warp owns
  const int j0 = half * NT;         // its first
  const int seq = chunk_seq[c], q0 = chunk_q0[c];
  const int start = sb.seq_start[seq] + q0, n = min(CH, sb.seq_new[seq] - q0);
  const __nv_bfloat16* row0 = proj + size_t(start) * stride;
  {
    StagedWords<DK, 256> qw, kw;
    StagedWords<DV, 256> vw;
    qw.load(row0 + h * DK, stride, n, tid);
    kw.load(row0 + heads * DK + h * DK, stride, n, tid);
    vw.load(row0 + 2 * heads * DK + h * DV, stride, n, tid);
    qw.store(q_s, 0, tid);
    kw.store(k_s, 0, tid);
    vw.store(v_s, 0, tid);
  }
  if ((tid >> 5) == 0) chunk_gates(gates, start, n, h, heads, lane, b_s, c_s, M_s);
  if (tid < DK) n0_s[tid] = n_before[(size_t(c) * heads + h) * DK + tid];
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
  {   // q_t . n0: four threads a token, a quarter of the entries each
    const int row = tid >> 2, part = tid & 3;
    float acc = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < DK / 32; ++w8) {
      const int cc = part * (DK / 32) + w8;
      float f[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(q_s + swz<DK>(row, cc)), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc = fmaf(f[e], n0_s[cc * 8 + e], acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (part == 0) qn_s[row] = acc;
  }
  __syncthreads();
  const uint32_t qs = smem_u32(q_s), ks = smem_u32(k_s), vs = smem_u32(v_s), shi = smem_u32(s_hi), slo = smem_u32(s_lo);
  const int g4 = lane >> 2, t4 = lane & 3, m = lane >> 3;

  // the warp's queries as A fragments
  uint32_t qa[DK / 16][4];
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk)
    ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], qs + swz<DK>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));

  // o = e_t q_t^T S0
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
  const float m0 = m_before[size_t(c) * heads + h];
  const float mm_lo = fmaxf(m0, M_s[r_lo]), mm_hi = fmaxf(m0, M_s[r_hi]);
  float den_lo, den_hi;
  {
    const float e_lo = expf(m0 - mm_lo), e_hi = expf(m0 - mm_hi);
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= e_lo; o[j][1] *= e_lo;
      o[j][2] *= e_hi; o[j][3] *= e_hi;
    }
    den_lo = e_lo * qn_s[r_lo];
    den_hi = e_hi * qn_s[r_hi];
  }
  // scores of the chunk, weighted and cut at the diagonal, then times the values: only key blocks up to the warp's own
  float part_lo = 0.f, part_hi = 0.f;       // this thread's share of sum_j D_tj (q_t . k_j)
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
        s[jj][e] = col <= row ? s[jj][e] * expf(c_s[col] - ((e >> 1) ? mm_hi : mm_lo)) : 0.f;
      }
      part_lo += s[jj][0] + s[jj][1];
      part_hi += s[jj][2] + s[jj][3];
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
  part_lo += __shfl_xor_sync(0xffffffffu, part_lo, 1);
  part_lo += __shfl_xor_sync(0xffffffffu, part_lo, 2);
  part_hi += __shfl_xor_sync(0xffffffffu, part_hi, 1);
  part_hi += __shfl_xor_sync(0xffffffffu, part_hi, 2);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = i ? r_hi : r_lo;
    if (r >= n) continue;
    const float den = q_scale * ((i ? den_hi : den_lo) + (i ? part_hi : part_lo));
    const float floor_ = expf(-(b_s[r] + (i ? mm_hi : mm_lo)));
    const float f = q_scale / (fmaxf(fabsf(den), floor_) + 1e-6f);
    float* dst = out + (size_t(start + r) * heads + h) * DV + j0 * 8 + t4 * 2;
#pragma unroll
    for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][2 * i] * f, o[j][2 * i + 1] * f);
  }
}

template <int DK, int DV>
int launch_sum(const void* proj, int stride, const float* gates, const StepBatch& sb, const int* chunk_seq, const int* chunk_q0,
               int n_chunks, float* sums, float* nsums, float* meta, int heads, cudaStream_t stream) {
  const size_t smem = size_t(2) * CH * DK * 2 + size_t(CH) * DV * 2 + 3 * CH * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(mlstm_chunk_sum_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  mlstm_chunk_sum_kernel<DK, DV><<<dim3(n_chunks, heads), DK * 2, smem, stream>>>((const __nv_bfloat16*)proj, stride, gates, sb,
                                                                                 chunk_seq, chunk_q0, sums, nsums, meta, heads);
  return launch_status();
}

template <int DK, int DV>
int launch_out(const void* proj, int stride, const float* gates, const StepBatch& sb, const int* chunk_seq, const int* chunk_q0,
               int n_chunks, const float* sums, const float* nsums, const float* m_before, float* out, int heads, float q_scale,
               cudaStream_t stream) {
  const size_t smem = size_t(2) * CH * DK * 2 + size_t(CH) * DV * 2 + size_t(2) * DK * DV * 2 + (4 * CH + DK) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(mlstm_chunk_out_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  mlstm_chunk_out_kernel<DK, DV><<<dim3(n_chunks, heads), 256, smem, stream>>>((const __nv_bfloat16*)proj, stride, gates, sb, chunk_seq,
                                                                              chunk_q0, sums, nsums, m_before, out, heads, q_scale);
  return launch_status();
}

}  // namespace

// Sizes that the chunked form takes: keys and values of 64 or 128 entries (bfloat16 projections whose q, k and v parts
// start at whole 16-byte words).
PTB_API int ptb_mlstm_chunks_supports(int dim, int v_dim) {
  return ((dim == 64 || dim == 128) && (v_dim == 64 || v_dim == 128)) ? 1 : 0;
}
PTB_API int ptb_mlstm_chunk_tokens() { return CH; }

// float32 scratch of the chunked form: every chunk's S, n, (total, maximum) and the maximum before it, and the
// maximum after every sequence's last chunk (sequences are no more than chunks)
PTB_API long long ptb_mlstm_chunks_scratch_floats(int n_chunks, int heads, int dim, int v_dim) {
  return (long long)n_chunks * heads * ((long long)dim * v_dim + dim + 4);
}

// The three passes over a step's chunks. proj, gates, state, slots and out as ptb_mlstm_scan takes them (bfloat16
// projections only); chunk_seq, chunk_q0 [n_chunks] and seq_chunk0 [sequences] describe the chunks of 64 tokens;
// scratch holds ptb_mlstm_chunks_scratch_floats floats.
PTB_API int ptb_mlstm_chunks(const void* proj, int stride, const float* gates, float* state, int state_stride, const int* slots,
                             const StepBatch* sb, const int* chunk_seq, const int* chunk_q0, const int* seq_chunk0, int n_chunks,
                             float* scratch, float* out, int heads, int dim, int v_dim, float q_scale, cudaStream_t stream) {
  if (sb->n_tokens <= 0 || n_chunks <= 0) return PTB_OK;
  if (!ptb_mlstm_chunks_supports(dim, v_dim) || heads <= 0 || heads > 65535 || sb->n_seqs > 65535 || sb->n_seqs > n_chunks ||
      stride < 2 * heads * dim + heads * v_dim || state_stride < heads * (dim * v_dim + ((v_dim + VB - 1) / VB) * (dim + 1)))
    return PTB_ERR_SIZE;
  if (!aligned16(proj) || stride % 8 != 0 || !aligned16(scratch)) return PTB_ERR_ALIGN;
  float* sums = scratch;
  float* nsums = sums + size_t(n_chunks) * heads * dim * v_dim;
  float* meta = nsums + size_t(n_chunks) * heads * dim;
  float* m_before = meta + size_t(n_chunks) * heads * 2;
  float* m_after = m_before + size_t(n_chunks) * heads;
  int rc;
#define PTB_ML(DK, DV)                                                                                                          \
  do {                                                                                                                          \
    rc = launch_sum<DK, DV>(proj, stride, gates, *sb, chunk_seq, chunk_q0, n_chunks, sums, nsums, meta, heads, stream);         \
    if (rc != PTB_OK) return rc;                                                                                                \
    mlstm_chunk_decay_kernel<<<dim3(unsigned((heads + 3) / 4), sb->n_seqs), 128, 0, stream>>>(                                  \
        meta, m_before, m_after, state, state_stride, slots, *sb, seq_chunk0, heads, DK, DV);                                   \
    rc = launch_status();                                                                                                       \
    if (rc != PTB_OK) return rc;                                                                                                \
    const size_t per = size_t(heads) * (size_t(DK) * DV + DK) / 4;                                                              \
    mlstm_chunk_join_kernel<<<dim3(unsigned((per + 127) / 128), sb->n_seqs), 128, 0, stream>>>(                                 \
        sums, nsums, meta, m_after, state, state_stride, slots, *sb, seq_chunk0, heads, DK, DV);                                \
    rc = launch_status();                                                                                                       \
    if (rc != PTB_OK) return rc;                                                                                                \
    return launch_out<DK, DV>(proj, stride, gates, *sb, chunk_seq, chunk_q0, n_chunks, sums, nsums, m_before, out, heads,       \
                              q_scale, stream);                                                                                 \
  } while (0)
  if (dim == 64 && v_dim == 64) PTB_ML(64, 64);
  if (dim == 64 && v_dim == 128) PTB_ML(64, 128);
  if (dim == 128 && v_dim == 64) PTB_ML(128, 64);
  PTB_ML(128, 128);
#undef PTB_ML
}
