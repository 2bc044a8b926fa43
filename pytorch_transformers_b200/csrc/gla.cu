// Gated linear attention: a decaying sum of key-value outer products whose decay is given per token and per key
// channel.
//
// Per head, with q_t, k_t [dim], v_t [v_dim] the projections of token t and a_t [dim] in (0, 1] its decays:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T (q_t * q_scale),      S = 0 before the first token.
// S [dim, v_dim] lives in float32 in the cache's per-sequence state area, laid out [heads][dim][v_dim]. The decays
// come as their logarithms (float32 [tokens, heads * dim]); a row of S is updated as S + (expm1(log a) S + k v), so
// that a decay close to one keeps its digits. All arithmetic on S is float32 whatever the model dtype.
//
// One kernel walks tokens in order with S in registers: a block owns VB or 2 VB value columns of one head, warp w the
// rows [w ROWS, (w + 1) ROWS) of S, lane j column j (and j + 32); the tokens' q, k and decays are staged in shared memory a batch
// ahead, and the warps' partial outputs meet there in a fixed order. It runs in three roles: over a sequence's new
// tokens from and to the state area (steps of any length); over one chunk of 64 tokens from zero, leaving the
// chunk's own sum and its total decay (pass 1 of the chunked form); over one chunk from the state before it, with
// outputs (pass 3). Pass 2 joins the chunks of a sequence in order. The chunked form differs from the plain walk by
// the order of float32 operations only. With bfloat16 projections and keys and values of 64 or 128 entries pass 1 is a
// product on the tensor cores instead (csrc/gla_mma.cu: the decayed keys enter it as two bfloat16 terms).
#include "common.cuh"

namespace {

constexpr int VB = 32;          // value columns of a block
constexpr int MAX_WARPS = 8;    // rows of S: up to 8 * 32
constexpr int CH = 64;          // tokens of a chunk

enum { GLA_WALK = 0, GLA_CHUNK_SUM = 1, GLA_CHUNK_OUT = 2 };

// tokens of a batch of the walk, by the rows of S a warp owns and the value columns a lane owns (what fits the
// registers that hold the next batch, and 48 KB of shared memory)
__host__ __device__ constexpr int walk_batch(int rows, int cols) { return (rows == 32 || cols == 2) ? 8 : 16; }

// Two float32 lanes in one 64-bit register and their fused multiply-add in one instruction (each lane rounds as fmaf does).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// z <- logsigmoid(z + bias) / tau: the logarithm of sigmoid(z + bias)^(1 / tau)
__global__ void gla_decay_kernel(float* __restrict__ z, const float* __restrict__ bias, long long total, int width,
                                 float inv_tau) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = z[i] + (bias ? bias[i % width] : 0.f);
  z[i] = (fminf(v, 0.f) - log1pf(expf(-fabsf(v)))) * inv_tau;
}

// proj row t: [q: heads * dim | k: heads * dim | v: heads * v_dim | ...], `stride` elements apart.
// role GLA_WALK: blockIdx.x = sequence; GLA_CHUNK_*: blockIdx.x = chunk (chunk_seq, chunk_q0 say which tokens).
// sums [chunks][heads][dim][v_dim]; chunk_decay [chunks][heads][dim]: the sum of the chunk's logarithms of decays.
//
// Tokens are staged in batches of SB: while a batch is computed from shared memory, the next one's q, k, decays and
// values are already on their way into registers (a token's loads alone take longer than its arithmetic), and the
// warps' partial outputs of a whole batch meet once: two block barriers a batch, none a token. With dim a multiple of
// 4 a warp reads four neighbouring rows' q, k and decays in one 16-byte word each.
// DIMC: the number of key channels where the instance is compiled for one (64, 128: the rows' tests and the addresses in
// shared memory are then constants), 0 for any.
template <typename T, int ROWS, int COLS, int DIMC>
__global__ void __launch_bounds__(32 * MAX_WARPS, ROWS == 32 ? 1 : 2)
gla_walk_kernel(const T* __restrict__ proj, int stride, const float* __restrict__ log_decay, float* __restrict__ state,
                int state_stride, const int* __restrict__ slots, StepBatch sb, const int* __restrict__ chunk_seq,
                const int* __restrict__ chunk_q0, float* __restrict__ sums, float* __restrict__ chunk_decay,
                float* __restrict__ out, int heads, int dim_any, int v_dim, float q_scale, int role) {
  const int dim = DIMC > 0 ? DIMC : dim_any;
  constexpr int SB = walk_batch(ROWS, COLS);   // tokens of a batch
  constexpr int IT = SB * ROWS / 32;           // (token, channel) pairs a thread stages of each of q, k and the decays
  constexpr int VBC = VB * COLS;               // value columns of a block: lane l owns columns l, l + 32, ...
  extern __shared__ __align__(16) float sm[];
  const int pitch = (dim + 3) & ~3;            // a token's row of channels, at whole 16-byte words
  float* qs = sm;                              // [SB][pitch]
  float* ks = qs + SB * pitch;
  float* es = ks + SB * pitch;
  float* vs = es + SB * pitch;                 // [SB][VBC]
  float* part = vs + SB * VBC;                 // [SB][warps][VBC]
  // every block has 32 * MAX_WARPS threads: warps whose rows lie past dim stage and sum with the others and hold zeros
  constexpr int nthreads = 32 * MAX_WARPS, warps = MAX_WARPS, RV = SB * VBC / nthreads;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int h = blockIdx.y, j0 = blockIdx.z * VBC;
  int seq, first, n;
  if (role == GLA_WALK) {
    seq = blockIdx.x;
    first = sb.seq_start[seq];
    n = sb.seq_new[seq];
  } else {
    seq = chunk_seq[blockIdx.x];
    const int q0 = chunk_q0[blockIdx.x];
    first = sb.seq_start[seq] + q0;
    n = min(CH, sb.seq_new[seq] - q0);
  }
  const size_t per_head = size_t(dim) * v_dim;
  float* st = nullptr;
  if (role == GLA_WALK) st = state + size_t(slots[seq]) * state_stride + size_t(h) * per_head;
  else st = sums + (size_t(blockIdx.x) * heads + h) * per_head;
  // Where the key size is compiled in, two neighbouring rows of a column share a 64-bit register and every update of
  // the pair is one instruction: half as many to issue. The outputs then sum even and odd rows apart.
  constexpr bool PACK = DIMC > 0;
  float S[PACK ? 1 : ROWS][COLS];
  f32x2 S2[PACK ? ROWS / 2 : 1][COLS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = warp * ROWS + r;
#pragma unroll
    for (int c = 0; c < COLS; ++c) {
      const int j = j0 + c * 32 + lane;
      const float s0 = (role != GLA_CHUNK_SUM && j < v_dim && d < dim) ? st[size_t(d) * v_dim + j] : 0.f;
      if constexpr (PACK) {
        if (r & 1) {
          float lo, hi;
          unpack2(S2[r / 2][c], lo, hi);
          S2[r / 2][c] = pack2(lo, s0);
        } else {
          S2[r / 2][c] = pack2(s0, 0.f);
        }
      } else {
        S[r][c] = s0;
      }
    }
  }
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  const bool with_out = role != GLA_CHUNK_SUM;
  const bool vec = (dim & 3) == 0;
  // staged values stay as they were loaded (no arithmetic that would wait for a load between two loads)
  T rq[IT], rk[IT], rv[RV];
  float re[IT];
  // the (token, channel) pairs this thread stages: pair it is tid + it * nthreads, walked without divisions
  const int t_first = tid / dim, d_first = tid - t_first * dim, t_step = nthreads / dim, d_step = nthreads - t_step * dim;

  // the loads of the batch that starts at token t0 (nb tokens), into registers
  auto fetch = [&](int t0, int nb) {
    int t = t_first, d = d_first;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int tt = min(t, nb - 1);      // a pair past the batch reads the batch's last token and is not stored
      const T* row = proj + size_t(first + t0 + tt) * stride + h * dim + d;
      rq[it] = row[0];
      rk[it] = row[k_off];
      re[it] = log_decay[size_t(first + t0 + tt) * k_off + h * dim + d];
      t += t_step;
      d += d_step;
      if (d >= dim) {
        d -= dim;
        ++t;
      }
    }
#pragma unroll
    for (int it = 0; it < RV; ++it) {
      const int idx = tid + it * nthreads;       // (token, column): idx / VBC, idx % VBC
      const int tt = min(idx / VBC, nb - 1), col = min(j0 + (idx % VBC), v_dim - 1);
      rv[it] = proj[size_t(first + t0 + tt) * stride + v_off + h * v_dim + col];
    }
  };
  auto store = [&](int nb) {
    int t = t_first, d = d_first;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      if (t < nb) {
        qs[t * pitch + d] = to_f(rq[it]) * q_scale;
        ks[t * pitch + d] = to_f(rk[it]);
        es[t * pitch + d] = expm1f(re[it]);
      }
      t += t_step;
      d += d_step;
      if (d >= dim) {
        d -= dim;
        ++t;
      }
    }
#pragma unroll
    for (int it = 0; it < RV; ++it) {
      const int idx = tid + it * nthreads;
      if (idx < nb * VBC) vs[idx] = (j0 + (idx % VBC) < v_dim) ? to_f(rv[it]) : 0.f;
    }
  };

  if (n > 0) fetch(0, min(SB, n));
  for (int t0 = 0; t0 < n; t0 += SB) {
    const int nb = min(SB, n - t0);
    store(nb);
    __syncthreads();                                   // the batch is staged
    if (t0 + SB < n) fetch(t0 + SB, min(SB, n - t0 - SB));   // the next batch's loads run under this batch's arithmetic
    // unrolled over the batch's tokens: the next token's reads of shared memory are issued under this token's arithmetic
    // (the partial outputs are kept in registers until the batch's end, so no store stands between two tokens' reads)
    float ob[SB][COLS];
#pragma unroll
    for (int t = 0; t < SB; ++t) {
      if (t >= nb) break;
      float v[COLS], o[COLS];
#pragma unroll
      for (int c = 0; c < COLS; ++c) {
        v[c] = vs[t * VBC + c * 32 + lane];
        o[c] = 0.f;
      }
      const float* qr = qs + t * pitch + warp * ROWS;
      const float* kr = ks + t * pitch + warp * ROWS;
      const float* er = es + t * pitch + warp * ROWS;
      // a row's update: S + expm1(log a) S, then + k v: two fused multiply-adds
      if constexpr (PACK) {
        f32x2 vv[COLS], o2[COLS];
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          vv[c] = pack2(v[c], v[c]);
          o2[c] = pack2(0.f, 0.f);
        }
#pragma unroll
        for (int r = 0; r < ROWS; r += 4) {
          const float4 e4 = *reinterpret_cast<const float4*>(er + r);
          const float4 k4 = *reinterpret_cast<const float4*>(kr + r);
          const float4 q4 = with_out ? *reinterpret_cast<const float4*>(qr + r) : make_float4(0.f, 0.f, 0.f, 0.f);
          const f32x2 e01 = pack2(e4.x, e4.y), e23 = pack2(e4.z, e4.w), k01 = pack2(k4.x, k4.y), k23 = pack2(k4.z, k4.w);
          const f32x2 q01 = pack2(q4.x, q4.y), q23 = pack2(q4.z, q4.w);
#pragma unroll
          for (int c = 0; c < COLS; ++c) {
            S2[r / 2][c] = fma2(k01, vv[c], fma2(e01, S2[r / 2][c], S2[r / 2][c]));
            S2[r / 2 + 1][c] = fma2(k23, vv[c], fma2(e23, S2[r / 2 + 1][c], S2[r / 2 + 1][c]));
            if (with_out) o2[c] = fma2(S2[r / 2 + 1][c], q23, fma2(S2[r / 2][c], q01, o2[c]));
          }
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          float lo, hi;
          unpack2(o2[c], lo, hi);
          o[c] = lo + hi;
        }
      } else if (vec) {
#pragma unroll
        for (int r = 0; r < ROWS; r += 4) {
          if (warp * ROWS + r < dim) {        // whole quads: dim and ROWS are multiples of 4
            const float4 e4 = *reinterpret_cast<const float4*>(er + r);
            const float4 k4 = *reinterpret_cast<const float4*>(kr + r);
            const float4 q4 = with_out ? *reinterpret_cast<const float4*>(qr + r) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
              S[r][c] = fmaf(k4.x, v[c], fmaf(e4.x, S[r][c], S[r][c]));
              S[r + 1][c] = fmaf(k4.y, v[c], fmaf(e4.y, S[r + 1][c], S[r + 1][c]));
              S[r + 2][c] = fmaf(k4.z, v[c], fmaf(e4.z, S[r + 2][c], S[r + 2][c]));
              S[r + 3][c] = fmaf(k4.w, v[c], fmaf(e4.w, S[r + 3][c], S[r + 3][c]));
              if (with_out) o[c] = fmaf(S[r + 3][c], q4.w, fmaf(S[r + 2][c], q4.z, fmaf(S[r + 1][c], q4.y, fmaf(S[r][c], q4.x, o[c]))));
            }
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          if (warp * ROWS + r < dim) {
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
              S[r][c] = fmaf(kr[r], v[c], fmaf(er[r], S[r][c], S[r][c]));
              if (with_out) o[c] = fmaf(S[r][c], qr[r], o[c]);
            }
          }
        }
      }
#pragma unroll
      for (int c = 0; c < COLS; ++c) ob[t][c] = o[c];
    }
    if (with_out) {
#pragma unroll
      for (int t = 0; t < SB; ++t) {
        if (t < nb) {
#pragma unroll
          for (int c = 0; c < COLS; ++c) part[(t * warps + warp) * VBC + c * 32 + lane] = ob[t][c];
        }
      }
    }
    __syncthreads();                                   // the batch's partial outputs are written; its rows are no longer read
    if (with_out) {
      for (int idx = tid; idx < nb * VBC; idx += nthreads) {
        const int t = idx / VBC, l = idx % VBC;
        if (j0 + l < v_dim) {
          float o = 0.f;
          for (int w = 0; w < warps; ++w) o += part[(t * warps + w) * VBC + l];     // a fixed order
          out[(size_t(first + t0 + t) * heads + h) * v_dim + j0 + l] = o;
        }
      }
    }
    // the next store writes rows that were last read before the barrier above; `part` is written again only after the
    // next batch's first barrier, which every thread reaches after this sum
  }
  if (role != GLA_CHUNK_OUT) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int d = warp * ROWS + r;
#pragma unroll
      for (int c = 0; c < COLS; ++c) {
        const int j = j0 + c * 32 + lane;
        float s1;
        if constexpr (PACK) {
          float lo, hi;
          unpack2(S2[r / 2][c], lo, hi);
          s1 = (r & 1) ? hi : lo;
        } else {
          s1 = S[r][c];
        }
        if (d < dim && j < v_dim) st[size_t(d) * v_dim + j] = s1;
      }
    }
  }
  if (role == GLA_CHUNK_SUM && blockIdx.z == 0) {
    for (int d = tid; d < dim; d += nthreads) {        // the chunk's total decay per channel, tokens in order
      float total = 0.f;
#pragma unroll 8
      for (int i = 0; i < n; ++i) total += log_decay[size_t(first + i) * k_off + h * dim + d];
      chunk_decay[(size_t(blockIdx.x) * heads + h) * dim + d] = total;
    }
  }
}

// One thread per (sequence, head, element of S): walks the sequence's chunks in order; sums[c] becomes the state
// BEFORE chunk c, and the state area receives the state after the last chunk.
__global__ void gla_chunk_join_kernel(float* __restrict__ sums, const float* __restrict__ chunk_decay,
                                      float* __restrict__ state, int state_stride, const int* __restrict__ slots,
                                      StepBatch sb, const int* __restrict__ seq_chunk0, int heads, int dim, int v_dim) {
  const int seq = blockIdx.y;
  const size_t per_head = size_t(dim) * v_dim, per = per_head * heads;
  const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= per) return;
  const int h = int(e / per_head), d = int((e % per_head) / v_dim);
  const int n_new = sb.seq_new[seq], c0 = seq_chunk0[seq];
  const int n_chunks = (n_new + CH - 1) / CH;
  float* st = state + size_t(slots[seq]) * state_stride + e;
  float s = *st;
  constexpr int AHEAD = 8;      // chunks whose own sums are loaded before the chain of updates needs them
  for (int g0 = 0; g0 < n_chunks; g0 += AHEAD) {
    float own[AHEAD], dec[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      const bool on = g0 + i < n_chunks;
      own[i] = on ? sums[size_t(c0 + g0 + i) * per + e] : 0.f;
      dec[i] = on ? chunk_decay[(size_t(c0 + g0 + i) * heads + h) * dim + d] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
      if (g0 + i >= n_chunks) break;
      sums[size_t(c0 + g0 + i) * per + e] = s;
      s = fmaf(expf(dec[i]), s, own[i]);
    }
  }
  *st = s;
}

template <typename T>
int launch_walk(const void* proj, int stride, const float* log_decay, float* state, int state_stride, const int* slots,
                const StepBatch& sb, const int* chunk_seq, const int* chunk_q0, int n_blocks, float* sums, float* chunk_decay,
                float* out, int heads, int dim, int v_dim, float q_scale, int role, cudaStream_t stream) {
  const int rows = dim <= 8 * MAX_WARPS ? 8 : (dim <= 16 * MAX_WARPS ? 16 : 32);
  const int warps = MAX_WARPS;
  const int cols = v_dim > VB ? 2 : 1;       // two value columns a lane where a head's values are wider than a warp
  dim3 grid(n_blocks, heads, (v_dim + VB * cols - 1) / (VB * cols));
  const int batch = walk_batch(rows, cols), pitch = (dim + 3) & ~3;
  const size_t smem = sizeof(float) * (size_t(3) * batch * pitch + size_t(batch) * VB * cols + size_t(batch) * warps * VB * cols);
#define PTB_GLA(ROWS, COLS, DIMC)                                                                                        \
  gla_walk_kernel<T, ROWS, COLS, DIMC><<<grid, 32 * warps, smem, stream>>>((const T*)proj, stride, log_decay, state,      \
                                                                           state_stride, slots, sb, chunk_seq, chunk_q0,  \
                                                                           sums, chunk_decay, out, heads, dim, v_dim,     \
                                                                           q_scale, role)
  if (cols == 1) {
    if (dim == 64) PTB_GLA(8, 1, 64);
    else if (dim == 128) PTB_GLA(16, 1, 128);
    else if (rows == 8) PTB_GLA(8, 1, 0);
    else if (rows == 16) PTB_GLA(16, 1, 0);
    else PTB_GLA(32, 1, 0);
  } else {
    if (dim == 64) PTB_GLA(8, 2, 64);
    else if (dim == 128) PTB_GLA(16, 2, 128);
    else if (rows == 8) PTB_GLA(8, 2, 0);
    else if (rows == 16) PTB_GLA(16, 2, 0);
    else PTB_GLA(32, 2, 0);
  }
#undef PTB_GLA
  return launch_status();
}

}  // namespace

// pass 1 on the tensor cores (csrc/gla_mma.cu)
PTB_API int ptb_gla_chunk_sum_mma_supports(int dtype, const void* proj, int stride, const float* log_decay, int dim, int v_dim);
PTB_API int ptb_gla_chunk_sum_mma(const void* proj, int stride, const float* log_decay, const StepBatch* sb, const int* chunk_seq,
                                  const int* chunk_q0, int n_chunks, float* sums, float* chunk_decay, int heads, int dim,
                                  int v_dim, cudaStream_t stream);

PTB_API int ptb_gla_max_dim() { return 32 * MAX_WARPS; }
PTB_API int ptb_gla_chunk_tokens() { return CH; }

// z: float32 [n, width] sums of the decay's projection; replaced by logsigmoid(z + bias) / tau. bias [width] or null.
PTB_API int ptb_gla_decay(float* z, const float* bias, int n, int width, float tau, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || !(tau > 0.f)) return PTB_ERR_SIZE;
  const long long total = (long long)n * width;
  gla_decay_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(z, bias, total, width, 1.f / tau);
  return launch_status();
}

// The step's tokens, every sequence walked in order from and to its state. out float32 [tokens, heads * v_dim].
PTB_API int ptb_gla_walk(int dtype, const void* proj, int stride, const float* log_decay, float* state, int state_stride,
                         const int* slots, const StepBatch* sb, float* out, int heads, int dim, int v_dim, float q_scale,
                         cudaStream_t stream) {
  if (sb->n_tokens <= 0 || sb->n_seqs <= 0) return PTB_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || dim > 32 * MAX_WARPS || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim)
    return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return launch_walk<float>(proj, stride, log_decay, state, state_stride, slots, *sb, nullptr, nullptr, sb->n_seqs, nullptr,
                              nullptr, out, heads, dim, v_dim, q_scale, GLA_WALK, stream);
  if (dtype == PTB_BF16)
    return launch_walk<__nv_bfloat16>(proj, stride, log_decay, state, state_stride, slots, *sb, nullptr, nullptr, sb->n_seqs,
                                      nullptr, nullptr, out, heads, dim, v_dim, q_scale, GLA_WALK, stream);
  return PTB_ERR_DTYPE;
}

// The chunked form for prompts: sums float32 [n_chunks, heads, dim, v_dim] and chunk_decay float32 [n_chunks, heads, dim]
// are scratch; seq_chunk0[b] is sequence b's first chunk. Three kernels.
PTB_API int ptb_gla_chunks(int dtype, const void* proj, int stride, const float* log_decay, float* state, int state_stride,
                           const int* slots, const StepBatch* sb, const int* chunk_seq, const int* chunk_q0,
                           const int* seq_chunk0, int n_chunks, float* sums, float* chunk_decay, float* out, int heads,
                           int dim, int v_dim, float q_scale, cudaStream_t stream) {
  if (sb->n_tokens <= 0 || n_chunks <= 0) return PTB_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || dim > 32 * MAX_WARPS || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim ||
      sb->n_seqs > 65535)
    return PTB_ERR_SIZE;
  // a chunk's own sum is a product of the decayed keys by the values: on the tensor cores where the sizes allow
  const bool sum_mma = ptb_gla_chunk_sum_mma_supports(dtype, proj, stride, log_decay, dim, v_dim) != 0;
  for (int role = GLA_CHUNK_SUM; role <= GLA_CHUNK_OUT; ++role) {
    int rc;
    if (role == GLA_CHUNK_SUM && sum_mma)
      rc = ptb_gla_chunk_sum_mma(proj, stride, log_decay, sb, chunk_seq, chunk_q0, n_chunks, sums, chunk_decay, heads, dim, v_dim,
                                 stream);
    else if (dtype == PTB_F32)
      rc = launch_walk<float>(proj, stride, log_decay, state, state_stride, slots, *sb, chunk_seq, chunk_q0, n_chunks, sums,
                              chunk_decay, out, heads, dim, v_dim, q_scale, role, stream);
    else if (dtype == PTB_BF16)
      rc = launch_walk<__nv_bfloat16>(proj, stride, log_decay, state, state_stride, slots, *sb, chunk_seq, chunk_q0, n_chunks,
                                      sums, chunk_decay, out, heads, dim, v_dim, q_scale, role, stream);
    else
      return PTB_ERR_DTYPE;
    if (rc != PTB_OK) return rc;
    if (role == GLA_CHUNK_SUM) {
      const size_t per = size_t(heads) * dim * v_dim;
      dim3 grid(unsigned((per + 255) / 256), sb->n_seqs);
      gla_chunk_join_kernel<<<grid, 256, 0, stream>>>(sums, chunk_decay, state, state_stride, slots, *sb, seq_chunk0, heads,
                                                      dim, v_dim);
      if (launch_status() != PTB_OK) return PTB_ERR_LAUNCH;
    }
  }
  return PTB_OK;
}
