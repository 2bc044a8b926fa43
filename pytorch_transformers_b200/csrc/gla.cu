// Gated linear attention: a decaying sum of key-value outer products whose decay is given per token and per key
// channel.
//
// Per head, with q_t, k_t [dim], v_t [v_dim] the projections of token t and a_t [dim] in (0, 1] its decays:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T (q_t * q_scale),      S = 0 before the first token.
// S [dim, v_dim] lives in float32 in the cache's per-sequence state area, laid out [heads][dim][v_dim]. The decays
// come as their logarithms (float32 [tokens, heads * dim]); a row of S is updated as S + (expm1(log a) S + k v), so
// that a decay close to one keeps its digits. All arithmetic on S is float32 whatever the model dtype.
//
// One kernel walks tokens in order with S in registers: a block owns VB value columns of one head, warp w the rows
// [w ROWS, (w + 1) ROWS) of S, lane j column j; a token's q, k and decays are staged in shared memory one token
// ahead, and the warps' partial outputs meet there in a fixed order. It runs in three roles: over a sequence's new
// tokens from and to the state area (steps of any length); over one chunk of 64 tokens from zero, leaving the
// chunk's own sum and its total decay (pass 1 of the chunked form); over one chunk from the state before it, with
// outputs (pass 3). Pass 2 joins the chunks of a sequence in order. The chunked form differs from the plain walk by
// the order of float32 operations only.
#include "common.cuh"

namespace {

constexpr int VB = 32;          // value columns of a block
constexpr int MAX_WARPS = 8;    // rows of S: up to 8 * 32
constexpr int CH = 64;          // tokens of a chunk

enum { GLA_WALK = 0, GLA_CHUNK_SUM = 1, GLA_CHUNK_OUT = 2 };

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
template <typename T, int ROWS>
__global__ void __launch_bounds__(32 * MAX_WARPS)
gla_walk_kernel(const T* __restrict__ proj, int stride, const float* __restrict__ log_decay, float* __restrict__ state,
                int state_stride, const int* __restrict__ slots, StepBatch sb, const int* __restrict__ chunk_seq,
                const int* __restrict__ chunk_q0, float* __restrict__ sums, float* __restrict__ chunk_decay,
                float* __restrict__ out, int heads, int dim, int v_dim, float q_scale, int role) {
  __shared__ float qs[2][32 * MAX_WARPS], ks[2][32 * MAX_WARPS], es[2][32 * MAX_WARPS];
  __shared__ float part[2][MAX_WARPS][VB];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, warps = blockDim.x / 32;
  const int h = blockIdx.y, j = blockIdx.z * VB + lane;
  const bool mine = j < v_dim;
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
  float S[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int d = warp * ROWS + r;
    S[r] = (role != GLA_CHUNK_SUM && mine && d < dim) ? st[size_t(d) * v_dim + j] : 0.f;
  }
  const int k_off = heads * dim, v_off = 2 * heads * dim;
  const int sd = threadIdx.x;            // the channel this thread stages
  const bool stages = sd < dim;
  float total_log = 0.f;
  // token 0 is staged before the loop, token i + 1 while token i is computed
  float nq = 0.f, nk = 0.f, ne = 0.f, nv = 0.f;
  if (n > 0) {
    const T* row = proj + size_t(first) * stride;
    if (stages) {
      nq = to_f(row[h * dim + sd]) * q_scale;
      nk = to_f(row[k_off + h * dim + sd]);
      const float la = log_decay[size_t(first) * k_off + h * dim + sd];
      total_log += la;
      ne = expm1f(la);
    }
    if (mine) nv = to_f(row[v_off + h * v_dim + j]);
    if (stages) {
      qs[0][sd] = nq;
      ks[0][sd] = nk;
      es[0][sd] = ne;
    }
  }
  for (int i = 0; i < n; ++i) {
    const int b = i & 1;
    const float v = nv;
    __syncthreads();      // token i is staged; the partial outputs of token i - 1 are written
    if (i + 1 < n) {      // the next token's loads are issued now and stored after this token's arithmetic
      const T* row = proj + size_t(first + i + 1) * stride;
      if (stages) {
        nq = to_f(row[h * dim + sd]) * q_scale;
        nk = to_f(row[k_off + h * dim + sd]);
        ne = log_decay[size_t(first + i + 1) * k_off + h * dim + sd];
      }
      if (mine) nv = to_f(row[v_off + h * v_dim + j]);
    }
    if (role != GLA_CHUNK_SUM && i > 0 && warp == 0 && mine) {
      float o = 0.f;
      for (int w = 0; w < warps; ++w) o += part[b ^ 1][w][lane];
      out[(size_t(first + i - 1) * heads + h) * v_dim + j] = o;
    }
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int d = warp * ROWS + r;       // rows past dim hold zeros and read staged zeros or stale values times zero
      if (d < dim) {
        S[r] = S[r] + fmaf(es[b][d], S[r], ks[b][d] * v);
        o = fmaf(S[r], qs[b][d], o);
      }
    }
    if (role != GLA_CHUNK_SUM) part[b][warp][lane] = o;
    if (i + 1 < n && stages) {
      total_log += ne;
      qs[b ^ 1][sd] = nq;
      ks[b ^ 1][sd] = nk;
      es[b ^ 1][sd] = expm1f(ne);
    }
  }
  if (role != GLA_CHUNK_SUM && n > 0) {
    __syncthreads();
    if (warp == 0 && mine) {
      float o = 0.f;
      for (int w = 0; w < warps; ++w) o += part[(n - 1) & 1][w][lane];
      out[(size_t(first + n - 1) * heads + h) * v_dim + j] = o;
    }
  }
  if (role != GLA_CHUNK_OUT && mine) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int d = warp * ROWS + r;
      if (d < dim) st[size_t(d) * v_dim + j] = S[r];
    }
  }
  if (role == GLA_CHUNK_SUM && blockIdx.z == 0 && stages)
    chunk_decay[(size_t(blockIdx.x) * heads + h) * dim + sd] = total_log;
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
  const int warps = (dim + rows - 1) / rows;
  dim3 grid(n_blocks, heads, (v_dim + VB - 1) / VB);
#define PTB_GLA(ROWS)                                                                                                  \
  gla_walk_kernel<T, ROWS><<<grid, 32 * warps, 0, stream>>>((const T*)proj, stride, log_decay, state, state_stride, slots, \
                                                            sb, chunk_seq, chunk_q0, sums, chunk_decay, out, heads, dim,   \
                                                            v_dim, q_scale, role)
  if (rows == 8) PTB_GLA(8);
  else if (rows == 16) PTB_GLA(16);
  else PTB_GLA(32);
#undef PTB_GLA
  return launch_status();
}

}  // namespace

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
  for (int role = GLA_CHUNK_SUM; role <= GLA_CHUNK_OUT; ++role) {
    int rc;
    if (dtype == PTB_F32)
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
