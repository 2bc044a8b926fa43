// The matrix memory with exponential gates (mLSTM): per head a state S [dim][v_dim], a normaliser n [dim] and a
// running maximum m of the gates' logarithms, all float32 per sequence.
//
//   i_t = cap tanh((gi_t + bi) / cap),   f_t = logsigmoid(cap tanh((gf_t + bf) / cap))      (logarithms of the gates)
//   m_t = max(f_t + m_(t-1), i_t)                                   m = 0, S = 0, n = 0 before the first token
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,      n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// gi, gf are the gate projections' float32 sums; q (times q_scale), k, v come from one projection in the model's
// type. Gates, decays, state and the division are float32. The state of a sequence lies in the cache's state
// area as S [heads][dim][v_dim], then for every head and every stretch of 32 value columns a copy of n [dim] and m [1]:
// the blocks that share a head each read and write a copy of their own, so none waits for another.
#include "common.cuh"

namespace {

constexpr int VB = 32;        // value columns of a block: one lane each
constexpr int WARPS = 8;      // row groups: warp w owns rows w, w + 8, ...
constexpr int MAX_DIM = 256;  // rows of S that the registers hold (32 a thread)

__device__ __forceinline__ float capped(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// logarithms of the input and forget gates of every (token, head): float32 [n, 2 heads] in place of the sums
__global__ void mlstm_gates_kernel(float* __restrict__ gates, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                                   int n, int heads, float cap) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * 2 * heads) return;
  const int col = i % (2 * heads);
  if (col < heads)
    gates[i] = capped(gates[i] + bias_i[col], cap);
  else
    gates[i] = log_sigmoid(capped(gates[i] + bias_f[col - heads], cap));
}

// One block per (sequence, head, 32 value columns) walks the sequence's tokens of the step. Thread (warp w, lane v)
// keeps S[w + 8 i][v0 + v] in registers; lane l of warp w also keeps n[w + 8 l]. One barrier a token: q, k, v of the
// next token and the partial sums of this one go through buffers that take turns.
template <typename T, int ROWS>
__global__ void __launch_bounds__(VB * WARPS)
mlstm_scan_kernel(const T* __restrict__ proj, int stride, const float* __restrict__ gates, float* __restrict__ state,
                  int state_stride, const int* __restrict__ slots, StepBatch sb, float* __restrict__ out, int heads, int dim,
                  int v_dim, float q_scale) {
  __shared__ float qs[2][MAX_DIM], ks[2][MAX_DIM], vs[2][VB], red_o[2][WARPS][VB], red_n[2][WARPS];
  const int seq = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VB;
  const int w = threadIdx.x / 32, lane = threadIdx.x % 32, tid = threadIdx.x;
  const int start = sb.seq_start[seq], n_new = sb.seq_new[seq];
  const bool col_ok = v0 + lane < v_dim;
  float* st = state + size_t(slots[seq]) * state_stride;
  float* S_g = st + size_t(h) * dim * v_dim;
  float* n_g = st + size_t(heads) * dim * v_dim + (size_t(h) * gridDim.z + blockIdx.z) * (dim + 1);
  float* m_g = n_g + dim;

  float S[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int r = w + WARPS * i;
    S[i] = (r < dim && col_ok) ? S_g[size_t(r) * v_dim + v0 + lane] : 0.f;
  }
  const int n_row = w + WARPS * lane;           // this lane's entry of n
  float n_val = (n_row < dim) ? n_g[n_row] : 0.f;
  float m = m_g[0];

  const T* q_base = proj + size_t(h) * dim;
  const T* k_base = proj + size_t(heads) * dim + size_t(h) * dim;
  const T* v_base = proj + 2 * size_t(heads) * dim + size_t(h) * v_dim + v0;
  auto load = [&](int t, int buf) {
    const size_t off = size_t(start + t) * stride;
    for (int e = tid; e < dim; e += VB * WARPS) {
      qs[buf][e] = to_f(q_base[off + e]) * q_scale;
      ks[buf][e] = to_f(k_base[off + e]);
    }
    if (tid < VB) vs[buf][tid] = (v0 + tid < v_dim) ? to_f(v_base[off + tid]) : 0.f;
  };
  auto finish = [&](int t, int buf, float m_t) {   // warp 0: the token's output from the warps' partial sums
    float o = 0.f, nq = 0.f;
#pragma unroll
    for (int ww = 0; ww < WARPS; ++ww) {
      o += red_o[buf][ww][lane];
      nq += red_n[buf][ww];
    }
    const float den = fmaxf(fabsf(nq), expf(-m_t)) + 1e-6f;
    if (col_ok) out[size_t(start + t) * heads * v_dim + size_t(h) * v_dim + v0 + lane] = o / den;
  };

  load(0, 0);
  float m_prev_token = m;
  for (int t = 0; t < n_new; ++t) {
    const int buf = t & 1;
    __syncthreads();
    if (t > 0 && w == 0) finish(t - 1, buf ^ 1, m_prev_token);
    const float gi = gates[size_t(start + t) * 2 * heads + h], gf = gates[size_t(start + t) * 2 * heads + heads + h];
    const float m_new = fmaxf(gf + m, gi);
    const float a = expf(gf + m - m_new), b = expf(gi - m_new);
    m = m_new;
    m_prev_token = m_new;
    const float bv = b * vs[buf][lane];
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int r = w + WARPS * i;
      if (r < dim) {
        S[i] = fmaf(a, S[i], ks[buf][r] * bv);
        part = fmaf(S[i], qs[buf][r], part);
      }
    }
    float part_n = 0.f;
    if (n_row < dim) {
      n_val = fmaf(a, n_val, b * ks[buf][n_row]);
      part_n = n_val * qs[buf][n_row];
    }
    part_n = warp_sum(part_n);
    red_o[buf][w][lane] = part;
    if (lane == 0) red_n[buf][w] = part_n;
    if (t + 1 < n_new) load(t + 1, buf ^ 1);
  }
  __syncthreads();
  if (w == 0 && n_new > 0) finish(n_new - 1, (n_new - 1) & 1, m_prev_token);
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int r = w + WARPS * i;
    if (r < dim && col_ok) S_g[size_t(r) * v_dim + v0 + lane] = S[i];
  }
  if (n_row < dim) n_g[n_row] = n_val;
  if (tid == 0) m_g[0] = m;
}

// out[t][h][e] = x[t][h][e] / rms(x[t][h][:]) * gain[h * v_dim + e] * sigmoid(gate[t][h * v_dim + e]); a warp per (token, head)
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ gain, const T* __restrict__ gate,
                                      int gate_stride, T* __restrict__ out, int out_stride, int n, int heads, int v_dim,
                                      float eps, int gate_silu) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
  if (warp >= n * heads) return;
  const int t = warp / heads, h = warp % heads;
  const float* row = x + (size_t(t) * heads + h) * v_dim;
  float ss = 0.f;
  for (int e = lane; e < v_dim; e += 32) ss = fmaf(row[e], row[e], ss);
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / float(v_dim) + eps);
  for (int e = lane; e < v_dim; e += 32) {
    float y = row[e] * rstd * gain[size_t(h) * v_dim + e];
    if (gate) {
      const float g = to_f(gate[size_t(t) * gate_stride + size_t(h) * v_dim + e]);
      y *= (gate_silu ? g : 1.f) / (1.f + expf(-g));      // sigmoid(g), or silu(g) = g sigmoid(g)
    }
    out[size_t(t) * out_stride + size_t(h) * v_dim + e] = from_f<T>(y);
  }
}

template <typename T>
int launch_scan(const void* proj, int stride, const float* gates, float* state, int state_stride, const int* slots,
                const StepBatch& sb, float* out, int heads, int dim, int v_dim, float q_scale, cudaStream_t stream) {
  dim3 grid(sb.n_seqs, heads, (v_dim + VB - 1) / VB);
#define PTB_SCAN(ROWS)                                                                                                       \
  mlstm_scan_kernel<T, ROWS><<<grid, VB * WARPS, 0, stream>>>((const T*)proj, stride, gates, state, state_stride, slots, sb, \
                                                              out, heads, dim, v_dim, q_scale)
  if (dim <= 8 * WARPS)
    PTB_SCAN(8);
  else if (dim <= 16 * WARPS)
    PTB_SCAN(16);
  else
    PTB_SCAN(32);
#undef PTB_SCAN
  return launch_status();
}

}  // namespace

// gates: float32 [n, 2 heads], the two gate projections' sums side by side (input gates, then forget gates); replaced by
// the gates' logarithms. cap <= 0: no cap.
PTB_API int ptb_mlstm_gates(float* gates, const float* bias_i, const float* bias_f, int n, int heads, float cap,
                            cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (heads <= 0) return PTB_ERR_SIZE;
  const int total = n * 2 * heads;
  mlstm_gates_kernel<<<(total + 255) / 256, 256, 0, stream>>>(gates, bias_i, bias_f, n, heads, cap);
  return launch_status();
}

// proj [tokens, >= 2 heads dim + heads v_dim] holds q, k, v side by side (rows `stride` apart); gates as ptb_mlstm_gates
// leaves them; state [slots, >= ptb_mlstm_state_floats(heads, dim, v_dim)] float32; out float32 [tokens, heads * v_dim].
PTB_API int ptb_mlstm_scan(int dtype, const void* proj, int stride, const float* gates, float* state, int state_stride,
                           const int* slots, const StepBatch* sb, float* out, int heads, int dim, int v_dim, float q_scale,
                           cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || dim > MAX_DIM || v_dim <= 0 || stride < 2 * heads * dim + heads * v_dim ||
      state_stride < heads * (dim * v_dim + ((v_dim + VB - 1) / VB) * (dim + 1)))
    return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return launch_scan<float>(proj, stride, gates, state, state_stride, slots, *sb, out, heads, dim, v_dim, q_scale, stream);
  if (dtype == PTB_BF16)
    return launch_scan<__nv_bfloat16>(proj, stride, gates, state, state_stride, slots, *sb, out, heads, dim, v_dim, q_scale,
                                      stream);
  return PTB_ERR_DTYPE;
}

PTB_API int ptb_mlstm_max_dim() { return MAX_DIM; }
PTB_API int ptb_mlstm_state_floats(int heads, int dim, int v_dim) {
  return heads * (dim * v_dim + ((v_dim + VB - 1) / VB) * (dim + 1));
}

// x float32 [n, heads * v_dim]; gain float32 [heads * v_dim]; gate (may be null) and out of `dtype`, rows gate_stride and
// out_stride apart.
PTB_API int ptb_head_norm_gate_act(const float* x, const float* gain, int dtype, const void* gate, int gate_stride, void* out,
                               int out_stride, int n, int heads, int v_dim, float eps, int gate_silu, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (heads <= 0 || v_dim <= 0 || out_stride < heads * v_dim) return PTB_ERR_SIZE;
  const long long warps = (long long)n * heads;
  const int threads = 256;
  const unsigned blocks = unsigned((warps * 32 + threads - 1) / threads);
  if (dtype == PTB_F32)
    head_norm_gate_kernel<float><<<blocks, threads, 0, stream>>>(x, gain, (const float*)gate, gate_stride, (float*)out,
                                                                 out_stride, n, heads, v_dim, eps, gate_silu);
  else if (dtype == PTB_BF16)
    head_norm_gate_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(x, gain, (const __nv_bfloat16*)gate, gate_stride,
                                                                         (__nv_bfloat16*)out, out_stride, n, heads, v_dim, eps, gate_silu);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_head_norm_gate(const float* x, const float* gain, int dtype, const void* gate, int gate_stride, void* out,
                               int out_stride, int n, int heads, int v_dim, float eps, cudaStream_t stream) {
  return ptb_head_norm_gate_act(x, gain, dtype, gate, gate_stride, out, out_stride, n, heads, v_dim, eps, 0, stream);
}
