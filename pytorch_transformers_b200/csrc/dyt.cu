// The Dynamic Tanh norm, alone or with the short causal convolution that some designs put on a mixer's input.
//
//   h[t][c] = tanh(alpha * x[t][c]) * w[c] + b[c]                    (no mean, no variance: elementwise)
//   y[t][c] = h[t][c] + sum_j conv[c][j] * h[t - taps + 1 + j][c]    (j = 0 .. taps - 1; zeros before the sequence)
//
// Everything is float32 arithmetic whatever the tensors' types. The convolution's inputs from before the step
// are the sequence's last taps - 1 values of h, kept per slot in the state area (oldest first, zero when a
// sequence starts); inputs from inside the step are formed again from x, which costs a tanh and saves a pass.
// The rows may come as a sum that has not been formed yet: x + (pending + pending_bias), a float32 stream and a branch's
// float32 result (with the bias [width] of its last product, or none). The kernel then also writes the sum (`sum_out`,
// another buffer than x: rows of x are read again as other tokens' earlier inputs), which is one pass over the stream
// instead of two.
// A step of single tokens reads and rewrites the state in the one kernel (the same thread does both); a step
// with longer portions leaves the state to a second small kernel that runs after every reader.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float dyt_value(float x, float alpha, float w, float b) { return fmaf(tanhf(alpha * x), w, b); }

// What a row is the sum of, beyond x: null pointers when x is the row itself.
struct Pending {
  const float* rows;    // [n, width] float32
  const float* bias;    // [width] float32 or null
  float* sum_out;       // [n, width] float32: x + (rows + bias)
};

template <typename TI>
__device__ __forceinline__ float row_value(const TI* __restrict__ x, const Pending& pd, size_t off, int c) {
  float v = to_f(x[off]);
  if (pd.rows) v += pd.rows[off] + (pd.bias ? pd.bias[c] : 0.f);
  return v;
}

template <typename TI, typename TO>
__global__ void dyt_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                           const float* __restrict__ b, TO* __restrict__ y, long long total, int width, Pending pd) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = int(i % width);
  const float v = row_value(x, pd, size_t(i), c);
  if (pd.sum_out) pd.sum_out[i] = v;
  y[i] = from_f<TO>(dyt_value(v, alpha[0], w[c], b ? b[c] : 0.f));
}

// grid (ceil(width / threads), tokens)
template <typename TI, typename TO>
__global__ void dyt_conv_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                                const float* __restrict__ b, const float* __restrict__ conv, float* __restrict__ state,
                                int state_stride, const int* __restrict__ slots, StepBatch sb, TO* __restrict__ y, int width,
                                int taps, int write_state, Pending pd) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int t = blockIdx.y;
  const int seq = sb.tok_seq[t], start = sb.seq_start[seq];
  const int idx = t - start;                              // the token's place among the sequence's tokens of this step
  float* st = state + size_t(slots[seq]) * state_stride;  // [taps - 1][width]
  const float a = alpha[0], wc = w[c], bc = b ? b[c] : 0.f;
  float h[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps) break;
    const int src = idx - (taps - 1) + j;
    if (src >= 0) {
      const float v = row_value(x, pd, size_t(start + src) * width + c, c);
      if (pd.sum_out && src == idx) pd.sum_out[size_t(t) * width + c] = v;
      h[j] = dyt_value(v, a, wc, bc);
    } else {
      h[j] = st[size_t(taps - 1 + src) * width + c];
    }
  }
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps) break;
    acc = fmaf(conv[size_t(c) * taps + j], h[j], acc);
  }
  float own = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j)
    if (j == taps - 1) own = h[j];
  y[size_t(t) * width + c] = from_f<TO>(own + acc);
  if (write_state && idx == 0) {
    // every sequence brings one token: h[1 .. taps - 1] are the last taps - 1 inputs now
#pragma unroll
    for (int j = 1; j < MAX_TAPS; ++j) {
      if (j >= taps) break;
      st[size_t(j - 1) * width + c] = h[j];
    }
  }
}

// ---- four channels a thread (width a multiple of 4, rows at whole 16-byte words): 16-byte loads, and in the
// convolution a run of tokens per thread whose window of earlier inputs slides, so that every tanh is formed once
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 dyt4(float4 x, float a, float4 w, float4 b) {
  return make_float4(dyt_value(x.x, a, w.x, b.x), dyt_value(x.y, a, w.y, b.y), dyt_value(x.z, a, w.z, b.z),
                     dyt_value(x.w, a, w.w, b.w));
}
__device__ __forceinline__ float4 fma4(float4 a, float4 b, float4 c) {
  return make_float4(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y), fmaf(a.z, b.z, c.z), fmaf(a.w, b.w, c.w));
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
template <typename TI>
__device__ __forceinline__ float4 row_value4(const TI* __restrict__ x, const Pending& pd, float4 pb, size_t off) {
  float4 v = load4(x + off);
  if (pd.rows) v = add4(v, add4(load4(pd.rows + off), pb));
  return v;
}

template <typename TI, typename TO>
__global__ void dyt_vec_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                               const float* __restrict__ b, TO* __restrict__ y, long long total4, int width, Pending pd) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  const int c = int((i * 4) % width);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 bc = b ? load4(b + c) : zero;
  const float4 v = row_value4(x, pd, pd.bias ? load4(pd.bias + c) : zero, size_t(i) * 4);
  if (pd.sum_out) store4(pd.sum_out + i * 4, v);
  store4(y + i * 4, dyt4(v, alpha[0], load4(w + c), bc));
}

// grid (ceil(width / 4 / threads), ceil(tokens / RUN)): a thread walks RUN tokens of the step in order; their inputs
// are all loaded before the first is used. MT: the most taps this instance takes (its registers hold MT weights and
// MT - 1 earlier inputs of four channels)
template <typename TI, typename TO, int RUN, int MT>
__global__ void dyt_conv_vec_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                                    const float* __restrict__ b, const float* __restrict__ conv, float* __restrict__ state,
                                    int state_stride, const int* __restrict__ slots, StepBatch sb, TO* __restrict__ y,
                                    int n, int width, int taps, int write_state, Pending pd) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= width) return;
  const int t0 = blockIdx.y * RUN, t1 = min(n, t0 + RUN);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 pb = pd.bias ? load4(pd.bias + c) : zero;
  float4 xv[RUN];
#pragma unroll
  for (int u = 0; u < RUN; ++u) xv[u] = t0 + u < t1 ? row_value4(x, pd, pb, size_t(t0 + u) * width + c) : zero;
  // the taps - 1 inputs before the run's first token, oldest first: rows of this step where the sequence has that many
  // in it, else the slot's state; loaded with the run's own rows, so that the thread waits for memory once
  const int seq0 = sb.tok_seq[t0], start0 = sb.seq_start[seq0], idx0 = t0 - start0;
  float4 wraw[MT - 1];
#pragma unroll
  for (int j = 0; j < MT - 1; ++j) {
    if (j >= taps - 1) break;
    const int src = idx0 - (taps - 1) + j;
    wraw[j] = (src >= 0) ? row_value4(x, pd, pb, size_t(start0 + src) * width + c)
                         : load4(state + size_t(slots[seq0]) * state_stride + size_t(taps - 1 + src) * width + c);
  }
  if (pd.sum_out) {
#pragma unroll
    for (int u = 0; u < RUN; ++u)
      if (t0 + u < t1) store4(pd.sum_out + size_t(t0 + u) * width + c, xv[u]);
  }
  const float a = alpha[0];
  const float4 wc = load4(w + c), bc = b ? load4(b + c) : zero;
  float4 cw[MT], win[MT - 1];
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    if (j >= taps) break;
    cw[j] = make_float4(conv[size_t(c) * taps + j], conv[size_t(c + 1) * taps + j], conv[size_t(c + 2) * taps + j],
                        conv[size_t(c + 3) * taps + j]);
  }
#pragma unroll
  for (int u = 0; u < RUN; ++u) {
    const int t = t0 + u;
    if (t >= t1) break;
    const int seq = sb.tok_seq[t], start = sb.seq_start[seq];
    const int idx = t - start;
    float* st = state + size_t(slots[seq]) * state_stride;
    if (t == t0) {                    // the window of the taps - 1 inputs before this token, oldest first
#pragma unroll
      for (int j = 0; j < MT - 1; ++j) {
        if (j >= taps - 1) break;
        win[j] = (idx - (taps - 1) + j >= 0) ? dyt4(wraw[j], a, wc, bc) : wraw[j];
      }
    } else if (idx == 0) {            // a sequence that starts inside the run: all of its window is its slot's state
#pragma unroll
      for (int j = 0; j < MT - 1; ++j) {
        if (j >= taps - 1) break;
        win[j] = load4(st + size_t(j) * width + c);
      }
    }
    const float4 own = dyt4(xv[u], a, wc, bc);
    float4 acc = own;
#pragma unroll
    for (int j = 0; j < MT - 1; ++j) {
      if (j >= taps - 1) break;
      acc = fma4(cw[j], win[j], acc);
    }
#pragma unroll
    for (int j = 0; j < MT; ++j)
      if (j == taps - 1) acc = fma4(cw[j], own, acc);
    store4(y + size_t(t) * width + c, acc);
#pragma unroll
    for (int j = 0; j < MT - 1; ++j) {      // slide
      if (j >= taps - 1) break;
      win[j] = (j + 1 < taps - 1) ? win[j + 1 < MT - 1 ? j + 1 : j] : own;
    }
    if (write_state && idx == 0) {
      // every sequence brings one token: the window after the slide is the state
#pragma unroll
      for (int j = 0; j < MT - 1; ++j) {
        if (j >= taps - 1) break;
        store4(st + size_t(j) * width + c, win[j]);
      }
    }
  }
}

// grid (ceil(width / threads), sequences): the state after the step
template <typename TI>
__global__ void dyt_conv_state_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                                      const float* __restrict__ b, float* __restrict__ state, int state_stride,
                                      const int* __restrict__ slots, StepBatch sb, int width, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int seq = blockIdx.y, start = sb.seq_start[seq], n_new = sb.seq_new[seq];
  float* st = state + size_t(slots[seq]) * state_stride;
  const float a = alpha[0], wc = w[c], bc = b ? b[c] : 0.f;
  float h[MAX_TAPS];
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i) {
    if (i >= taps - 1) break;
    const int rel = n_new - (taps - 1) + i;      // the input that becomes entry i
    h[i] = (rel >= 0) ? dyt_value(to_f(x[size_t(start + rel) * width + c]), a, wc, bc) : st[size_t(i + n_new) * width + c];
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i) {
    if (i >= taps - 1) break;
    st[size_t(i) * width + c] = h[i];
  }
}

template <typename TI, typename TO>
int launch_dyt(const void* x, const float* alpha, const float* w, const float* b, void* y, int n, int width,
               const float* conv, float* state, int state_stride, const int* slots, const StepBatch* sb, int taps,
               int single_tokens, Pending pd, cudaStream_t stream) {
  const int threads = 256;
  const bool vec = width % 4 == 0 && (pd.rows == nullptr || (aligned16(pd.rows) && aligned16(pd.sum_out) &&
                                                              (pd.bias == nullptr || aligned16(pd.bias)))) && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(TI))) == 0 &&
                   (reinterpret_cast<uintptr_t>(y) % (4 * sizeof(TO))) == 0 && aligned16(w) && (b == nullptr || aligned16(b)) &&
                   (conv == nullptr || taps <= 1 || (aligned16(state) && state_stride % 4 == 0));
  if (conv == nullptr) {
    const long long total = (long long)n * width;
    if (vec)
      dyt_vec_kernel<TI, TO><<<unsigned((total / 4 + threads - 1) / threads), threads, 0, stream>>>((const TI*)x, alpha, w, b,
                                                                                                  (TO*)y, total / 4, width, pd);
    else
      dyt_kernel<TI, TO><<<unsigned((total + threads - 1) / threads), threads, 0, stream>>>((const TI*)x, alpha, w, b, (TO*)y,
                                                                                           total, width, pd);
    return launch_status();
  }
  if (vec) {
    const int vthreads = 128, across = (width / 4 + vthreads - 1) / vthreads;
#define PTB_DYT_RUN(RUN)                                                                                                  \
  do {                                                                                                                    \
    if (taps <= 4)                                                                                                        \
      dyt_conv_vec_kernel<TI, TO, RUN, 4><<<dim3(across, (n + RUN - 1) / RUN), vthreads, 0, stream>>>(                    \
          (const TI*)x, alpha, w, b, conv, state, state_stride, slots, *sb, (TO*)y, n, width, taps, single_tokens, pd);   \
    else                                                                                                                  \
      dyt_conv_vec_kernel<TI, TO, RUN, MAX_TAPS><<<dim3(across, (n + RUN - 1) / RUN), vthreads, 0, stream>>>(             \
          (const TI*)x, alpha, w, b, conv, state, state_stride, slots, *sb, (TO*)y, n, width, taps, single_tokens, pd);   \
  } while (0)
    // the longest run that still gives every SM a thousand threads: a run of RUN tokens forms RUN + taps - 1 values of
    // tanh instead of RUN * taps, but a step has to fill the machine first (a run of 8 at 2,048 x 2,048 left it a
    // fifth occupied and took four times a plain pass)
    const long long want = 148LL * 1024, lanes = (long long)across * vthreads;
    if (lanes * ((n + 7) / 8) >= want)
      PTB_DYT_RUN(8);
    else if (lanes * ((n + 3) / 4) >= want)
      PTB_DYT_RUN(4);
    else if (lanes * ((n + 1) / 2) >= want)
      PTB_DYT_RUN(2);
    else
      PTB_DYT_RUN(1);
#undef PTB_DYT_RUN
  } else {
    dim3 grid((width + threads - 1) / threads, n);
    dyt_conv_kernel<TI, TO><<<grid, threads, 0, stream>>>((const TI*)x, alpha, w, b, conv, state, state_stride, slots, *sb,
                                                          (TO*)y, width, taps, single_tokens, pd);
  }
  int code = launch_status();
  if (code != PTB_OK || single_tokens || taps <= 1) return code;
  dim3 grid2((width + threads - 1) / threads, sb->n_seqs);
  // the state's inputs come from the sum where the first kernel has formed it (TI is float then)
  dyt_conv_state_kernel<TI><<<grid2, threads, 0, stream>>>(pd.rows ? (const TI*)pd.sum_out : (const TI*)x, alpha, w, b, state, state_stride, slots, *sb, width,
                                                           taps);
  return launch_status();
}

}  // namespace

// x [n, width] (float32 or bfloat16) -> y [n, width] (float32 or bfloat16). alpha: one float32 on the device; w, b: float32
// [width] (b may be null). With conv (float32 [width, taps]): the convolution over each sequence's tokens, with
// state [slots, >= (taps - 1) * width] float32 (rows state_stride apart); single_tokens: every sequence brings one token.
// pending (float32 [n, width], with x float32; pending_bias float32 [width] or null): the rows are x + (pending +
// pending_bias), and sum_out (float32 [n, width], not x) receives them.
PTB_API int ptb_dyt(int in_dtype, const void* x, const float* alpha, const float* w, const float* b, int out_dtype, void* y,
                    int n, int width, const float* conv, float* state, int state_stride, const int* slots,
                    const StepBatch* sb, int taps, int single_tokens, const float* pending, const float* pending_bias,
                    float* sum_out, cudaStream_t stream) {
  if (n <= 0 || width <= 0) return PTB_OK;
  if (pending == nullptr && (pending_bias != nullptr || sum_out != nullptr)) return PTB_ERR_SIZE;
  if (pending != nullptr && (sum_out == nullptr || (const void*)sum_out == x)) return PTB_ERR_SIZE;
  if (pending != nullptr && in_dtype != PTB_F32) return PTB_ERR_DTYPE;
  const Pending pd{pending, pending_bias, sum_out};
  if (conv != nullptr && (taps < 1 || taps > MAX_TAPS || sb == nullptr || sb->n_tokens != n || slots == nullptr ||
                          (taps > 1 && (state == nullptr || state_stride < (taps - 1) * width))))
    return PTB_ERR_SIZE;
#define PTB_DYT(TI, TO) \
  return launch_dyt<TI, TO>(x, alpha, w, b, y, n, width, conv, state, state_stride, slots, sb, taps, single_tokens, pd, stream)
  if (in_dtype == PTB_F32 && out_dtype == PTB_F32) PTB_DYT(float, float);
  if (in_dtype == PTB_F32 && out_dtype == PTB_BF16) PTB_DYT(float, __nv_bfloat16);
  if (in_dtype == PTB_BF16 && out_dtype == PTB_BF16) PTB_DYT(__nv_bfloat16, __nv_bfloat16);
  if (in_dtype == PTB_BF16 && out_dtype == PTB_F32) PTB_DYT(__nv_bfloat16, float);
#undef PTB_DYT
  return PTB_ERR_DTYPE;
}
