// The Dynamic Tanh norm, alone or with the short causal convolution that some designs put on a mixer's input.
//
//   h[t][c] = tanh(alpha * x[t][c]) * w[c] + b[c]                    (no mean, no variance: elementwise)
//   y[t][c] = h[t][c] + sum_j conv[c][j] * h[t - taps + 1 + j][c]    (j = 0 .. taps - 1; zeros before the sequence)
//
// Everything is float32 arithmetic whatever the tensors' types. The convolution's inputs from before the step
// are the sequence's last taps - 1 values of h, kept per slot in the state area (oldest first, zero when a
// sequence starts); inputs from inside the step are formed again from x, which costs a tanh and saves a pass.
// A step of single tokens reads and rewrites the state in the one kernel (the same thread does both); a step
// with longer portions leaves the state to a second small kernel that runs after every reader.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float dyt_value(float x, float alpha, float w, float b) { return fmaf(tanhf(alpha * x), w, b); }

template <typename TI, typename TO>
__global__ void dyt_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                           const float* __restrict__ b, TO* __restrict__ y, long long total, int width) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = int(i % width);
  y[i] = from_f<TO>(dyt_value(to_f(x[i]), alpha[0], w[c], b ? b[c] : 0.f));
}

// grid (ceil(width / threads), tokens)
template <typename TI, typename TO>
__global__ void dyt_conv_kernel(const TI* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ w,
                                const float* __restrict__ b, const float* __restrict__ conv, float* __restrict__ state,
                                int state_stride, const int* __restrict__ slots, StepBatch sb, TO* __restrict__ y, int width,
                                int taps, int write_state) {
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
    h[j] = (src >= 0) ? dyt_value(to_f(x[size_t(start + src) * width + c]), a, wc, bc) : st[size_t(taps - 1 + src) * width + c];
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
               int single_tokens, cudaStream_t stream) {
  const int threads = 256;
  if (conv == nullptr) {
    const long long total = (long long)n * width;
    dyt_kernel<TI, TO><<<unsigned((total + threads - 1) / threads), threads, 0, stream>>>((const TI*)x, alpha, w, b, (TO*)y,
                                                                                         total, width);
    return launch_status();
  }
  dim3 grid((width + threads - 1) / threads, n);
  dyt_conv_kernel<TI, TO><<<grid, threads, 0, stream>>>((const TI*)x, alpha, w, b, conv, state, state_stride, slots, *sb,
                                                        (TO*)y, width, taps, single_tokens);
  int code = launch_status();
  if (code != PTB_OK || single_tokens || taps <= 1) return code;
  dim3 grid2((width + threads - 1) / threads, sb->n_seqs);
  dyt_conv_state_kernel<TI><<<grid2, threads, 0, stream>>>((const TI*)x, alpha, w, b, state, state_stride, slots, *sb, width,
                                                           taps);
  return launch_status();
}

}  // namespace

// x [n, width] (float32 or bfloat16) -> y [n, width] (float32 or bfloat16). alpha: one float32 on the device; w, b: float32
// [width] (b may be null). With conv (float32 [width, taps]): the convolution over each sequence's tokens, with
// state [slots, >= (taps - 1) * width] float32 (rows state_stride apart); single_tokens: every sequence brings one token.
PTB_API int ptb_dyt(int in_dtype, const void* x, const float* alpha, const float* w, const float* b, int out_dtype, void* y,
                    int n, int width, const float* conv, float* state, int state_stride, const int* slots,
                    const StepBatch* sb, int taps, int single_tokens, cudaStream_t stream) {
  if (n <= 0 || width <= 0) return PTB_OK;
  if (conv != nullptr && (taps < 1 || taps > MAX_TAPS || sb == nullptr || sb->n_tokens != n || slots == nullptr ||
                          (taps > 1 && (state == nullptr || state_stride < (taps - 1) * width))))
    return PTB_ERR_SIZE;
#define PTB_DYT(TI, TO) \
  return launch_dyt<TI, TO>(x, alpha, w, b, y, n, width, conv, state, state_stride, slots, sb, taps, single_tokens, stream)
  if (in_dtype == PTB_F32 && out_dtype == PTB_F32) PTB_DYT(float, float);
  if (in_dtype == PTB_F32 && out_dtype == PTB_BF16) PTB_DYT(float, __nv_bfloat16);
  if (in_dtype == PTB_BF16 && out_dtype == PTB_BF16) PTB_DYT(__nv_bfloat16, __nv_bfloat16);
  if (in_dtype == PTB_BF16 && out_dtype == PTB_F32) PTB_DYT(__nv_bfloat16, float);
#undef PTB_DYT
  return PTB_ERR_DTYPE;
}
