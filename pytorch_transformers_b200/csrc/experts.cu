// Routed experts: the router (scores, group-limited choice), the plan that sorts (token, choice)
// pairs by expert into tiles, the experts' grouped matrix products and the weighted sum.
//
// Router, per token, in float32: z = W_r h, s = softmax(z) over all n outputs; choice scores
// s + correction; outputs form `n_groups` equal groups of neighbours, a group's score is its largest
// choice score, only the `keep` best groups stay eligible; the `top` largest eligible choice scores
// are chosen (ties: lowest index); the weight of a chosen output is s * route_scale (not renormalised).
// The last n - n_experts outputs are identity experts: they pass their input on.
// score_kind 1: s = sigmoid(z) per output instead of the softmax. correction may be null (none).
#include "common.cuh"

namespace {

constexpr int ROUTE_VPL = 16;   // router outputs per lane: up to 512 outputs
constexpr int ROUTE_WARPS = 8;

constexpr int ROUTE_TOKENS = 8;   // tokens of a block of the logits kernel for prompts: a matrix row is read once for them

// Router logits z[t, e] = W_r[e] . h[t] in float32: a warp per output, lanes along the width, TPB tokens a
// block; a token's sums have one fixed order whatever else is in the batch.
template <typename T, int TPB>
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
route_logits_kernel(const T* __restrict__ h, const float* __restrict__ w_router, float* __restrict__ z, int n_tokens,
                    int width, int n) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t0 = blockIdx.x * TPB, e = blockIdx.y * ROUTE_WARPS + warp;
  if (e >= n) return;
  const float* wr = w_router + size_t(e) * width;
  float d[TPB];
  const T* rows[TPB];      // a token past the end reads the block's first token; its result is not written
#pragma unroll
  for (int i = 0; i < TPB; ++i) {
    d[i] = 0.f;
    rows[i] = h + size_t(t0 + i < n_tokens ? t0 + i : t0) * width;
  }
#pragma unroll 4
  for (int k = lane; k < width; k += 32) {
    const float wv = wr[k];
#pragma unroll
    for (int i = 0; i < TPB; ++i) d[i] = fmaf(wv, to_f(rows[i][k]), d[i]);
  }
#pragma unroll
  for (int i = 0; i < TPB; ++i) {
    const float v = warp_sum(d[i]);
    if (lane == 0 && t0 + i < n_tokens) z[size_t(t0 + i) * n + e] = v;
  }
}

// Scores and choice from the logits: a warp per token.
__global__ void __launch_bounds__(32 * ROUTE_WARPS)
route_select_kernel(const float* __restrict__ zs_all, const float* __restrict__ correction, int* __restrict__ ids,
                    float* __restrict__ gates, int n_tokens, int n, int n_groups, int keep, int top,
                    float route_scale, int score_kind, int z_stride, int group_top, int normalize) {
  extern __shared__ float sm[];   // per warp: n choice scores, n_groups group scores
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  const float* zs = zs_all + size_t(t) * z_stride;
  float* choice = sm + size_t(warp) * (n + n_groups);
  float* gscore = choice + n;
  float z[ROUTE_VPL], s[ROUTE_VPL];
  float zmax = -INFINITY;
#pragma unroll
  for (int v = 0; v < ROUTE_VPL; ++v) {
    const int e = lane + 32 * v;
    z[v] = (e < n) ? zs[e] : -INFINITY;
    zmax = fmaxf(zmax, z[v]);
  }
  zmax = warp_max(zmax);
  float sum = 0.f;
#pragma unroll
  for (int v = 0; v < ROUTE_VPL; ++v) {
    const int e = lane + 32 * v;
    s[v] = (e < n) ? expf(z[v] - zmax) : 0.f;
    sum += s[v];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int v = 0; v < ROUTE_VPL; ++v) {
    const int e = lane + 32 * v;
    if (score_kind == 1) s[v] = (e < n) ? 1.f / (1.f + expf(-z[v])) : 0.f;
    else s[v] = s[v] / sum;
    if (e < n) choice[e] = s[v] + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  const int per = n / n_groups;
  for (int g = lane; g < n_groups; g += 32) {
    float m = -INFINITY, m2 = -INFINITY;      // the group's largest and second largest choice scores
    for (int i = 0; i < per; ++i) {
      const float c = choice[g * per + i];
      if (c > m) {
        m2 = m;
        m = c;
      } else {
        m2 = fmaxf(m2, c);
      }
    }
    gscore[g] = (group_top == 2 && per > 1) ? m + m2 : m;
  }
  __syncwarp();
  if (keep < n_groups) {
    // a group stays if fewer than `keep` groups beat it (a larger score, or the same with a lower index)
    for (int g = lane; g < n_groups; g += 32) {
      const float mine = gscore[g];
      int better = 0;
      for (int o = 0; o < n_groups; ++o) better += (gscore[o] > mine || (gscore[o] == mine && o < g)) ? 1 : 0;
      if (better >= keep)
        for (int i = 0; i < per; ++i) choice[g * per + i] = -INFINITY;
    }
    __syncwarp();
  }
  float cs[ROUTE_VPL];
  bool open[ROUTE_VPL];
#pragma unroll
  for (int v = 0; v < ROUTE_VPL; ++v) {
    const int e = lane + 32 * v;
    cs[v] = (e < n) ? choice[e] : -INFINITY;
    open[v] = e < n;
  }
  float chosen_sum = 0.f;     // of the chosen outputs' scores, in the order of the choice (every lane holds it)
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int v = 0; v < ROUTE_VPL; ++v) {
      const int e = lane + 32 * v;
      if (open[v] && (best_e == 0x7fffffff || cs[v] > best)) {   // lane's entries come in ascending index
        best = cs[v];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) {
        best = ob;
        best_e = oe;
      }
    }
    float sv = 0.f;
    if (best_e % 32 == lane) {
      const int v = best_e / 32;
#pragma unroll
      for (int u = 0; u < ROUTE_VPL; ++u)
        if (u == v) {
          sv = s[u];
          open[u] = false;
        }
      ids[size_t(t) * top + k] = best_e;
      if (!normalize) gates[size_t(t) * top + k] = sv * route_scale;
    }
    if (normalize) {
      sv = __shfl_sync(0xffffffffu, sv, best_e % 32);
      chosen_sum += sv;
      if (lane == 0) gates[size_t(t) * top + k] = sv;
    }
  }
  if (normalize && lane == 0) {
    // weights = scores / (their sum + 1e-20) * scale
    const float total = chosen_sum + 1e-20f;
    for (int k = 0; k < top; ++k) gates[size_t(t) * top + k] = gates[size_t(t) * top + k] / total * route_scale;
  }
}

// One block sorts the pairs (token, choice) by expert. plan (int32):
//   [0]                         number of tiles
//   [1, 1 + max_tiles)          expert of each tile
//   [.., + max_tiles)           first sorted row of each tile
//   [.., + max_tiles)           rows of each tile
//   then row_of_pair [pairs] (-1 for an identity expert) and pair_of_row [pairs]
// Pairs of one expert take consecutive rows; their order among themselves is not fixed, and no
// result depends on it (every row is computed alone and summed per token in the order of the choice).
__global__ void __launch_bounds__(1024)
expert_plan_kernel(const int* __restrict__ ids, int* __restrict__ plan, int pairs, int n_experts, int tile_rows,
                   int max_tiles) {
  extern __shared__ int si[];   // counts [n_experts], offsets [n_experts + 1], cursor [n_experts]
  int* count = si;
  int* offset = count + n_experts;
  int* cursor = offset + n_experts + 1;
  int* tile_expert = plan + 1;
  int* tile_row0 = tile_expert + max_tiles;
  int* tile_n = tile_row0 + max_tiles;
  int* row_of_pair = tile_n + max_tiles;
  int* pair_of_row = row_of_pair + pairs;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e < n_experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < n_experts; ++e) {
      offset[e] = rows;
      for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
        tile_expert[tiles] = e;
        tile_row0[tiles] = rows + r0;
        tile_n[tiles] = min(tile_rows, count[e] - r0);
        ++tiles;
      }
      rows += count[e];
    }
    offset[n_experts] = rows;
    plan[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    int row = -1;
    if (e < n_experts) {
      row = offset[e] + atomicAdd(&cursor[e], 1);
      pair_of_row[row] = p;
    }
    row_of_pair[p] = row;
  }
}

// Grouped product over the plan's tiles. MODE 0: rows are gathered from h by token (pair / top),
// W [experts, 2 F, K] holds gate rows then up rows, out[row, f] = silu(gate) * up in the model dtype.
// MODE 1: rows are `x`'s sorted rows [pairs, K], W [experts, N, K], out [pairs, N] float32.
// MODE 2: rows gathered from h as in MODE 0, W [experts, N, K] (an expert without a gate),
// out[row, n] = act(row_scale[pair] * (W h)) in the model dtype: the expert's first product of the pair's
// weight times the token's row (the weight commutes with the product).
// float32 FMAs in ascending k (16 products summed apart, then into the total): a row's result does
// not depend on its tile. A block computes TM * 16 rows x 64 outputs.
constexpr int EBN = 64, EBK = 16, ETN = 4;

template <typename T, typename TO, int MODE, int TM>
__global__ void __launch_bounds__(256)
expert_linear_kernel(const T* __restrict__ x, const T* __restrict__ w, TO* __restrict__ out,
                     const int* __restrict__ plan, int pairs, int max_tiles, int top, int N, int K,
                     const float* __restrict__ row_scale, int act) {
  constexpr int EBM = TM * 16;
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int expert = plan[1 + tile], row0 = plan[1 + max_tiles + tile], rows = plan[1 + 2 * max_tiles + tile];
  const int* pair_of_row = plan + 1 + 3 * max_tiles + pairs;
  __shared__ float xs[EBK][EBM + 4];
  __shared__ float ws[MODE == 0 ? 2 : 1][EBK][EBN + 4];
  __shared__ int src_row[EBM];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * EBN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * ETN;
  if (tid < EBM) src_row[tid] = (tid < rows) ? (MODE != 1 ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const T* we = w + size_t(expert) * (MODE == 0 ? 2 : 1) * N * K;
  float acc[MODE == 0 ? 2 : 1][TM][ETN];
#pragma unroll
  for (int s = 0; s < (MODE == 0 ? 2 : 1); ++s)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < ETN; ++j) acc[s][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += EBK) {
    for (int i = tid; i < EBM * EBK; i += 256) {
      const int rr = i / EBK, kk = i % EBK;
      const int sr = src_row[rr], k = k0 + kk;
      xs[kk][rr] = (sr >= 0 && k < K) ? to_f(x[size_t(sr) * K + k]) : 0.f;
    }
    for (int i = tid; i < EBN * EBK; i += 256) {
      const int nn = i / EBK, kk = i % EBK;
      const int gn = n0 + nn, k = k0 + kk;
      const bool ok = gn < N && k < K;
      ws[0][kk][nn] = ok ? to_f(we[size_t(gn) * K + k]) : 0.f;
      if (MODE == 0) ws[MODE == 0 ? 1 : 0][kk][nn] = ok ? to_f(we[size_t(N + gn) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < (MODE == 0 ? 2 : 1); ++s) {
      float part[TM][ETN];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < ETN; ++j) part[i][j] = 0.f;
#pragma unroll
      for (int k = 0; k < EBK; ++k) {
        float a[TM], b[ETN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
        for (int j = 0; j < ETN; ++j) b[j] = ws[s][k][tn + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < ETN; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < ETN; ++j) acc[s][i][j] += part[i][j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    if (tm + i >= rows) continue;
#pragma unroll
    for (int j = 0; j < ETN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[0][i][j];
      if (MODE == 0) v = v / (1.f + expf(-v)) * acc[MODE == 0 ? 1 : 0][i][j];
      if (MODE == 2) v = apply_activation(v * (row_scale ? row_scale[pair_of_row[row0 + tm + i]] : 1.f), act);
      out[size_t(row0 + tm + i) * N + gn] = from_f<TO>(v);
    }
  }
}

// out[t] = base[t] + sum_k gate[t, k] * (expert output row of the pair, or h[t] for an identity expert),
// summed in float32 in the order of the choice (gate null: every weight is one); base and out are float32 or of
// the model dtype (TB). With `shared` (float32 [tokens, width]) the result also holds sigmoid(shared_gate[t]) * shared[t]
// (shared_gate null: the rows as they are).
// One block per token.
template <typename T, typename TB>
__global__ void expert_combine_kernel(const TB* __restrict__ base, const T* __restrict__ h,
                                      const float* __restrict__ y, const int* __restrict__ ids,
                                      const float* __restrict__ gates, const int* __restrict__ row_of_pair,
                                      TB* __restrict__ out, int width, int top, const float* __restrict__ shared,
                                      const float* __restrict__ shared_gate, int shared_gate_stride) {
  const int t = blockIdx.x;
  // an expert that every token uses: its float32 rows times sigmoid(one logit per token), added last
  const float sg = shared ? (shared_gate ? 1.f / (1.f + expf(-shared_gate[size_t(t) * shared_gate_stride])) : 1.f) : 0.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = row_of_pair[size_t(t) * top + k];
      const float v = (row >= 0) ? y[size_t(row) * width + i] : to_f(h[size_t(t) * width + i]);
      s = fmaf(gates ? gates[size_t(t) * top + k] : 1.f, v, s);
    }
    if (shared) s = fmaf(sg, shared[size_t(t) * width + i], s);
    out[size_t(t) * width + i] = from_f<TB>((base ? to_f(base[size_t(t) * width + i]) : 0.f) + s);
  }
}

template <typename T, typename TO, int MODE>
int launch_expert_linear(const void* x, const void* w, void* out, const int* plan, int pairs, int max_tiles, int top,
                         int N, int K, int tile_rows, const float* row_scale, int act, cudaStream_t stream) {
  dim3 grid((N + EBN - 1) / EBN, max_tiles);
  if (tile_rows == 16)
    expert_linear_kernel<T, TO, MODE, 1><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, (TO*)out, plan, pairs,
                                                                   max_tiles, top, N, K, row_scale, act);
  else if (tile_rows == 64)
    expert_linear_kernel<T, TO, MODE, 4><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, (TO*)out, plan, pairs,
                                                                   max_tiles, top, N, K, row_scale, act);
  else
    return PTB_ERR_SIZE;
  return launch_status();
}

}  // namespace

// `logits`: float32 [n_tokens, n + extra]: the router matrix has `extra` more rows whose logits are formed with the
// others and take no part in the choice (a gate that reads the same input). group_top 1 or 2: a group is scored by its
// largest choice score or by the sum of its two largest. normalize: weights = scores / (sum of the chosen + 1e-20) * scale.
PTB_API int ptb_route_grouped(int dtype, const void* h, const float* w_router, const float* correction, float* logits, int* ids,
                      float* gates, int n_tokens, int width, int n, int n_groups, int keep, int top, float route_scale,
                      int score_kind, int extra, int group_top, int normalize, cudaStream_t stream) {
  if (n_tokens <= 0) return PTB_OK;
  if (n <= 0 || n > 32 * ROUTE_VPL || n_groups <= 0 || n % n_groups != 0 || keep <= 0 || keep > n_groups || top <= 0 ||
      top > (n / n_groups) * keep || width <= 0 || score_kind < 0 || score_kind > 1 || extra < 0 || group_top < 1 || group_top > 2)
    return PTB_ERR_SIZE;
  // few tokens (steps of single tokens): one token a block, so that the blocks fill the device
  const int tpb = n_tokens >= 2 * sm_count() ? ROUTE_TOKENS : 1;
  dim3 grid((n_tokens + tpb - 1) / tpb, (n + extra + ROUTE_WARPS - 1) / ROUTE_WARPS);
#define PTB_ROUTE(TT, NTOK) \
  route_logits_kernel<TT, NTOK><<<grid, 32 * ROUTE_WARPS, 0, stream>>>((const TT*)h, w_router, logits, n_tokens, width, n + extra)
  if (dtype == PTB_F32) {
    if (tpb == 1) PTB_ROUTE(float, 1);
    else PTB_ROUTE(float, ROUTE_TOKENS);
  } else if (dtype == PTB_BF16) {
    if (tpb == 1) PTB_ROUTE(__nv_bfloat16, 1);
    else PTB_ROUTE(__nv_bfloat16, ROUTE_TOKENS);
  } else {
    return PTB_ERR_DTYPE;
  }
#undef PTB_ROUTE
  if (launch_status() != PTB_OK) return PTB_ERR_LAUNCH;
  const size_t smem = size_t(ROUTE_WARPS) * (n + n_groups) * sizeof(float);
  route_select_kernel<<<(n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS, 32 * ROUTE_WARPS, smem, stream>>>(
      logits, correction, ids, gates, n_tokens, n, n_groups, keep, top, route_scale, score_kind, n + extra, group_top, normalize);
  return launch_status();
}

PTB_API int ptb_route(int dtype, const void* h, const float* w_router, const float* correction, float* logits, int* ids,
                      float* gates, int n_tokens, int width, int n, int n_groups, int keep, int top, float route_scale,
                      int score_kind, cudaStream_t stream) {
  return ptb_route_grouped(dtype, h, w_router, correction, logits, ids, gates, n_tokens, width, n, n_groups, keep, top,
                           route_scale, score_kind, 0, 1, 0, stream);
}

// int32 words of a plan for `pairs` pairs and `max_tiles` tiles
PTB_API long long ptb_expert_plan_words(int pairs, int max_tiles) { return 1 + 3LL * max_tiles + 2LL * pairs; }

PTB_API int ptb_expert_plan(const int* ids, int* plan, int pairs, int n_experts, int tile_rows, int max_tiles,
                            cudaStream_t stream) {
  if (pairs <= 0) return PTB_OK;
  if (n_experts <= 0 || n_experts > 4000 || tile_rows <= 0 || max_tiles < pairs / tile_rows + (pairs < n_experts ? pairs : n_experts))
    return PTB_ERR_SIZE;
  const size_t smem = (3 * size_t(n_experts) + 1) * sizeof(int);
  expert_plan_kernel<<<1, 1024, smem, stream>>>(ids, plan, pairs, n_experts, tile_rows, max_tiles);
  return launch_status();
}

// mode 0: gate and up with silu(gate) * up, out in the model dtype; mode 1: down, out float32; mode 2: one product
// with act(row_scale * .), out in the model dtype (row_scale [pairs] float32 or null, act: an activation code)
PTB_API int ptb_expert_linear(int dtype, int mode, const void* x, const void* w, void* out, const int* plan, int pairs,
                              int max_tiles, int top, int N, int K, int tile_rows, const float* row_scale, int act,
                              cudaStream_t stream) {
  if (pairs <= 0 || max_tiles <= 0) return PTB_OK;
  if (N <= 0 || K <= 0 || max_tiles > 65535 || top <= 0 || mode < 0 || mode > 2 || !activation_known(act))
    return PTB_ERR_SIZE;
#define PTB_EL(TT, TTO, MM) \
  launch_expert_linear<TT, TTO, MM>(x, w, out, plan, pairs, max_tiles, top, N, K, tile_rows, row_scale, act, stream)
  if (dtype == PTB_F32) return mode == 0 ? PTB_EL(float, float, 0) : mode == 1 ? PTB_EL(float, float, 1) : PTB_EL(float, float, 2);
  if (dtype == PTB_BF16)
    return mode == 0 ? PTB_EL(__nv_bfloat16, __nv_bfloat16, 0)
                     : mode == 1 ? PTB_EL(__nv_bfloat16, float, 1) : PTB_EL(__nv_bfloat16, __nv_bfloat16, 2);
#undef PTB_EL
  return PTB_ERR_DTYPE;
}

PTB_API int ptb_expert_combine_shared(int dtype, int out_dtype, const void* base, const void* h, const float* y,
                               const int* ids, const float* gates, const int* row_of_pair, void* out, int n_tokens,
                               int width, int top, const float* shared, const float* shared_gate, int shared_gate_stride,
                                      cudaStream_t stream) {
  if (n_tokens <= 0) return PTB_OK;
  if (width <= 0 || top <= 0) return PTB_ERR_SIZE;
  const int threads = width >= 1024 ? 256 : 128;
  // few tokens: several blocks a token, so that the blocks fill the device
  const int per_token = n_tokens >= 2 * sm_count() ? 1 : (width + threads - 1) / threads;
  const dim3 n_tokens_grid(n_tokens, per_token);
  if (dtype == PTB_F32 && out_dtype == PTB_F32)
    expert_combine_kernel<float, float><<<n_tokens_grid, threads, 0, stream>>>(
        (const float*)base, (const float*)h, y, ids, gates, row_of_pair, (float*)out, width, top, shared, shared_gate,
        shared_gate_stride);
  else if (dtype == PTB_BF16 && out_dtype == PTB_F32)
    expert_combine_kernel<__nv_bfloat16, float><<<n_tokens_grid, threads, 0, stream>>>(
        (const float*)base, (const __nv_bfloat16*)h, y, ids, gates, row_of_pair, (float*)out, width, top, shared, shared_gate,
        shared_gate_stride);
  else if (dtype == PTB_BF16 && out_dtype == PTB_BF16)
    expert_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<n_tokens_grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)base, (const __nv_bfloat16*)h, y, ids, gates, row_of_pair, (__nv_bfloat16*)out, width,
        top, shared, shared_gate, shared_gate_stride);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_expert_combine(int dtype, int out_dtype, const void* base, const void* h, const float* y,
                               const int* ids, const float* gates, const int* row_of_pair, void* out, int n_tokens,
                               int width, int top, cudaStream_t stream) {
  return ptb_expert_combine_shared(dtype, out_dtype, base, h, y, ids, gates, row_of_pair, out, n_tokens, width, top, nullptr,
                                   nullptr, 0, stream);
}
