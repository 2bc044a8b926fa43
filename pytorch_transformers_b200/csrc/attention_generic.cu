// Attention over the paged cache, general form (CUDA cores, float32 arithmetic), and the kernel
// that splits a fused projection into rotated queries and cache entries.
//
// The general attention kernel takes every head size up to 256, any number of heads and groups,
// float32 or bfloat16 tensors, rotary or ALiBi models, an optional window, prompts and single
// tokens alike. It is the kernel of the float32 path and the fallback of the bfloat16 path for
// sizes that the tensor-core kernels refuse. Every query row is reduced over its keys in blocks
// of 64 aligned to absolute positions, in ascending order, whatever else is in the launch: the
// result of a position does not depend on how tokens were cut into steps or batched.
#include "common.cuh"

namespace {

constexpr int BQ = 16;        // query rows of a tile
constexpr int THREADS = 128;  // 8 threads per query row
constexpr int MAX_D = 256;    // head sizes up to this
constexpr int DPT = MAX_D / 8;

// a float as the tensors' type holds it
template <typename T> __device__ __forceinline__ float round_store(float v) { return to_f(from_f<T>(v)); }

// ------------------------------------------------------------------------------------------------
// Fused projection [n_tokens, kv_heads * (q_per_kv + 2) * head_dim], rows grouped per K/V head as
// (q_per_kv query heads, K, V), to: q_out [n_tokens, heads, head_dim] (query head = group *
// q_per_kv + index in group) and the K and V pools of one layer. With inv_freq != nullptr the
// first 2 * rot_pairs dims of every query and key head are rotated: pairs (i, i + rot_pairs), or with
// `interleaved` pairs (2 i, 2 i + 1);
// angle = position * inv_freq[i] in float32, x' = x cos - y sin, y' = y cos + x sin. With a table
// (rope_cos, rope_sin: [n_tokens, rot_pairs], made by rope_table_kernel from the same product) the
// cosines and sines are read instead of computed. One block per token.
template <typename T>
__global__ void split_rotate_store_kernel(const T* __restrict__ fused, T* __restrict__ q_out, T* __restrict__ k_pool,
                                          T* __restrict__ v_pool, StepBatch sb, const float* __restrict__ inv_freq,
                                          const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                                          int rot_pairs, int kv_heads, int q_per_kv, int head_dim, int write_cache,
                                          int interleaved) {
  const int t = blockIdx.x;
  const int pos = sb.tok_pos[t];
  const int seq = sb.tok_seq[t];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
  const int in_page = pos % PTB_PAGE;
  const int rows = q_per_kv + 2;
  const int fused_width = kv_heads * rows * head_dim;
  const T* src_tok = fused + size_t(t) * fused_width;
  const int heads = kv_heads * q_per_kv;
  // work items: (group g, row r in group, pair or plain element)
  const int rot_dims = 2 * rot_pairs;
  // bfloat16 with head sizes and rotation widths in multiples of 8 and a table of cosines: 16-byte words
  if (sizeof(T) == 2 && head_dim % 8 == 0 && rot_pairs % 8 == 0 && (rot_pairs == 0 || (rope_cos != nullptr && !interleaved)) &&
      aligned16(fused) && aligned16(q_out) && (!write_cache || (aligned16(k_pool) && aligned16(v_pool)))) {
    const int chunks = head_dim / 8, rot_chunks = rot_pairs / 8;
    const int total_v = kv_heads * rows * chunks;
    for (int w = threadIdx.x; w < total_v; w += blockDim.x) {
      const int c = w % chunks;
      const int gr = w / chunks;
      const int r = gr % rows, g = gr / rows;
      const T* src = src_tok + size_t(g * rows + r) * head_dim;
      T* dst;
      if (r < q_per_kv) {
        dst = q_out + (size_t(t) * heads + (g * q_per_kv + r)) * head_dim;
      } else {
        if (!write_cache) continue;
        dst = ((r == q_per_kv) ? k_pool : v_pool) + kv_offset(page, g, in_page, kv_heads, head_dim);
      }
      const bool rotated_row = (r <= q_per_kv) && rot_chunks > 0;
      if (rotated_row && c < rot_chunks) {
        float a[8], b[8], cs[8], sn[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src + c * 8), a);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src + rot_pairs + c * 8), b);
        const float4* cp = reinterpret_cast<const float4*>(rope_cos + size_t(t) * rot_pairs + c * 8);
        const float4* sp = reinterpret_cast<const float4*>(rope_sin + size_t(t) * rot_pairs + c * 8);
        *reinterpret_cast<float4*>(cs) = cp[0];
        *reinterpret_cast<float4*>(cs + 4) = cp[1];
        *reinterpret_cast<float4*>(sn) = sp[0];
        *reinterpret_cast<float4*>(sn + 4) = sp[1];
#pragma unroll
        for (int e = 0; e < 8; ++e) rotate_pair(a[e], b[e], cs[e], sn[e], a[e], b[e]);
        *reinterpret_cast<uint4*>(dst + c * 8) = pack_bf16x8(a);
        *reinterpret_cast<uint4*>(dst + rot_pairs + c * 8) = pack_bf16x8(b);
      } else if (rotated_row && c < 2 * rot_chunks) {
        // the upper half of a rotated pair: written by the thread that holds the lower half
      } else {
        *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
      }
    }
    return;
  }
  const int per_row = rot_pairs + (head_dim - rot_dims);  // rotated pairs, then untouched dims
  const int total = kv_heads * rows * per_row;
  for (int w = threadIdx.x; w < total; w += blockDim.x) {
    const int e = w % per_row;
    const int gr = w / per_row;
    const int r = gr % rows;
    const int g = gr / rows;
    const T* src = src_tok + size_t(g * rows + r) * head_dim;
    T* dst;
    if (r < q_per_kv) {
      dst = q_out + (size_t(t) * heads + (g * q_per_kv + r)) * head_dim;
    } else {
      if (!write_cache) continue;
      T* pool = (r == q_per_kv) ? k_pool : v_pool;
      dst = pool + kv_offset(page, g, in_page, kv_heads, head_dim);
    }
    const bool rotated_row = (r <= q_per_kv) && (inv_freq != nullptr || rope_cos != nullptr);  // queries and K, not V
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;   // the pair's two dims
      const float a = to_f(src[ia]);
      const float b = to_f(src[ib]);
      if (rotated_row) {
        float s, c, ra, rb;
        if (rope_cos) {
          c = rope_cos[size_t(t) * rot_pairs + e];
          s = rope_sin[size_t(t) * rot_pairs + e];
        } else {
          sincosf(float(pos) * inv_freq[e], &s, &c);
        }
        rotate_pair(a, b, c, s, ra, rb);
        dst[ia] = from_f<T>(ra);
        dst[ib] = from_f<T>(rb);
      } else {
        dst[ia] = src[ia];
        dst[ib] = src[ib];
      }
    } else {
      const int i = rot_dims + (e - rot_pairs);
      dst[i] = src[i];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// One block = one tile of BQ consecutive new tokens of one sequence x one query head.
//   tile_seq[i], tile_q0[i]: sequence index and first token (within the sequence's new tokens)
// q [n_tokens, heads, head_dim]; out [n_tokens, heads * head_dim].
// score(q at position p, key at position j) = (q . k_j + alibi_h(j)) * scale for j <= p
// (and j > p - window when window > 0); softmax over those keys in float32; out = sum p_j v_j.
// Values may have a size of their own (v_dim; the V pool is [pages][kv_heads][PTB_PAGE][v_dim]).
// With `sinks` [heads] every row's softmax denominator holds one more term, exp(sink_h), taken as stored
// (`scale` is not applied to it); no key or value is read for it. With `gate` (row t, head h at gate[t * gate_stride + h]) the head's
// output is multiplied by sigmoid(gate); with `gate_wide` the gate has a number per output entry instead (row t, head h,
// entry e at gate[t * gate_stride + h * v_dim + e]); `out_scale` multiplies everything. Output row t, head h starts
// at out[t * out_stride + h * v_dim]. `softcap` > 0: score <- softcap * tanh(score / softcap) after the scale.
template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, StepBatch sb, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_q0, const float* __restrict__ alibi_slopes, int heads,
                         int kv_heads, int head_dim, float scale, int window, int v_dim,
                         const float* __restrict__ sinks, const T* __restrict__ gate, int gate_stride, float out_scale,
                         int out_stride, int keep_first, float* __restrict__ out_wide, float softcap, int gate_wide) {
  extern __shared__ float smem[];
  const int wide = max(head_dim, v_dim);
  float* qs = smem;                                 // [BQ][head_dim]
  float* kv = qs + BQ * head_dim;                   // [PTB_PAGE][wide + 1], K then V
  float* ps = kv + PTB_PAGE * (wide + 1);           // [BQ][PTB_PAGE]
  const int kstride = head_dim + 1, vstride = v_dim + 1;

  const int tile = blockIdx.x, h = blockIdx.y;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int rows = min(BQ, n_new - q0);
  const int g = h / (heads / kv_heads);
  // with out_wide the grid's third dimension names the K/V head whose values this block reads (the scores are
  // head h's own): every head's weights meet every K/V head's values, for a mixing of the heads' weights afterwards
  const int gv = out_wide ? int(blockIdx.z) : g;
  const int tid = threadIdx.x;
  const int r = tid / 8, c = tid % 8;
  const int my_pos = (r < rows) ? past + q0 + r : -1;  // -1: no key is visible, nothing is stored
  const float slope = alibi_slopes ? alibi_slopes[h] : 0.f;

  for (int i = tid; i < BQ * head_dim; i += THREADS) {
    const int rr = i / head_dim, e = i % head_dim;
    qs[i] = (rr < rows) ? to_f(q[(size_t(start + q0 + rr) * heads + h) * head_dim + e]) : 0.f;
  }
  float acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int last_pos = past + q0 + rows - 1;
  const int first_pos = past + q0;
  int kb_lo = 0;
  if (window > 0) kb_lo = max(0, first_pos - window + 1) / PTB_PAGE;
  const int kb_hi = last_pos / PTB_PAGE;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;
  // the first keep_first positions stay visible left of the window: their pages are walked first
  const int kept_pages = (window > 0 && keep_first > 0) ? min((keep_first + PTB_PAGE - 1) / PTB_PAGE, kb_lo) : 0;

  for (int kb = (kept_pages > 0 ? 0 : kb_lo); kb <= kb_hi; ++kb) {
    if (kb == kept_pages && kb < kb_lo) kb = kb_lo;
    const int page = pages[kb];
    const int valid = min(PTB_PAGE, last_pos + 1 - kb * PTB_PAGE);  // keys of this block that exist
    const T* kp = k_pool + kv_offset(page, g, 0, kv_heads, head_dim);
    const T* vp = v_pool + kv_offset(page, gv, 0, kv_heads, v_dim);
    __syncthreads();  // previous block's V and ps are no longer read
    for (int i = tid; i < PTB_PAGE * head_dim; i += THREADS) {
      const int j = i / head_dim, e = i % head_dim;
      kv[j * kstride + e] = (j < valid) ? to_f(kp[i]) : 0.f;
    }
    __syncthreads();
    // scores: this thread owns keys j = c + 8 jj of row r
    float s[8];
    float m_blk = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int j = c + 8 * jj;
      const int key_pos = kb * PTB_PAGE + j;
      float dot = 0.f;
      const float* qr = qs + r * head_dim;
      const float* kr = kv + j * kstride;
      for (int e = 0; e < head_dim; ++e) dot = fmaf(qr[e], kr[e], dot);
      bool visible = key_pos <= my_pos;
      if (window > 0) visible = visible && (key_pos > my_pos - window || key_pos < keep_first);
      float sc = -INFINITY;
      if (visible) {
        if (alibi_slopes) dot += alibi_bias(slope, key_pos);
        sc = dot * scale;
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      }
      s[jj] = sc;
      m_blk = fmaxf(m_blk, sc);
    }
    // row maximum and sum over the 8 threads of the row (lanes 8 r' .. 8 r' + 7 of a warp)
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m_blk = fmaxf(m_blk, __shfl_xor_sync(0xffffffffu, m_blk, o));
    const float m_new = fmaxf(m_run, m_blk);
    float corr = 1.f, l_blk = 0.f;
    if (m_new == -INFINITY) {
      // nothing visible so far (rows beyond the tile, or keys left of a window)
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) ps[r * PTB_PAGE + c + 8 * jj] = 0.f;
    } else {
      corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float p = (s[jj] == -INFINITY) ? 0.f : expf(s[jj] - m_new);
        ps[r * PTB_PAGE + c + 8 * jj] = p;
        l_blk += p;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) l_blk += __shfl_xor_sync(0xffffffffu, l_blk, o);
    l_run = l_run * corr + l_blk;
    m_run = m_new;
    __syncthreads();  // all scores of this block are written, K is no longer read
    for (int i = tid; i < PTB_PAGE * v_dim; i += THREADS) {
      const int j = i / v_dim, e = i % v_dim;
      kv[j * vstride + e] = (j < valid) ? to_f(vp[i]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] *= corr;
    for (int j = 0; j < PTB_PAGE; ++j) {
      const float p = ps[r * PTB_PAGE + j];
      const float* vr = kv + j * vstride;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int e = c + 8 * i;
        if (e < v_dim) acc[i] = fmaf(p, vr[e], acc[i]);
      }
    }
  }
  if (r < rows) {
    float keep = 1.f;      // what the keys' share of the denominator shrinks by when the sink raises the reference
    if (sinks) {
      const float sink = sinks[h], m_all = fmaxf(m_run, sink);
      keep = (m_run == -INFINITY) ? 0.f : expf(m_run - m_all);
      l_run = l_run * keep + expf(sink - m_all);
    }
    float inv = (l_run > 0.f ? 1.f / l_run : 0.f) * keep * out_scale;
    if (gate && !gate_wide) inv *= 1.f / (1.f + expf(-to_f(gate[size_t(start + q0 + r) * gate_stride + h])));
    if (out_wide) {
      // float32 [token][head][K/V head][v_dim]
      float* o = out_wide + ((size_t(start + q0 + r) * heads + h) * kv_heads + gv) * v_dim;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int e = c + 8 * i;
        if (e < v_dim) o[e] = acc[i] * inv;
      }
      return;
    }
    T* o = out + size_t(start + q0 + r) * out_stride + size_t(h) * v_dim;
    const T* ge = (gate && gate_wide) ? gate + size_t(start + q0 + r) * gate_stride + size_t(h) * v_dim : nullptr;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int e = c + 8 * i;
      if (e < v_dim) o[e] = from_f<T>(acc[i] * inv * (ge ? 1.f / (1.f + expf(-to_f(ge[e]))) : 1.f));
    }
  }
}

// two neighbouring entries in one access (the address a whole pair)
__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// four neighbouring entries in one access (the address a whole quad)
__device__ __forceinline__ float4 load_quad(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load_quad(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store_quad(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store_quad(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
// one half of rotate_pair: the entry `own` of a pair whose other entry is `other` (first: own c - other s; second:
// own c + other s), with rotate_pair's roundings
__device__ __forceinline__ float rotate_own(float own, float other, float c, float s, bool first) {
  return first ? __fsub_rn(__fmul_rn(own, c), __fmul_rn(other, s)) : __fadd_rn(__fmul_rn(own, c), __fmul_rn(other, s));
}

// ------------------------------------------------------------------------------------------------
// Separate projections q | k | v side by side in a row of `proj` (rows `stride` apart), an optional bias on all of
// them (float32, added here in float32), then for every query and key head: rotation of the first 2 rot_pairs
// entries (pairs (i, i + rot_pairs); the table holds cos and sin of the token's angles, with whatever factor the
// position part puts on them), then, with `unit_norm`, division by the head's root mean square (eps inside the
// root, no gain). Values: v <- (1 - lam) v + lam v_first with the values of the same token that an earlier layer
// kept (`v_first`, rows v_first_stride apart; lam one float32 on the device); `v_keep` receives this layer's own
// values (with bias, before any mixing) for later layers. Keys and values go into the paged pools at the tokens'
// positions, queries to q_out [tokens, heads, dim]. With `norm_first` the norm comes before the rotation and takes
// gains (`q_gain`, `k_gain` [dim] float32, null: none). With temp_every > 0 a query at position p is multiplied by
// 1 + temp_coef ln(floor((p + 1) / temp_every) + 1) at the end, in float32. A warp per (token, head): query heads, then key heads, then the
// K/V heads' values; the warps of a block share nothing, so a head's chain of loads, rotation, sum and stores waits
// for no other.
template <typename T>
__global__ void rope_norm_store_kernel(const T* __restrict__ proj, int stride, const float* __restrict__ bias,
                                       T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, StepBatch sb,
                                       const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int rot_pairs,
                                       int heads, int kv_heads, int dim, int v_dim, float eps, int unit_norm,
                                       const T* __restrict__ v_first, int v_first_stride, const float* __restrict__ lam,
                                       T* __restrict__ v_keep, int write_cache, int pairs, int quads,
                                       const float* __restrict__ q_gain, const float* __restrict__ k_gain, int norm_first,
                                       float temp_coef, int temp_every) {
  extern __shared__ float rows[];   // per warp: a row of `dim` floats, then cos and sin of the rotated pairs
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x, hh = blockIdx.y * (blockDim.x / 32) + warp;      // grid (tokens, groups of a block's warps)
  if (hh >= heads + 2 * kv_heads) return;
  const T* row = proj + size_t(t) * stride;
  if (hh >= heads + kv_heads) {     // the values of one K/V head
    const int g = hh - heads - kv_heads;
    const T* vsrc = row + size_t(heads + kv_heads) * dim + size_t(g) * v_dim;
    const float* vb = bias ? bias + size_t(heads + kv_heads) * dim + size_t(g) * v_dim : nullptr;
    const float l = (v_first != nullptr) ? lam[0] : 0.f;
    T* dst = nullptr;
    if (write_cache) {
      const int pos = sb.tok_pos[t], seq = sb.tok_seq[t];
      const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
      dst = v_pool + kv_offset(page, g, pos % PTB_PAGE, kv_heads, v_dim);
    }
    for (int e = lane; e < v_dim; e += 32) {
      float v = to_f(vsrc[e]) + (vb ? vb[e] : 0.f);
      if (v_keep) v_keep[(size_t(t) * kv_heads + g) * v_dim + e] = from_f<T>(v);
      if (v_first != nullptr) v = (1.f - l) * round_store<T>(v) + l * to_f(v_first[size_t(t) * v_first_stride + size_t(g) * v_dim + e]);
      if (dst) dst[e] = from_f<T>(v);
    }
    return;
  }
  const bool is_q = hh < heads;
  if (!is_q && !write_cache) return;
  float* buf = rows + size_t(warp) * (dim + 2 * rot_pairs);
  float* cs = buf + dim;
  const T* src = row + size_t(hh) * dim;
  const float* bsrc = bias ? bias + size_t(hh) * dim : nullptr;
  T* dst;
  const float* gain = is_q ? q_gain : k_gain;     // null: the norm has no gains
  float last = 1.f;     // what the finished row is multiplied by: the query temperature of the token's position
  if (is_q) {
    dst = q_out + (size_t(t) * heads + hh) * dim;
    if (temp_every > 0) last = 1.f + temp_coef * logf(float((sb.tok_pos[t] + 1) / temp_every) + 1.f);
  } else {
    const int pos = sb.tok_pos[t], seq = sb.tok_seq[t];
    const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
    dst = k_pool + kv_offset(page, hh - heads, pos % PTB_PAGE, kv_heads, dim);
  }
  if (quads) {
    // heads of up to 128 entries whose rotated part is a multiple of 8: four entries a lane in registers, the other
    // entry of a rotated pair from the lane rot_pairs / 4 further (or back) by shuffle; no shared memory
    const unsigned full = 0xffffffffu;
    const int e = 4 * lane, P = rot_pairs / 4;
    const bool on = e < dim;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 x = on ? load_quad(src + e) : zero;
    if (bsrc && on) {
      const float4 b = *reinterpret_cast<const float4*>(bsrc + e);
      x = make_float4(x.x + b.x, x.y + b.y, x.z + b.z, x.w + b.w);
    }
    if (unit_norm && norm_first) {      // the norm (with its gains) comes before the rotation
      const float ss = fmaf(x.w, x.w, fmaf(x.z, x.z, fmaf(x.y, x.y, x.x * x.x)));
      const float r = 1.0f / sqrtf(warp_sum(ss) / float(dim) + eps);
      const float4 g = (gain && on) ? *reinterpret_cast<const float4*>(gain + e) : make_float4(1.f, 1.f, 1.f, 1.f);
      x = make_float4(x.x * r * g.x, x.y * r * g.y, x.z * r * g.z, x.w * r * g.w);
    }
    if (P > 0) {
      const bool first = lane < P, rotated = lane < 2 * P;
      const int other = first ? lane + P : (rotated ? lane - P : lane);
      float4 c = zero, sn = zero;
      if (rotated) {
        c = *reinterpret_cast<const float4*>(rope_cos + size_t(t) * rot_pairs + 4 * (first ? lane : lane - P));
        sn = *reinterpret_cast<const float4*>(rope_sin + size_t(t) * rot_pairs + 4 * (first ? lane : lane - P));
      }
      const float4 y = make_float4(__shfl_sync(full, x.x, other), __shfl_sync(full, x.y, other), __shfl_sync(full, x.z, other),
                                   __shfl_sync(full, x.w, other));
      if (rotated)
        x = make_float4(rotate_own(x.x, y.x, c.x, sn.x, first), rotate_own(x.y, y.y, c.y, sn.y, first),
                        rotate_own(x.z, y.z, c.z, sn.z, first), rotate_own(x.w, y.w, c.w, sn.w, first));
    }
    float rstd = last;
    if (unit_norm && !norm_first) {
      const float ss = fmaf(x.w, x.w, fmaf(x.z, x.z, fmaf(x.y, x.y, x.x * x.x)));
      rstd = last / sqrtf(warp_sum(ss) / float(dim) + eps);
    }
    if (on) store_quad(dst + e, make_float4(x.x * rstd, x.y * rstd, x.z * rstd, x.w * rstd));
    return;
  }
  for (int i = lane; i < rot_pairs; i += 32) {       // issued with the row's loads
    cs[i] = rope_cos[size_t(t) * rot_pairs + i];
    cs[rot_pairs + i] = rope_sin[size_t(t) * rot_pairs + i];
  }
  if (pairs) {      // two entries a load (dim even, rows at whole pairs)
    for (int e = 2 * lane; e < dim; e += 64) {
      const float2 x = load_pair(src + e);
      buf[e] = x.x + (bsrc ? bsrc[e] : 0.f);
      buf[e + 1] = x.y + (bsrc ? bsrc[e + 1] : 0.f);
    }
  } else {
    for (int e = lane; e < dim; e += 32) buf[e] = to_f(src[e]) + (bsrc ? bsrc[e] : 0.f);
  }
  __syncwarp();
  if (unit_norm && norm_first) {
    float ss = 0.f;
    for (int e = lane; e < dim; e += 32) ss = fmaf(buf[e], buf[e], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / float(dim) + eps);
    for (int e = lane; e < dim; e += 32) buf[e] = buf[e] * r * (gain ? gain[e] : 1.f);
    __syncwarp();
  }
  for (int i = lane; i < rot_pairs; i += 32) {
    float a, b;
    rotate_pair(buf[i], buf[i + rot_pairs], cs[i], cs[rot_pairs + i], a, b);
    buf[i] = a;
    buf[i + rot_pairs] = b;
  }
  __syncwarp();
  float rstd = last;
  if (unit_norm && !norm_first) {
    float ss = 0.f;
    for (int e = lane; e < dim; e += 32) ss = fmaf(buf[e], buf[e], ss);
    rstd = last / sqrtf(warp_sum(ss) / float(dim) + eps);
  }
  if (pairs) {
    for (int e = 2 * lane; e < dim; e += 64) store_pair(dst + e, buf[e] * rstd, buf[e + 1] * rstd);
  } else {
    for (int e = lane; e < dim; e += 32) dst[e] = from_f<T>(buf[e] * rstd);
  }
}

// out[t][h][:] = sum_g talk[h][g] * wide[t][g][kv head of h][:]: the heads' softmax weights mixed after the softmax,
// applied to head h's own values, written as the sum over g of what every head's weights gave on those values.
// wide float32 [tokens][heads][kv_heads][v_dim]; talk float32 [heads][heads]; ascending g, float32.
template <typename T>
__global__ void talk_mix_kernel(const float* __restrict__ wide, const float* __restrict__ talk, T* __restrict__ out,
                                int out_stride, long long total, int heads, int kv_heads, int v_dim) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int e = int(i % v_dim), h = int((i / v_dim) % heads);
  const long long t = i / (v_dim * (long long)heads);
  const int c = h / (heads / kv_heads);
  const float* src = wide + (size_t(t) * heads * kv_heads + c) * v_dim + e;
  float acc = 0.f;
  for (int g = 0; g < heads; ++g) acc = fmaf(talk[size_t(h) * heads + g], src[size_t(g) * kv_heads * v_dim], acc);
  out[size_t(t) * out_stride + size_t(h) * v_dim + e] = from_f<T>(acc);
}

// The same with four value columns a thread and all heads of a K/V group in it: what every head's weights gave on the
// group's values is read once (16-byte loads) and meets the group's rows of `talk` in registers, eight heads at a time.
template <typename T>
__global__ void talk_mix_vec_kernel(const float* __restrict__ wide, const float* __restrict__ talk, T* __restrict__ out,
                                    int out_stride, long long total, int heads, int kv_heads, int v_dim) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int quads = v_dim / 4, qpk = heads / kv_heads;
  const int e = int(i % quads) * 4, c = int((i / quads) % kv_heads);
  const long long t = i / (quads * (long long)kv_heads);
  const float* src = wide + (size_t(t) * heads * kv_heads + c) * v_dim + e;
  for (int h0 = 0; h0 < qpk; h0 += 8) {
    float4 acc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* trow = talk + size_t(c * qpk + h0) * heads;
    for (int g = 0; g < heads; ++g) {
      const float4 v = *reinterpret_cast<const float4*>(src + size_t(g) * kv_heads * v_dim);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (h0 + u < qpk) {
          const float w = trow[size_t(u) * heads + g];
          acc[u].x = fmaf(w, v.x, acc[u].x);
          acc[u].y = fmaf(w, v.y, acc[u].y);
          acc[u].z = fmaf(w, v.z, acc[u].z);
          acc[u].w = fmaf(w, v.w, acc[u].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (h0 + u < qpk) {
        T* dst = out + size_t(t) * out_stride + size_t(c * qpk + h0 + u) * v_dim + e;
        dst[0] = from_f<T>(acc[u].x);
        dst[1] = from_f<T>(acc[u].y);
        dst[2] = from_f<T>(acc[u].z);
        dst[3] = from_f<T>(acc[u].w);
      }
    }
  }
}

template <typename T>
int launch_attention(const void* q, const void* k_pool, const void* v_pool, void* out, const StepBatch& sb,
                     const int* tile_seq, const int* tile_q0, int n_tiles, const float* slopes, int heads,
                     int kv_heads, int head_dim, float scale, int window, int v_dim, const float* sinks, const void* gate,
                     int gate_stride, float out_scale, int out_stride, int keep_first, float* out_wide, float softcap,
                     int gate_wide, cudaStream_t stream) {
  const int wide = head_dim > v_dim ? head_dim : v_dim;
  const size_t smem = sizeof(float) * (size_t(BQ) * head_dim + size_t(PTB_PAGE) * (wide + 1) + BQ * PTB_PAGE);
  static size_t configured = 48 * 1024;  // per element type: raised when a larger head size first comes
  if (smem > configured) {
    if (cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  dim3 grid(n_tiles, heads, out_wide ? kv_heads : 1);
  attention_generic_kernel<T><<<grid, THREADS, smem, stream>>>((const T*)q, (const T*)k_pool, (const T*)v_pool,
                                                               (T*)out, sb, tile_seq, tile_q0, slopes, heads, kv_heads,
                                                               head_dim, scale, window, v_dim, sinks, (const T*)gate,
                                                               gate_stride, out_scale, out_stride, keep_first, out_wide,
                                                               softcap, gate_wide);
  return launch_status();
}

}  // namespace

// cos and sin of position * inv_freq[i] for every token of the step, each times `factor` (a product in float32; 1 for a
// plain rotation): [n_tokens, pairs] each, float32.
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int n_tokens, int pairs,
                                  float factor) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * pairs) return;
  float s, c;
  sincosf(float(tok_pos[i / pairs]) * inv_freq[i % pairs], &s, &c);
  cos_out[i] = factor == 1.f ? c : c * factor;
  sin_out[i] = factor == 1.f ? s : s * factor;
}

PTB_API int ptb_rope_table(const int* tok_pos, const float* inv_freq, float* cos_out, float* sin_out, int n_tokens,
                           int pairs, float factor, cudaStream_t stream) {
  if (n_tokens <= 0 || pairs <= 0) return PTB_OK;
  const int total = n_tokens * pairs;
  rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(tok_pos, inv_freq, cos_out, sin_out, n_tokens, pairs, factor);
  return launch_status();
}

PTB_API int ptb_split_rotate_store(int dtype, const void* fused, void* q_out, void* k_pool, void* v_pool,
                                   const StepBatch* sb, const float* inv_freq, const float* rope_cos,
                                   const float* rope_sin, int rot_pairs, int kv_heads, int q_per_kv, int head_dim,
                                   int write_cache, int interleaved, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (kv_heads <= 0 || q_per_kv <= 0 || head_dim <= 0 || rot_pairs < 0 || 2 * rot_pairs > head_dim)
    return PTB_ERR_SIZE;
  if (inv_freq == nullptr && rope_cos == nullptr) rot_pairs = 0;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return PTB_ERR_SIZE;
  const int threads = 256;
  if (dtype == PTB_F32)
    split_rotate_store_kernel<float><<<sb->n_tokens, threads, 0, stream>>>(
        (const float*)fused, (float*)q_out, (float*)k_pool, (float*)v_pool, *sb, inv_freq, rope_cos, rope_sin,
        rot_pairs, kv_heads, q_per_kv, head_dim, write_cache, interleaved);
  else if (dtype == PTB_BF16)
    split_rotate_store_kernel<__nv_bfloat16><<<sb->n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)fused, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, *sb,
        inv_freq, rope_cos, rope_sin, rot_pairs, kv_heads, q_per_kv, head_dim, write_cache, interleaved);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_attention_generic_capped(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const StepBatch* sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                                  const float* alibi_slopes, int heads, int kv_heads, int head_dim, float scale,
                                  int window, int v_dim, const float* sinks, const void* gate, int gate_stride,
                                  float out_scale, int out_stride, int keep_first, float* out_wide, float softcap, int gate_wide,
                                         cudaStream_t stream) {
  // softcap > 0: scores are soft-capped; gate_wide: the gate has heads * v_dim numbers a token (gate_stride at least that)
  // keep_first: with a window, the sequence's first keep_first positions stay visible too. out_wide (float32
  // [tokens][heads][kv_heads][v_dim], or null): every head's weights on every K/V head's values instead of `out`.
  if (n_tiles <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim <= 0 || head_dim > MAX_D || heads > 65535 ||
      v_dim <= 0 || v_dim > MAX_D || (out_wide == nullptr && out_stride < heads * v_dim) || keep_first < 0 ||
      (out_wide != nullptr && kv_heads > 65535) || softcap < 0.f ||
      (gate != nullptr && gate_stride < (gate_wide ? heads * v_dim : heads)))
    return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return launch_attention<float>(q, k_pool, v_pool, out, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes, heads,
                                   kv_heads, head_dim, scale, window, v_dim, sinks, gate, gate_stride, out_scale, out_stride,
                                   keep_first, out_wide, softcap, gate_wide, stream);
  if (dtype == PTB_BF16)
    return launch_attention<__nv_bfloat16>(q, k_pool, v_pool, out, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes,
                                           heads, kv_heads, head_dim, scale, window, v_dim, sinks, gate, gate_stride,
                                           out_scale, out_stride, keep_first, out_wide, softcap, gate_wide, stream);
  return PTB_ERR_DTYPE;
}

PTB_API int ptb_attention_generic(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const StepBatch* sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                                  const float* alibi_slopes, int heads, int kv_heads, int head_dim, float scale,
                                  int window, int v_dim, const float* sinks, const void* gate, int gate_stride,
                                  float out_scale, int out_stride, int keep_first, float* out_wide, cudaStream_t stream) {
  return ptb_attention_generic_capped(dtype, q, k_pool, v_pool, out, sb, tile_seq, tile_q0, n_tiles, alibi_slopes, heads,
                                      kv_heads, head_dim, scale, window, v_dim, sinks, gate, gate_stride, out_scale, out_stride,
                                      keep_first, out_wide, 0.f, 0, stream);
}

// rows of a tile of the general kernel, for the host that builds the tile lists
PTB_API int ptb_attention_generic_tile_rows() { return BQ; }

// bias: float32 [(heads + kv_heads) dim + kv_heads v_dim] or null; rope_cos / rope_sin: float32 [tokens, rot_pairs] or null;
// v_first (rows v_first_stride apart), lam, v_keep [tokens, kv_heads v_dim]: null where not used.
PTB_API int ptb_qk_prepare_store(int dtype, const void* proj, int stride, const float* bias, void* q_out, void* k_pool,
                                void* v_pool, const StepBatch* sb, const float* rope_cos, const float* rope_sin, int rot_pairs,
                                int heads, int kv_heads, int dim, int v_dim, float eps, int unit_norm, const void* v_first,
                                int v_first_stride, const float* lam, void* v_keep, int write_cache, const float* q_gain,
                                 const float* k_gain, int norm_first, float temp_coef, int temp_every, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || dim <= 0 || v_dim <= 0 || stride < (heads + kv_heads) * dim + kv_heads * v_dim ||
      rot_pairs < 0 || 2 * rot_pairs > dim || (rot_pairs > 0 && (rope_cos == nullptr || rope_sin == nullptr)) ||
      (v_first != nullptr && lam == nullptr) || dim > 4096 || temp_every < 0 ||
      ((q_gain != nullptr || k_gain != nullptr) && !(unit_norm && norm_first)))
    return PTB_ERR_SIZE;
  const int warps = 8, threads = 32 * warps;
  const size_t smem = size_t(warps) * (dim + 2 * size_t(rot_pairs)) * sizeof(float);
  if (smem > 48 * 1024) return PTB_ERR_SIZE;
  const int units = heads + 2 * kv_heads;
  if ((units + warps - 1) / warps > 65535) return PTB_ERR_SIZE;
  const dim3 blocks(sb->n_tokens, (units + warps - 1) / warps);
  const size_t pair_bytes = dtype == PTB_F32 ? 8 : 4;
  const int pairs = (dim % 2 == 0 && stride % 2 == 0 && reinterpret_cast<uintptr_t>(proj) % pair_bytes == 0 &&
                     reinterpret_cast<uintptr_t>(q_out) % pair_bytes == 0 && reinterpret_cast<uintptr_t>(k_pool) % pair_bytes == 0)
                        ? 1 : 0;
  const size_t quad_bytes = 2 * pair_bytes;
  const int quads = (dim % 4 == 0 && dim <= 128 && rot_pairs % 4 == 0 && stride % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(proj) % quad_bytes == 0 && reinterpret_cast<uintptr_t>(q_out) % quad_bytes == 0 &&
                     reinterpret_cast<uintptr_t>(k_pool) % quad_bytes == 0 && (bias == nullptr || aligned16(bias)) && (q_gain == nullptr || aligned16(q_gain)) &&
                     (k_gain == nullptr || aligned16(k_gain)) &&
                     (rot_pairs == 0 || (aligned16(rope_cos) && aligned16(rope_sin))))
                        ? 1 : 0;
  if (dtype == PTB_F32)
    rope_norm_store_kernel<float><<<blocks, threads, smem, stream>>>(
        (const float*)proj, stride, bias, (float*)q_out, (float*)k_pool, (float*)v_pool, *sb, rope_cos, rope_sin, rot_pairs,
        heads, kv_heads, dim, v_dim, eps, unit_norm, (const float*)v_first, v_first_stride, lam, (float*)v_keep, write_cache,
        pairs, quads, q_gain, k_gain, norm_first, temp_coef, temp_every);
  else if (dtype == PTB_BF16)
    rope_norm_store_kernel<__nv_bfloat16><<<blocks, threads, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, bias, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, *sb,
        rope_cos, rope_sin, rot_pairs, heads, kv_heads, dim, v_dim, eps, unit_norm, (const __nv_bfloat16*)v_first,
        v_first_stride, lam, (__nv_bfloat16*)v_keep, write_cache, pairs, quads, q_gain, k_gain, norm_first, temp_coef,
        temp_every);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_rope_norm_store(int dtype, const void* proj, int stride, const float* bias, void* q_out, void* k_pool,
                                void* v_pool, const StepBatch* sb, const float* rope_cos, const float* rope_sin, int rot_pairs,
                                int heads, int kv_heads, int dim, int v_dim, float eps, int unit_norm, const void* v_first,
                                int v_first_stride, const float* lam, void* v_keep, int write_cache, cudaStream_t stream) {
  return ptb_qk_prepare_store(dtype, proj, stride, bias, q_out, k_pool, v_pool, sb, rope_cos, rope_sin, rot_pairs, heads,
                              kv_heads, dim, v_dim, eps, unit_norm, v_first, v_first_stride, lam, v_keep, write_cache, nullptr,
                              nullptr, 0, 0.f, 0, stream);
}

PTB_API int ptb_talk_mix(int dtype, const float* wide, const float* talk, void* out, int out_stride, int n_tokens, int heads,
                         int kv_heads, int v_dim, cudaStream_t stream) {
  if (n_tokens <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || v_dim <= 0 || out_stride < heads * v_dim) return PTB_ERR_SIZE;
  if (v_dim % 4 == 0 && aligned16(wide)) {
    const long long total = (long long)n_tokens * kv_heads * (v_dim / 4);
    const unsigned blocks = unsigned((total + 127) / 128);
    if (dtype == PTB_F32)
      talk_mix_vec_kernel<float><<<blocks, 128, 0, stream>>>(wide, talk, (float*)out, out_stride, total, heads, kv_heads, v_dim);
    else if (dtype == PTB_BF16)
      talk_mix_vec_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(wide, talk, (__nv_bfloat16*)out, out_stride, total, heads,
                                                                     kv_heads, v_dim);
    else
      return PTB_ERR_DTYPE;
    return launch_status();
  }
  const long long total = (long long)n_tokens * heads * v_dim;
  const unsigned blocks = unsigned((total + 255) / 256);
  if (dtype == PTB_F32)
    talk_mix_kernel<float><<<blocks, 256, 0, stream>>>(wide, talk, (float*)out, out_stride, total, heads, kv_heads, v_dim);
  else if (dtype == PTB_BF16)
    talk_mix_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(wide, talk, (__nv_bfloat16*)out, out_stride, total, heads,
                                                               kv_heads, v_dim);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
