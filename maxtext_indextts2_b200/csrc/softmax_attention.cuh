// Causal softmax attention with grouped key heads and rotary positions, over the paged cache and a ragged batch.
//
// For the query row at position i of page group s and query head h (key head g = h / (H / G)):
//
//   s(j)  = scale * <rot(q_h, i), rot(k_g(j), j)>        for lo <= j <= i, lo = max(0, i - window + 1) (window 0: lo = 0)
//   p(j)  = exp(s(j) - max_j s) / sum_j exp(s(j) - max_j s)
//   out_h = out_scale * sum_j p(j) v_g(j)
//
// rot(t, p) turns the channel pairs (2c, 2c + 1), c < rot_dims / 2, of a head by the angle p * rot_freq[c]; the product and its
// reduction to [-pi, pi] are formed in double (so that the angle of a late position is no worse than that of an early one),
// sine and cosine in fp32; the remaining channels pass.  A design whose values are the un-rotated keys (values_are_keys) gets the key
// projection written twice: rotated into the key pool, as projected into the value pool.
//
// Optional parts, each off when its pointer is null: a distance penalty slopes[h] * (i - j) taken off the scaled score; a sink
// (exp(sink[h]) in the denominator, with no key and no value); a gate sigmoid(gate[row, h]) on head h's output; RMS norms of the
// query and key heads before the rotation; the rotation's other pairing (i, i + rot_dims / 2); keys and values taken from the
// pools of an earlier layer (the layer then appends nothing); RMS norms over the whole query / key projection instead of head by
// head; a cap on the scaled score, cap * tanh(s / cap); and pooled blocks: beside the window's tokens a query at i sees one mean
// key / value per block of `pool` tokens that ends at or before i - window (block b = positions b pool .. b pool + pool - 1), in
// the same softmax.  The means live in pools of their own with pool_slots blocks per page, on the sequence's page map (block b in
// page b / pool_slots), and the kernels walk them as a first segment of keys before the window's tokens.
//
//   rope_append_kernel         per row: bias already in the projection; rotates q and k, writes q, appends k and v to the pages
//   qk_prepare_append_kernel   the same with the optional head norms, either pairing, and layers that append nothing
//   pool_append_kernel         per row that completes a block: the means of the block's cached keys and values into the pooled pools
//   softmax_attention_rows_kernel<T>   one CTA per (query tile of <= 16 rows of one sequence, query head); keys walked in tiles
//                              staged as fp32 in shared memory; running maximum and sum per row; everything fp32 (T is only the
//                              dtype of q, the pools and the output).  Serves float32 engines, every geometry, and decode rows.
//   softmax_attention_mma_kernel       bf16: one CTA per (query tile, key head); a warp per (query head of the group, slice of the
//                              value columns); S = Q K^T and O += P V on mma.sync m16n8k16 with fp32 accumulators, scores, running
//                              maximum and sum in fp32 registers, K / V tiles double-buffered in shared memory by cp.async through the
//                              page map.  For vdim == dim in {16, 32, 48, 64, 96, 128, 256}.
//   softmax_attention_decode_kernel    bf16, steps of single tokens: one CTA per (row, key head, chunk of eight query heads, key
//                              split) with the products TRANSPOSED (S^T = K Q^T, O^T = V^T P^T): the 16-row side of the MMA carries
//                              keys / value columns, the 8-column side the chunk's query heads, so no tensor-core row is spent on
//                              padding; when keys and values are the same rows of one pool a tile is staged once; each of the four warps takes 16 keys of every 64-key tile and the warps' partial results
//                              are merged through shared memory.
//   softmax_attention_merge_kernel     adds the key splits' partial results.
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"
#include "linear_any.cuh"
#include "window_attention_mma.cuh"     // mma_bf16_16816, cp_async_16
#include "window_attention_decode.cuh"  // cp_async_commit, cp_async_wait_pending

namespace mtx {

template <typename T>
struct RopeAppendArgs {
  const float* proj;     // [rows, ld]: q at column q_col, k at k_col, v at v_col (v_col < 0: the values are the keys)
  long long ld;
  int q_col, k_col, v_col;
  const double* rot_freq;  // [rot_dims / 2]
  T* q_out;               // [rows, H * d]
  T* k_pages;
  T* v_pages;
  const int* group;
  const int* pos;
  const int* page_map;
  int heads, kv_heads, dim, vdim, rot_dims;
  int num_pages, tokens_per_page, max_pages;
};

template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, half = d / 2, rh = a.rot_dims / 2;
  const float* row = a.proj + size_t(r) * a.ld;
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  const double dp = double(p);
  // pairs of q and of k: unit u = (head, pair)
  const int q_pairs = H * half, k_pairs = G * half;
  for (int u = tid; u < q_pairs + k_pairs; u += blockDim.x) {
    const bool is_q = u < q_pairs;
    const int v = is_q ? u : u - q_pairs, head = v / half, c = v % half;
    const float* src = row + (is_q ? a.q_col : a.k_col) + head * d + 2 * c;
    float x0 = src[0], x1 = src[1];
    if (c < rh) {
      float sn, cs;
      const double ang = dp * a.rot_freq[c];
      sincosf(float(ang - 6.283185307179586 * rint(ang * 0.15915494309189535)), &sn, &cs);
      const float y0 = x0 * cs - x1 * sn, y1 = x1 * cs + x0 * sn;
      x0 = y0;
      x1 = y1;
    }
    T* dst = is_q ? a.q_out + size_t(r) * H * d + head * d + 2 * c
                  : a.k_pages + (size_t(head) * a.num_pages * a.tokens_per_page + slot) * d + 2 * c;
    dst[0] = to_act<T>(x0);
    dst[1] = to_act<T>(x1);
  }
  if (d & 1) {  // an odd last channel is never rotated
    for (int u = tid; u < H + G; u += blockDim.x) {
      const bool is_q = u < H;
      const int head = is_q ? u : u - H;
      const float x = row[(is_q ? a.q_col : a.k_col) + head * d + d - 1];
      if (is_q) a.q_out[size_t(r) * H * d + head * d + d - 1] = to_act<T>(x);
      else a.k_pages[(size_t(head) * a.num_pages * a.tokens_per_page + slot) * d + d - 1] = to_act<T>(x);
    }
  }
  const int vsrc = a.v_col < 0 ? a.k_col : a.v_col;
  for (int e = tid; e < G * dv; e += blockDim.x) {
    const int kv = e / dv, c = e % dv;
    a.v_pages[(size_t(kv) * a.num_pages * a.tokens_per_page + slot) * dv + c] = to_act<T>(row[vsrc + e]);
  }
}

template <typename T>
struct QkPrepareArgs {
  const float* proj;     // [rows, ld]: q at column q_col, k at k_col, v at v_col
  long long ld;
  int q_col, k_col, v_col;
  const float* q_norm;   // [d] or null
  const float* k_norm;   // [d] or null
  const double* rot_freq;  // [rot_dims / 2] (rot_dims == 0: null)
  T* q_out;              // [rows, H * d]
  T* k_pages;
  T* v_pages;
  const int* group;
  const int* pos;
  const int* page_map;
  int heads, kv_heads, dim, vdim, rot_dims, rot_half, shared_kv;
  int num_pages, tokens_per_page, max_pages;
  float eps;
  int norm_whole;        // 1: q_norm [H * d] / k_norm [G * d]: the whole projection is brought to unit RMS at once
};

// angle of channel pair c at position p, reduced to [-pi, pi] in double before the fp32 sine and cosine
__device__ __forceinline__ void rot_sincos(double p, double freq, float* sn, float* cs) {
  const double ang = p * freq;
  sincosf(float(ang - 6.283185307179586 * rint(ang * 0.15915494309189535)), sn, cs);
}

// one CTA per row, a warp per head (query heads, then key heads): norm, rotation, write; then the values
template <typename T>
__global__ void __launch_bounds__(256) qk_prepare_append_kernel(const QkPrepareArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  const int H = a.heads, G = a.shared_kv ? 0 : a.kv_heads, d = a.dim, dv = a.vdim, rh = a.rot_dims / 2;
  const float* row = a.proj + size_t(r) * a.ld;
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  const double dp = double(p);
  float inv_all[2] = {1.0f, 1.0f};  // norm_whole: of the query / the key projection
  if (a.norm_whole) {
    __shared__ float red[8];
    for (int which = 0; which < 2; ++which) {
      const int n = which == 0 ? H * d : G * d;
      if (n == 0 || !(which == 0 ? a.q_norm : a.k_norm)) continue;
      const float* src = row + (which == 0 ? a.q_col : a.k_col);
      float ss = 0.0f;
      for (int c = tid; c < n; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
      inv_all[which] = 1.0f / sqrtf(block_sum(ss, red) / float(n) + a.eps);
    }
  }
  for (int u = warp; u < H + G; u += nw) {
    const bool is_q = u < H;
    const float* src = row + (is_q ? a.q_col + u * d : a.k_col + (u - H) * d);
    const float* w = is_q ? a.q_norm : a.k_norm;
    float inv = 1.0f;
    if (w && a.norm_whole) {
      inv = inv_all[is_q ? 0 : 1];
      w += (is_q ? u : u - H) * d;
    } else if (w) {
      float ss = 0.0f;
      for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / float(d) + a.eps);
    }
    T* dst = is_q ? a.q_out + size_t(r) * H * d + u * d : a.k_pages + (size_t(u - H) * a.num_pages * a.tokens_per_page + slot) * d;
    auto val = [&](int c) { return w ? src[c] * inv * w[c] : src[c]; };
    for (int i = lane; i < rh; i += 32) {  // the pairs that turn
      const int c0 = a.rot_half ? i : 2 * i, c1 = a.rot_half ? i + rh : 2 * i + 1;
      float sn, cs;
      rot_sincos(dp, a.rot_freq[i], &sn, &cs);
      const float x0 = val(c0), x1 = val(c1);
      dst[c0] = to_act<T>(x0 * cs - x1 * sn);
      dst[c1] = to_act<T>(x1 * cs + x0 * sn);
    }
    for (int c = 2 * rh + lane; c < d; c += 32) dst[c] = to_act<T>(val(c));
  }
  if (a.shared_kv) return;
  for (int e = tid; e < G * dv; e += blockDim.x) {
    const int kv = e / dv, c = e % dv;
    a.v_pages[(size_t(kv) * a.num_pages * a.tokens_per_page + slot) * dv + c] = to_act<T>(row[a.v_col + e]);
  }
}

template <typename T>
struct PoolAppendArgs {
  const T* k_pages;
  const T* v_pages;
  T* kp_pages;  // [G, num_pages, pool_slots, d]
  T* vp_pages;  // [G, num_pages, pool_slots, dv]
  const int* group;
  const int* pos;
  const int* page_map;
  int kv_heads, dim, vdim, pool, pool_slots;
  int num_pages, tokens_per_page, max_pages;
};

// one CTA per row; the row whose position ends a block of `pool` tokens adds the block's cached keys and values up in order of
// position (fp32) and writes their means; every other CTA leaves at once
template <typename T>
__global__ void __launch_bounds__(256) pool_append_kernel(const PoolAppendArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, p = a.pos[r], P = a.pool;
  if ((p + 1) % P != 0) return;
  const int b = p / P, d = a.dim, dv = a.vdim, G = a.kv_heads, tpp = a.tokens_per_page;
  const int* pages = a.page_map + size_t(a.group[r]) * a.max_pages;
  const size_t dst = size_t(pages[b / a.pool_slots]) * a.pool_slots + b % a.pool_slots;
  const float inv = 1.0f / float(P);
  for (int e = threadIdx.x; e < G * (d + dv); e += blockDim.x) {
    const bool is_k = e < G * d;
    const int f = is_k ? e : e - G * d, w = is_k ? d : dv, kv = f / w, c = f % w;
    const T* src = is_k ? a.k_pages : a.v_pages;
    float acc = 0.0f;
    for (int j = b * P; j <= p; ++j) {
      const size_t row = size_t(kv) * a.num_pages * tpp + size_t(pages[j / tpp]) * tpp + j % tpp;
      acc += act_f32(src[row * w + c]);
    }
    T* out = is_k ? a.kp_pages : a.vp_pages;
    out[(size_t(kv) * a.num_pages * a.pool_slots + dst) * w + c] = to_act<T>(acc * inv);
  }
}

template <typename T>
struct SoftmaxAttnArgs {
  const T* q;            // [rows, H * d]
  T* out;                // [rows, ld_out]; head h writes columns [h * dv, (h + 1) * dv)
  long long ld_out;
  const T* k_pages;
  const T* v_pages;
  const int* group;
  const int* pos;
  const int* page_map;
  const int* tile_row0;  // [n_tiles + 1]
  int heads, kv_heads, dim, vdim, window;
  int num_pages, tokens_per_page, max_pages;
  float scale, out_scale;
  // key splits of the tensor-core arm (splits > 1: blockIdx.z walks every splits-th part of the key tiles and leaves an
  // unnormalised partial result; softmax_attention_merge_kernel adds the parts)
  int splits, rows;
  float* part_o;   // [splits, rows, H, dv]
  float* part_ml;  // [splits, rows, H, 2]: running maximum, sum
  // optional parts (null: none)
  const float* slopes;  // [H]: slopes[h] * (i - j) is taken off the scaled score
  const float* sink;    // [H]: exp(sink[h]) joins the denominator (it enters the first key split's running maximum and sum)
  const float* gate;    // [rows, ld_gate]: head h's output is multiplied by sigmoid(gate[row, h])
  long long ld_gate;
  float softcap;        // > 0: the scaled score becomes softcap * tanh(score / softcap)
  int pool, pool_slots; // pool > 0: pooled blocks (see the head of this file); needs window > 0
  const T* kp_pages;    // [G, num_pages, pool_slots, d]
  const T* vp_pages;    // [G, num_pages, pool_slots, dv]
};

// blocks of `pool` tokens that the query at position i sees: those that end at or before i - window
__device__ __forceinline__ int smax_blocks_seen(int i, int window, int pool) {
  const int past = i - window + 1;  // tokens before the window
  return (pool > 0 && past > 0) ? past / pool : 0;
}

__device__ __forceinline__ float smax_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float smax_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// cap * tanh(raw * scale / cap) = cap - 2 cap / (1 + 2^(raw * mul)) with mul = scale * 2 log2(e) / cap: one multiplication, two
// special-function instructions and a fused multiply-add per score; absolute error of a few 1e-7 * cap
__device__ __forceinline__ float smax_softcap_scaled(float raw, float mul, float cap) {
  return fmaf(-2.0f * cap, smax_rcp(1.0f + smax_ex2(raw * mul)), cap);
}

__device__ __forceinline__ float smax_gate(const float* gate, long long ld, int row, int h) {
  return gate ? 1.0f / (1.0f + expf(-gate[size_t(row) * ld + h])) : 1.0f;
}

constexpr int kSmaxThreads = 256, kSmaxRows = 16, kSmaxKeys = 32;
constexpr int kSmaxMaxAcc = 32;  // kSmaxRows * vdim <= kSmaxThreads * kSmaxMaxAcc: vdim <= 512

inline size_t softmax_attn_smem_bytes(int dim, int vdim) {
  return sizeof(float) * (size_t(kSmaxRows) * dim + size_t(kSmaxKeys) * (dim + 1) + size_t(kSmaxKeys) * vdim + size_t(kSmaxRows) * kSmaxKeys +
                          3 * kSmaxRows);
}

template <typename T>
__global__ void __launch_bounds__(kSmaxThreads) softmax_attention_rows_kernel(const SoftmaxAttnArgs<T> a) {
  extern __shared__ float smem[];
  const int d = a.dim, dv = a.vdim, rep = a.heads / a.kv_heads;
  float* sq = smem;                        // [16][d]
  float* sk = sq + kSmaxRows * d;          // [32][d + 1]
  float* sv = sk + kSmaxKeys * (d + 1);    // [32][dv]
  float* sp = sv + kSmaxKeys * dv;         // [16][32]
  float* s_max = sp + kSmaxRows * kSmaxKeys;  // [16] running maximum
  float* s_sum = s_max + kSmaxRows;           // [16] running sum
  float* s_fix = s_sum + kSmaxRows;           // [16] factor that brings the old accumulators to the new maximum
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  griddep_wait();
  const int r0 = a.tile_row0[blockIdx.x], nr = a.tile_row0[blockIdx.x + 1] - r0, h = blockIdx.y, g = h / rep;
  const int p0 = a.pos[r0], grp = a.group[r0];  // row r0 + i has position p0 + i
  const int p_last = p0 + nr - 1;
  int lo = 0;
  if (a.window > 0 && p0 - a.window + 1 > 0) lo = p0 - a.window + 1;
  for (int e = tid; e < nr * d; e += kSmaxThreads) sq[e] = act_f32(a.q[size_t(r0 + e / d) * a.heads * d + h * d + e % d]) * a.scale;
  if (tid < kSmaxRows) {
    s_max[tid] = a.sink ? a.sink[h] : -INFINITY;
    s_sum[tid] = a.sink ? 1.0f : 0.0f;
  }
  const float slope = a.slopes ? a.slopes[h] : 0.0f;
  float acc[kSmaxMaxAcc];
#pragma unroll
  for (int u = 0; u < kSmaxMaxAcc; ++u) acc[u] = 0.0f;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  const int nb_last = smax_blocks_seen(p_last, a.window, a.pool);
  // two segments of keys: the pooled blocks 0 .. nb_last - 1 (if any), then the tokens lo .. p_last
  for (int seg = nb_last > 0 ? 0 : 1; seg < 2; ++seg) {
  const bool pooled = seg == 0;
  const int begin = pooled ? 0 : lo, end = pooled ? nb_last - 1 : p_last, tpp = pooled ? a.pool_slots : a.tokens_per_page;
  const T* kpool = pooled ? a.kp_pages : a.k_pages;
  const T* vpool = pooled ? a.vp_pages : a.v_pages;
  const size_t head_rows = size_t(g) * a.num_pages * tpp;
  for (int j0 = begin; j0 <= end; j0 += kSmaxKeys) {
    const int nk = end - j0 + 1 < kSmaxKeys ? end - j0 + 1 : kSmaxKeys;
    __syncthreads();
    for (int e = tid; e < nk * d; e += kSmaxThreads) {
      const int jj = e / d, c = e % d, j = j0 + jj;
      const size_t row = head_rows + size_t(pages[j / tpp]) * tpp + j % tpp;
      sk[jj * (d + 1) + c] = act_f32(kpool[row * d + c]);
    }
    for (int e = tid; e < nk * dv; e += kSmaxThreads) {
      const int jj = e / dv, c = e % dv, j = j0 + jj;
      const size_t row = head_rows + size_t(pages[j / tpp]) * tpp + j % tpp;
      sv[jj * dv + c] = act_f32(vpool[row * dv + c]);
    }
    __syncthreads();
    for (int e = tid; e < nr * kSmaxKeys; e += kSmaxThreads) {
      const int i = e / kSmaxKeys, jj = e % kSmaxKeys, j = j0 + jj, pi = p0 + i;
      float s = -INFINITY;
      const bool seen = pooled ? j < smax_blocks_seen(pi, a.window, a.pool) : (j <= pi && (a.window <= 0 || pi - j < a.window));
      if (jj < nk && seen) {
        const float* qv = sq + i * d;
        const float* kv = sk + jj * (d + 1);
        s = 0.0f;
        for (int c = 0; c < d; ++c) s = fmaf(qv[c], kv[c], s);
        if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
        if (!pooled) s -= slope * float(pi - j);
      }
      sp[e] = s;
    }
    __syncthreads();
    for (int i = warp; i < nr; i += kSmaxThreads / 32) {  // kSmaxKeys == 32: one key per lane
      const float s = sp[i * kSmaxKeys + lane];
      float m = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float m_old = s_max[i], m_new = fmaxf(m_old, m);
      const float p = (m_new == -INFINITY || s == -INFINITY) ? 0.0f : expf(s - m_new);
      const float fix = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
      const float sum = warp_sum(p);
      sp[i * kSmaxKeys + lane] = p;
      if (lane == 0) {
        s_max[i] = m_new;
        s_sum[i] = s_sum[i] * fix + sum;
        s_fix[i] = fix;
      }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kSmaxMaxAcc; ++u) {
      const int o = tid + u * kSmaxThreads;
      if (o < nr * dv) {
        const int i = o / dv, c = o % dv;
        const float* pv = sp + i * kSmaxKeys;
        float s = acc[u] * s_fix[i];
        for (int jj = 0; jj < nk; ++jj) s = fmaf(pv[jj], sv[jj * dv + c], s);
        acc[u] = s;
      }
    }
  }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < kSmaxMaxAcc; ++u) {
    const int o = tid + u * kSmaxThreads;
    if (o < nr * dv) {
      const int i = o / dv, c = o % dv;
      a.out[size_t(r0 + i) * a.ld_out + h * dv + c] = to_act<T>(acc[u] * a.out_scale / s_sum[i] * smax_gate(a.gate, a.ld_gate, r0 + i, h));
    }
  }
}

// ---- bf16 tensor-core arm ------------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smax_pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct SoftmaxMmaPlan {
  bool ok;
  int d16, parts, key_tile, warps, chunks;  // chunks: CTAs per (tile, key head), each with `warps` warps
  size_t smem;
};

// D16 = dim / 16 (vdim == dim); PARTS = slices of the value columns, a warp each (keeps the output accumulators in registers)
inline SoftmaxMmaPlan softmax_mma_plan(int heads, int kv_heads, int dim, int vdim) {
  SoftmaxMmaPlan p = {false, 0, 1, 64, 1, 1, 0};
  if (dim != vdim || dim % 16 != 0) return p;
  const int d16 = dim / 16;
  if (!(d16 == 1 || d16 == 2 || d16 == 3 || d16 == 4 || d16 == 6 || d16 == 8 || d16 == 16)) return p;
  p.ok = true;
  p.d16 = d16;
  p.parts = d16 == 16 ? 2 : 1;
  p.key_tile = d16 == 16 ? 32 : 64;
  const int units = (heads / kv_heads) * p.parts;  // warps' worth of work per (tile, key head)
  p.warps = units < 4 ? units : 4;
  p.chunks = (units + p.warps - 1) / p.warps;
  p.smem = size_t(2) * p.key_tile * 2 * (dim + 8) * sizeof(bf16);
  return p;
}

template <int D16, int PARTS, int KT>
__global__ void __launch_bounds__(128) softmax_attention_mma_kernel(const SoftmaxAttnArgs<bf16> a, int chunks) {
  extern __shared__ __align__(16) unsigned char smax_raw[];
  constexpr int D = 16 * D16, PITCH = D + 8, DVW = D / PARTS, NB = DVW / 8;  // NB: 8-column blocks of a warp's output
  bf16* const stage0 = reinterpret_cast<bf16*>(smax_raw);                     // stage s: K [KT][PITCH], then V [KT][PITCH]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3, nthreads = blockDim.x, nwarps = nthreads >> 5;
  griddep_wait();
  const int rep = a.heads / a.kv_heads;
  const int kvh = blockIdx.y / chunks, unit = (blockIdx.y % chunks) * nwarps + warp;  // unit = (head of the group, part)
  const bool active = unit < rep * PARTS;
  const int h = kvh * rep + (active ? unit / PARTS : 0), part = active ? unit % PARTS : 0;
  const int r0 = a.tile_row0[blockIdx.x], nr = a.tile_row0[blockIdx.x + 1] - r0;
  const int p0 = a.pos[r0], grp = a.group[r0], p_last = p0 + nr - 1;
  int lo = 0;
  if (a.window > 0 && p0 - a.window + 1 > 0) lo = p0 - a.window + 1;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  const size_t head_rows = size_t(kvh) * a.num_pages * a.tokens_per_page;
  const int page_shift = (a.tokens_per_page & (a.tokens_per_page - 1)) == 0 ? __ffs(a.tokens_per_page) - 1 : -1;  // pages of 2^n tokens: no division per key
  // the key tiles: first those of the pooled blocks 0 .. nb_last - 1 (if any), then those of the tokens lo .. p_last
  const int nb_last = smax_blocks_seen(p_last, a.window, a.pool), pool_tiles = (nb_last + KT - 1) / KT;
  const int pool_shift = (a.pool_slots & (a.pool_slots - 1)) == 0 && a.pool_slots > 0 ? __ffs(a.pool_slots) - 1 : -1;
  const size_t pool_head_rows = size_t(kvh) * a.num_pages * a.pool_slots;
  const int all_key_tiles = pool_tiles + (p_last - lo) / KT + 1;
  int tile_lo = 0, n_key_tiles = all_key_tiles;
  if (a.splits > 1) {
    const int per = (all_key_tiles + a.splits - 1) / a.splits;
    tile_lo = int(blockIdx.z) * per;
    n_key_tiles = all_key_tiles - tile_lo < per ? all_key_tiles - tile_lo : per;
    if (n_key_tiles < 0) n_key_tiles = 0;
  }

  const bool same_kv = a.k_pages == a.v_pages;  // the values are the cached keys' rows themselves: one copy of a tile serves both
  auto load_tile = [&](int it, int stage) {
    bf16* sk = stage0 + size_t(stage) * 2 * KT * PITCH;
    bf16* sv = sk + KT * PITCH;
    const int gt = tile_lo + it;
    const bool pooled = gt < pool_tiles;
    const int j0 = pooled ? gt * KT : lo + (gt - pool_tiles) * KT, last = pooled ? nb_last - 1 : p_last;
    const int tpp = pooled ? a.pool_slots : a.tokens_per_page, shift = pooled ? pool_shift : page_shift;
    const size_t hr = pooled ? pool_head_rows : head_rows;
    const bf16* kpool = pooled ? a.kp_pages : a.k_pages;
    const bf16* vpool = pooled ? a.vp_pages : a.v_pages;
    constexpr int CH = D / 8;  // 16-byte chunks per row
    for (int e = tid; e < KT * CH; e += nthreads) {
      const int jj = e / CH, c = e % CH, j = j0 + jj;
      const bool ok = j <= last;
      const int pg = shift >= 0 ? (j >> shift) : j / tpp;
      const size_t row = ok ? hr + size_t(pages[pg]) * tpp + (j - pg * tpp) : 0;
      cp_async_16(sk + jj * PITCH + c * 8, kpool + row * D + c * 8, ok);
      if (!same_kv) cp_async_16(sv + jj * PITCH + c * 8, vpool + row * D + c * 8, ok);
    }
    cp_async_commit();
  };

  // Q fragments of rows g and g + 8 (rows beyond the tile: zero)
  uint32_t qf[D16][4];
  {
    const bf16* q0 = a.q + size_t(r0 + g) * a.heads * D + h * D;
    const bf16* q1 = q0 + size_t(8) * a.heads * D;
    const bool ok0 = active && g < nr, ok1 = active && g + 8 < nr;
#pragma unroll
    for (int kk = 0; kk < D16; ++kk) {
      qf[kk][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 2 * t) : 0u;
      qf[kk][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 2 * t) : 0u;
      qf[kk][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + 2 * t) : 0u;
      qf[kk][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + 2 * t) : 0u;
    }
  }
  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  if (a.sink && blockIdx.z == 0) {  // (the four lanes of a row are added at the end: lane t == 0 carries the sink's 1)
    m_run[0] = m_run[1] = a.sink[h];
    l_run[0] = l_run[1] = t == 0 ? 1.0f : 0.0f;
  }
  const float slope = a.slopes ? a.slopes[h] : 0.0f;
  const int pi0 = p0 + g, pi1 = p0 + g + 8;
  const int nb0 = smax_blocks_seen(pi0, a.window, a.pool), nb1 = smax_blocks_seen(pi1, a.window, a.pool);
  const int nb_first = smax_blocks_seen(p0, a.window, a.pool);
  const bool capped = a.softcap > 0.0f, sloped = a.slopes != nullptr;
  const float cap_mul = capped ? a.scale * 2.8853900817779268f / a.softcap : 0.0f;

  if (n_key_tiles > 0) load_tile(0, 0);
  for (int it = 0; it < n_key_tiles; ++it) {
    if (it + 1 < n_key_tiles) {
      load_tile(it + 1, (it + 1) & 1);
      cp_async_wait_pending(1);
    } else {
      cp_async_wait_pending(0);
    }
    __syncthreads();
    if (active) {
      const bf16* sk = stage0 + size_t(it & 1) * 2 * KT * PITCH;
      const bf16* sv = same_kv ? sk : sk + KT * PITCH;
      const int gt = tile_lo + it;
      const bool pooled = gt < pool_tiles;
      const int j0 = pooled ? gt * KT : lo + (gt - pool_tiles) * KT;
      // a tile whose every key every row of the query tile sees (most tiles of a long window) needs no masks
      const bool every_key_seen = pooled ? j0 + KT <= nb_first : (j0 + KT - 1 <= p0 && (a.window <= 0 || p_last - j0 < a.window));
      float s[KT / 8][4];
#pragma unroll
      for (int nb = 0; nb < KT / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nb][e] = 0.0f;
        const bf16* kr = sk + (nb * 8 + g) * PITCH + 2 * t;
#pragma unroll
        for (int kk = 0; kk < D16; ++kk)
          mma_bf16_16816(s[nb], qf[kk], *reinterpret_cast<const uint32_t*>(kr + kk * 16), *reinterpret_cast<const uint32_t*>(kr + kk * 16 + 8));
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < KT / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float sc = capped ? smax_softcap_scaled(s[nb][e], cap_mul, a.softcap) : s[nb][e] * a.scale;
          if (!every_key_seen || (sloped && !pooled)) {
            const int j = j0 + nb * 8 + 2 * t + (e & 1), pi = (e & 2) ? pi1 : pi0;
            const bool seen = pooled ? j < ((e & 2) ? nb1 : nb0) : (j <= pi && (a.window <= 0 || pi - j < a.window));
            if (sloped && !pooled) sc -= slope * float(pi - j);
            sc = seen ? sc : -INFINITY;
          }
          s[nb][e] = sc;
        }
        mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;
      const float fix0 = __expf(m_run[0] - base0), fix1 = __expf(m_run[1] - base1);  // (exp(-inf) = 0 while a row has seen no key)
      m_run[0] = mn0;
      m_run[1] = mn1;
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int nb = 0; nb < KT / 8; ++nb) {
        s[nb][0] = __expf(s[nb][0] - base0);
        s[nb][1] = __expf(s[nb][1] - base0);
        s[nb][2] = __expf(s[nb][2] - base1);
        s[nb][3] = __expf(s[nb][3] - base1);
        sum0 += s[nb][0] + s[nb][1];
        sum1 += s[nb][2] + s[nb][3];
      }
      l_run[0] = l_run[0] * fix0 + sum0;  // (per-thread partial sums; the four lanes of a row are added at the end)
      l_run[1] = l_run[1] * fix1 + sum1;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        o[nb][0] *= fix0;
        o[nb][1] *= fix0;
        o[nb][2] *= fix1;
        o[nb][3] *= fix1;
      }
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t pf[4];
        pf[0] = smax_pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[1] = smax_pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[2] = smax_pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[3] = smax_pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        // V [key][column] -> the B fragments of two 8-column blocks at once: lanes 0-15 name the 16 key rows of the first block,
        // lanes 16-31 those of the second
        const bf16* vrow = sv + (kk * 16 + (lane & 15)) * PITCH + part * DVW + (lane >> 4) * 8;
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
          uint32_t b0, b1, b2, b3;
          const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(vrow + nb * 8));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
          mma_bf16_16816(o[nb], pf, b0, b1);
          mma_bf16_16816(o[nb + 1], pf, b2, b3);
        }
      }
    }
    __syncthreads();  // the stage is free for the load after next
  }
  if (!active) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (a.splits > 1) {
    const size_t base0 = (size_t(blockIdx.z) * a.rows + r0 + g) * a.heads + h, base1 = base0 + size_t(8) * a.heads;
    if (g < nr && t == 0 && part == 0) {
      a.part_ml[base0 * 2] = m_run[0];
      a.part_ml[base0 * 2 + 1] = l_run[0];
    }
    if (g + 8 < nr && t == 0 && part == 0) {
      a.part_ml[base1 * 2] = m_run[1];
      a.part_ml[base1 * 2 + 1] = l_run[1];
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int col = part * DVW + nb * 8 + 2 * t;
      if (g < nr) *reinterpret_cast<float2*>(a.part_o + base0 * D + col) = make_float2(o[nb][0], o[nb][1]);
      if (g + 8 < nr) *reinterpret_cast<float2*>(a.part_o + base1 * D + col) = make_float2(o[nb][2], o[nb][3]);
    }
    return;
  }
  const float f0 = a.out_scale / l_run[0] * (g < nr ? smax_gate(a.gate, a.ld_gate, r0 + g, h) : 1.0f);
  const float f1 = a.out_scale / l_run[1] * (g + 8 < nr ? smax_gate(a.gate, a.ld_gate, r0 + g + 8, h) : 1.0f);
  bf16* out0 = a.out + size_t(r0 + g) * a.ld_out + h * D + part * DVW + 2 * t;
  bf16* out1 = out0 + size_t(8) * a.ld_out;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    if (g < nr) *reinterpret_cast<uint32_t*>(out0 + nb * 8) = smax_pack_bf16(o[nb][0] * f0, o[nb][1] * f0);
    if (g + 8 < nr) *reinterpret_cast<uint32_t*>(out1 + nb * 8) = smax_pack_bf16(o[nb][2] * f1, o[nb][3] * f1);
  }
}

// ---- bf16, single-token rows: transposed products ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smax_movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

constexpr int kSdecWarps = 4, kSdecKeys = 64;

// (same_kv: keys and values are the same rows of one pool, so a tile is staged once)
inline size_t softmax_decode_smem_bytes(int dim, bool same_kv = false) {
  const size_t ring = size_t(2) * kSdecKeys * (same_kv ? 1 : 2) * (dim + 8) * sizeof(bf16), merge = sizeof(float) * kSdecWarps * (8 * size_t(dim) + 16);
  return ring > merge ? ring : merge;
}

template <int D16>
__global__ void __launch_bounds__(kSdecWarps * 32) softmax_attention_decode_kernel(const SoftmaxAttnArgs<bf16> a) {
  extern __shared__ __align__(16) unsigned char sdec_raw[];
  constexpr int D = 16 * D16, PITCH = D + 8, KT = kSdecKeys, NT = kSdecWarps * 32;
  bf16* const stage0 = reinterpret_cast<bf16*>(sdec_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  griddep_wait();
  // a key head's query heads in chunks of eight (the MMA's 8-column side): blockIdx.y = (key head, chunk)
  const int rep_all = a.heads / a.kv_heads, chunks = (rep_all + 7) / 8;
  const int row = blockIdx.x, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int rep = rep_all - chunk * 8 < 8 ? rep_all - chunk * 8 : 8, head0 = kvh * rep_all + chunk * 8;
  const bool same_kv = a.k_pages == a.v_pages;  // the values are the cached keys' rows themselves: one copy of a tile serves both
  const int stage_elems = (same_kv ? 1 : 2) * KT * PITCH;
  const int pos = a.pos[row], grp = a.group[row];
  int lo = 0;
  if (a.window > 0 && pos - a.window + 1 > 0) lo = pos - a.window + 1;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  const size_t head_rows = size_t(kvh) * a.num_pages * a.tokens_per_page;
  const int page_shift = (a.tokens_per_page & (a.tokens_per_page - 1)) == 0 ? __ffs(a.tokens_per_page) - 1 : -1;  // pages of 2^n tokens: no division per key
  // the key tiles: first those of the pooled blocks 0 .. nb - 1 (if any), then those of the tokens lo .. pos
  const int nb = smax_blocks_seen(pos, a.window, a.pool), pool_tiles = (nb + KT - 1) / KT;
  const int pool_shift = (a.pool_slots & (a.pool_slots - 1)) == 0 && a.pool_slots > 0 ? __ffs(a.pool_slots) - 1 : -1;
  const size_t pool_head_rows = size_t(kvh) * a.num_pages * a.pool_slots;
  const int all_key_tiles = pool_tiles + (pos - lo) / KT + 1;
  const int per = (all_key_tiles + a.splits - 1) / a.splits;
  const int tile_lo = int(blockIdx.z) * per;
  int n_key_tiles = all_key_tiles - tile_lo < per ? all_key_tiles - tile_lo : per;
  if (n_key_tiles < 0) n_key_tiles = 0;

  auto load_tile = [&](int it, int stage) {
    bf16* sk = stage0 + size_t(stage) * stage_elems;
    bf16* sv = sk + KT * PITCH;
    const int gt = tile_lo + it;
    const bool pooled = gt < pool_tiles;
    const int j0 = pooled ? gt * KT : lo + (gt - pool_tiles) * KT, last = pooled ? nb - 1 : pos;
    const int tpp = pooled ? a.pool_slots : a.tokens_per_page, shift = pooled ? pool_shift : page_shift;
    const size_t hr = pooled ? pool_head_rows : head_rows;
    const bf16* kpool = pooled ? a.kp_pages : a.k_pages;
    const bf16* vpool = pooled ? a.vp_pages : a.v_pages;
    constexpr int CH = D / 8;
    for (int e = tid; e < KT * CH; e += NT) {
      const int jj = e / CH, c = e % CH, j = j0 + jj;
      const bool ok = j <= last;
      const int pg = shift >= 0 ? (j >> shift) : j / tpp;
      const size_t r = ok ? hr + size_t(pages[pg]) * tpp + (j - pg * tpp) : 0;
      cp_async_16(sk + jj * PITCH + c * 8, kpool + r * D + c * 8, ok);
      if (!same_kv) cp_async_16(sv + jj * PITCH + c * 8, vpool + r * D + c * 8, ok);
    }
    cp_async_commit();
  };

  // the group's queries as the B operand: lane (g, t) holds head g's channels kk * 16 + 2t, + 1 and + 8 + 2t, + 9
  uint32_t qf[D16][2];
  {
    const bf16* q = a.q + size_t(row) * a.heads * D + (head0 + (g < rep ? g : 0)) * D;
#pragma unroll
    for (int kk = 0; kk < D16; ++kk) {
      qf[kk][0] = g < rep ? *reinterpret_cast<const uint32_t*>(q + kk * 16 + 2 * t) : 0u;
      qf[kk][1] = g < rep ? *reinterpret_cast<const uint32_t*>(q + kk * 16 + 8 + 2 * t) : 0u;
    }
  }
  float o[D16][4];  // O^T: (column mb * 16 + g / g + 8, head 2t / 2t + 1)
#pragma unroll
  for (int mb = 0; mb < D16; ++mb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[mb][e] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // heads 2t, 2t + 1
  const float cap_mul = a.softcap > 0.0f ? a.scale * 2.8853900817779268f / a.softcap : 0.0f;
  float slope0 = 0.0f, slope1 = 0.0f;
  if (a.slopes) {
    slope0 = 2 * t < rep ? a.slopes[head0 + 2 * t] : 0.0f;
    slope1 = 2 * t + 1 < rep ? a.slopes[head0 + 2 * t + 1] : 0.0f;
  }
  if (a.sink && warp == 0 && blockIdx.z == 0) {  // (the first warp of the first split carries the sink; its eight lanes of a head are added at the end)
    if (2 * t < rep) m_run[0] = a.sink[head0 + 2 * t], l_run[0] = g == 0 ? 1.0f : 0.0f;
    if (2 * t + 1 < rep) m_run[1] = a.sink[head0 + 2 * t + 1], l_run[1] = g == 0 ? 1.0f : 0.0f;
  }

  if (n_key_tiles > 0) load_tile(0, 0);
  for (int it = 0; it < n_key_tiles; ++it) {
    if (it + 1 < n_key_tiles) {
      load_tile(it + 1, (it + 1) & 1);
      cp_async_wait_pending(1);
    } else {
      cp_async_wait_pending(0);
    }
    __syncthreads();
    const bf16* sk = stage0 + size_t(it & 1) * stage_elems;
    const bf16* sv = same_kv ? sk : sk + KT * PITCH;
    const int gt = tile_lo + it;
    const bool pooled = gt < pool_tiles;
    const int j0 = (pooled ? gt * KT : lo + (gt - pool_tiles) * KT) + warp * 16;  // this warp's 16 keys
    if (j0 <= (pooled ? nb - 1 : pos)) {
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const bf16* k0 = sk + (warp * 16 + g) * PITCH + 2 * t;
#pragma unroll
      for (int kk = 0; kk < D16; ++kk) {
        uint32_t af[4];
        af[0] = *reinterpret_cast<const uint32_t*>(k0 + kk * 16);
        af[1] = *reinterpret_cast<const uint32_t*>(k0 + 8 * PITCH + kk * 16);
        af[2] = *reinterpret_cast<const uint32_t*>(k0 + kk * 16 + 8);
        af[3] = *reinterpret_cast<const uint32_t*>(k0 + 8 * PITCH + kk * 16 + 8);
        mma_bf16_16816(c, af, qf[kk][0], qf[kk][1]);
      }
      // c[0], c[1]: key j0 + g, heads 2t, 2t + 1;  c[2], c[3]: key j0 + g + 8
      const int ja = j0 + g, jb = j0 + g + 8;
      const bool sa_ = pooled ? ja < nb : (ja <= pos && (a.window <= 0 || pos - ja < a.window));
      const bool sb_ = pooled ? jb < nb : (jb <= pos && (a.window <= 0 || pos - jb < a.window));
#pragma unroll
      for (int e = 0; e < 4; ++e) c[e] = a.softcap > 0.0f ? smax_softcap_scaled(c[e], cap_mul, a.softcap) : c[e] * a.scale;
      const float da = pooled ? 0.0f : float(pos - ja), db = pooled ? 0.0f : float(pos - jb);
      c[0] = sa_ ? c[0] - slope0 * da : -INFINITY;
      c[1] = sa_ ? c[1] - slope1 * da : -INFINITY;
      c[2] = sb_ ? c[2] - slope0 * db : -INFINITY;
      c[3] = sb_ ? c[3] - slope1 * db : -INFINITY;
      float mx0 = fmaxf(c[0], c[2]), mx1 = fmaxf(c[1], c[3]);
#pragma unroll
      for (int sh = 4; sh < 32; sh <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float b0 = mn0 == -INFINITY ? 0.0f : mn0, b1 = mn1 == -INFINITY ? 0.0f : mn1;
      const float fix0 = __expf(m_run[0] - b0), fix1 = __expf(m_run[1] - b1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      c[0] = __expf(c[0] - b0);
      c[1] = __expf(c[1] - b1);
      c[2] = __expf(c[2] - b0);
      c[3] = __expf(c[3] - b1);
      l_run[0] = l_run[0] * fix0 + c[0] + c[2];  // (this lane's keys; the eight lanes of a head are added at the end)
      l_run[1] = l_run[1] * fix1 + c[1] + c[3];
      const uint32_t pb0 = smax_movmatrix_trans(smax_pack_bf16(c[0], c[1])), pb1 = smax_movmatrix_trans(smax_pack_bf16(c[2], c[3]));
      // V^T as the A operand: four 8 x 8 blocks (keys 0-7 / 8-15) x (columns 0-7 / 8-15) of the warp's 16 keys, transposed on load
      const bf16* v0 = sv + (warp * 16 + (lane & 7) + 8 * (lane >> 4)) * PITCH + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int mb = 0; mb < D16; ++mb) {
        uint32_t vf[4];
        const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(v0 + mb * 16));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(vf[0]), "=r"(vf[1]), "=r"(vf[2]), "=r"(vf[3]) : "r"(addr));
        o[mb][0] *= fix0;
        o[mb][1] *= fix1;
        o[mb][2] *= fix0;
        o[mb][3] *= fix1;
        mma_bf16_16816(o[mb], vf, pb0, pb1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int sh = 4; sh < 32; sh <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], sh);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], sh);
  }
  // merge of the four warps (the ring is free: the loop ended with a barrier)
  float* mo = reinterpret_cast<float*>(sdec_raw);       // [warp][8 heads][D]
  float* mm = mo + kSdecWarps * 8 * D;                  // [warp][8] maxima, then [warp][8] sums
  float* ml = mm + kSdecWarps * 8;
#pragma unroll
  for (int mb = 0; mb < D16; ++mb) {
    mo[(warp * 8 + 2 * t) * D + mb * 16 + g] = o[mb][0];
    mo[(warp * 8 + 2 * t + 1) * D + mb * 16 + g] = o[mb][1];
    mo[(warp * 8 + 2 * t) * D + mb * 16 + g + 8] = o[mb][2];
    mo[(warp * 8 + 2 * t + 1) * D + mb * 16 + g + 8] = o[mb][3];
  }
  if (g == 0) {
    mm[warp * 8 + 2 * t] = m_run[0];
    mm[warp * 8 + 2 * t + 1] = m_run[1];
    ml[warp * 8 + 2 * t] = l_run[0];
    ml[warp * 8 + 2 * t + 1] = l_run[1];
  }
  __syncthreads();
  for (int e = tid; e < rep * D; e += NT) {
    const int hh = e / D, col = e % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSdecWarps; ++w) M = fmaxf(M, mm[w * 8 + hh]);
    float L = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < kSdecWarps; ++w) {
      const float mw = mm[w * 8 + hh];
      if (mw != -INFINITY) {
        const float f = __expf(mw - M);
        L = fmaf(f, ml[w * 8 + hh], L);
        acc = fmaf(f, mo[(w * 8 + hh) * D + col], acc);
      }
    }
    const int h = head0 + hh;
    if (a.splits > 1) {
      const size_t base = (size_t(blockIdx.z) * a.rows + row) * a.heads + h;
      a.part_o[base * D + col] = acc;
      if (col == 0) {
        a.part_ml[base * 2] = M;
        a.part_ml[base * 2 + 1] = L;
      }
    } else {
      a.out[size_t(row) * a.ld_out + h * D + col] = __float2bfloat16_rn(acc * a.out_scale / L * smax_gate(a.gate, a.ld_gate, row, h));
    }
  }
}

// out[row, h] = out_scale * sum_z e^(m_z - M) o_z / sum_z e^(m_z - M) l_z, M = max_z m_z; one warp per (row, head)
__global__ void __launch_bounds__(128) softmax_attention_merge_kernel(const SoftmaxAttnArgs<bf16> a) {
  griddep_wait();
  const int unit = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (unit >= a.rows * a.heads) return;
  const int row = unit / a.heads, h = unit % a.heads, D = a.vdim;
  float M = -INFINITY;
  for (int z = 0; z < a.splits; ++z) M = fmaxf(M, a.part_ml[((size_t(z) * a.rows + row) * a.heads + h) * 2]);
  float L = 0.0f;
  for (int z = 0; z < a.splits; ++z) {
    const float* ml = a.part_ml + ((size_t(z) * a.rows + row) * a.heads + h) * 2;
    if (ml[0] != -INFINITY) L += __expf(ml[0] - M) * ml[1];
  }
  const float gate = smax_gate(a.gate, a.ld_gate, row, h);
  for (int c = lane; c < D; c += 32) {
    float acc = 0.0f;
    for (int z = 0; z < a.splits; ++z) {
      const size_t base = (size_t(z) * a.rows + row) * a.heads + h;
      const float mz = a.part_ml[base * 2];
      if (mz != -INFINITY) acc = fmaf(__expf(mz - M), a.part_o[base * D + c], acc);
    }
    a.out[size_t(row) * a.ld_out + h * D + c] = __float2bfloat16_rn(acc * a.out_scale / L * gate);
  }
}

}  // namespace mtx
