// Attention whose keys and values are expansions of a cached latent, served in the latent space.
//
// Per token the cache holds one row [c | k_rot]: c = rmsnorm(the first kv_rank outputs of the down-projection) * weight, and the
// last rot_dim outputs turned by the token's position (one rotated key part for all heads).  Head h's key would be
// [w_uk_h c | k_rot] and its value w_uv_h c; instead of expanding every cached token at every step, the query goes the other way:
//
//   score_h(i, j) = scale * (<w_uk_h^T q_plain_h(i), c(j)> + <q_rot_h(i), k_rot(j)>)
//   out_h(i)      = w_uv_h * sum_j p_h(i, j) c(j)
//
// so the attention itself is the one-key-head softmax attention of softmax_attention.cuh over rows of kv_rank + rot_dim channels
// whose values are the cached rows themselves (the rotated tail of the weighted sum is not read by anyone), and the two
// expansions become per-head matrix products over the step's rows (linear_any.cuh, batched mode).
//
//   latent_prepare_kernel<T>   per row: the query latent (normed, in the matmul dtype) and the cache row (normed latent, rotated tail)
//   latent_query_kernel<T>     per row and head: the plain query part for the product with w_uk_h^T, the rotated part into place
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"
#include "softmax_attention.cuh"

namespace mtx {

template <typename T>
struct LatentPrepareArgs {
  const float* proj;      // [rows, ld]: the query's down-projection at q_col (q_rank columns), the key / value one at kv_col (kv_rank + rot_dim)
  long long ld;
  int q_col, kv_col, q_rank, kv_rank, rot_dim, rot_half;
  const float* q_norm;    // [q_rank]
  const float* kv_norm;   // [kv_rank]
  const double* rot_freq; // [rot_dim / 2]
  T* cq_out;              // [rows, q_rank]
  T* pages;               // [num_pages * tokens_per_page, kv_rank + rot_dim]
  const int* group;
  const int* pos;
  const int* page_map;
  int tokens_per_page, max_pages;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const LatentPrepareArgs<T> a) {
  __shared__ float red[8];
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* rq = a.proj + size_t(r) * a.ld + a.q_col;
  const float* rk = a.proj + size_t(r) * a.ld + a.kv_col;
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  T* dst = a.pages + slot * size_t(a.kv_rank + a.rot_dim);
  float ss = 0.0f;
  for (int c = tid; c < a.q_rank; c += blockDim.x) ss = fmaf(rq[c], rq[c], ss);
  ss = block_sum(ss, red);
  const float fq = 1.0f / sqrtf(ss / float(a.q_rank) + a.eps);
  for (int c = tid; c < a.q_rank; c += blockDim.x) a.cq_out[size_t(r) * a.q_rank + c] = to_act<T>(rq[c] * fq * a.q_norm[c]);
  float sk = 0.0f;
  for (int c = tid; c < a.kv_rank; c += blockDim.x) sk = fmaf(rk[c], rk[c], sk);
  sk = block_sum(sk, red);
  const float fk = 1.0f / sqrtf(sk / float(a.kv_rank) + a.eps);
  for (int c = tid; c < a.kv_rank; c += blockDim.x) dst[c] = to_act<T>(rk[c] * fk * a.kv_norm[c]);
  const int rh = a.rot_dim / 2;
  const float* tail = rk + a.kv_rank;
  for (int i = tid; i < rh; i += blockDim.x) {
    const int c0 = a.rot_half ? i : 2 * i, c1 = a.rot_half ? i + rh : 2 * i + 1;
    float sn, cs;
    rot_sincos(double(p), a.rot_freq[i], &sn, &cs);
    dst[a.kv_rank + c0] = to_act<T>(tail[c0] * cs - tail[c1] * sn);
    dst[a.kv_rank + c1] = to_act<T>(tail[c1] * cs + tail[c0] * sn);
  }
  if ((a.rot_dim & 1) && tid == 0) dst[a.kv_rank + a.rot_dim - 1] = to_act<T>(tail[a.rot_dim - 1]);
}

template <typename T>
struct LatentQueryArgs {
  const float* q;        // [rows, H * (dim + rot_dim)]
  T* q_plain;            // [rows, H * dim]
  T* q_full;             // [rows, H * (kv_rank + rot_dim)]: the rotated part is written at column kv_rank of every head
  const double* rot_freq;
  const int* pos;
  int heads, dim, rot_dim, kv_rank, rot_half;
};

template <typename T>
__global__ void __launch_bounds__(256) latent_query_kernel(const LatentQueryArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, H = a.heads, d = a.dim, dr = a.rot_dim, rh = dr / 2, dq = d + dr, dl = a.kv_rank + dr;
  const float* q = a.q + size_t(r) * H * dq;
  const double dp = double(a.pos[r]);
  for (int e = threadIdx.x; e < H * d; e += blockDim.x) a.q_plain[size_t(r) * H * d + e] = to_act<T>(q[(e / d) * dq + e % d]);
  for (int e = threadIdx.x; e < H * rh; e += blockDim.x) {
    const int h = e / rh, i = e % rh;
    const int c0 = a.rot_half ? i : 2 * i, c1 = a.rot_half ? i + rh : 2 * i + 1;
    const float* src = q + h * dq + d;
    T* dst = a.q_full + size_t(r) * H * dl + h * dl + a.kv_rank;
    float sn, cs;
    rot_sincos(dp, a.rot_freq[i], &sn, &cs);
    dst[c0] = to_act<T>(src[c0] * cs - src[c1] * sn);
    dst[c1] = to_act<T>(src[c1] * cs + src[c0] * sn);
  }
  if (dr & 1)
    for (int h = threadIdx.x; h < H; h += blockDim.x) a.q_full[size_t(r) * H * dl + h * dl + a.kv_rank + dr - 1] = to_act<T>(q[h * dq + d + dr - 1]);
}

}  // namespace mtx
