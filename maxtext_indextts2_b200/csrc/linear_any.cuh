// out[rows, n] = a[rows, k] . w[n, k]^T for ANY rows / n / k (no multiple-of-64 rule), with small fused epilogues.
//
// Two kernels behind one argument block:
//   * linear_mma_kernel   bf16 operands on the warp-level tensor-core path (mma.sync m16n8k16), fp32 accumulation;
//   * linear_f32_kernel   fp32 operands, fp32 FMA accumulation (no reduced-precision matrix mode): the exact arm of a model
//                         that is served in float32.
// The layered engine routes a projection here when its shape does not fit the 128 x 64 tiles of the tcgen05 GEMMs
// (gemm_rows.cuh), and always in float32.  Edges are handled by guarded loads (zero fill) and guarded stores.
//
// Epilogues: LIN_PLAIN  out = acc                      (fp32)
//            LIN_BIAS   out = acc + bias[col]          (fp32)
//            LIN_GATED  act[r, f] = gelu_tanh(acc[r, 2f]) * acc[r, 2f + 1]   (the weight rows are interleaved gate / up)
//            LIN_GATED_CLAMP  act[r, f] = g sigmoid(1.702 g) (u + 1), g = min(acc[r, 2f], limit), u = clamp(acc[r, 2f + 1], -limit, limit);
//                             limit <= 0: act[r, f] = silu(acc[r, 2f]) * acc[r, 2f + 1], no limits
//            LIN_ACT    act[r, c] = acc                  (in the matmul dtype, row pitch ldo: the input of another product)
//            LIN_RELU2  act[r, c] = max(acc, 0)^2
//
// Batched mode (batch_a != 0 or batch_o != 0; group_off null): blockIdx.z names one of several products over the same rows whose
// operands lie side by side: `a` moves by batch_a columns, the weight by w_group_stride elements and the output by batch_o columns
// per batch (the per-head products of an attention that works in a latent space).
//
// Grouped mode (group_off != null; a mixture of experts): blockIdx.z names a group with its own weight matrix; the group's rows are
// the slots [group_off[g], group_off[g + 1]); slot s reads row a_row[s] of `a` (or row s when a_row is null) and writes row s of the
// output.  CTAs beyond a group's last row tile leave at once, so the grid is sized for the worst case without a host round trip;
// with `groups` set the grid's y walks the groups' row tiles one group after the other (at most ceil(slots / tile) + groups tiles
// in all), which leaves few CTAs without work when there are many groups.
#pragma once

#include "common.cuh"

namespace mtx {

enum { LIN_PLAIN = 0, LIN_BIAS = 1, LIN_GATED = 2, LIN_GATED_CLAMP = 3, LIN_ACT = 4, LIN_RELU2 = 5 };

template <typename T>
struct LinArgs {
  const T* a;         // [rows, k], row pitch lda
  const T* w;         // [n, k] contiguous
  const float* bias;  // [n] (LIN_BIAS)
  float* out;         // [rows, n] fp32, row pitch ldo (LIN_PLAIN / LIN_BIAS)
  T* act;             // [rows, n / 2], row pitch ldo (LIN_GATED)
  long long lda, ldo;
  int rows, n, k;
  float limit;             // LIN_GATED_CLAMP
  const int* group_off;    // grouped mode: [groups + 1] slot ranges
  const int* a_row;        // grouped mode: [slots] row of `a` per slot, or null
  long long w_group_stride;  // grouped / batched mode: elements between two groups' weights
  long long batch_a, batch_o;  // batched mode: columns between two batches' inputs / outputs
  int groups;              // grouped mode, > 0: the grid's y walks the groups' row tiles one group after the other (gridDim.z == 1,
                           // gridDim.y >= ceil(slots / tile) + groups) instead of every group owning a worst-case range of y
};

// grouped mode: the argument block of this CTA's group (false: the CTA has no rows)
template <typename T>
__device__ __forceinline__ bool lin_enter_group(LinArgs<T>& p, int tile_rows, int& row_tile) {
  row_tile = blockIdx.y;
  if (p.group_off == nullptr) {
    if (p.batch_a != 0 || p.batch_o != 0) {
      const size_t b = blockIdx.z;
      p.a += b * p.batch_a;
      p.w += b * p.w_group_stride;
      if (p.out) p.out += b * p.batch_o;
      if (p.act) p.act += b * p.batch_o;
    }
    return true;
  }
  int g = blockIdx.z;
  if (p.groups > 0) {  // whose tile is this?
    int t = blockIdx.y;
    for (g = 0; g < p.groups; ++g) {
      const int nt = (p.group_off[g + 1] - p.group_off[g] + tile_rows - 1) / tile_rows;
      if (t < nt) break;
      t -= nt;
    }
    if (g == p.groups) return false;
    row_tile = t;
  }
  const int s0 = p.group_off[g], cnt = p.group_off[g + 1] - s0;
  if (row_tile * tile_rows >= cnt) return false;
  p.rows = cnt;
  p.w += size_t(g) * p.w_group_stride;
  if (p.a_row) p.a_row += s0;
  else p.a += size_t(s0) * p.lda;
  if (p.out) p.out += size_t(s0) * p.ldo;
  if (p.act) p.act += size_t(s0) * p.ldo;
  return true;
}

__device__ __forceinline__ float clamped_gate_f(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

// silu(g) * u
__device__ __forceinline__ float silu_gate_f(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__device__ __forceinline__ float gelu_tanh_f(float z) {
  const float c = 0.7978845608028654f;  // sqrt(2 / pi)
  return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
}

template <typename T>
__device__ __forceinline__ T to_act(float v);
template <>
__device__ __forceinline__ float to_act<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 to_act<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float act_f32(float v) { return v; }
__device__ __forceinline__ float act_f32(bf16 v) { return __bfloat162float(v); }

// one (row, column pair) of the accumulator tile
template <typename T, int EPI>
__device__ __forceinline__ void lin_store_pair(const LinArgs<T>& p, int r, int c, float v0, float v1) {
  if (r >= p.rows || c >= p.n) return;
  if (EPI == LIN_GATED) {  // c is even: (gate, up) of feature c / 2
    p.act[size_t(r) * p.ldo + (c >> 1)] = to_act<T>(gelu_tanh_f(v0) * v1);
    return;
  }
  if (EPI == LIN_GATED_CLAMP) {
    p.act[size_t(r) * p.ldo + (c >> 1)] = to_act<T>(p.limit > 0.0f ? clamped_gate_f(v0, v1, p.limit) : silu_gate_f(v0, v1));
    return;
  }
  if (EPI == LIN_ACT || EPI == LIN_RELU2) {
    if (EPI == LIN_RELU2) {
      v0 = fmaxf(v0, 0.0f);
      v1 = fmaxf(v1, 0.0f);
      v0 *= v0;
      v1 *= v1;
    }
    T* o = p.act + size_t(r) * p.ldo + c;
    o[0] = to_act<T>(v0);
    if (c + 1 < p.n) o[1] = to_act<T>(v1);
    return;
  }
  float* o = p.out + size_t(r) * p.ldo + c;
  if (EPI == LIN_BIAS) {
    v0 += p.bias[c];
    if (c + 1 < p.n) v1 += p.bias[c + 1];
  }
  o[0] = v0;
  if (c + 1 < p.n) o[1] = v1;
}

// ---- bf16: 64 x 64 x 64 tiles, four warps of 32 x 32 ---------------------------------------------------------------------
constexpr int kLinThreads = 128;
constexpr int kLinBM = 64, kLinBN = 64, kLinBK = 64, kLinPitch = kLinBK + 8;  // 144-byte rows: fragment reads hit 32 banks

// 64 rows x 64 columns of an operand: 512 chunks of 8 elements, four per thread; fetched into registers one k step ahead of their
// use (the loads of step k + 1 are in flight while step k's tensor-core work runs), then stored to shared memory
__device__ __forceinline__ void lin_fetch_tile(const bf16* src, long long ld, int row0, int n_rows, int k0, int k, bool vec, uint4 (&v)[4], int tid,
                                               const int* row_map = nullptr) {
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int chunk = tid + it * kLinThreads, r = chunk >> 3, c = (chunk & 7) * 8;
    const int gr = row0 + r, gc = k0 + c;
    v[it] = make_uint4(0u, 0u, 0u, 0u);
    if (gr < n_rows && gc < k) {
      const bf16* s = src + size_t(row_map ? row_map[gr] : gr) * ld + gc;
      if (vec && gc + 8 <= k) {
        v[it] = *reinterpret_cast<const uint4*>(s);
      } else {
        bf16 tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = (gc + e < k) ? s[e] : __float2bfloat16_rn(0.0f);
        v[it] = *reinterpret_cast<const uint4*>(tmp);
      }
    }
  }
}

__device__ __forceinline__ void lin_store_tile(const uint4 (&v)[4], bf16* dst, int tid) {
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int chunk = tid + it * kLinThreads, r = chunk >> 3, c = (chunk & 7) * 8;
    *reinterpret_cast<uint4*>(dst + r * kLinPitch + c) = v[it];
  }
}

template <int EPI>
__global__ void __launch_bounds__(kLinThreads) linear_mma_kernel(const LinArgs<bf16> p_in) {
  __shared__ __align__(16) bf16 sa[kLinBM * kLinPitch];
  __shared__ __align__(16) bf16 sb[kLinBN * kLinPitch];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  griddep_wait();
  LinArgs<bf16> p = p_in;
  int row_tile;
  if (!lin_enter_group(p, kLinBM, row_tile)) return;
  const int row0 = row_tile * kLinBM, col0 = blockIdx.x * kLinBN;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const bool vec_a = (p.lda % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0);
  const bool vec_w = (p.k % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.w) & 15) == 0);
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
  uint4 ra[4], rb[4];
  lin_fetch_tile(p.a, p.lda, row0, p.rows, 0, p.k, vec_a, ra, tid, p.a_row);
  lin_fetch_tile(p.w, p.k, col0, p.n, 0, p.k, vec_w, rb, tid);
  for (int k0 = 0; k0 < p.k; k0 += kLinBK) {
    lin_store_tile(ra, sa, tid);
    lin_store_tile(rb, sb, tid);
    __syncthreads();
    if (k0 + kLinBK < p.k) {
      lin_fetch_tile(p.a, p.lda, row0, p.rows, k0 + kLinBK, p.k, vec_a, ra, tid, p.a_row);
      lin_fetch_tile(p.w, p.k, col0, p.n, k0 + kLinBK, p.k, vec_w, rb, tid);
    }
#pragma unroll
    for (int kk = 0; kk < kLinBK; kk += 16) {
      uint32_t af[2][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bf16* base = sa + (wm + i * 16 + g) * kLinPitch + kk + 2 * t;
        af[i][0] = *reinterpret_cast<const uint32_t*>(base);
        af[i][1] = *reinterpret_cast<const uint32_t*>(base + 8 * kLinPitch);
        af[i][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        af[i][3] = *reinterpret_cast<const uint32_t*>(base + 8 * kLinPitch + 8);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bf16* base = sb + (wn + j * 8 + g) * kLinPitch + kk + 2 * t;
        bfr[j][0] = *reinterpret_cast<const uint32_t*>(base);
        bfr[j][1] = *reinterpret_cast<const uint32_t*>(base + 8);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                       : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bfr[j][0]), "r"(bfr[j][1]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + wm + i * 16 + g, c = col0 + wn + j * 8 + 2 * t;
      lin_store_pair<bf16, EPI>(p, r, c, acc[i][j][0], acc[i][j][1]);
      lin_store_pair<bf16, EPI>(p, r + 8, c, acc[i][j][2], acc[i][j][3]);
    }
}

// ---- fp32: 64 x 64 x 16 tiles, 256 threads of 4 x 4 ------------------------------------------------------------------------
constexpr int kLinF32Threads = 256;

template <int EPI>
__global__ void __launch_bounds__(kLinF32Threads) linear_f32_kernel(const LinArgs<float> p_in) {
  __shared__ float sa[16][64 + 4];  // [k][row]
  __shared__ float sb[16][64 + 4];  // [k][col]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  griddep_wait();
  LinArgs<float> p = p_in;
  int row_tile;
  if (!lin_enter_group(p, 64, row_tile)) return;
  const int row0 = row_tile * 64, col0 = blockIdx.x * 64;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < p.k; k0 += 16) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {  // 64 x 16 elements of each operand, four per thread; consecutive threads walk k
      const int idx = tid + it * kLinF32Threads, r = idx >> 4, c = idx & 15;
      const int gk = k0 + c;
      sa[c][r] = (row0 + r < p.rows && gk < p.k) ? p.a[size_t(p.a_row ? p.a_row[row0 + r] : row0 + r) * p.lda + gk] : 0.0f;
      sb[c][r] = (col0 + r < p.n && gk < p.k) ? p.w[size_t(col0 + r) * p.k + gk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i, c = col0 + tx * 4;
    lin_store_pair<float, EPI>(p, r, c, acc[i][0], acc[i][1]);
    lin_store_pair<float, EPI>(p, r, c + 2, acc[i][2], acc[i][3]);
  }
}

}  // namespace mtx
