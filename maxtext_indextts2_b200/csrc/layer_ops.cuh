// Row-wise steps of a layered model between its matrix products, for a ragged batch (every row = one token of some sequence):
//
//   embed_rows_kernel       x = embedding[token] * scale (fp32 residual) and its copy in the matmul dtype
//   qkv_post_kernel         per-head RMS norm of q and k (a weight vector shared by the heads), mixing of the values with the
//                           values an earlier layer computed for the same token, append of k and v to the paged cache
//   norm_residual_kernel    x += gain * y / sqrt(mean(y^2) + eps)   (a normalisation with ONE gain, on the sublayer's OUTPUT)
//   scalar_norm_rows_kernel n = gain * x[row] / sqrt(mean(x[row]^2) + eps) for a gathered subset of rows (before the logits)
//   sandwich_step_kernel    norms with a weight vector stored around zero, before AND after a sublayer:
//                           x += wnorm(y + bias, post); x += embedding output; x += vector; xa = wnorm(x, pre)   (each part optional)
//                           with wnorm(y, w) = y / sqrt(mean(y^2) + eps) * (1 + w)
//   weighted_norm_rows_kernel  wnorm of a gathered subset of rows;  softcap_kernel  z = cap * tanh(z / cap)
//   group_norm_step_kernel  x += mult * y (optional); h = gnorm(x) * w (w null: no h), the row normed in `groups` consecutive parts of their own (fp32 out)
//   input_conv_kernel       per-channel causal convolutions over time on h: a = h + conv1(h), b = h + conv2(h) in the matmul dtype; rows
//                           before a run's first come from the sequence's state (a ring of the last taps - 1 normed rows)
//   conv_state_update_kernel  the last rows of every run go into that ring
//   group_norm_rows_kernel  gnorm of a gathered subset of rows;  logit_post_kernel  z = cap * tanh(scale * z / cap)
//   pre_norm_step_kernel    pre-norm layers: x = unit(x) * w0 (optional); x += y or x += unit(y) * wy (optional); a copy of x in the matmul
//                           dtype (optional); unit(x) * w to the fp32 plane of normed rows and / or the matmul dtype (optional), or,
//                           in steps of single tokens, straight through the next mixer's input convolution and into its ring
//   side_act_kernel         act = gelu_tanh(gate) * table[token, col ..]: the gated rows of a per-layer token input
//
// Everything here is fp32 arithmetic; T is the dtype the matrix products and the cache use (bf16, or float for a float32 engine).
#pragma once

#include "common.cuh"
#include "linear_any.cuh"

namespace mtx {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// sum over the block; every thread gets the result.  `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.0f;
  for (int w = 0; w < nw; ++w) r += red[w];  // fixed order
  return r;
}

// (x0: a second copy of the embedding output for layers that add it again, or null)
template <typename T>
__global__ void embed_rows_kernel(const int* token, const T* embedding, int vocab, float scale, float* x, T* xa, int width, float* x0) {
  griddep_wait();
  const int r = blockIdx.x;
  int tok = token[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = act_f32(embedding[size_t(tok) * width + c]) * scale;
    x[size_t(r) * width + c] = v;
    xa[size_t(r) * width + c] = to_act<T>(v);
    if (x0) x0[size_t(r) * width + c] = v;
  }
}

struct SandwichArgs {
  const float* y;         // [rows, width] the sublayer's output, or null: no residual update in this call
  const float* y_bias;    // [width] added to y before its norm, or null
  const float* post;      // [width] weight of the norm on y
  const float* x0;        // [rows, width] added to x after the update, or null
  const float* add_vec;   // [width] added to x after that, or null
  const float* pre;       // [width] weight of the norm whose result goes to xa, or null: xa is not written
  float* x;               // [rows, width]
  float eps;
  int width;
};

// one CTA per row; the row of x stays in registers between the two reductions.  V = 4: the row moves as float4s (width a
// multiple of 4, <= 256 * 4 * kSandwichVec); V = 1: any width <= 256 * kSandwichMax.
constexpr int kSandwichMax = 32, kSandwichVec = 8;

template <typename T, int V>
__global__ void __launch_bounds__(256) sandwich_step_kernel(const SandwichArgs a, T* xa) {
  __shared__ float red[8];
  constexpr int N = V == 4 ? kSandwichVec : kSandwichMax;  // register groups of V floats per thread
  griddep_wait();
  const int r = blockIdx.x, W = a.width;
  float* xr = a.x + size_t(r) * W;
  const float* yr = a.y ? a.y + size_t(r) * W : nullptr;
  const float* x0r = a.x0 ? a.x0 + size_t(r) * W : nullptr;
  auto load = [&](const float* p, int c, float (&v)[V]) {
    if (V == 4) {
      const float4 q = *reinterpret_cast<const float4*>(p + c);
      v[0] = q.x, v[V > 1 ? 1 : 0] = q.y, v[V > 2 ? 2 : 0] = q.z, v[V > 3 ? 3 : 0] = q.w;
    } else {
      v[0] = p[c];
    }
  };
  float yv[N][V];
  float f = 0.0f;
  if (yr) {
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < N; ++u) {
      const int c = (threadIdx.x + u * 256) * V;
      if (c < W) {
        float b[V];
        load(yr, c, yv[u]);
        if (a.y_bias) {
          load(a.y_bias, c, b);
#pragma unroll
          for (int e = 0; e < V; ++e) yv[u][e] += b[e];
        }
#pragma unroll
        for (int e = 0; e < V; ++e) ss = fmaf(yv[u][e], yv[u][e], ss);
      }
    }
    ss = block_sum(ss, red);
    f = 1.0f / sqrtf(ss / float(W) + a.eps);
  }
  float ss2 = 0.0f;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const int c = (threadIdx.x + u * 256) * V;
    if (c < W) {
      float v[V], w[V];
      load(xr, c, v);
      if (yr) {
        load(a.post, c, w);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] += yv[u][e] * f * (1.0f + w[e]);
      }
      if (x0r) {
        load(x0r, c, w);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] += w[e];
      }
      if (a.add_vec) {
        load(a.add_vec, c, w);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] += w[e];
      }
#pragma unroll
      for (int e = 0; e < V; ++e) {
        yv[u][e] = v[e];  // (the registers now hold the new x)
        ss2 = fmaf(v[e], v[e], ss2);
      }
      if (yr || x0r || a.add_vec) {
        if (V == 4) *reinterpret_cast<float4*>(xr + c) = make_float4(v[0], v[V > 1 ? 1 : 0], v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
        else xr[c] = v[0];
      }
    }
  }
  if (!a.pre) return;
  ss2 = block_sum(ss2, red);
  const float f2 = 1.0f / sqrtf(ss2 / float(W) + a.eps);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const int c = (threadIdx.x + u * 256) * V;
    if (c < W) {
      float w[V];
      load(a.pre, c, w);
#pragma unroll
      for (int e = 0; e < V; ++e) xa[size_t(r) * W + c + e] = to_act<T>(yv[u][e] * f2 * (1.0f + w[e]));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) weighted_norm_rows_kernel(const float* x, const int* rows, const float* w, float eps, T* out, int width) {
  __shared__ float red[8];
  griddep_wait();
  const int src = rows ? rows[blockIdx.x] : int(blockIdx.x);
  const float* xr = x + size_t(src) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
  ss = block_sum(ss, red);
  const float f = 1.0f / sqrtf(ss / float(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[size_t(blockIdx.x) * width + c] = to_act<T>(xr[c] * f * (1.0f + w[c]));
}

__global__ void softcap_kernel(float* z, float cap, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    z[i] = cap * tanhf(z[i] / cap);
}

template <typename T>
struct InputConvArgs {
  const float* h;        // [rows, width] the normed rows of this step
  const float* w1;       // [taps, width]: tap j multiplies the row taps - 1 - j steps back (the last tap the row itself)
  const float* w2;       // the same for the second output, or null
  float* state;          // [slots, taps - 1, width]: the normed row of position p of a sequence at index p % (taps - 1)
  T* out1;               // [rows, width] h + conv1(h)
  T* out2;               // [rows, width] h + conv2(h) (w2 null: h itself), or null: not written
  const int* group;
  const int* pos;
  int rows, width, taps;
};

// CTAs of eight warps.  A group's sum of squares is added in a fixed order: with eight groups or more a CTA takes a row and each of
// its warps whole groups; with fewer the grid is (rows, groups) and the eight warps' partial sums of a group meet in shared memory.
// FUSED (steps in which every row is a single token of its own sequence): the row's normed values do not go to the plane h but
// straight through the input convolutions (the earlier rows come from the sequence's ring) and into the ring.  The arithmetic is
// that of input_conv_kernel, value by value, so a position's result does not depend on which of the two paths served it.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(256) group_norm_step_kernel(const float* y, float mult, float* x, const float* w, float eps, float* h, int width,
                                                              int groups, const InputConvArgs<T> cv) {
  __shared__ float red[8];
  griddep_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gs = width / groups;
  float* xr = x + size_t(r) * width;
  const float* yr = y ? y + size_t(r) * width : nullptr;
  float* hr = h + size_t(r) * width;
  const int p = FUSED ? cv.pos[r] : 0, grp = FUSED ? cv.group[r] : 0, ring = cv.taps - 1;
  auto emit = [&](int c, float hv) {
    if constexpr (!FUSED) {
      hr[c] = hv;
    } else {
      const int W = width;
      float s1 = hv * cv.w1[size_t(ring) * W + c], s2 = cv.w2 ? hv * cv.w2[size_t(ring) * W + c] : 0.0f;
      for (int back = 1; back <= ring && back <= p; ++back) {
        const float v = cv.state[(size_t(grp) * ring + (p - back) % ring) * W + c];
        s1 = fmaf(v, cv.w1[size_t(ring - back) * W + c], s1);
        if (cv.w2) s2 = fmaf(v, cv.w2[size_t(ring - back) * W + c], s2);
      }
      cv.out1[size_t(r) * W + c] = to_act<T>(hv + s1);
      if (cv.out2) cv.out2[size_t(r) * W + c] = to_act<T>(hv + s2);
      if (ring > 0) cv.state[(size_t(grp) * ring + p % ring) * W + c] = hv;  // (the slot of position p - ring, read just above by this thread)
    }
  };
  if (groups >= 8) {
    for (int g = warp; g < groups; g += 8) {
      const int base = g * gs;
      float ss = 0.0f;
      for (int c = lane; c < gs; c += 32) {
        float v = xr[base + c];
        if (yr) {
          v = fmaf(mult, yr[base + c], v);
          xr[base + c] = v;
        }
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      const float f = 1.0f / sqrtf(ss / float(gs) + eps);
      if (w)
        for (int c = lane; c < gs; c += 32) emit(base + c, xr[base + c] * f * w[base + c]);
    }
    return;
  }
  const int base = int(blockIdx.y) * gs;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < gs; c += 256) {
    float v = xr[base + c];
    if (yr) {
      v = fmaf(mult, yr[base + c], v);
      xr[base + c] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (!w) return;
  float tot = 0.0f;
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float f = 1.0f / sqrtf(tot / float(gs) + eps);
#pragma unroll 2
  for (int c = threadIdx.x; c < gs; c += 256) emit(base + c, xr[base + c] * f * w[base + c]);
}

template <typename T>
__global__ void __launch_bounds__(256) group_norm_rows_kernel(const float* x, const int* rows, const float* w, float eps, T* out, int width, int groups) {
  __shared__ float red[8];
  griddep_wait();
  const int src = rows ? rows[blockIdx.x] : int(blockIdx.x), warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gs = width / groups;
  const float* xr = x + size_t(src) * width;
  if (groups == 1) {  // a plain RMS norm: the whole CTA on the one group
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    const float f = 1.0f / sqrtf(block_sum(ss, red) / float(width) + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[size_t(blockIdx.x) * width + c] = to_act<T>(xr[c] * f * w[c]);
    return;
  }
  for (int g = warp; g < groups; g += 8) {  // (only the rows whose logits are wanted come here: a warp per group is enough)
    const int base = g * gs;
    float ss = 0.0f;
    for (int c = lane; c < gs; c += 32) ss = fmaf(xr[base + c], xr[base + c], ss);
    ss = warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / float(gs) + eps);
    for (int c = lane; c < gs; c += 32) out[size_t(blockIdx.x) * width + base + c] = to_act<T>(xr[base + c] * f * w[base + c]);
  }
}

__global__ void logit_post_kernel(float* z, float scale, float cap, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float v = z[i] * scale;
    z[i] = cap > 0.0f ? cap * tanhf(v / cap) : v;
  }
}


// one CTA per row.  The row `back` steps before row r is row r - back of the batch when that is the same sequence's previous
// position (rows of a run are consecutive), a row of the state when the run began later, and zero before the sequence's start.
// Where each of them lies is found once per CTA (up to kConvMaxBack earlier rows; more taps take the per-element path).
constexpr int kConvMaxBack = 16;

template <typename T>
__global__ void __launch_bounds__(256) input_conv_kernel(const InputConvArgs<T> a) {
  __shared__ const float* s_src[kConvMaxBack];
  griddep_wait();
  const int r = blockIdx.x, W = a.width, p = a.pos[r], grp = a.group[r], ring = a.taps - 1;
  const int n_back = ring < p ? ring : p;
  if (ring <= kConvMaxBack) {
    if (threadIdx.x < n_back) {
      const int back = threadIdx.x + 1, rr = r - back;
      const bool in_batch = rr >= 0 && a.group[rr] == grp && a.pos[rr] == p - back;
      s_src[threadIdx.x] = in_batch ? a.h + size_t(rr) * W : a.state + (size_t(grp) * ring + (p - back) % ring) * W;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float own = a.h[size_t(r) * W + c];
      float s1 = own * a.w1[size_t(ring) * W + c], s2 = a.w2 ? own * a.w2[size_t(ring) * W + c] : 0.0f;
      for (int back = 1; back <= n_back; ++back) {
        const float v = s_src[back - 1][c];
        s1 = fmaf(v, a.w1[size_t(ring - back) * W + c], s1);
        if (a.w2) s2 = fmaf(v, a.w2[size_t(ring - back) * W + c], s2);
      }
      a.out1[size_t(r) * W + c] = to_act<T>(own + s1);
      if (a.out2) a.out2[size_t(r) * W + c] = to_act<T>(own + s2);
    }
    return;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float own = a.h[size_t(r) * W + c];
    float s1 = own * a.w1[size_t(ring) * W + c], s2 = a.w2 ? own * a.w2[size_t(ring) * W + c] : 0.0f;
    for (int back = 1; back <= n_back; ++back) {
      const int rr = r - back;
      const bool in_batch = rr >= 0 && a.group[rr] == grp && a.pos[rr] == p - back;
      const float v = in_batch ? a.h[size_t(rr) * W + c] : a.state[(size_t(grp) * ring + (p - back) % ring) * W + c];
      s1 = fmaf(v, a.w1[size_t(ring - back) * W + c], s1);
      if (a.w2) s2 = fmaf(v, a.w2[size_t(ring - back) * W + c], s2);
    }
    a.out1[size_t(r) * W + c] = to_act<T>(own + s1);
    if (a.out2) a.out2[size_t(r) * W + c] = to_act<T>(own + s2);
  }
}

// grid (runs, taps - 1): CTA (run, i) keeps the run's i-th row from its end, if the run is that long (`ld`: row pitch of h)
__global__ void __launch_bounds__(256) conv_state_update_kernel(const float* h, float* state, const int* run_row0, const int* group, const int* pos,
                                                                int width, int taps, long long ld) {
  griddep_wait();
  const int r0 = run_row0[blockIdx.x], r1 = run_row0[blockIdx.x + 1], r = r1 - 1 - int(blockIdx.y), ring = taps - 1;
  if (r < r0) return;
  float* dst = state + (size_t(group[r]) * ring + pos[r] % ring) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = h[size_t(r) * ld + c];
}

struct PreNormArgs {
  const float* y;       // [rows, width] joins x, or null
  const float* y_w;     // [width]: x += unit(y) * y_w; null: x += y
  const float* self_w;  // [width]: before anything else x = unit(x) * self_w (the norm of the embedding output); null: not
  float* x;             // [rows, width]
  const float* w;       // [width] weight of the norm that is written out; null: none is
  float* h;             // [rows, width] unit(x) * w in fp32 (what an input convolution reads), or null
  float eps;
  int width;
};

// one CTA per row.  FUSED (steps in which every row is a single token of its own sequence): the normed values go straight through
// the input convolution `cv` (the earlier rows come from the sequence's ring) and into the ring, with the arithmetic of
// input_conv_kernel value by value.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(256) pre_norm_step_kernel(const PreNormArgs a, T* x_copy, T* out, const InputConvArgs<T> cv) {
  __shared__ float red[8];
  griddep_wait();
  const int r = blockIdx.x, W = a.width;
  float* xr = a.x + size_t(r) * W;
  const float* yr = a.y ? a.y + size_t(r) * W : nullptr;
  float fy = 1.0f, fs = 1.0f;
  if (yr && a.y_w) {
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += 256) ss = fmaf(yr[c], yr[c], ss);
    fy = 1.0f / sqrtf(block_sum(ss, red) / float(W) + a.eps);
  }
  if (a.self_w) {
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += 256) ss = fmaf(xr[c], xr[c], ss);
    fs = 1.0f / sqrtf(block_sum(ss, red) / float(W) + a.eps);
  }
  float ss2 = 0.0f;
  for (int c = threadIdx.x; c < W; c += 256) {
    float v = xr[c];
    if (a.self_w) v = v * fs * a.self_w[c];
    if (yr) v += a.y_w ? yr[c] * fy * a.y_w[c] : yr[c];
    if (yr || a.self_w) xr[c] = v;
    if (x_copy) x_copy[size_t(r) * W + c] = to_act<T>(v);
    ss2 = fmaf(v, v, ss2);
  }
  if (!a.w) return;
  const float f2 = 1.0f / sqrtf(block_sum(ss2, red) / float(W) + a.eps);
  const int p = FUSED ? cv.pos[r] : 0, grp = FUSED ? cv.group[r] : 0, ring = cv.taps - 1;
  for (int c = threadIdx.x; c < W; c += 256) {
    const float hv = xr[c] * f2 * a.w[c];  // (xr[c]: this thread's own write above)
    if constexpr (!FUSED) {
      if (a.h) a.h[size_t(r) * W + c] = hv;
      if (out) out[size_t(r) * W + c] = to_act<T>(hv);
    } else {
      float s1 = hv * cv.w1[size_t(ring) * W + c];
      for (int back = 1; back <= ring && back <= p; ++back)
        s1 = fmaf(cv.state[(size_t(grp) * ring + (p - back) % ring) * W + c], cv.w1[size_t(ring - back) * W + c], s1);
      cv.out1[size_t(r) * W + c] = to_act<T>(hv + s1);
      if (ring > 0) cv.state[(size_t(grp) * ring + p % ring) * W + c] = hv;  // (the slot of position p - ring, read just above by this thread)
    }
  }
}

// act[r, c] = gelu_tanh(gate[r, c]) * table[token[r], col + c], c < dim
template <typename T>
__global__ void __launch_bounds__(256) side_act_kernel(const float* gate, long long ld_gate, const int* token, const T* table, long long ld_table, int col,
                                                       int vocab, T* act, int dim, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / dim;
    const int c = int(i % dim);
    int tok = token[r];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    act[i] = to_act<T>(gelu_tanh_f(gate[r * ld_gate + c]) * act_f32(table[size_t(tok) * ld_table + col + c]));
  }
}

template <typename T>
struct QkvPostArgs {
  const float* qkv;   // [rows, H*d + G*d + G*dv]: the projection with its bias, or null:
  const bf16* qkv_bf16;  // the projection as the tcgen05 GEMM left it (bf16, no bias) and
  const float* bias;     // its bias [H*d + G*d + G*dv] (or null)
  const float* q_norm;  // [d] or null (no normalisation)
  const float* k_norm;  // [d] or null
  T* q_out;           // [rows, H*d]
  T* k_pages;         // [G, num_pages, tokens_per_page, d]
  T* v_pages;         // [G, num_pages, tokens_per_page, dv]
  float* v_shared;    // [rows, G*dv] values of the layer the others mix in (written when value_mix == 1, read when == 2)
  const int* group;
  const int* pos;
  const int* page_map;
  int heads, kv_heads, dim, vdim;
  int num_pages, tokens_per_page, max_pages;
  int value_mix;      // 0: none, 1: keep these values for later layers, 2: v = (1 - lambda) v + lambda v_shared
  float value_lambda, eps;
};

// one CTA per row; a warp per head for the norms
template <typename T>
__global__ void __launch_bounds__(256) qkv_post_kernel(const QkvPostArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim;
  const int n_all = H * d + G * d + G * dv;
  const float* rowf = a.qkv ? a.qkv + size_t(r) * n_all : nullptr;
  const bf16* rowb = a.qkv ? nullptr : a.qkv_bf16 + size_t(r) * n_all;
  auto val = [&](int c) { return rowf ? rowf[c] : __bfloat162float(rowb[c]) + (a.bias ? a.bias[c] : 0.0f); };
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  for (int u = warp; u < H + G; u += nw) {  // unit u: query head u, or key head u - H
    const bool is_q = u < H;
    const int src = is_q ? u * d : H * d + (u - H) * d;
    const float* w = is_q ? a.q_norm : a.k_norm;
    float ss = 0.0f;
    for (int c = lane; c < d; c += 32) {
      const float v = val(src + c);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = w ? 1.0f / sqrtf(ss / float(d) + a.eps) : 1.0f;
    T* dst = is_q ? a.q_out + size_t(r) * H * d + u * d
                  : a.k_pages + (size_t(u - H) * a.num_pages * a.tokens_per_page + slot) * d;
    for (int c = lane; c < d; c += 32) dst[c] = to_act<T>(w ? val(src + c) * inv * w[c] : val(src + c));
  }
  const int vsrc = H * d + G * d;
  for (int e = tid; e < G * dv; e += blockDim.x) {
    float v = val(vsrc + e);
    if (a.value_mix == 1) a.v_shared[size_t(r) * G * dv + e] = v;
    else if (a.value_mix == 2) v = (1.0f - a.value_lambda) * v + a.value_lambda * a.v_shared[size_t(r) * G * dv + e];
    const int kv = e / dv, c = e % dv;
    a.v_pages[(size_t(kv) * a.num_pages * a.tokens_per_page + slot) * dv + c] = to_act<T>(v);
  }
}

// (y as fp32, or -- y null -- as the bf16 matrix y_bf16 a tcgen05 GEMM left)
template <typename T>
__global__ void __launch_bounds__(256) norm_residual_kernel(const float* y, const bf16* y_bf16, float gain, float eps, float* x, T* xa, int width) {
  __shared__ float red[8];
  griddep_wait();
  const int r = blockIdx.x;
  const float* yf = y ? y + size_t(r) * width : nullptr;
  const bf16* yb = y ? nullptr : y_bf16 + size_t(r) * width;
  auto val = [&](int c) { return yf ? yf[c] : __bfloat162float(yb[c]); };
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = val(c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float f = gain / sqrtf(ss / float(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x[size_t(r) * width + c] + val(c) * f;
    x[size_t(r) * width + c] = v;
    xa[size_t(r) * width + c] = to_act<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) scalar_norm_rows_kernel(const float* x, const int* rows, float gain, float eps, T* out, int width) {
  __shared__ float red[8];
  griddep_wait();
  const int src = rows ? rows[blockIdx.x] : int(blockIdx.x);
  const float* xr = x + size_t(src) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
  ss = block_sum(ss, red);
  const float f = gain / sqrtf(ss / float(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[size_t(blockIdx.x) * width + c] = to_act<T>(xr[c] * f);
}

}  // namespace mtx
