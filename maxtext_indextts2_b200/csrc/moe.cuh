// Routing of a mixture of experts for a ragged batch (the experts' matrix products are the grouped mode of linear_any.cuh).
//
//   moe_router_kernel   per row: the router's logits, fp32 accumulation
//   moe_route_kernel    per row: s = sigmoid(logits) (or, softmax set, the softmax over all experts); choice = s + correction; the experts of all but the keep_groups best groups
//                       (a group's score = the sum of its two largest choice scores) are barred; the `top` largest remaining choice
//                       scores are chosen (the lower index wins a tie); weights = s of the chosen / (their sum + 1e-20), or, plain set, s of the
//                       chosen as it is.  fp32.
//   moe_sort_kernel     one CTA: counts the (row, choice) entries per expert, lays the experts' slot ranges side by side
//                       (group_off), gives every entry a slot in its expert's range and records the row each slot reads.
//   moe_combine_kernel  y[row] (+)= sum over the row's choices, in the order of the choices, of weight * expert output of its slot.
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"

namespace mtx {

// logits[r, e] = <x[r, :], w[e, :]> with fp32 accumulation: one CTA per row, a warp per expert in turn (few experts, so a tile of
// a matrix-product kernel would be mostly padding and its k loop one long chain)
template <typename T>
__global__ void __launch_bounds__(256) moe_router_kernel(const T* x, const T* w, float* logits, int experts, int width) {
  griddep_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* xr = x + size_t(r) * width;
  // bf16 rows of whole 16-byte chunks: eight channels per load
  const bool vec = sizeof(T) == 2 && width % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  for (int e = warp; e < experts; e += 8) {
    const T* we = w + size_t(e) * width;
    float acc0 = 0.0f, acc1 = 0.0f;
    if (vec) {
      for (int c = lane * 8; c < width; c += 256) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xr + c), wv = *reinterpret_cast<const uint4*>(we + c);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __bfloat1622float2(xp[i]), wf = __bfloat1622float2(wp[i]);
          acc0 = fmaf(xf.x, wf.x, acc0);
          acc1 = fmaf(xf.y, wf.y, acc1);
        }
      }
    } else {
      int c = lane * 2;
      for (; c + 1 < width; c += 64) {
        acc0 = fmaf(act_f32(xr[c]), act_f32(we[c]), acc0);
        acc1 = fmaf(act_f32(xr[c + 1]), act_f32(we[c + 1]), acc1);
      }
      if (c < width) acc0 = fmaf(act_f32(xr[c]), act_f32(we[c]), acc0);
    }
    const float sum = warp_sum(acc0 + acc1);
    if (lane == 0) logits[size_t(r) * experts + e] = sum;
  }
}

struct MoeRouteArgs {
  const float* logits;      // [rows, experts]
  const float* correction;  // [experts] or null
  int* chosen;              // [rows, top]
  float* weight;            // [rows, top]
  int experts, top, groups, keep;
  int softmax;              // 1: s = softmax(logits) over all experts
  int plain;                // 1: weights = s of the chosen, not renormalised
};

// one warp per row; shared memory: 2 * experts + groups floats
__global__ void __launch_bounds__(32) moe_route_kernel(const MoeRouteArgs a) {
  extern __shared__ float sm[];
  float* s = sm;                  // [E] scores
  float* c = s + a.experts;       // [E] choice scores
  float* gs = c + a.experts;      // [groups]
  griddep_wait();
  const int r = blockIdx.x, lane = threadIdx.x, E = a.experts, per = E / a.groups;
  float zmax = -INFINITY, zsum = 1.0f;
  if (a.softmax) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, a.logits[size_t(r) * E + e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    zsum = 0.0f;
    for (int e = lane; e < E; e += 32) zsum += expf(a.logits[size_t(r) * E + e] - zmax);
    zsum = warp_sum(zsum);
  }
  for (int e = lane; e < E; e += 32) {
    const float z = a.logits[size_t(r) * E + e];
    const float v = a.softmax ? expf(z - zmax) / zsum : 1.0f / (1.0f + expf(-z));
    s[e] = v;
    c[e] = v + (a.correction ? a.correction[e] : 0.0f);
  }
  __syncwarp();
  if (a.groups > 1 && a.keep < a.groups) {
    for (int g = lane; g < a.groups; g += 32) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = c[e];
        if (v > b1) {
          b2 = b1;
          b1 = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      gs[g] = per >= 2 ? b1 + b2 : b1;
    }
    __syncwarp();
    for (int g = lane; g < a.groups; g += 32) {
      int ahead = 0;
      for (int o = 0; o < a.groups; ++o) ahead += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
      if (ahead >= a.keep)
        for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.0f;
  for (int k = 0; k < a.top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > best) {  // (ascending e: the lowest index of equal scores stays)
        best = c[e];
        at = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (at == 0x7fffffff) at = 0;  // (fewer admissible experts than `top`: cannot happen for a valid config)
    total += s[at];
    if (lane == 0) {
      a.chosen[size_t(r) * a.top + k] = at;
      c[at] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = lane; k < a.top; k += 32) a.weight[size_t(r) * a.top + k] = s[a.chosen[size_t(r) * a.top + k]] / (a.plain ? 1.0f : total + 1e-20f);
}

// shared memory: (2 * experts + 1) ints
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* chosen, int entries, int top, int experts, int* group_off, int* slot_of, int* a_row) {
  extern __shared__ int si[];
  int* count = si;               // [E]
  int* start = count + experts;  // [E + 1]
  griddep_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) atomicAdd(&count[chosen[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      at += count[e];
    }
    start[experts] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) group_off[e] = start[e];
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int p = atomicAdd(&start[chosen[i]], 1);
    slot_of[i] = p;
    a_row[p] = i / top;
  }
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float* ye, const int* slot_of, const float* weight, int top, int width, int add, float* y) {
  griddep_wait();
  const int r = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = add ? y[size_t(r) * width + c] : 0.0f;
    for (int k = 0; k < top; ++k) v = fmaf(weight[size_t(r) * top + k], ye[size_t(slot_of[size_t(r) * top + k]) * width + c], v);
    y[size_t(r) * width + c] = v;
  }
}

}  // namespace mtx
