// Token selection kernels: greedy argmax over the (vocab-parallel) logits,
// temperature / top-k / top-p sampling, and the MoE router (softmax + top-k +
// renormalise, both orders used by the model families).
//
// Reference parity: greedy_sampling in examples/models/qwen3/kernels/sampling.py:113-147
// (local top-1 -> gather over ranks -> global id = rank * V/tp + local); Qwen3
// router order softmax -> top-k -> renorm in
// examples/models/qwen3/kernels/transformer_layer.py:86-91; gpt-oss order
// top-k on raw logits -> softmax over the selected in
// examples/models/gpt_oss/kernels/feedforward.py:59-68.
#include "common.cuh"
#include "api.h"
#include <float.h>

namespace nkb {

__device__ __forceinline__ float load_logit(const void* p, int is_fp32, long long i) {
  return is_fp32 ? reinterpret_cast<const float*>(p)[i]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Larger value wins; on ties the smaller index wins (first occurrence).
__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

__global__ void argmax_kernel(const void* __restrict__ logits, int is_fp32, int* __restrict__ out_ids,
                              float* __restrict__ out_vals, int vocab, long long ld) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const long long row = blockIdx.x;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  griddep_wait();
  griddep_launch();
  if (!is_fp32 && (ld % 8 == 0)) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(logits) + row * ld);
    const int nvec = vocab >> 3;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 r = p[v];
      uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = unpack_bf16x2(w[e]);
        argmax_combine(best, bi, f.x, v * 8 + 2 * e);
        argmax_combine(best, bi, f.y, v * 8 + 2 * e + 1);
      }
    }
    for (int i = (nvec << 3) + threadIdx.x; i < vocab; i += blockDim.x)
      argmax_combine(best, bi, load_logit(logits, 0, row * ld + i), i);
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
      argmax_combine(best, bi, load_logit(logits, is_fp32, row * ld + i), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine(best, bi, ov, oi);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sv[lane] : -FLT_MAX;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_combine(best, bi, ov, oi);
    }
    if (lane == 0) {
      out_ids[row] = bi;
      if (out_vals) out_vals[row] = best;
    }
  }
}

// ---------------------------------------------------------------------------
// Sampling: candidates = the (at most) kCand most likely tokens of the row,
// found with a 4-pass radix select on the order-preserving integer image of the
// logits; then sorted in shared memory, softmax with temperature, top-k / top-p
// cut, inverse-CDF draw with a counter-based hash RNG.
// ---------------------------------------------------------------------------
constexpr int kCand = 1024;

__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending order-preserving
}
__device__ __forceinline__ uint32_t hash_u32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return uint32_t(x >> 16);
}

__global__ void __launch_bounds__(1024) sample_kernel(const void* __restrict__ logits, int is_fp32,
                                                      int* __restrict__ out_ids, int vocab, long long ld,
                                                      float temperature, int top_k, float top_p,
                                                      unsigned long long seed, unsigned long long step) {
  __shared__ int hist[256];
  __shared__ float cval[kCand];
  __shared__ int cidx[kCand];
  __shared__ int s_count;
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ float s_red[32];
  const long long row = blockIdx.x;
  griddep_wait();
  griddep_launch();
  const int want = (top_k > 0 && top_k < kCand) ? top_k : kCand;
  const int k = want < vocab ? want : vocab;

  // radix select the k-th largest key
  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      uint32_t key = float_key(load_logit(logits, is_fp32, row * ld + i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int rem = s_remaining, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= rem) break;
        rem -= hist[b];
      }
      s_prefix = prefix | (uint32_t(b) << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;  // key of the k-th largest logit
  if (threadIdx.x == 0) s_count = 0;
  for (int i = threadIdx.x; i < kCand; i += blockDim.x) { cval[i] = -FLT_MAX; cidx[i] = 0x7fffffff; }
  __syncthreads();
  // strictly greater first, then fill ties up to k (lowest indices are not guaranteed among ties)
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = load_logit(logits, is_fp32, row * ld + i);
    if (float_key(v) > kth) {
      int p = atomicAdd(&s_count, 1);
      if (p < kCand) { cval[p] = v; cidx[p] = i; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = load_logit(logits, is_fp32, row * ld + i);
    if (float_key(v) == kth) {
      int p = atomicAdd(&s_count, 1);
      if (p < k) { cval[p] = v; cidx[p] = i; }
    }
  }
  __syncthreads();
  // bitonic sort, descending by (value, then ascending index)
  for (int size = 2; size <= kCand; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < kCand / 2; t += blockDim.x) {
        int lo = (t / stride) * stride * 2 + (t % stride);
        int hi = lo + stride;
        bool desc = ((lo & size) == 0);
        float a = cval[lo], b = cval[hi];
        int ia = cidx[lo], ib = cidx[hi];
        bool a_first = (a > b) || (a == b && ia < ib);
        if (a_first != desc) { cval[lo] = b; cval[hi] = a; cidx[lo] = ib; cidx[hi] = ia; }
      }
      __syncthreads();
    }
  }
  // softmax over the k candidates with temperature
  const float inv_t = 1.f / fmaxf(temperature, 1e-6f);
  const float mx = cval[0];
  float local = 0.f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    float e = __expf((cval[i] - mx) * inv_t);
    cval[i] = e;
    local += e;
  }
  local = warp_sum(local);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) tot += s_red[w];
    // nucleus cut: smallest prefix with mass >= top_p
    float target = (top_p > 0.f && top_p < 1.f) ? top_p * tot : tot;
    float acc = 0.f;
    int n = 0;
    for (; n < k; ++n) {
      acc += cval[n];
      if (acc >= target) { ++n; break; }
    }
    if (n > k) n = k;
    if (n < 1) n = 1;
    float mass = 0.f;
    for (int i = 0; i < n; ++i) mass += cval[i];
    uint32_t r = hash_u32(seed * 0x9E3779B97F4A7C15ULL + step * 0xD1B54A32D192ED03ULL + uint64_t(row));
    float u = (float(r >> 8) + 0.5f) * (1.f / 16777216.f) * mass;
    float c = 0.f;
    int pick = n - 1;
    for (int i = 0; i < n; ++i) {
      c += cval[i];
      if (u <= c) { pick = i; break; }
    }
    out_ids[row] = cidx[pick];
  }
}

// ---------------------------------------------------------------------------
// MoE router: one warp per token, num_experts <= 1024.
//   mode 0: softmax over all experts -> top-k -> divide by the selected sum
//   mode 1: top-k on raw logits -> softmax over the selected
// ---------------------------------------------------------------------------
// logits may be bf16 / fp32 [tokens, E] or fp32 split-K partials [splits, tokens, E] (summed here, plus bias)
__global__ void router_topk_kernel(const void* __restrict__ logits, int is_fp32, int splits, long long split_stride,
                                   const __nv_bfloat16* __restrict__ bias, float* __restrict__ weights,
                                   int* __restrict__ experts, int tokens, int num_experts, int top_k, int mode) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  griddep_wait();
  griddep_launch();
  if (warp >= tokens) return;
  constexpr int kPer = 32;
  float v[kPer];
  const int per = (num_experts + 31) / 32;
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int e = j * 32 + lane;
    if (j < per && e < num_experts) {
      float a = load_logit(logits, is_fp32, (long long)warp * num_experts + e);
      for (int s = 1; s < splits; ++s)
        a += reinterpret_cast<const float*>(logits)[s * split_stride + (long long)warp * num_experts + e];
      if (bias) a += __bfloat162float(bias[e]);
      v[j] = a;
    } else {
      v[j] = -FLT_MAX;
    }
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float denom = 1.f;
  if (mode == 0) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kPer; ++j)
      if (j < per && v[j] > -FLT_MAX) s += __expf(v[j] - mx);
    denom = warp_sum(s);
  }
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int r = 0; r < top_k; ++r) {
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kPer; ++j)
      if (j < per) argmax_combine(best, bi, v[j], j * 32 + lane);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_combine(best, bi, ov, oi);
    }
    // mode 0 weight = softmax prob; mode 1 weight = exp(logit - max selected) (first pick is the max)
    const float wgt = (mode == 0) ? __expf(best - mx) / denom : __expf(best - mx);
    sel_sum += wgt;
    if (lane == r % 32 && r / 32 == 0) { my_w = wgt; my_e = bi; }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kPer; ++j)
        if (j == (bi >> 5)) v[j] = -FLT_MAX;
    }
  }
  if (lane < top_k) {
    weights[(long long)warp * top_k + lane] = my_w / sel_sum;
    experts[(long long)warp * top_k + lane] = my_e;
  }
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_argmax(const void* logits, int is_fp32, int* out_ids, float* out_vals, int rows, int vocab,
                          long long ld, void* stream) {
  if (rows <= 0) return 0;
  return launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), logits, is_fp32,
                    out_ids, out_vals, vocab, ld);
}

extern "C" int nkb_sample(const void* logits, int is_fp32, int* out_ids, int rows, int vocab, long long ld,
                          float temperature, int top_k, float top_p, unsigned long long seed,
                          unsigned long long step, void* stream) {
  if (rows <= 0) return 0;
  return launch_pdl(sample_kernel, dim3(rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), logits, is_fp32,
                    out_ids, vocab, ld, temperature, top_k, top_p, seed, step);
}

extern "C" int nkb_router_topk(const void* logits, int is_fp32, int splits, long long split_stride, const void* bias,
                               float* weights, int* experts, int tokens, int num_experts, int top_k, int mode,
                               void* stream) {
  if (tokens <= 0) return 0;
  if (num_experts > 1024 || top_k > 32 || top_k > num_experts) return -2;
  const int threads = 128;
  const int blocks = (tokens * 32 + threads - 1) / threads;
  if (splits < 1) splits = 1;
  if (splits > 1 && !is_fp32) return -2;
  return launch_pdl(router_topk_kernel, dim3(blocks), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), logits,
                    is_fp32, splits, split_stride, (const __nv_bfloat16*)bias, weights, experts, tokens, num_experts,
                    top_k, mode);
}
