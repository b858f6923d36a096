// Memory-bound helper kernels of the model layer: RMSNorm (optionally fused with
// the split-K / tensor-parallel partial-sum reduction and the residual add),
// SwiGLU gate, embedding gather, RoPE + QK-norm + paged KV-cache append.
//
// Reference parity (behaviour, not code): rmsnorm_kernel in
// examples/models/qwen3/kernels/rmsnorm.py:4-21 (fp32 statistics, eps inside the
// sqrt, weight multiply, cast back); rotate-halves RoPE in
// examples/models/qwen3/kernels/rope.py:23-48; SwiGLU in
// examples/models/qwen3/kernels/feedforward.py:4-18 and the clamped variant in
// examples/models/gpt_oss/kernels/feedforward.py:6-18; in-place KV-cache write
// in examples/models/qwen3/kernels/attention.py:100-106.
#include "common.cuh"
#include "api.h"

namespace nkb {

constexpr int kNormMaxIters = 4;  // 8 elements per thread per iteration

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// h = sum_s partials[s] (+ x) (+ bias) (+ residual_in);  residual_out = h;
// normed_out = h * rsqrt(mean(h^2) + eps) * w        (skipped when w == nullptr)
__global__ void add_rmsnorm_kernel(const float* __restrict__ partials, int splits, long long split_stride,
                                   const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual_in,
                                   const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ residual_out, __nv_bfloat16* __restrict__ normed_out,
                                   int hidden, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = hidden >> 3;
  griddep_wait();
  griddep_launch();
  float h[kNormMaxIters][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kNormMaxIters; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      const long long off = row * hidden + (long long)v * 8;
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float4* p = reinterpret_cast<const float4*>(partials + s * split_stride + off);
        float4 p0 = p[0], p1 = p[1];
        a[0] += p0.x; a[1] += p0.y; a[2] += p0.z; a[3] += p0.w;
        a[4] += p1.x; a[5] += p1.y; a[6] += p1.z; a[7] += p1.w;
      }
      auto add_bf16 = [&](const __nv_bfloat16* src, long long o) {
        uint4 r = *reinterpret_cast<const uint4*>(src + o);
        uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = unpack_bf16x2(rw[e]);
          a[2 * e] += f.x;
          a[2 * e + 1] += f.y;
        }
      };
      if (x) add_bf16(x, off);
      if (bias) add_bf16(bias, (long long)v * 8);
      if (residual_in) add_bf16(residual_in, off);
      if (residual_out) {
        uint4 o;
        o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
        o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
        *reinterpret_cast<uint4*>(residual_out + off) = o;
        // statistics are taken from the bf16-rounded stream, exactly what an
        // unfused norm reading the stored residual would see
        uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = unpack_bf16x2(ow[e]);
          a[2 * e] = f.x;
          a[2 * e + 1] = f.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        h[it][j] = a[j];
        ss += a[j] * a[j];
      }
    }
  }
  if (!w) return;
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / float(hidden) + eps);
#pragma unroll
  for (int it = 0; it < kNormMaxIters; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      const long long off = row * hidden + (long long)v * 8;
      uint4 wr = *reinterpret_cast<const uint4*>(w + (long long)v * 8);
      uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = unpack_bf16x2(ww[e]);
        o[e] = pack_bf16x2(h[it][2 * e] * inv * f.x, h[it][2 * e + 1] * inv * f.y);
      }
      *reinterpret_cast<uint4*>(normed_out + off) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// out[t, i] = act(gate[t, i]) * up[t, i], gate_up = [gate | up] along the last axis.
// limit <= 0: plain SiLU gate.  limit > 0: clamped variant
//   gate = min(gate, limit); up = clamp(up, -limit, limit); out = (up + 1) * gate * sigmoid(alpha * gate)
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows,
                                int inter, float limit, float alpha) {
  const long long nvec = (long long)rows * (inter >> 3);
  griddep_wait();
  griddep_launch();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (inter >> 3);
    const int c = int(i % (inter >> 3)) * 8;
    uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + c);
    uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + inter + c);
    uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 gf = unpack_bf16x2(gw[e]), uf = unpack_bf16x2(uw[e]);
      float r0, r1;
      if (limit > 0.f) {
        float g0 = fminf(gf.x, limit), g1 = fminf(gf.y, limit);
        float u0 = fminf(fmaxf(uf.x, -limit), limit), u1 = fminf(fmaxf(uf.y, -limit), limit);
        r0 = (u0 + 1.f) * g0 / (1.f + __expf(-alpha * g0));
        r1 = (u1 + 1.f) * g1 / (1.f + __expf(-alpha * g1));
      } else {
        r0 = gf.x / (1.f + __expf(-gf.x)) * uf.x;
        r1 = gf.y / (1.f + __expf(-gf.y)) * uf.y;
      }
      o[e] = pack_bf16x2(r0, r1);
    }
    *reinterpret_cast<uint4*>(out + r * inter + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Same gate, fed by split-K fp32 partials [S, rows, 2 * inter] of the gate_up GEMM
// (used when the fused-gate GEMM would have too few tiles to fill the GPU).
__global__ void silu_mul_partials_kernel(const float* __restrict__ parts, int splits, long long stride,
                                         const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                         int rows, int inter, float limit, float alpha) {
  const long long nvec = (long long)rows * (inter >> 2);
  griddep_wait();
  griddep_launch();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (inter >> 2);
    const int c = int(i % (inter >> 2)) * 4;
    float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float4 gv = *reinterpret_cast<const float4*>(parts + s * stride + r * 2 * inter + c);
      const float4 uv = *reinterpret_cast<const float4*>(parts + s * stride + r * 2 * inter + inter + c);
      g[0] += gv.x; g[1] += gv.y; g[2] += gv.z; g[3] += gv.w;
      u[0] += uv.x; u[1] += uv.y; u[2] += uv.z; u[3] += uv.w;
    }
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float gg = g[e], uu = u[e];
      if (bias) {
        gg += __bfloat162float(bias[c + e]);
        uu += __bfloat162float(bias[inter + c + e]);
      }
      if (limit > 0.f) {
        gg = fminf(gg, limit);
        uu = fminf(fmaxf(uu, -limit), limit);
        o[e] = (uu + 1.f) * gg / (1.f + __expf(-alpha * gg));
      } else {
        o[e] = gg / (1.f + __expf(-gg)) * uu;
      }
    }
    uint2 pk;
    pk.x = pack_bf16x2(o[0], o[1]);
    pk.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(out + r * inter + c) = pk;
  }
}

__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int n, int hidden, int vocab) {
  const int t = blockIdx.x;
  griddep_wait();
  griddep_launch();
  int id = ids[t];
  if (id < 0) id = 0;
  if (id >= vocab) id = vocab - 1;
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)id * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * hidden);
  for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) dst[v] = src[v];
}

// One warp per (token, head).  Heads [0, nq) are queries, [nq, nq+nkv) keys,
// [nq+nkv, nq+2nkv) values of the fused QKV row.  Queries/keys optionally get a
// per-head RMSNorm (Qwen3) and then the rotate-halves rotation; keys and values
// are written to their slot (block * block_size + offset) of the paged cache
// [block, kv_head, token_in_block, head_dim].
// head_dim must be 64, 128 or 256 (each lane owns pairs (i, i + d/2)).
template <int D>
__global__ void rope_kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ partials,
                                      int splits, long long split_stride, const __nv_bfloat16* __restrict__ bias,
                                      const int* __restrict__ positions, const int* __restrict__ slots,
                                      const float* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ q_norm_w,
                                      const __nv_bfloat16* __restrict__ k_norm_w, float norm_eps,
                                      __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                      __nv_bfloat16* __restrict__ v_cache, int tokens, int nq, int nkv, int max_pos,
                                      int block_size) {
  constexpr int PER = D / 64;  // elements per lane in each half
  const int heads = nq + 2 * nkv;
  const long long gw = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  griddep_wait();
  griddep_launch();
  if (gw >= (long long)tokens * heads) return;
  const int t = int(gw / heads), h = int(gw % heads);
  const int width = heads * D;
  const long long base = (long long)t * width + (long long)h * D;
  float lo[PER], hi[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane * PER + j;
    float a = 0.f, b = 0.f;
    if (partials) {
      for (int s = 0; s < splits; ++s) {
        a += partials[s * split_stride + base + i];
        b += partials[s * split_stride + base + D / 2 + i];
      }
    } else {
      a = __bfloat162float(qkv[base + i]);
      b = __bfloat162float(qkv[base + D / 2 + i]);
    }
    if (bias) {
      a += __bfloat162float(bias[h * D + i]);
      b += __bfloat162float(bias[h * D + D / 2 + i]);
    }
    lo[j] = a;
    hi[j] = b;
  }
  const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
  const int slot = slots ? slots[t] : -1;
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / float(D) + norm_eps);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane * PER + j;
        // round to bf16 after the norm like an unfused implementation would
        lo[j] = __bfloat162float(__float2bfloat16(lo[j] * inv * __bfloat162float(nw[i])));
        hi[j] = __bfloat162float(__float2bfloat16(hi[j] * inv * __bfloat162float(nw[D / 2 + i])));
      }
    }
    if (cos_sin) {
      int pos = positions[t];
      pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
      const float* cs = cos_sin + (long long)pos * D;  // [cos(d/2) | sin(d/2)]
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane * PER + j;
        const float c = cs[i], s = cs[D / 2 + i];
        const float a = lo[j], b = hi[j];
        lo[j] = a * c - b * s;
        hi[j] = b * c + a * s;
      }
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (long long)t * nq * D + (long long)h * D;
  } else {
    if (slot < 0) return;
    const int kh = is_k ? h - nq : h - nq - nkv;
    // cache layout [block, kv_head, token_in_block, D]
    const long long blk = slot / block_size, off = slot % block_size;
    dst = (is_k ? k_cache : v_cache) + ((blk * nkv + kh) * block_size + off) * D;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane * PER + j;
    dst[i] = __float2bfloat16(lo[j]);
    dst[D / 2 + i] = __float2bfloat16(hi[j]);
  }
}

}  // namespace nkb

using namespace nkb;

static inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" int nkb_add_rmsnorm(const float* partials, int splits, long long split_stride, const void* x,
                               const void* residual_in, const void* bias, const void* w, void* residual_out,
                               void* normed_out, int rows, int hidden, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (hidden & 7) return -2;
  const int nvec = hidden >> 3;
  if (nvec > 1024 * kNormMaxIters) return -2;
  int threads = ((nvec + kNormMaxIters - 1) / kNormMaxIters + 31) / 32 * 32;
  if (nvec <= 1024) threads = (nvec + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (!partials) splits = 0;
  return launch_pdl(add_rmsnorm_kernel, dim3(rows), dim3(threads), 0, S(stream), partials, splits, split_stride,
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual_in, (const __nv_bfloat16*)bias,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)residual_out, (__nv_bfloat16*)normed_out, hidden, eps);
}

extern "C" int nkb_rmsnorm(const void* x, const void* w, void* out, int rows, int hidden, float eps, void* stream) {
  return nkb_add_rmsnorm(nullptr, 0, 0, x, nullptr, nullptr, w, nullptr, out, rows, hidden, eps, stream);
}

extern "C" int nkb_silu_mul(const void* gate_up, void* out, int rows, int inter, float limit, float alpha,
                            void* stream) {
  if (rows <= 0) return 0;
  if (inter & 7) return -2;
  long long nvec = (long long)rows * (inter >> 3);
  int blocks = int((nvec + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), 0, S(stream), (const __nv_bfloat16*)gate_up,
                    (__nv_bfloat16*)out, rows, inter, limit, alpha);
}

extern "C" int nkb_silu_mul_partials(const float* partials, int splits, long long stride, const void* bias, void* out,
                                     int rows, int inter, float limit, float alpha, void* stream) {
  if (rows <= 0) return 0;
  if (inter & 3) return -2;
  long long nvec = (long long)rows * (inter >> 2);
  int blocks = int((nvec + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_pdl(silu_mul_partials_kernel, dim3(blocks), dim3(256), 0, S(stream), partials, splits, stride,
                    (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, rows, inter, limit, alpha);
}

extern "C" int nkb_embedding(const int* ids, const void* table, void* out, int n, int hidden, int vocab,
                             void* stream) {
  if (n <= 0) return 0;
  if (hidden & 7) return -2;
  return launch_pdl(embedding_kernel, dim3(n), dim3(128), 0, S(stream), ids, (const __nv_bfloat16*)table,
                    (__nv_bfloat16*)out, n, hidden, vocab);
}

extern "C" int nkb_rope_kv_append(const void* qkv_bf16, const float* qkv_partials, int splits, long long split_stride,
                                  const void* bias, const int* positions, const int* slots, const float* cos_sin,
                                  const void* q_norm_w, const void* k_norm_w, float norm_eps, void* q_out,
                                  void* k_cache, void* v_cache, int tokens, int nq, int nkv, int head_dim, int max_pos,
                                  int block_size, void* stream) {
  if (tokens <= 0) return 0;
  const long long warps = (long long)tokens * (nq + 2 * nkv);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
#define NKB_ROPE(D)                                                                                               \
  return launch_pdl(rope_kv_append_kernel<D>, dim3((unsigned)blocks), dim3(threads), 0, S(stream),                \
                    (const __nv_bfloat16*)qkv_bf16, qkv_partials, splits, split_stride,                           \
                    (const __nv_bfloat16*)bias, positions, slots, cos_sin, (const __nv_bfloat16*)q_norm_w,        \
                    (const __nv_bfloat16*)k_norm_w, norm_eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,     \
                    (__nv_bfloat16*)v_cache, tokens, nq, nkv, max_pos, block_size)
  switch (head_dim) {
    case 64: NKB_ROPE(64);
    case 128: NKB_ROPE(128);
    case 256: NKB_ROPE(256);
    default: return -2;
  }
#undef NKB_ROPE
}

namespace nkb {
// Per-step bookkeeping of a decode batch, done on the device so a captured
// graph can be replayed without host writes: the new token of sequence b goes
// to position context_lens[b]; its cache slot comes from the block table; the
// context length grows by q_len.  Inactive sequences (context_lens < 0) are
// skipped and get slot -1.
__global__ void decode_advance_kernel(int* __restrict__ context_lens, const int* __restrict__ block_table,
                                      int* __restrict__ positions, int* __restrict__ slots, int batch, int q_len,
                                      int max_blocks, int block_size) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  griddep_wait();
  griddep_launch();
  if (i >= batch * q_len) return;
  const int b = i / q_len, j = i % q_len;
  const int ctx = context_lens[b];
  if (ctx < 0) {
    positions[i] = 0;
    slots[i] = -1;
    return;
  }
  const int pos = ctx + j;
  const int page = pos / block_size;
  positions[i] = pos;
  slots[i] = page < max_blocks ? block_table[(long long)b * max_blocks + page] * block_size + pos % block_size : -1;
}
__global__ void add_int_kernel(int* __restrict__ v, int n, int delta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  griddep_wait();
  griddep_launch();
  if (i < n && v[i] >= 0) v[i] += delta;
}
}  // namespace nkb

extern "C" int nkb_decode_advance(int* context_lens, const int* block_table, int* positions, int* slots, int batch,
                                  int q_len, int max_blocks, int block_size, void* stream) {
  if (batch <= 0) return 0;
  const int n = batch * q_len;
  int rc = launch_pdl(nkb::decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, S(stream), context_lens,
                      block_table, positions, slots, batch, q_len, max_blocks, block_size);
  if (rc) return rc;
  return launch_pdl(nkb::add_int_kernel, dim3((batch + 127) / 128), dim3(128), 0, S(stream), context_lens, batch,
                    q_len);
}
