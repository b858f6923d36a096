// Paged-KV decode attention (flash-decoding) for sm_100a.
//
// One CTA per (kv split, kv head, sequence).  The query rows of a CTA are the
// q_len new tokens x the GQA group of this kv head (at most 16 rows), held as
// MMA A-fragments in registers for the whole kernel.  Each of the four warps
// walks its own subset of 32-token KV pages: the page is fetched with TMA
// (128-byte swizzle, through the per-sequence block table) into a private
// 3-stage shared-memory ring, scores and P*V run on the tensor cores with
// m16n8k16 fragments fed by ldmatrix, and the online-softmax state stays in
// registers.  Warps are merged through shared memory; for long contexts the KV
// range is split over several CTAs, each writes its partial (accumulator, running
// maximum, denominator) to a scratch buffer and the CTA that arrives last at a
// per-(sequence, kv head) counter merges them, so the whole op is one launch.
//
// This op is bound by HBM traffic (the whole KV cache is read once per step),
// which is why it uses register-fragment MMAs instead of tcgen05: a 128-row
// TMEM tile would be 8-32x padded for 4-16 query rows, and the per-row softmax
// would be serialised on a handful of threads.
//
// KV cache layout: [num_blocks, kv_heads, block_size = 32, head_dim] bf16, so a
// page of one head is one contiguous 32 x head_dim slab.
//
// Reference parity: the decode branch of attention_kernel in
// examples/models/qwen3/kernels/attention.py:104-137 (scores against the whole
// static cache with an additive mask); sliding window and attention sinks from
// examples/models/gpt_oss/kernels/attention.py:116-148.  Paging, block tables
// and prefix sharing are new here.
#include "common.cuh"
#include "api.h"
#include <math.h>

namespace nkb {

constexpr int kPage = 32;
constexpr int kDecStages = 3;
// The scratch buffer starts with the arrival counters (one per sequence x kv head, at most this many), the
// split partials follow.  Counters must be zero before the first call and are reset by the merging CTA.
constexpr int kDecCounters = 16384;

struct DecodeParams {
  const __nv_bfloat16* q;
  const int* block_table;
  const int* context_lens;
  __nv_bfloat16* out;
  float* scratch;            // partials (behind the counters); nullptr when num_splits == 1
  unsigned int* counters;    // arrival counters of the split merge
  const float* sinks;
  int* status;
  int batch, q_len, nq, nkv, group, max_blocks, num_splits, window;
  float scale_log2;
  // Fused mode (qkv_partials != nullptr, q_len == 1): the kernel takes the split-K partials of the fused QKV
  // projection [splits][batch][(nq + 2 nkv) * D] instead of finished queries.  Every CTA builds its group's
  // query rows itself (sum, bias, QK-norm, rotate-halves RoPE); the CTA of split 0 also builds the new
  // token's key and value, writes them to their cache slot for later steps and adds them to the softmax
  // as one extra key, so the pages it streams stop one token earlier.  This removes the separate
  // RoPE + append launch from every layer of a decode step.
  const float* qkv_partials;
  long long qkv_split_stride;
  const __nv_bfloat16* qkv_bias;
  const int* positions;
  const int* slots;
  const float* cos_sin;
  const __nv_bfloat16* q_norm_w;
  const __nv_bfloat16* k_norm_w;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  float norm_eps;
  int qkv_splits, max_pos;
};

// One head row of the fused QKV output for token `tok`, in two steps so that a warp can have the loads of two
// heads in flight at once: `load` issues every global read the row needs (the partials of up to kFuseChunk splits,
// bias, norm weight, the cos / sin row), `finish` sums, normalises, rotates and rounds to bf16 the way the
// stand-alone RoPE kernel does.  One warp; lane owns elements lane * PER + j of each half.
constexpr int kFuseChunk = 8;
template <int D>
struct FusedRow {
  static constexpr int PER = D / 64;
  float x[kFuseChunk][PER], y[kFuseChunk][PER];
  float bx[PER], by[PER], wx[PER], wy[PER], c[PER], sn[PER];
  long long base;
  bool has_norm, rotate;

  __device__ __forceinline__ void load(const DecodeParams& p, int tok, int head, const __nv_bfloat16* norm_w,
                                       bool rot, int lane) {
    const int width = (p.nq + 2 * p.nkv) * D;
    base = (long long)tok * width + (long long)head * D + lane * PER;
    has_norm = norm_w != nullptr;
    rotate = rot && p.cos_sin != nullptr;
    int pos = rotate ? p.positions[tok] : 0;
#pragma unroll
    for (int q = 0; q < kFuseChunk; ++q) {
      const bool on = q < p.qkv_splits;
      const float* src = p.qkv_partials + (long long)q * p.qkv_split_stride + base;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        x[q][j] = on ? __ldcg(src + j) : 0.f;
        y[q][j] = on ? __ldcg(src + D / 2 + j) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane * PER + j;
      bx[j] = p.qkv_bias ? __bfloat162float(p.qkv_bias[head * D + i]) : 0.f;
      by[j] = p.qkv_bias ? __bfloat162float(p.qkv_bias[head * D + D / 2 + i]) : 0.f;
      wx[j] = has_norm ? __bfloat162float(norm_w[i]) : 1.f;
      wy[j] = has_norm ? __bfloat162float(norm_w[D / 2 + i]) : 1.f;
    }
    pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane * PER + j;
      c[j] = rotate ? p.cos_sin[(long long)pos * D + i] : 1.f;
      sn[j] = rotate ? p.cos_sin[(long long)pos * D + D / 2 + i] : 0.f;
    }
  }

  __device__ __forceinline__ void finish(const DecodeParams& p, float (&lo)[PER], float (&hi)[PER]) {
#pragma unroll
    for (int j = 0; j < PER; ++j) lo[j] = hi[j] = 0.f;
#pragma unroll
    for (int q = 0; q < kFuseChunk; ++q) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        lo[j] += x[q][j];
        hi[j] += y[q][j];
      }
    }
    // more splits than one chunk holds (rare): the rest in order, without the overlap
    for (int q = kFuseChunk; q < p.qkv_splits; ++q) {
      const float* src = p.qkv_partials + (long long)q * p.qkv_split_stride + base;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        lo[j] += __ldcg(src + j);
        hi[j] += __ldcg(src + D / 2 + j);
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      lo[j] += bx[j];
      hi[j] += by[j];
    }
    if (has_norm) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / float(D) + p.norm_eps);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        lo[j] = __bfloat162float(__float2bfloat16(lo[j] * inv * wx[j]));
        hi[j] = __bfloat162float(__float2bfloat16(hi[j] * inv * wy[j]));
      }
    }
    if (rotate) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const float a = lo[j], b = hi[j];
        lo[j] = a * c[j] - b * sn[j];
        hi[j] = b * c[j] + a * sn[j];
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      lo[j] = __bfloat162float(__float2bfloat16(lo[j]));
      hi[j] = __bfloat162float(__float2bfloat16(hi[j]));
    }
  }
};


__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}


template <int D, int kDecWarps>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const DecodeParams p) {
  constexpr int NH = D / 64;                 // 128-byte halves per row
  constexpr int kHalfBytes = kPage * 128;    // one [32 x 64] swizzled slab
  constexpr int kMatBytes = NH * kHalfBytes; // K (or V) page
  constexpr int kStageBytes = 2 * kMatBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[kDecWarps][kDecStages];
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int rows = p.q_len * p.group;

  if (threadIdx.x == 0) {
    for (int w = 0; w < kDecWarps; ++w)
      for (int s = 0; s < kDecStages; ++s) mbar_init(&bars[w][s], 1);
    abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  __syncthreads();
  griddep_wait();   // q, the cache and the tables come from the preceding kernels
  griddep_launch();
  const int ctx = p.context_lens[b];
  const bool fused = p.qkv_partials != nullptr;       // then q_len == 1
  const bool owner = fused && split == 0 && ctx > 0;   // this CTA handles the new token's key and value
  // tokens that are read from the cache pages: all of them, or all but the new one
  const int ctx_paged = fused ? ctx - 1 : ctx;

  // ---- page range of this split
  int first_tok = 0;
  if (p.window > 0) first_tok = max(0, ctx - p.q_len - p.window + 1);
  const int page_lo = first_tok / kPage, page_hi = (ctx_paged + kPage - 1) / kPage;
  const int npages = max(page_hi - page_lo, 0);
  const int per_split = (npages + p.num_splits - 1) / p.num_splits;
  const int p0 = page_lo + split * per_split;
  const int p1 = min(page_hi, p0 + per_split);
  const int* table = p.block_table + (long long)b * p.max_blocks;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  uint8_t* my_smem = smem + warp * kDecStages * kStageBytes;
  auto issue = [&](int page, int stage) {
    if (lane == 0) {
      const int blk = table[page];
      uint8_t* dst = my_smem + stage * kStageBytes;
      mbar_expect_tx(&bars[warp][stage], kStageBytes);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_4d(dst + h * kHalfBytes, &tmK, &bars[warp][stage], h * 64, 0, kvh, blk);
        tma_load_4d(dst + kMatBytes + h * kHalfBytes, &tmV, &bars[warp][stage], h * 64, 0, kvh, blk);
      }
    }
  };

  // ---- prologue
  const int my_first = p0 + warp;
#pragma unroll
  for (int s = 0; s < kDecStages; ++s) {
    const int pg = my_first + s * kDecWarps;
    if (pg < p1) issue(pg, s);
  }
  // (the first pages are in flight while the queries are built)
  __shared__ __align__(16) __nv_bfloat16 q_s[16 * D]; // the group's query rows (fused mode)
  __shared__ float kn_s[D], vn_s[D], snew_s[16];
  if (fused) {
    constexpr int PER = D / 64;
    // heads of this CTA: the group's queries, then (owner only) the key and the value of this kv head; a warp
    // takes two of them per round so that both rows' loads are in flight together
    const int nheads = p.group + (owner ? 2 : 0);
    const int slot = p.slots ? p.slots[b] : -1;
    auto head_of = [&](int hh) { return hh < p.group ? kvh * p.group + hh : (hh == p.group ? p.nq + kvh : p.nq + p.nkv + kvh); };
    auto store = [&](int hh, const float (&lo)[PER], const float (&hi)[PER]) {
      if (hh < p.group) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          q_s[hh * D + lane * PER + j] = __float2bfloat16(lo[j]);
          q_s[hh * D + D / 2 + lane * PER + j] = __float2bfloat16(hi[j]);
        }
        return;
      }
      const bool is_k = hh == p.group;
      float* dst_s = is_k ? kn_s : vn_s;
      __nv_bfloat16* dst = nullptr;
      if (slot >= 0) {
        const long long blk = slot / kPage, off = slot % kPage;
        dst = (is_k ? p.k_cache : p.v_cache) + ((blk * p.nkv + kvh) * kPage + off) * D;
      }
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane * PER + j;
        dst_s[i] = lo[j];
        dst_s[D / 2 + i] = hi[j];
        if (dst) {
          dst[i] = __float2bfloat16(lo[j]);
          dst[D / 2 + i] = __float2bfloat16(hi[j]);
        }
      }
    };
    for (int h0 = warp; h0 < nheads; h0 += 2 * kDecWarps) {
      const int h1 = h0 + kDecWarps;
      FusedRow<D> ra, rb;
      float lo[PER], hi[PER];
      ra.load(p, b, head_of(h0), h0 < p.group ? p.q_norm_w : (h0 == p.group ? p.k_norm_w : nullptr), h0 <= p.group, lane);
      if (h1 < nheads)
        rb.load(p, b, head_of(h1), h1 < p.group ? p.q_norm_w : (h1 == p.group ? p.k_norm_w : nullptr), h1 <= p.group, lane);
      ra.finish(p, lo, hi);
      store(h0, lo, hi);
      if (h1 < nheads) {
        rb.finish(p, lo, hi);
        store(h1, lo, hi);
      }
    }
    __syncthreads();
    if (owner) {
      // scores of the new token against the group's queries (log2 domain like the paged part)
      for (int r = warp; r < p.group; r += kDecWarps) {
        float acc = 0.f;
        for (int i = lane; i < D; i += 32) acc += __bfloat162float(q_s[r * D + i]) * kn_s[i];
        acc = warp_sum(acc);
        if (lane == 0) snew_s[r] = acc * p.scale_log2;
      }
    }
  }
  // ---- query fragments
  uint32_t qf[D / 16][4];
  {
    const int r0 = g, r1 = g + 8;
    const __nv_bfloat16* q0 = nullptr;
    const __nv_bfloat16* q1 = nullptr;
    if (r0 < rows)
      q0 = fused ? q_s + r0 * D
                 : p.q + (((long long)b * p.q_len + r0 / p.group) * p.nq + kvh * p.group + r0 % p.group) * D;
    if (r1 < rows)
      q1 = fused ? q_s + r1 * D
                 : p.q + (((long long)b * p.q_len + r1 / p.group) * p.nq + kvh * p.group + r1 % p.group) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
      qf[ks][1] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
      qf[ks][2] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
      qf[ks][3] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  // last visible kv position (inclusive) and first visible one, per owned row
  const int qpos0 = ctx - p.q_len + (g < rows ? g / p.group : 0);
  const int qpos1 = ctx - p.q_len + (g + 8 < rows ? (g + 8) / p.group : 0);
  const int lim0 = fused ? qpos0 - 1 : qpos0, lim1 = fused ? qpos1 - 1 : qpos1;   // fused: the new token is not paged
  const int low0 = p.window > 0 ? qpos0 - p.window + 1 : 0;
  const int low1 = p.window > 0 ? qpos1 - p.window + 1 : 0;

  int stage = 0;
  uint32_t phase = 0;
  for (int pg = my_first; pg < p1; pg += kDecWarps) {
    bool ok = mbar_wait(&bars[warp][stage], phase, &abort_flag, p.status, ERR_WAIT_SMEM_FULL);
    if (!__all_sync(0xffffffffu, ok)) break;
    const uint32_t kbase = smem_u32(my_smem + stage * kStageBytes);
    const uint32_t vbase = kbase + kMatBytes;

    // S = Q K^T for the 32 tokens of the page
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int kp = 0; kp < D / 32; ++kp) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int tok = nt * 8 + (lane & 7);
        const int chunk = 4 * kp + (lane >> 3);
        const uint32_t addr = kbase + (chunk >> 3) * kHalfBytes + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(addr, b0, b1, b2, b3);
        mma_16816(s[nt], qf[2 * kp], b0, b1);
        mma_16816(s[nt], qf[2 * kp + 1], b2, b3);
      }
    }
    // online softmax (base-2 domain)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = pg * kPage + nt * 8 + 2 * t + e;
        float v0 = s[nt][e] * p.scale_log2, v1 = s[nt][2 + e] * p.scale_log2;
        if (tok > lim0 || tok < low0) v0 = -INFINITY;
        if (tok > lim1 || tok < low1) v1 = -INFINITY;
        s[nt][e] = v0;
        s[nt][2 + e] = v1;
        mx0 = fmaxf(mx0, v0);
        mx1 = fmaxf(mx1, v1);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float a0 = exp2f(m0 - base0), a1 = exp2f(m1 - base1);
    m0 = mn0;
    m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[nt][e] = exp2f(s[nt][e] - base0);
        s[nt][2 + e] = exp2f(s[nt][2 + e] - base1);
        sum0 += s[nt][e];
        sum1 += s[nt][2 + e];
      }
    }
    l0 = l0 * a0 + sum0;
    l1 = l1 * a1 + sum1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= a0; o[i][1] *= a0;
      o[i][2] *= a1; o[i][3] *= a1;
    }
    // O += P V
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * j][0], s[2 * j][1]);
      pa[1] = pack_bf16x2(s[2 * j][2], s[2 * j][3]);
      pa[2] = pack_bf16x2(s[2 * j + 1][0], s[2 * j + 1][1]);
      pa[3] = pack_bf16x2(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        const int tok = 16 * j + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int chunk = 2 * dp + (lane >> 4);
        const uint32_t addr = vbase + (chunk >> 3) * kHalfBytes + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4);
        uint32_t v0, v1, v2, v3;
        ldsm_x4_t(addr, v0, v1, v2, v3);
        mma_16816(o[2 * dp], pa, v0, v1);
        mma_16816(o[2 * dp + 1], pa, v2, v3);
      }
    }
    __syncwarp();
    const int next = pg + kDecStages * kDecWarps;
    if (next < p1) issue(next, stage);
    if (++stage == kDecStages) { stage = 0; phase ^= 1u; }
  }
  // quad-reduce the row sums
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  if (abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();  // every load consumed: the ring can be reused as merge space

  // ---- merge the four warps through shared memory
  float* mo = reinterpret_cast<float*>(smem);             // [warp][16][D]
  float* mm = mo + kDecWarps * 16 * D;                    // [warp][16]
  float* ml = mm + kDecWarps * 16;                        // [warp][16]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    float* r0 = mo + (warp * 16 + g) * D + i * 8 + 2 * t;
    float* r1 = mo + (warp * 16 + g + 8) * D + i * 8 + 2 * t;
    r0[0] = o[i][0]; r0[1] = o[i][1];
    r1[0] = o[i][2]; r1[1] = o[i][3];
  }
  if (t == 0) {
    mm[warp * 16 + g] = m0; mm[warp * 16 + g + 8] = m1;
    ml[warp * 16 + g] = l0; ml[warp * 16 + g + 8] = l1;
  }
  __syncthreads();
  float* part = p.scratch
      ? p.scratch + (((long long)b * p.nkv + kvh) * p.num_splits + split) * (16 * D + 32)
      : nullptr;
  for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    float mf = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mf = fmaxf(mf, mm[w * 16 + r]);
    if (owner) mf = fmaxf(mf, snew_s[r]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mm[w * 16 + r];
      const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - mf);
      acc += sc * mo[(w * 16 + r) * D + d];
      l += sc * ml[w * 16 + r];
    }
    if (owner) {
      // the new token: one more key with probability mass exp2(score - max) and its value row
      const float sc = exp2f(snew_s[r] - mf);
      acc += sc * vn_s[d];
      l += sc;
    }
    if (p.num_splits == 1) {
      const int head = kvh * p.group + r % p.group;
      if (p.sinks) {
        const float sk = p.sinks[head] * 1.4426950408889634f;
        const float m2 = fmaxf(mf, sk);
        const float sc = (mf == -INFINITY) ? 0.f : exp2f(mf - m2);
        acc *= sc;
        l = l * sc + exp2f(sk - m2);
      }
      const float v = l > 0.f ? acc / l : 0.f;
      p.out[(((long long)b * p.q_len + r / p.group) * p.nq + head) * D + d] = __float2bfloat16(v);
    } else {
      part[r * D + d] = acc;
      if (d == 0) {
        part[16 * D + r] = mf;
        part[16 * D + 16 + r] = l;
      }
    }
  }
  if (p.num_splits == 1) return;

  // ---- split merge by the CTA that arrives last at this (sequence, kv head)'s counter
  __shared__ int is_last;
  __threadfence();                 // this CTA's partial is visible device-wide before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* ctr = p.counters + (long long)b * p.nkv + kvh;
    const unsigned int old = atomicAdd(ctr, 1u);
    const int last = old == unsigned(p.num_splits - 1);
    if (last) *ctr = 0u;           // ready for the next call (the next kernel starts after this grid)
    is_last = last;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* base = p.scratch + (((long long)b * p.nkv + kvh) * p.num_splits) * (16 * D + 32);
  for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    float mf = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) mf = fmaxf(mf, __ldcg(base + s * (16 * D + 32) + 16 * D + r));
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
      const float* ps = base + s * (16 * D + 32);
      const float ms = __ldcg(ps + 16 * D + r);
      const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - mf);
      acc += sc * __ldcg(ps + r * D + d);
      l += sc * __ldcg(ps + 16 * D + 16 + r);
    }
    const int head = kvh * p.group + r % p.group;
    if (p.sinks) {
      const float sk = p.sinks[head] * 1.4426950408889634f;
      const float m2 = fmaxf(mf, sk);
      const float sc = (mf == -INFINITY) ? 0.f : exp2f(mf - m2);
      acc *= sc;
      l = l * sc + exp2f(sk - m2);
    }
    const float v = l > 0.f ? acc / l : 0.f;
    p.out[(((long long)b * p.q_len + r / p.group) * p.nq + head) * D + d] = __float2bfloat16(v);
  }
}

template <int D, int kDecWarps>
static int launch_decode(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p, cudaStream_t s) {
  constexpr int kStageBytes = 2 * (D / 64) * kPage * 128;
  constexpr int smem = kDecWarps * kDecStages * kStageBytes + 1024;
  static_assert(kDecWarps * kDecStages * kStageBytes >= int((kDecWarps * 16 * D + kDecWarps * 32) * sizeof(float)),
                "merge space must fit in the KV ring");
  // the attribute is per device: remember which devices of this process have it
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(paged_attn_decode_kernel<D, kDecWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    attr_set[dev] = true;
  }
  dim3 grid(p.num_splits, p.nkv, p.batch);
  return launch_pdl(paged_attn_decode_kernel<D, kDecWarps>, grid, dim3(kDecWarps * 32), size_t(smem), s, tk, tv, p);
}

// Warps per CTA: every warp streams its own pages through a private 3-stage ring (48 KB at D = 128), so an SM
// holds four warps' rings whatever the CTA size.  The grid should fit the resident slots in one wave (a second,
// partly filled wave costs as much as a full one): four-warp CTAs while there is at most one CTA per SM, two-warp
// CTAs up to two per SM, one-warp CTAs (four per SM) beyond.
static int dispatch_decode(int head_dim, long long ctas, int sms, const CUtensorMap& tk, const CUtensorMap& tv,
                           const DecodeParams& p, cudaStream_t s) {
  const int warps = ctas <= sms ? 4 : (ctas <= 2LL * sms ? 2 : 1);
  if (head_dim == 128) {
    if (warps == 4) return launch_decode<128, 4>(tk, tv, p, s);
    if (warps == 2) return launch_decode<128, 2>(tk, tv, p, s);
    return launch_decode<128, 1>(tk, tv, p, s);
  }
  if (head_dim == 64) {
    if (warps == 4) return launch_decode<64, 4>(tk, tv, p, s);
    if (warps == 2) return launch_decode<64, 2>(tk, tv, p, s);
    return launch_decode<64, 1>(tk, tv, p, s);
  }
  return -2;
}

}  // namespace nkb

using namespace nkb;

extern "C" long long nkb_paged_attn_decode_scratch_floats(int batch, int q_len, int nq, int head_dim,
                                                          int num_splits) {
  (void)q_len;
  if (num_splits <= 1) return 0;
  // arrival counters first, then (upper bound) one partial per (sequence, kv head, split); kv heads <= nq
  return kDecCounters + (long long)batch * nq * num_splits * (16 * head_dim + 32);
}

extern "C" int nkb_paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     const int* context_lens, void* out, float* scratch, int batch, int q_len, int nq,
                                     int nkv, int head_dim, int block_size, int num_blocks, int max_blocks_per_seq,
                                     float scale, int window, const float* sinks, int num_splits, void* stream) {
  if (batch <= 0) return 0;
  if (block_size != kPage || nq % nkv != 0) return -2;
  const int group = nq / nkv;
  if (q_len * group > 16) return -2;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!scratch || (long long)batch * nkv > kDecCounters)) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  DecodeParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.block_table = block_table;
  p.context_lens = context_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.scratch = num_splits > 1 ? scratch + kDecCounters : nullptr;
  p.counters = reinterpret_cast<unsigned int*>(scratch);
  p.sinks = sinks;
  p.status = status_word();
  p.batch = batch; p.q_len = q_len; p.nq = nq; p.nkv = nkv; p.group = group;
  p.max_blocks = max_blocks_per_seq; p.num_splits = num_splits; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tk, tv;
  const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(kPage), uint64_t(nkv), uint64_t(num_blocks)};
  const uint64_t strides[3] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * kPage * 2,
                               uint64_t(head_dim) * kPage * nkv * 2};
  const uint32_t box[4] = {64, uint32_t(kPage), 1, 1};
  if (encode_tmap_bf16(&tk, k_cache, 4, dims, strides, box)) return -4;
  if (encode_tmap_bf16(&tv, v_cache, 4, dims, strides, box)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_decode(head_dim, (long long)batch * nkv * num_splits, num_sms(), tk, tv, p, s);
}

// Decode attention that starts from the split-K partials of the fused QKV projection: bias, QK-norm, RoPE and the
// append of the new token's key and value to the paged cache happen inside the attention kernel (q_len == 1).
// `context_lens` already counts the new token; `slots[b]` is its flat cache slot (negative: not stored).
extern "C" int nkb_paged_attn_decode_fused(const float* qkv_partials, int qkv_splits, long long qkv_split_stride,
                                           const void* qkv_bias, const int* positions, const int* slots,
                                           const float* cos_sin, const void* q_norm_w, const void* k_norm_w,
                                           float norm_eps, int max_pos, void* k_cache, void* v_cache,
                                           const int* block_table, const int* context_lens, void* out, float* scratch,
                                           int batch, int nq, int nkv, int head_dim, int block_size, int num_blocks,
                                           int max_blocks_per_seq, float scale, int window, const float* sinks,
                                           int num_splits, void* stream) {
  if (batch <= 0) return 0;
  if (block_size != kPage || nq % nkv != 0 || !qkv_partials || qkv_splits < 1 || !positions || !slots) return -2;
  const int group = nq / nkv;
  if (group > 16) return -2;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!scratch || (long long)batch * nkv > kDecCounters)) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  DecodeParams p{};
  p.block_table = block_table;
  p.context_lens = context_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.scratch = num_splits > 1 ? scratch + kDecCounters : nullptr;
  p.counters = reinterpret_cast<unsigned int*>(scratch);
  p.sinks = sinks;
  p.status = status_word();
  p.batch = batch; p.q_len = 1; p.nq = nq; p.nkv = nkv; p.group = group;
  p.max_blocks = max_blocks_per_seq; p.num_splits = num_splits; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.qkv_partials = qkv_partials;
  p.qkv_split_stride = qkv_split_stride;
  p.qkv_splits = qkv_splits;
  p.qkv_bias = reinterpret_cast<const __nv_bfloat16*>(qkv_bias);
  p.positions = positions;
  p.slots = slots;
  p.cos_sin = cos_sin;
  p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  p.norm_eps = norm_eps;
  p.max_pos = max_pos;
  CUtensorMap tk, tv;
  const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(kPage), uint64_t(nkv), uint64_t(num_blocks)};
  const uint64_t strides[3] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * kPage * 2,
                               uint64_t(head_dim) * kPage * nkv * 2};
  const uint32_t box[4] = {64, uint32_t(kPage), 1, 1};
  if (encode_tmap_bf16(&tk, k_cache, 4, dims, strides, box)) return -4;
  if (encode_tmap_bf16(&tv, v_cache, 4, dims, strides, box)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_decode(head_dim, (long long)batch * nkv * num_splits, num_sms(), tk, tv, p, s);
}

// ---------------------------------------------------------------------------
// Allocation-free variant (see no_alloc.h for who needs it and its limits).
// ---------------------------------------------------------------------------
#include "no_alloc.h"
#include <mutex>
#include <stdio.h>

namespace nkb {
// Arrival counters and split-KV partial results live here instead of in a caller-provided buffer.
// In host code this name is only a stand-in for the symbol: the device address
// is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[NKB_NOALLOC_SCRATCH_FLOATS];
static __device__ int g_noalloc_status;

struct NoAllocDevice {
  bool ready;
  float* scratch;
  int* status;
  int sms;
};
constexpr int kNoAllocMaxDevices = 64;
static NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
static std::mutex g_noalloc_mutex;   // the first calls of two host threads may meet in the set-up

// Once per device, with that device current: resolve the device addresses.
static int noalloc_setup(NoAllocDevice** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return NKB_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.ready) {
    void* sp = nullptr;
    void* st = nullptr;
    if (cudaGetSymbolAddress(&sp, g_noalloc_scratch) != cudaSuccess || sp == nullptr) return NKB_NOALLOC_SETUP_FAILED;
    if (cudaGetSymbolAddress(&st, g_noalloc_status) != cudaSuccess || st == nullptr) return NKB_NOALLOC_SETUP_FAILED;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return NKB_NOALLOC_SETUP_FAILED;
    d.scratch = static_cast<float*>(sp);
    d.status = static_cast<int*>(st);
    d.sms = sms;
    d.ready = true;
  }
  *out = &d;
  return 0;
}
}  // namespace nkb

extern "C" int nkb_noalloc_status(int reset) {
  NoAllocDevice* d = nullptr;
  if (int rc = noalloc_setup(&d)) return rc;
  int v = 0;
  if (cudaMemcpy(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return NKB_NOALLOC_SETUP_FAILED;
  if (reset && v) {
    const int zero = 0;
    cudaMemcpy(d->status, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

extern "C" int nkb_paged_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                             const int* block_table, const int* context_lens, void* out, int batch,
                                             int q_len, int nq, int nkv, int head_dim, int block_size, int num_blocks,
                                             int max_blocks_per_seq, float scale, int window, const float* sinks,
                                             int num_splits, void* stream) {
  if (batch <= 0) return 0;
  if (block_size != kPage || nkv <= 0 || nq % nkv != 0) return -2;
  const int group = nq / nkv;
  if (q_len * group > 16) return -2;
  if (head_dim != 64 && head_dim != 128) return -2;
  if (num_splits < 1) num_splits = 1;
  const long long counters = (long long)batch * nkv;
  const long long need =
      num_splits > 1 ? kDecCounters + (long long)batch * nkv * num_splits * (16 * head_dim + 32) : 0;
  if (need > NKB_NOALLOC_SCRATCH_FLOATS || (num_splits > 1 && counters > kDecCounters)) {
    fprintf(stderr,
            "nkb_paged_attn_decode_noalloc: needs %lld scratch floats (batch %d x kv heads %d x splits %d), the "
            "built-in array holds %lld; use fewer splits / a smaller batch or the allocating entry point\n",
            need, batch, nkv, num_splits, (long long)NKB_NOALLOC_SCRATCH_FLOATS);
    return NKB_NOALLOC_TOO_LARGE;
  }
  NoAllocDevice* d = nullptr;
  if (int rc = noalloc_setup(&d)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (num_splits > 1) {
    // The merge counts arrivals from zero.  A finished call leaves its counters at zero, but a call that gave
    // up in a bounded wait may not have: clear the ones this call uses (a memset, not an allocation).
    cudaError_t e = cudaMemsetAsync(d->scratch, 0, size_t(counters) * sizeof(unsigned int), s);
    if (e != cudaSuccess) return int(e);
  }
  DecodeParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.block_table = block_table;
  p.context_lens = context_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.scratch = num_splits > 1 ? d->scratch + kDecCounters : nullptr;
  p.counters = reinterpret_cast<unsigned int*>(d->scratch);
  p.sinks = sinks;
  p.status = d->status;
  p.batch = batch; p.q_len = q_len; p.nq = nq; p.nkv = nkv; p.group = group;
  p.max_blocks = max_blocks_per_seq; p.num_splits = num_splits; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tk, tv;
  const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(kPage), uint64_t(nkv), uint64_t(num_blocks)};
  const uint64_t strides[3] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * kPage * 2,
                               uint64_t(head_dim) * kPage * nkv * 2};
  const uint32_t box[4] = {64, uint32_t(kPage), 1, 1};
  if (encode_tmap_bf16(&tk, k_cache, 4, dims, strides, box)) return -4;
  if (encode_tmap_bf16(&tv, v_cache, 4, dims, strides, box)) return -4;
  return dispatch_decode(head_dim, (long long)batch * nkv * num_splits, d->sms, tk, tv, p, s);
}
