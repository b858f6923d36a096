// Split-K "fix-up" epilogues of the decode-orientation GEMM (gemm_tcgen05.cuh).
//
// A decode-sized projection has too few 128-feature tiles to fill the GPU, so its
// contraction is split over several CTAs.  Each CTA stores its fp32 partial tile to a
// scratch array in global memory (it stays in L2) and bumps a per-tile arrival
// counter; the CTA that arrives last sums the partials of the tile and applies the
// epilogue that needs finished values right there, inside the GEMM kernel:
//
//   FIX_STORE   bf16 output (+ bias, + residual)
//   FIX_SWIGLU  silu(gate) * up for the [gate; up] projection (the gate tile and the up tile of
//               the same 128 output features share one counter)
//   FIX_ROPE    the fused QKV projection: bias, per-head QK-RMSNorm, rotate-halves RoPE, the write
//               of K / V into the paged cache and of Q into its buffer
//   FIX_PUSH    one bf16 partial per rank stored into every tensor-parallel peer's symmetric
//               buffer (plain peer stores over NVLink): the producer half of the fused all-reduce
//
// so the separate "sum the partials" kernels (and their launches) disappear from the decode step.
// Counters must be zero before the first launch; the last arriver resets its counter.
//
// Reference parity: the reference compiles projection + activation / rotary embedding / all-reduce into one
// device program per layer (examples/models/qwen3/kernels/attention.py:72-154, kernels/feedforward.py:4-18).
#pragma once
#include "common.cuh"
#include "gemm_args.h"

namespace nkb {

enum : int { FIX_NONE = 0, FIX_STORE = 1, FIX_SWIGLU = 2, FIX_ROPE = 3, FIX_PUSH = 4 };

struct FixCommon {
  float* partials;               // [splits][tokens][ld] fp32 scratch
  unsigned int* tile_counters;   // one per row tile (SWIGLU: per gate / up tile pair)
  long long ld;                  // row length of the partial array = number of GEMM rows (features)
  const __nv_bfloat16* bias;     // [features] or nullptr
};

struct NoFix {
  static constexpr int kind = FIX_NONE;
  struct Args {};
};
struct StoreFix {
  static constexpr int kind = FIX_STORE;
  struct Args {
    FixCommon c;
    __nv_bfloat16* out;          // [tokens, ldo]
    const __nv_bfloat16* residual;
    long long ldo;
  };
};
struct SwigluFix {
  static constexpr int kind = FIX_SWIGLU;
  struct Args {
    FixCommon c;
    __nv_bfloat16* out;          // [tokens, ldo] with `inter` valid columns
    long long ldo;
    int inter;                   // output features = rows of the gate half (a multiple of 128)
    float act_limit;             // > 0: clamped form (up + 1) * gate * sigmoid(act_alpha * gate)
    float act_alpha;
  };
};
struct RopeFix {
  static constexpr int kind = FIX_ROPE;
  struct Args {
    FixCommon c;
    const int* positions;
    const int* slots;
    const float* cos_sin;
    const __nv_bfloat16* q_norm_w;
    const __nv_bfloat16* k_norm_w;
    __nv_bfloat16* q_out;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    float norm_eps;
    int nq, nkv, head_dim, max_pos, block_size;
  };
};
struct PushFix {
  static constexpr int kind = FIX_PUSH;
  struct Args {
    FixCommon c;
    PushArgs push;
  };
};

__device__ __forceinline__ float fix_silu(float g) { return g / (1.f + __expf(-g)); }

// Sum of the `splits` partials of 32 consecutive tokens for one feature row.
__device__ __forceinline__ void fix_sum(const FixCommon& c, int splits, long long split_stride, int row, int tok0,
                                        int n, float bias, float (&acc)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) acc[j] = bias;
  for (int s = 0; s < splits; ++s) {
    const float* p = c.partials + s * split_stride + (long long)tok0 * c.ld + row;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < n) acc[j] += __ldcg(p + (long long)j * c.ld);
  }
}

// Runs on the four epilogue warps (threads 64..191, et = threadIdx.x - 64) of the CTA that arrived last at
// the tile's counter.  rt = row tile, rows = GEMM rows (features), tokens = GEMM columns.
// `stage` is an 8 KB shared-memory staging tile (PUSH only); `red` a [4][32] float array (ROPE with QK-norm).
template <class Fix>
__device__ __forceinline__ void run_fix(const typename Fix::Args& fx, int rt, int rows, int tokens, int splits,
                                        long long split_stride, __nv_bfloat16* stage, float* red) {
  const int et = threadIdx.x - 64;
  const int quad = et >> 5, lane = et & 31;
  const FixCommon& c = fx.c;
  if constexpr (Fix::kind == FIX_STORE) {
    const int row = rt * kTileRows + et;
    const bool ok = row < rows;
    const float b = (c.bias && ok) ? __bfloat162float(c.bias[row]) : 0.f;
    for (int t0 = 0; t0 < tokens; t0 += 32) {
      const int n = min(32, tokens - t0);
      if (!ok) continue;
      float acc[32];
      fix_sum(c, splits, split_stride, row, t0, n, b, acc);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < n) {
          const long long idx = (long long)(t0 + j) * fx.ldo + row;
          float x = acc[j];
          if (fx.residual) x += __bfloat162float(fx.residual[idx]);
          fx.out[idx] = __float2bfloat16(x);
        }
      }
    }
  } else if constexpr (Fix::kind == FIX_SWIGLU) {
    // rt indexes the gate tile; the up tile of the same features sits `inter` rows further
    const int feat = rt * kTileRows + et;
    const bool ok = feat < fx.inter;
    const float bg = (c.bias && ok) ? __bfloat162float(c.bias[feat]) : 0.f;
    const float bu = (c.bias && ok) ? __bfloat162float(c.bias[fx.inter + feat]) : 0.f;
    const float lim = fx.act_limit, alpha = fx.act_alpha;
    for (int t0 = 0; t0 < tokens; t0 += 32) {
      const int n = min(32, tokens - t0);
      if (!ok) continue;
      float g[32], u[32];
      fix_sum(c, splits, split_stride, feat, t0, n, bg, g);
      fix_sum(c, splits, split_stride, fx.inter + feat, t0, n, bu, u);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < n) {
          float y;
          if (lim > 0.f) {
            const float gg = fminf(g[j], lim), uu = fminf(fmaxf(u[j], -lim), lim);
            y = (uu + 1.f) * gg / (1.f + __expf(-alpha * gg));
          } else {
            y = fix_silu(g[j]) * u[j];
          }
          fx.out[(long long)(t0 + j) * fx.ldo + feat] = __float2bfloat16(y);
        }
      }
    }
  } else if constexpr (Fix::kind == FIX_ROPE) {
    // A thread owns the rotation pair (i, i + D / 2) of one head, so no exchange is needed: with D = 128 the
    // tile is one head and threads 0..63 / 64..127 take alternate 32-token chunks; with D = 64 the tile holds
    // two heads and each half of the threads takes one of them.
    const int D = fx.head_dim, half = D >> 1;
    const int heads_per_tile = kTileRows / D;                 // 1 or 2
    const int grp = et >> 6, gi = et & 63;                    // two groups of 64 threads (two warps each)
    int head, i, chunk0, chunk_step;
    if (heads_per_tile == 1) {
      head = rt; i = gi; chunk0 = grp; chunk_step = 2;
    } else {
      head = rt * 2 + grp; i = gi & 31; chunk0 = (gi >> 5); chunk_step = 2;
    }
    const int nheads = fx.nq + 2 * fx.nkv;
    const bool head_ok = head < nheads;
    const bool is_q = head < fx.nq, is_k = !is_q && head < fx.nq + fx.nkv;
    const __nv_bfloat16* nw = is_q ? fx.q_norm_w : (is_k ? fx.k_norm_w : nullptr);
    const bool any_norm = fx.q_norm_w || fx.k_norm_w;
    const int row_lo = head * D + i, row_hi = row_lo + half;
    const float b_lo = (c.bias && head_ok) ? __bfloat162float(c.bias[row_lo]) : 0.f;
    const float b_hi = (c.bias && head_ok) ? __bfloat162float(c.bias[row_hi]) : 0.f;
    const float w_lo = (nw && head_ok) ? __bfloat162float(nw[i]) : 1.f;
    const float w_hi = (nw && head_ok) ? __bfloat162float(nw[half + i]) : 1.f;
    const int nchunks = (tokens + 31) / 32;
    // every thread walks the same number of iterations so that the barriers below stay uniform
    const int iters = (nchunks + chunk_step - 1) / chunk_step;
    for (int it = 0; it < iters; ++it) {
      const int ch = chunk0 + it * chunk_step;
      const int t0 = ch * 32;
      const int n = ch < nchunks ? min(32, tokens - t0) : 0;
      float lo[32], hi[32];
      if (head_ok && n > 0) {
        fix_sum(c, splits, split_stride, row_lo, t0, n, b_lo, lo);
        fix_sum(c, splits, split_stride, row_hi, t0, n, b_hi, hi);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) lo[j] = hi[j] = 0.f;
      }
      if (any_norm) {
        // sum of squares over the head: the threads of one head and chunk are one warp (D = 64) or two (D = 128)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float ss = warp_sum(lo[j] * lo[j] + hi[j] * hi[j]);
          if (lane == 0) red[quad * 32 + j] = ss;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (nw && head_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float tot = heads_per_tile == 1 ? red[(quad & 2) * 32 + j] + red[((quad & 2) + 1) * 32 + j]
                                                  : red[quad * 32 + j];
            const float inv = rsqrtf(tot / float(D) + fx.norm_eps);
            // round to bf16 after the norm like an unfused implementation would
            lo[j] = __bfloat162float(__float2bfloat16(lo[j] * inv * w_lo));
            hi[j] = __bfloat162float(__float2bfloat16(hi[j] * inv * w_hi));
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!head_ok) continue;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < n) {
          const int tok = t0 + j;
          float a = lo[j], b = hi[j];
          if (fx.cos_sin && (is_q || is_k)) {
            int pos = fx.positions[tok];
            pos = pos < 0 ? 0 : (pos >= fx.max_pos ? fx.max_pos - 1 : pos);
            const float* cs = fx.cos_sin + (long long)pos * D;
            const float cc = cs[i], sn = cs[half + i];
            const float ra = a * cc - b * sn, rb = b * cc + a * sn;
            a = ra;
            b = rb;
          }
          __nv_bfloat16* dst = nullptr;
          if (is_q) {
            dst = fx.q_out + ((long long)tok * fx.nq + head) * D;
          } else {
            const int slot = fx.slots ? fx.slots[tok] : -1;
            if (slot >= 0) {
              const int kh = is_k ? head - fx.nq : head - fx.nq - fx.nkv;
              const long long blk = slot / fx.block_size, off = slot % fx.block_size;
              dst = (is_k ? fx.k_cache : fx.v_cache) + ((blk * fx.nkv + kh) * fx.block_size + off) * D;
            }
          }
          if (dst) {
            dst[i] = __float2bfloat16(a);
            dst[half + i] = __float2bfloat16(b);
          }
        }
      }
    }
  } else if constexpr (Fix::kind == FIX_PUSH) {
    const PushArgs& push = fx.push;
    const int row = rt * kTileRows + et;
    const bool ok = row < rows;
    const float b = (c.bias && ok) ? __bfloat162float(c.bias[row]) : 0.f;
    const int row0 = rt * kTileRows;
    for (int t0 = 0; t0 < tokens; t0 += 32) {
      const int n = min(32, tokens - t0);
      float acc[32];
      if (ok) {
        fix_sum(c, splits, split_stride, row, t0, n, b, acc);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0.f;
      }
      // stage [token][feature] bf16, then store 16-byte pieces to every rank: each token row of the tile is
      // one contiguous 256-byte run in the destination's slot [rank][token][feature]
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < n) stage[j * kTileRows + et] = __float2bfloat16(acc[j]);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int idx = et; idx < n * 16; idx += 128) {
        const int tl = idx >> 4, chn = idx & 15;
        const int gtok = t0 + tl, gfeat = row0 + chn * 8;
        if (gfeat < rows) {
          const uint4 val = *reinterpret_cast<const uint4*>(stage + tl * kTileRows + chn * 8);
          const long long off = ((long long)push.rank * tokens + gtok) * c.ld + gfeat;
          push_store_16(push, off, val);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
  }
}

}  // namespace nkb
