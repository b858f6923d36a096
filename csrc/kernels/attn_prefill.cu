// Blockwise (flash) prefill attention on tcgen05 for sm_100a, reading K/V from
// the paged cache through the per-sequence block table.
//
// One CTA per (256 query rows, query head, sequence), as two 128-row query tiles in ping-pong:
//   warp 0     TMA producer: both Q tiles once, then a 3-stage ring of 128-token K and V tiles (four
//              32-token pages each, 128-byte swizzle, non-multicast)
//   warps 1, 2 issue tcgen05.mma, one warp per query tile t, per KV tile j in the order
//              S_t(j+1) = Q_t K(j+1)^T, then O_t += P_t(j) V(j) (V is an MN-major B operand).  S_t is free
//              as soon as the softmax holds it in registers, so the next scores are ready when the
//              softmax of tile j ends and the softmax warps do not wait for the tensor pipe.
//   warps 4-7  softmax of tile 0, warps 8-11 softmax of tile 1: one thread per query row reads its
//              128 scores from TMEM once, keeps them in registers, and writes P as bf16 to shared memory
//              in the swizzled K-major layout the MMA reads.  The two tiles take turns with their
//              exponentials (see the loop), so that one tile's MMAs, score loads and row maxima run
//              while the other tile has the special-function unit.
// O_0 and O_1 stay in TMEM for the whole KV loop (S_0, S_1, O_0, O_1 = 4 x 128 columns).  The row maximum
// that scales the exponentials is only raised when the true maximum has grown by more than 2^8 since it
// was last set; then the row's O is rescaled in TMEM (load, multiply, store).  With a stale maximum the
// probabilities are at most 2^8 too large, which fp32 sums and bf16 P hold without loss, and O / l is
// unchanged because both carry the same factor.  KV tiles past a query tile's causal diagonal or before
// its window are skipped for that tile; the mask is only evaluated on tiles that cross either edge.
// GQA needs no repeat of K/V: the query head picks its kv head.  Supports causal
// masking with a cached prefix (q_len <= context_len), sliding windows and
// attention-sink logits.
//
// What the structure answers to (measured on B200 with a cycle trace of one CTA and an issue-rate probe):
// * The tensor pipe runs a 128 x 128 x 16 MMA in 64 cycles from any operand source, but queues only a few of
//   them: whatever the issuing thread does between two groups of MMAs is time in which the pipe drains.  A single
//   thread runs one dependent instruction every few cycles, and a blocking wait for one query tile kept the
//   other tile's ready group from being issued.  Hence one issuer per query tile, issue by a single elected
//   thread without warp votes, descriptors prepared before four MMAs go out as one instruction sequence, and
//   warp roles the compiler can prove uniform.
// * 128 exponentials per row keep the special-function unit of a scheduler busy for about as long as the rest
//   of an iteration takes.  Left alone, the two query tiles fall into step (they share the K/V ring), compute
//   their exponentials at half speed at the same time and then wait at the same time.
// * Computing part of the exponentials with a polynomial on the FMA pipe, a branch per 32 scores in the
//   exponential loop (to skip fully masked groups) and probabilities in tensor memory (which ties Q K^T of
//   the next tile to P V of this one) were all measured slower than what is here.
//
// Reference parity: prefill branch of attention_kernel in
// examples/models/qwen3/kernels/attention.py:108-137 (materialised scores +
// additive -1e5 mask + softmax + P.V), window / sinks from
// examples/models/gpt_oss/kernels/attention.py:116-148, non-causal-free prefill
// of examples/models/qwen3_embedding/kernels/attention.py.
#include "common.cuh"
#include "api.h"
#include <math.h>

namespace nkb {

constexpr int kQTile = 128;          // rows of one MMA tile
constexpr int kQPair = 2 * kQTile;   // query rows per CTA
constexpr int kKVTile = 128;
constexpr int kPfPage = 32;
constexpr int kPfThreads = 384;      // warpgroup 0: TMA warp, two MMA warps, one idle; warpgroups 1, 2: softmax
constexpr int kKVStages = 3;
constexpr float kRescaleStep = 8.f;  // log2 of the growth of the row maximum that triggers a rescale of O

struct PrefillParams {
  const int* block_table;
  const int* q_start;
  const int* q_lens;
  const int* context_lens;
  __nv_bfloat16* out;
  const float* sinks;
  int* status;
  int nq, nkv, max_blocks, causal, window;
  float scale_log2;
};

struct PrefillCtrl {
  uint64_t q_full;
  uint64_t kv_full[kKVStages], kv_empty[kKVStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], o_full[2];
  uint64_t turn[2][4];
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Blackwell's three-input maximum and packed two-lane fp32 arithmetic halve the instructions of the row
// maximum, the scaling and the row sum.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  uint64_t rd;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(rd)
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)), "l"(reinterpret_cast<uint64_t&>(c)));
  return reinterpret_cast<float2&>(rd);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  uint64_t rd;
  asm("add.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return reinterpret_cast<float2&>(rd);
}

// Four MMAs (k-steps) of one accumulator as one instruction sequence, descriptors prepared beforehand.
__device__ __forceinline__ void umma4_ss(uint32_t d, const uint64_t (&a)[4], const uint64_t (&b)[4], uint32_t idesc,
                                         uint32_t acc_first) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1;\n"
      "setp.ne.b32 p0, %10, 0;\n"
      "setp.eq.b32 p1, %9, %9;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, p1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, p1;\n"
      "}\n" ::"r"(d),
      "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "r"(idesc), "r"(acc_first)
      : "memory");
}

// Bounded barrier wait whose slow path (timer, abort flag) is one shared out-of-line function: the kernel has two
// dozen waits and their inlined loops would push the hot code out of the instruction cache.
__device__ __noinline__ bool pf_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  return mbar_wait(bar, parity, abort_flag, status, code);
}
__device__ __forceinline__ bool pf_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                        int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return pf_wait_slow(bar, parity, abort_flag, status, code);
}

// KV tile range [lo, hi) that query tile `t` of the CTA attends to (empty when the tile has no rows).
struct TileRange {
  int lo, hi, pos0, rows;
};
__device__ __forceinline__ TileRange tile_range(const PrefillParams& p, int row0, int q_len, int ctx) {
  TileRange r{0, 0, 0, 0};
  if (row0 >= q_len) return r;
  r.rows = min(kQTile, q_len - row0);
  r.pos0 = ctx - q_len + row0;                       // kv position of the tile's first query
  r.hi = (ctx + kKVTile - 1) / kKVTile;
  if (p.causal) r.hi = min(r.hi, (r.pos0 + r.rows - 1) / kKVTile + 1);
  if (p.window > 0) r.lo = max(0, r.pos0 - p.window + 1) / kKVTile;
  if (r.hi < r.lo) r.hi = r.lo;
  return r;
}

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
flash_attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  constexpr int NH = D / 64;
  constexpr int kHalf = 128 * 128;          // [128 rows][64 bf16] swizzled slab = 16 KB
  constexpr int kQBytes = NH * kHalf;       // one query tile
  constexpr int kKVBytes = NH * kHalf;      // one K or V tile
  constexpr int kPBytes = 2 * kHalf;        // [128 rows][128 tokens]
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSCol = 0, kOCol = 256;   // S_t at kSCol + 128 t, O_t at kOCol + 128 t

  // the heaviest CTAs (last query rows of a causal sequence) start first
  const int qt = gridDim.x - 1 - blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  griddep_wait();
  griddep_launch();
  const int q_len = p.q_lens[b];
  if (qt * kQPair >= q_len) return;
  const int ctx = p.context_lens[b];
  const int q_row0 = p.q_start[b] + qt * kQPair;        // row in the packed q / out arrays
  const int kvh = head / (p.nq / p.nkv);
  const TileRange tr0 = tile_range(p, qt * kQPair, q_len, ctx);
  const TileRange tr1 = tile_range(p, qt * kQPair + kQTile, q_len, ctx);
  const bool two = tr1.rows > 0;
  // union of the two ranges; every tile of it is attended to by at least one query tile
  const int u_lo = tr0.lo, u_hi = two ? max(tr0.hi, tr1.hi) : tr0.hi;
  const int n_union = u_hi - u_lo;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                              // 2 query tiles
  uint8_t* kv_s = q_s + 2 * kQBytes;                // ring of K and V tiles
  uint8_t* p_s = kv_s + kKVStages * kKVBytes;       // 2 probability tiles
  PrefillCtrl* ctrl = reinterpret_cast<PrefillCtrl*>(p_s + 2 * kPBytes);

  const int warp = warp_idx_uniform(), lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(&ctrl->q_full, 1);
    for (int i = 0; i < kKVStages; ++i) {
      mbar_init(&ctrl->kv_full[i], 1);
      mbar_init(&ctrl->kv_empty[i], two ? 2 : 1);   // one release from each query tile's issuer
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->s_full[i], 1);
      mbar_init(&ctrl->s_empty[i], 4);
      mbar_init(&ctrl->p_full[i], 4);
      mbar_init(&ctrl->o_full[i], 1);
      for (int q = 0; q < 4; ++q) mbar_init(&ctrl->turn[i][q], 1);
    }
    ctrl->abort = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&ctrl->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, ctrl->tmem_base, 0);   // provably warp-uniform
  volatile int* abort_flag = &ctrl->abort;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(&ctrl->q_full, 2 * kQBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < NH; ++h)
          tma_load_3d(q_s + t * kQBytes + h * kHalf, &tmQ, &ctrl->q_full, h * 64, head, q_row0 + t * kQTile);
    }
    __syncwarp();
    const int* table = p.block_table + (long long)b * p.max_blocks;
    const int last_page = max((ctx + kPfPage - 1) / kPfPage - 1, 0);
    // Ring items in the order the issuers consume them: K(0), then per KV tile u: K(u+1), V(u).  Q K^T runs one
    // tile ahead of P V, so K(u+2) has the whole of iteration u to arrive.  Item `seq` lives in stage seq % 3.
    int seq = 0;
    bool live = true;
    auto load = [&](bool is_v, int x) {
      if (!live) return;
      const int j = u_lo + x;
      const int st = seq % kKVStages;
      const uint32_t ph = uint32_t(seq / kKVStages) & 1u;
      ++seq;
      bool ok = pf_wait(&ctrl->kv_empty[st], ph ^ 1u, abort_flag, p.status, ERR_WAIT_SMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) { live = false; return; }
      int blk[4];
#pragma unroll
      for (int pi = 0; pi < 4; ++pi) blk[pi] = table[min(j * 4 + pi, last_page)];
      if (lane == 0) {
        const CUtensorMap* tm = is_v ? &tmV : &tmK;
        uint8_t* dst = kv_s + st * kKVBytes;
        mbar_expect_tx(&ctrl->kv_full[st], kKVBytes);
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_4d(dst + h * kHalf + pi * (kPfPage * 128), tm, &ctrl->kv_full[st], h * 64, 0, kvh, blk[pi]);
      }
      __syncwarp();
    };
    if (n_union > 0) load(false, 0);
#pragma unroll 1
    for (int u = 0; u < n_union && live; ++u) {
      if (u + 1 < n_union) load(false, u + 1);
      load(true, u);
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------------------------------------------------------- MMA issuers, one per query tile
    // Both issuers walk all KV tiles of the CTA in the producer's order and release every ring stage (the barrier
    // counts two arrivals), also for KV tiles their query tile does not attend to; each waits for a stage to be
    // loaded before it releases it, so that an issuer can never arrive twice on one barrier phase.
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, kKVTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);  // B = V is MN-major
    const int t = warp - 1;
    const uint32_t q_lo = uint32_t(make_smem_desc_sw128(smem_u32(q_s + t * kQBytes), 0, 1024));
    const uint32_t kv_lo = uint32_t(make_smem_desc_sw128(smem_u32(kv_s), 0, 1024));
    const uint32_t p_lo = uint32_t(make_smem_desc_sw128(smem_u32(p_s + t * kPBytes), 0, 1024));
    const uint64_t hk = uint64_t(uint32_t(make_smem_desc_sw128(0, 0, 1024) >> 32)) << 32;   // SBO, version, swizzle
    const uint32_t lbo_v = (uint32_t(kHalf) >> 4) << 16;                                    // low-word part of V's LBO
    const int a_lo = t == 0 ? tr0.lo - u_lo : (two ? tr1.lo - u_lo : 0);
    const int a_hi = t == 0 ? tr0.hi - u_lo : (two ? tr1.hi - u_lo : 0);
    const uint32_t s_tmem = tmem_base + kSCol + t * 128, o_tmem = tmem_base + kOCol + t * 128;
    if ((t == 0 || two) && elect_one()) {
      bool ok = pf_wait(&ctrl->q_full, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      int seq = 0;                                   // ring item counter, in the producer's order
      // K tile x: S_t = Q_t K(x)^T if this query tile attends to it, then release its ring stage
      auto do_k = [&](int x) {
        if (x >= n_union || !ok) return;
        const int item = seq++, st = item % kKVStages;
        ok = pf_wait(&ctrl->kv_full[st], uint32_t(item / kKVStages) & 1u, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
        if (!ok) return;
        if (x >= a_lo && x < a_hi) {
          const uint32_t lit = uint32_t(x - a_lo);
          ok = pf_wait(&ctrl->s_empty[t], (lit & 1u) ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY);
          if (!ok) return;
          tc_fence_after();
          const uint32_t kvd = kv_lo + uint32_t(st * kKVBytes >> 4);
#pragma unroll
          for (int h = 0; h < NH; ++h) {
            uint64_t da[4], db[4];
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint32_t off = uint32_t(h * (kHalf >> 4) + k4 * 2);
              da[k4] = hk | (q_lo + off);
              db[k4] = hk | (kvd + off);
            }
            umma4_ss(s_tmem, da, db, idesc_qk, h > 0 ? 1u : 0u);
          }
          umma_commit(&ctrl->s_full[t]);
        }
        umma_commit(&ctrl->kv_empty[st]);
      };
      // V tile x: O_t (+)= P_t V(x) if this query tile attends to it, then release its ring stage
      auto do_v = [&](int x) {
        if (!ok) return;
        const int item = seq++, st = item % kKVStages;
        ok = pf_wait(&ctrl->kv_full[st], uint32_t(item / kKVStages) & 1u, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
        if (!ok) return;
        if (x >= a_lo && x < a_hi) {
          const uint32_t lit = uint32_t(x - a_lo);
          ok = pf_wait(&ctrl->p_full[t], lit & 1u, abort_flag, p.status, ERR_WAIT_SOFTMAX);
          if (!ok) return;
          tc_fence_after();
          const uint32_t kvd = kv_lo + uint32_t(st * kKVBytes >> 4);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint64_t da[4], db[4];
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // V tile: [token][64 dims] rows of 128 B; 16 tokens per step = 2 KB; next 64 dims one slab on
              db[k4] = hk | ((kvd + uint32_t((h * 4 + k4) * 128)) | lbo_v);
              da[k4] = hk | (p_lo + uint32_t(h * (kHalf >> 4) + k4 * 2));
            }
            umma4_ss(o_tmem, da, db, idesc_pv, (lit > 0 || h > 0) ? 1u : 0u);
          }
          umma_commit(&ctrl->o_full[t]);            // P_t has been read, O_t holds its product
        }
        umma_commit(&ctrl->kv_empty[st]);
      };
      do_k(0);
#pragma unroll 1
      for (int u = 0; u < n_union && ok; ++u) {
        do_k(u + 1);
        do_v(u);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax
    const int t = (warp - 4) >> 2;                  // query tile of this warp
    const int quad = warp & 3;                      // TMEM lanes this warp may touch
    const TileRange tr = t == 0 ? tr0 : tr1;
    const int r = quad * 32 + lane;                 // row of the query tile
    const int q_pos = tr.pos0 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + kSCol + t * 128;
    const uint32_t o_addr = tmem_base + lane_off + kOCol + t * 128;
    uint8_t* my_p = p_s + t * kPBytes + r * 128;
    const int n_tiles = tr.hi - tr.lo;
    const int n_other = t == 0 ? (two ? tr1.hi - tr1.lo : 0) : tr0.hi - tr0.lo;   // KV tiles of the other query tile
    float m = -INFINITY, l = 0.f;
    int hi_pos = ctx - 1;
    if (p.causal) hi_pos = min(hi_pos, q_pos);
    const int lo_pos = p.window > 0 ? q_pos - p.window + 1 : 0;
    bool alive = true;

    for (int it = 0; it < n_tiles; ++it) {
      const int kv0 = (tr.lo + it) * kKVTile;
      bool ok = pf_wait(&ctrl->s_full[t], uint32_t(it) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      tc_fence_after();
      uint32_t v[kKVTile];
#pragma unroll
      for (int c = 0; c < kKVTile / 32; ++c) tmem_ld_32x32(s_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(v[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->s_empty[t]);   // the scores are in registers: S_t may be overwritten

      // the mask only on tiles that cross the causal diagonal, the end of the context or the window edge
      const bool edge = kv0 + kKVTile - 1 > hi_pos || kv0 < lo_pos;
      if (__any_sync(0xffffffffu, edge)) {
        const int hi_rel = hi_pos - kv0, lo_rel = lo_pos - kv0;
#pragma unroll
        for (int i = 0; i < kKVTile; ++i)
          if (i > hi_rel || i < lo_rel) v[i] = 0xff800000u;   // -inf
      }
      // four independent chains of three-input maxima instead of one 128-long dependent chain
      float mx4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
#pragma unroll
      for (int i = 8; i < kKVTile; i += 2)
        mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= p.scale_log2;

      bool p_free = it == 0;     // the P_t buffer may be overwritten (P V of the previous tile has finished)
      if (it == 0) {
        m = mx;
      } else {
        const bool grow = mx > m + kRescaleStep || (m == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          // O_t holds all of the previous tile's contribution
          ok = pf_wait(&ctrl->o_full[t], uint32_t(it - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
          if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          p_free = true;
          tc_fence_after();
          const float alpha = grow ? exp2f(m - mx) : 1.f;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, o);
          }
          tmem_st_wait();
          l *= alpha;
          if (grow) m = mx;
        }
      }
      const float base = (m == -INFINITY) ? 0.f : m;
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nb2 = make_float2(-base, -base);
      float2 sum2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sum2[i] = make_float2(0.f, 0.f);
      // probabilities of 32 scores as 16 packed bf16 pairs
      auto exp_chunk = [&](int c32, uint32_t (&pk)[16]) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int k = c32 * 32 + 2 * i;
          const float2 x = ffma2(make_float2(__uint_as_float(v[k]), __uint_as_float(v[k + 1])), sc2, nb2);
          const float2 e = make_float2(exp2f(x.x), exp2f(x.y));
          sum2[i & 3] = fadd2(sum2[i & 3], e);
          pk[i] = pack_bf16x2(e.x, e.y);
        }
      };
      // 32 tokens = four 16-byte chunks of the row, swizzled like a TMA 128-byte-swizzle load places them
      auto store_chunk = [&](int c, const uint32_t (&pk)[16]) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(my_p + (c >> 1) * kHalf + ((((c & 1) * 4 + q) ^ (r & 7)) << 4)) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      };
      // P_t's buffer is free once P V of the previous tile has finished
      if (!p_free) {
        ok = pf_wait(&ctrl->o_full[t], uint32_t(it - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      }
      // The exponentials of the two query tiles take turns.  The warps of tile 0 and tile 1 that own the same TMEM
      // lanes share a scheduler and its special-function unit, which 128 exponentials per row keep busy for about
      // as long as the rest of an iteration takes; left alone the two tiles fall into step (they share the K/V
      // ring), both compute exponentials at half speed and then both wait.  Alternating lets one tile use the unit
      // at full speed while the other loads its scores, takes the maximum and publishes P.
      // Order: tile 0 (it), tile 1 (it), tile 0 (it + 1), ...; a tile that has run out of KV tiles is not waited for.
      if (t == 0 ? (it >= 1 && it - 1 < n_other) : (it < n_other)) {
        ok = pf_wait(&ctrl->turn[t][quad], uint32_t(t == 0 ? it - 1 : it) & 1u, abort_flag, p.status, ERR_WAIT_SOFTMAX);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      }
#pragma unroll
      for (int c = 0; c < kKVTile / 32; ++c) {
        uint32_t pk[16];
        exp_chunk(c, pk);
        store_chunk(c, pk);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->turn[1 - t][quad]);
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->p_full[t]);
      {
        const float2 s01 = fadd2(sum2[0], sum2[1]), s23 = fadd2(sum2[2], sum2[3]);
        const float2 s4 = fadd2(s01, s23);
        l += s4.x + s4.y;
      }
    }
    // ---- epilogue: O_t / l to global memory
    if (tr.rows > 0) {
      bool have_o = false;
      if (alive && n_tiles > 0) {
        bool ok = pf_wait(&ctrl->o_full[t], uint32_t(n_tiles - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
        have_o = __all_sync(0xffffffffu, ok);
        if (have_o) tc_fence_after();
      }
      float osc = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[head] * 1.4426950408889634f;
        const float m2 = fmaxf(m, sk);
        osc = (m == -INFINITY) ? 0.f : exp2f(m - m2);
        l = l * osc + exp2f(sk - m2);
      }
      const float inv = l > 0.f ? osc / l : 0.f;
      __nv_bfloat16* dst = p.out + ((long long)(q_row0 + t * kQTile + r) * p.nq + head) * D;
      const bool store = r < tr.rows && !*abort_flag;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (have_o) {
          tmem_ld_32x32(o_addr + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
          }
        }
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
static int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const PrefillParams& p, int batch, int max_q_len, cudaStream_t s) {
  constexpr int NH = D / 64;
  constexpr int smem = NH * 16384 * (2 + kKVStages) + 2 * 2 * 16384 + int(sizeof(PrefillCtrl)) + 1024 + 64;
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(flash_attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    attr_set[dev] = true;
  }
  dim3 grid((max_q_len + kQPair - 1) / kQPair, p.nq, batch);
  return launch_pdl(flash_attn_prefill_kernel<D>, grid, dim3(kPfThreads), size_t(smem), s, tq, tk, tv, p);
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_flash_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                      const int* q_start, const int* q_lens, const int* context_lens, void* out,
                                      int batch, int total_q, int max_q_len, int nq, int nkv, int head_dim,
                                      int block_size, int num_blocks, int max_blocks_per_seq, float scale, int causal,
                                      int window, const float* sinks, void* stream) {
  if (batch <= 0 || total_q <= 0) return 0;
  if (block_size != kPfPage || nq % nkv != 0) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  PrefillParams p{};
  p.block_table = block_table;
  p.q_start = q_start;
  p.q_lens = q_lens;
  p.context_lens = context_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.sinks = sinks;
  p.status = status_word();
  p.nq = nq; p.nkv = nkv; p.max_blocks = max_blocks_per_seq; p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tq, tk, tv;
  {
    const uint64_t dims[3] = {uint64_t(head_dim), uint64_t(nq), uint64_t(total_q)};
    const uint64_t strides[2] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * nq * 2};
    const uint32_t box[3] = {64, 1, uint32_t(kQTile)};
    if (encode_tmap_bf16(&tq, q, 3, dims, strides, box)) return -4;
  }
  {
    const uint64_t dims[4] = {uint64_t(head_dim), uint64_t(kPfPage), uint64_t(nkv), uint64_t(num_blocks)};
    const uint64_t strides[3] = {uint64_t(head_dim) * 2, uint64_t(head_dim) * kPfPage * 2,
                                 uint64_t(head_dim) * kPfPage * nkv * 2};
    const uint32_t box[4] = {64, uint32_t(kPfPage), 1, 1};
    if (encode_tmap_bf16(&tk, k_cache, 4, dims, strides, box)) return -4;
    if (encode_tmap_bf16(&tv, v_cache, 4, dims, strides, box)) return -4;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128) return launch_prefill<128>(tq, tk, tv, p, batch, max_q_len, s);
  if (head_dim == 64) return launch_prefill<64>(tq, tk, tv, p, batch, max_q_len, s);
  return -2;
}
