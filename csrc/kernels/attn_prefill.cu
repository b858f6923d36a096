// Blockwise (flash) prefill attention on tcgen05 for sm_100a, reading K/V from
// the paged cache through the per-sequence block table.
//
// One CTA per (256 query rows, query head, sequence), as two 128-row query tiles in ping-pong:
//   warp 0     TMA producer: both Q tiles once, then a 3-stage ring that holds the 128-token K and V
//              tiles in turn (four 32-token pages each, 128-byte swizzle, non-multicast)
//   warp 1     issues tcgen05.mma.  Per KV tile and query tile t: S_t = Q_t K^T (M = N = 128, fp32 in
//              TMEM) and O_t += P_t V with V as an MN-major B operand.  The order
//              PV_0(j), QK_0(j+1), PV_1(j), QK_1(j+1) keeps the tensor pipe busy with one tile's
//              MMAs while the other tile's softmax runs.
//   warps 4-7  softmax of tile 0, warps 8-11 softmax of tile 1: one thread per query row reads its
//              128 scores from TMEM once, keeps them in registers, writes P as bf16 to shared memory
//              in the swizzled K-major layout the MMA reads.
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
constexpr int kPfThreads = 384;          // warpgroup 0: TMA warp, MMA warp, two idle; warpgroups 1, 2: softmax
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
  uint8_t* kv_s = q_s + 2 * kQBytes;                // ring: K(j), V(j), K(j+1), ...
  uint8_t* p_s = kv_s + kKVStages * kKVBytes;       // 2 probability tiles
  PrefillCtrl* ctrl = reinterpret_cast<PrefillCtrl*>(p_s + 2 * kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(&ctrl->q_full, 1);
    for (int i = 0; i < kKVStages; ++i) {
      mbar_init(&ctrl->kv_full[i], 1);
      mbar_init(&ctrl->kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->s_full[i], 1);
      mbar_init(&ctrl->s_empty[i], 4);
      mbar_init(&ctrl->p_full[i], 4);
      mbar_init(&ctrl->o_full[i], 1);
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
  const uint32_t tmem_base = ctrl->tmem_base;
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
    for (int n = 0; n < 2 * n_union; ++n) {          // item n: K of tile n / 2 (even n) or its V (odd n)
      const int j = u_lo + (n >> 1);
      const int st = n % kKVStages;
      const uint32_t ph = uint32_t(n / kKVStages) & 1u;
      bool ok = mbar_wait(&ctrl->kv_empty[st], ph ^ 1u, abort_flag, p.status, ERR_WAIT_SMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) break;
      int blk[4];
#pragma unroll
      for (int pi = 0; pi < 4; ++pi) blk[pi] = table[min(j * 4 + pi, last_page)];
      if (lane == 0) {
        const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
        uint8_t* dst = kv_s + st * kKVBytes;
        mbar_expect_tx(&ctrl->kv_full[st], kKVBytes);
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_4d(dst + h * kHalf + pi * (kPfPage * 128), tm, &ctrl->kv_full[st], h * 64, 0, kvh, blk[pi]);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, kKVTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);  // B = V is MN-major
    bool alive = true;
    {
      bool ok = mbar_wait(&ctrl->q_full, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) alive = false;
    }
    auto active = [&](int t, int u) {
      const int j = u_lo + u;
      return t == 0 ? (j >= tr0.lo && j < tr0.hi) : (two && j >= tr1.lo && j < tr1.hi);
    };
    auto local_it = [&](int t, int u) { return u_lo + u - (t == 0 ? tr0.lo : tr1.lo); };
    auto wait_item = [&](int n) -> bool {
      bool ok = mbar_wait(&ctrl->kv_full[n % kKVStages], uint32_t(n / kKVStages) & 1u, abort_flag, p.status,
                          ERR_WAIT_SMEM_FULL);
      return __all_sync(0xffffffffu, ok);
    };
    auto release_item = [&](int n) {
      if (lane == 0) umma_commit(&ctrl->kv_empty[n % kKVStages]);
      __syncwarp();
    };
    // S_t = Q_t K(u)^T
    auto issue_qk = [&](int t, int u) -> bool {
      if (!wait_item(2 * u)) return false;
      const int lit = local_it(t, u);
      bool ok = mbar_wait(&ctrl->s_empty[t], (uint32_t(lit) & 1u) ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qa = smem_u32(q_s + t * kQBytes), ka = smem_u32(kv_s + ((2 * u) % kKVStages) * kKVBytes);
        const uint32_t d = tmem_base + kSCol + t * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 32;
          umma_f16(d, make_smem_desc_sw128(qa + off, 0, 1024), make_smem_desc_sw128(ka + off, 0, 1024), idesc_qk,
                   ks > 0 ? 1u : 0u);
        }
        umma_commit(&ctrl->s_full[t]);
      }
      __syncwarp();
      return true;
    };
    // O_t (+)= P_t V(u)
    auto issue_pv = [&](int t, int u) -> bool {
      const int lit = local_it(t, u);
      bool ok = mbar_wait(&ctrl->p_full[t], uint32_t(lit) & 1u, abort_flag, p.status, ERR_WAIT_SOFTMAX);
      if (!__all_sync(0xffffffffu, ok)) return false;
      if (!wait_item(2 * u + 1)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(p_s + t * kPBytes), va = smem_u32(kv_s + ((2 * u + 1) % kKVStages) * kKVBytes);
        const uint32_t d = tmem_base + kOCol + t * 128;
#pragma unroll
        for (int ks = 0; ks < kKVTile / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(pa + (ks >> 2) * kHalf + (ks & 3) * 32, 0, 1024);
          // V tile: [token][64 dims] rows of 128 B; 16 tokens per step = 2 KB; next 64 dims one slab on
          const uint64_t db = make_smem_desc_sw128(va + ks * 2048, kHalf, 1024);
          umma_f16(d, da, db, idesc_pv, (lit > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&ctrl->o_full[t]);
      }
      __syncwarp();
      return true;
    };
    if (alive && n_union > 0) {
      if (active(0, 0)) alive = issue_qk(0, 0);
      if (alive && active(1, 0)) alive = issue_qk(1, 0);
      if (alive) release_item(0);
    }
    for (int u = 0; u < n_union && alive; ++u) {
      const bool more = u + 1 < n_union;
      if (active(0, u)) alive = issue_pv(0, u);
      if (alive && more && active(0, u + 1)) alive = issue_qk(0, u + 1);
      if (alive && active(1, u)) alive = issue_pv(1, u);
      if (!alive) break;
      release_item(2 * u + 1);
      if (more) {
        if (active(1, u + 1)) alive = issue_qk(1, u + 1);
        if (alive) release_item(2 * u + 2);
      }
    }
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
    uint8_t* my_p = p_s + t * kPBytes;
    const int n_tiles = tr.hi - tr.lo;
    float m = -INFINITY, l = 0.f;
    int hi_pos = ctx - 1;
    if (p.causal) hi_pos = min(hi_pos, q_pos);
    const int lo_pos = p.window > 0 ? q_pos - p.window + 1 : 0;
    bool alive = true;

    for (int it = 0; it < n_tiles; ++it) {
      const int kv0 = (tr.lo + it) * kKVTile;
      bool ok = mbar_wait(&ctrl->s_full[t], uint32_t(it) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
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
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < kKVTile; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
      mx *= p.scale_log2;

      if (it == 0) {
        m = mx;
      } else {
        // P_t of the previous tile has been read and O_t holds its contribution
        ok = mbar_wait(&ctrl->o_full[t], uint32_t(it - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        const bool grow = mx > m + kRescaleStep || (m == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
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
      const float nbase = -base;
      float sum = 0.f;
#pragma unroll
      for (int c8 = 0; c8 < kKVTile / 8; ++c8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(fmaf(__uint_as_float(v[c8 * 8 + i]), p.scale_log2, nbase));
          sum += e[i];
        }
        // 16-byte chunk c8 of the row, swizzled like a TMA 128-byte-swizzle load would place it
        uint8_t* dst = my_p + (c8 >> 3) * kHalf + r * 128 + (((c8 & 7) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(e[0], e[1]), pack_bf16x2(e[2], e[3]),
                                                    pack_bf16x2(e[4], e[5]), pack_bf16x2(e[6], e[7]));
      }
      l += sum;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->p_full[t]);
    }
    // ---- epilogue: O_t / l to global memory
    if (tr.rows > 0) {
      bool have_o = false;
      if (alive && n_tiles > 0) {
        bool ok = mbar_wait(&ctrl->o_full[t], uint32_t(n_tiles - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(flash_attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    attr_set = true;
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
