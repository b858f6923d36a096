// bf16 GEMM on CTA pairs: D[m, n] = A[m, k] * B[n, k]^T with 256 x 256 output tiles.
//
// Two CTAs of a cluster (one SM each) work on one tile with `tcgen05.mma.cta_group::2`: CTA r of
// the pair holds rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the B tile in
// its shared memory and the matching 128 accumulator rows in its tensor memory; the MMA is issued by
// one thread of the pair's first CTA and reads both CTAs' shared memory.  Per k-slab each CTA therefore
// loads 32 KB for 128 x 256 outputs (the single-CTA kernel loads 48 KB), which takes the L2 -> shared-
// memory traffic of the prefill GEMMs from about 16 TB/s at tensor-core peak to about 11 TB/s, and the
// ring holds seven stages instead of four.
//
// Synchronisation (all mbarriers; every wait is bounded):
//   full[s]   lives in the first CTA: its TMA warp announces the bytes of both CTAs, both CTAs' loads
//             complete their bytes there;
//   empty[s]  one per CTA: after the MMAs of a stage the issuing thread commits to its own and to the
//             peer's barrier (two plain commits; no cluster-wide broadcast form is used anywhere);
//   tfull[a]  one per CTA, same two commits, wakes both epilogues;
//   tempty[a] lives in the first CTA, count 8: the four epilogue warps of both CTAs arrive.
// Loads are plain (non-broadcast) tiled TMA copies of this GPU's memory.
//
// Reference parity: same role as gemm_tcgen05.cuh (the `dot` lowering target, prefill orientation).
#include "gemm_tcgen05.cuh"
#include "api.h"
#include <stdlib.h>

namespace nkb {

struct Gemm2Args {            // <= 128 bytes (see GemmArgs)
  int m, n, k;
  int tiles_m, tiles_n;       // 256 x 256 tiles
  int kb_total, stages;
  int bias_on_cols;
  int group_m;                // row tiles that share one sweep over the column tiles (L2 reuse)
  int gated;                  // B holds [gate; up] rows: the pair's first CTA loads gate rows, the second up rows
  int gate_off;               // row offset of the up half in B
  long long ldo;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int* status;
};
static_assert(sizeof(Gemm2Args) <= 128, "Gemm2Args grew past the fast kernel-parameter size");

constexpr int k2TileN = 256;
constexpr int k2StageBytes = 2 * kATileBytes;     // A rows + B rows of this CTA, 16 KB each

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Gemm2Args args) {
  extern __shared__ uint8_t smem_raw[];
  // identical layout in both CTAs: [control 1 KB][ring]
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmCtrl* ctrl = reinterpret_cast<GemmCtrl*>(base);
  uint8_t* tiles = base + 1024;
  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = issues the MMAs
  const int stages = args.stages;
  constexpr uint32_t tmem_cols = 2 * k2TileN;     // two accumulators of 256 columns

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->tfull[i], 1);
      mbar_init(&ctrl->tempty[i], 8);
    }
    ctrl->abort = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctrl->tmem_base, tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // both CTAs' barriers exist before anything remote arrives
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort;

  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total_work = args.tiles_m * args.tiles_n;
  griddep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    griddep_wait();
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int w = pair; w < total_work && alive; w += npairs) {
      // group_m row tiles share a sweep over the column tiles so that A and B tiles are re-read from L2
      const int kGroup = args.group_m;
      const int per_group = kGroup * args.tiles_n;
      const int g = w / per_group;
      const int first = g * kGroup;
      const int gsz = min(args.tiles_m - first, kGroup);
      const int in = w - g * per_group;
      const int tm = first + in % gsz, tn = in / gsz;
      const int a_row = tm * 256 + int(rank) * 128;
      const int b_row = args.gated ? (int(rank) * args.gate_off + tn * 128) : (tn * 256 + int(rank) * 128);
      for (int kb = 0; kb < args.kb_total; ++kb) {
        bool ok = mbar_wait(&ctrl->empty[stage], phase ^ 1u, abort_flag, args.status, ERR_WAIT_SMEM_EMPTY);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        if (lane == 0) {
          const uint32_t full0 = map_to_cta(&ctrl->full[stage], 0);
          uint8_t* a_ptr = tiles + stage * k2StageBytes;
          // the first CTA announces the bytes of both CTAs; the second only lets its loads complete there
          // (its loads of this phase cannot start before the barrier entered the phase: they wait for the
          // stage to be released, which follows the previous phase's completion)
          if (rank == 0) mbar_expect_tx(&ctrl->full[stage], 2 * k2StageBytes);
          tma_load_2d_pair(a_ptr, &tmA, full0, kb * kBlockK, a_row);
          tma_load_2d_pair(a_ptr + kATileBytes, &tmB, full0, kb * kBlockK, b_row);
        }
        __syncwarp();
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (first CTA of the pair)
    // One elected thread runs the whole loop alone: the tensor pipe queues only a few MMAs, so warp votes,
    // reconvergence and descriptor arithmetic between two k-blocks are time in which it drains.
    constexpr uint32_t idesc = make_idesc_bf16(256, k2TileN, 0, 0);
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      const uint64_t d_tiles = make_smem_desc_sw128(smem_u32(tiles), 0, 1024);
      const uint64_t d_hi = d_tiles & 0xffffffff00000000ull;
      const uint32_t a_lo0 = uint32_t(d_tiles);
      const uint32_t empty0 = map_to_cta(&ctrl->empty[0], 0), empty1 = map_to_cta(&ctrl->empty[0], 1);
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += npairs) {
        ok = mbar_wait(&ctrl->tempty[acc], acc_phase ^ 1u, abort_flag, args.status, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        const uint32_t d0 = tmem_base + uint32_t(acc * k2TileN);
        for (int kb = 0; kb < args.kb_total; ++kb) {
          ok = mbar_wait(&ctrl->full[stage], phase, abort_flag, args.status, ERR_WAIT_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + uint32_t(stage) * uint32_t(k2StageBytes >> 4);
          const uint64_t da = d_hi | a_lo, db = d_hi | (a_lo + uint32_t(kATileBytes >> 4));
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k)
            umma_f16_pair(d0, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty0 + uint32_t(stage) * 8u);
          umma_commit_pair(empty1 + uint32_t(stage) * 8u);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(&ctrl->tfull[acc], 0));
        umma_commit_pair(map_to_cta(&ctrl->tfull[acc], 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    griddep_wait();
    int acc = 0;
    uint32_t acc_phase = 0;
    __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(args.out);
    for (int w = pair; w < total_work; w += npairs) {
      const int kGroup = args.group_m;
      const int per_group = kGroup * args.tiles_n;
      const int g = w / per_group;
      const int first = g * kGroup;
      const int gsz = min(args.tiles_m - first, kGroup);
      const int in = w - g * per_group;
      const int tm = first + in % gsz, tn = in / gsz;
      bool ok = mbar_wait(&ctrl->tfull[acc], acc_phase, abort_flag, args.status, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      const uint32_t t0 = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * k2TileN);
      const int row = tm * 256 + int(rank) * 128 + quad * 32 + lane;
      if (args.gated) {
        // accumulator columns [0, 128) = gate, [128, 256) = up: out[:, tn * 128 + j] = silu(gate_j) * up_j
        const int gcol0 = tn * 128;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t v[32], u[32];
          tmem_ld_32x32(t0 + c, v);
          tmem_ld_32x32(t0 + 128 + c, u);
          tmem_ld_wait();
          if (c + 32 >= 128) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&ctrl->tempty[acc], 0));
          }
          const int cbase = gcol0 + c;
          if (row >= args.m || cbase >= args.n) continue;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(silu_f(__uint_as_float(v[j])) * __uint_as_float(u[j]));
          const long long off = (long long)row * args.ldo + cbase;
          if (cbase + 32 <= args.n && ((off & 7) == 0)) {
            uint4* p = reinterpret_cast<uint4*>(out_h + off);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              p[q] = make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                                pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                                pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                                pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
          } else {
            for (int j = 0; j < 32; ++j)
              if (cbase + j < args.n) out_h[off + j] = __float2bfloat16(__uint_as_float(v[j]));
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      }
      const int col0 = tn * k2TileN;
#pragma unroll 1
      for (int c = 0; c < k2TileN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t0 + c, v);
        tmem_ld_wait();
        if (c + 32 >= k2TileN) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(&ctrl->tempty[acc], 0));
        }
        const int cbase = col0 + c;
        if (row >= args.m || cbase >= args.n) continue;
        if (args.bias && args.bias_on_cols) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (cbase + j < args.n)
              v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(args.bias[cbase + j]));
        }
        const long long off = (long long)row * args.ldo + cbase;
        if (cbase + 32 <= args.n && ((off & 7) == 0)) {
          uint32_t pk[16];
          if (args.residual) {
            const uint4* rp = reinterpret_cast<const uint4*>(args.residual + off);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 rr = rp[q];
              const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_bf16x2(rw[e]);
                pk[q * 4 + e] = pack_bf16x2(__uint_as_float(v[q * 8 + 2 * e]) + f.x,
                                            __uint_as_float(v[q * 8 + 2 * e + 1]) + f.y);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          }
          uint4* p = reinterpret_cast<uint4*>(out_h + off);
#pragma unroll
          for (int q = 0; q < 4; ++q) p[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        } else {
          for (int j = 0; j < 32; ++j) {
            if (cbase + j < args.n) {
              float x = __uint_as_float(v[j]);
              if (args.residual) x += __bfloat162float(args.residual[off + j]);
              out_h[off + j] = __float2bfloat16(x);
            }
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // neither CTA leaves (and frees shared / tensor memory) while its peer still works
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, tmem_cols);
  }
}

}  // namespace nkb

using namespace nkb;

// out[m, n] = A[m, k] * B[n, k]^T (+ bias[n]) (+ residual[m, n]); bf16 in and out, row strides in elements.
// For m, n of at least a few hundred; the launcher returns -5 for shapes it does not take (callers then use
// the single-CTA kernel).
// Number of CTA pairs that can be resident at once (0 before the first launch).
static int g_pairs_last = 0;
extern "C" int nkb_gemm_2cta_pairs() { return g_pairs_last; }

// gated != 0: B holds [gate; up] (2 x n rows, the up half starting at row gate_off) and out[m, n] =
// silu(A gate^T) * (A up^T); bias / residual are not applied in that mode.
extern "C" int nkb_gemm_bf16_2cta(const void* A, const void* B, void* out, int m, int n, int k, long long lda,
                                  long long ldb, long long ldo, const void* bias, const void* residual, int gated,
                                  int gate_off, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (m <= 0 || n <= 0 || k <= 0) return -2;
  if ((k & 7) || (lda & 7) || (ldb & 7)) return -2;
  if (m < 256 || n < 256) return -5;
  Gemm2Args a{};
  a.m = m; a.n = n; a.k = k;
  a.tiles_m = (m + 255) / 256;
  a.tiles_n = gated ? (n + 127) / 128 : (n + 255) / 256;
  a.gated = gated ? 1 : 0;
  a.gate_off = gate_off;
  if (gated && (bias || residual)) return -2;
  a.kb_total = (k + kBlockK - 1) / kBlockK;
  a.bias_on_cols = 1;
  static int group_m = 0;
  if (group_m == 0) {
    const char* e = getenv("NKIPY_B200_2CTA_GROUP");
    group_m = e ? atoi(e) : 16;
    if (group_m < 1) group_m = 16;
  }
  a.group_m = group_m;
  a.ldo = ldo;
  a.out = out;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.status = status_word();
  int stages = (232448 - 1024 - 1024) / k2StageBytes;
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  const int smem = stages * k2StageBytes + 2048;
  CUtensorMap ta, tb;
  if (encode_tmap_bf16_2d(&ta, A, k, m, lda, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, B, k, gated ? uint64_t(gate_off) + n : uint64_t(n), ldb, kBlockK, kTileRows)) return -4;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return int(e);
    attr_set = true;
  }
  const int total = a.tiles_m * a.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (num_sms() / 2));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = size_t(smem);
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The persistent loop strides by the number of pairs, so every pair must be resident at once: pairs need
  // two SMs of one GPC, and not every SM can be paired.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm2_kernel, &cfg);
    max_pairs = (e == cudaSuccess && n > 0) ? n : num_sms() / 4;
  }
  int pairs = max_pairs < total ? max_pairs : total;
  g_pairs_last = pairs;
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return int(cudaLaunchKernelEx(&cfg, gemm2_kernel, ta, tb, a));
}
