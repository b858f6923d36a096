// Persistent, warp-specialised bf16 GEMM for sm_100a (device code; included by the
// library launcher gemm_tcgen05.cu and by generated kernels).
//
//   D[r, c] = sum_k A[r, k] * B[c, k]          (both operands K-major, bf16)
//
// * operands are staged by TMA (128-byte swizzle, 64-wide K slabs) into a
//   multi-stage shared-memory ring,
// * one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into a
//   double-buffered TMEM accumulator,
// * four epilogue warps read the accumulator back with tcgen05.ld while the MMA
//   warp already works on the next tile.
//
// The same kernel serves both orientations used by the models:
//   "normal"  A = activations [tokens, K], B = weights [features, K]  (prefill)
//   "swapped" A = weights [features, K],  B = activations [tokens, K]  (decode:
//             the 128-row MMA dimension is filled by features, the token count
//             becomes the narrow N dimension), output written transposed.
// Optional fusions: split-K partials (fp32), bias, residual add, and the SwiGLU
// gate (two weight tiles per stage, silu(g)*u in the epilogue).
//
// Reference parity: this is the `dot` lowering target of the tracing frontend
// (nkipy/src/nkipy/core/ops/_hlo_impls.py:633-710 in the reference lowers
// np.matmul to an HLO dot executed by the Neuron tensor engine).
#pragma once
#include "common.cuh"
#include "gemm_args.h"
#include "splitk_fix.cuh"

namespace nkb {


struct GemmCtrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort;
  int fix_last;   // split-K fix-up: this CTA arrived last at the tile's counter
};

__device__ __forceinline__ void decode_tile(const GemmArgs& a, int w, int& row_tile, int& col_tile, int& split) {
  split = w % a.splits;
  int t = w / a.splits;
  constexpr int kGroup = 16;
  int per_group = kGroup * a.num_col_tiles;
  int g = t / per_group;
  int first = g * kGroup;
  int gsz = min(a.num_row_tiles - first, kGroup);
  int in = t - g * per_group;
  row_tile = first + in % gsz;
  col_tile = in / gsz;
}

struct WorkItem {
  int rt, ct, sp, group;
  int col0;       // first B row / output column of this tile (global)
  int cols_end;   // one past the last valid column (global)
  bool valid;
};

template <int BN, bool GROUPED>
__device__ __forceinline__ WorkItem decode_work(const GemmArgs& a, const GroupArgs& g, int w) {
  WorkItem wi;
  if constexpr (!GROUPED) {
    decode_tile(a, w, wi.rt, wi.ct, wi.sp);
    wi.group = 0;
    wi.col0 = wi.ct * BN;
    wi.cols_end = a.cols;
    wi.valid = true;
    return wi;
  }
  if (g.tile_list) {
    const int t = w / a.num_row_tiles;
    wi.rt = w - t * a.num_row_tiles;
    wi.sp = 0;
    if (t >= *g.tile_count) {
      wi.valid = false;
      wi.group = wi.ct = wi.col0 = wi.cols_end = 0;
      return wi;
    }
    wi.group = g.tile_list[2 * t];
    wi.ct = g.tile_list[2 * t + 1];
    wi.col0 = g.group_offsets[wi.group] + wi.ct * BN;
    wi.cols_end = g.group_offsets[wi.group + 1];
    wi.valid = true;
  } else if (g.num_groups > 0) {
    const int per_group = a.num_row_tiles * g.max_col_tiles;
    wi.group = w / per_group;
    const int rem = w - wi.group * per_group;
    wi.rt = rem % a.num_row_tiles;
    wi.ct = rem / a.num_row_tiles;
    wi.sp = 0;
    const int off = g.group_offsets[wi.group], end = g.group_offsets[wi.group + 1];
    wi.col0 = off + wi.ct * BN;
    wi.cols_end = end;
    wi.valid = wi.col0 < end;
  } else {
    wi.valid = false;
    wi.rt = wi.ct = wi.sp = wi.group = wi.col0 = wi.cols_end = 0;
  }
  return wi;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

// GROUPED selects the per-expert variant (3-D weight map, group offsets / tile list, expert
// biases and the clamped activation); the plain variant compiles none of that.
// Elementwise epilogue hook for generated kernels: a functor applied to every fp32 accumulator value
// (output row, output column) before the store of the non-transposed orientation.
struct NoElemEpi {
  static constexpr bool active = false;
  __device__ __forceinline__ float operator()(float x, long long, long long) const { return x; }
};

// Optional hook for kernels that run this body as one stage of a longer persistent kernel: `wait` is called
// once by the producer warp (after it has filled the ring with weight tiles, which depend on nothing) and once
// by every epilogue warp before their first use of data or buffers of the preceding stage.  It returns false
// when the wait gave up.
struct NoSync {
  static constexpr bool active = false;
  // lean: compile only the compact epilogue of the decode orientation (transposed output, bias per row; fp32
  // partials / bf16 (+ residual) / SwiGLU / push).  It reads the accumulator sixteen columns at a time in rolled
  // loops: an epilogue runs once per tile, so its instructions are always fetched cold, and the fully unrolled
  // general epilogue (tens of kilobytes of straight-line code) spent microseconds on instruction fetch alone.
  static constexpr bool lean = false;
  __device__ __forceinline__ bool wait(volatile int*) const { return true; }
  __device__ __forceinline__ void mark(int) const {}     // optional time stamps of the body's phases
};
struct LeanSync : NoSync {
  static constexpr bool lean = true;
};

// Fix selects a split-K fix-up epilogue (splitk_fix.cuh): the partial tiles go to fix.c.partials (the
// launcher points args.out there) and the CTA that completes a tile's arrival counter finishes the tile.
// Returns false when a bounded wait inside gave up (the status word then holds the reason).
template <int BN, bool PUSH, bool GROUPED, class Fix = NoFix, class ElemEpi = NoElemEpi, class Sync = NoSync>
__device__ __forceinline__ bool gemm_bf16_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args,
                                               const PushArgs& push, const GroupArgs& grp,
                                               const typename Fix::Args& fix = typename Fix::Args{},
                                               const ElemEpi& elem_epi = ElemEpi{}, const Sync& sync = Sync{}) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = PUSH ? int(threadIdx.x >> 5) : warp_idx_uniform();
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) sync.mark(0);
  const int a_tiles = (args.gated == 1) ? 2 : 1;
  const int b_tiles = (args.gated == 2) ? 2 : 1;
  constexpr int kBTileBytes = BN * kBlockK * 2;
  const int stage_bytes = a_tiles * kATileBytes + b_tiles * kBTileBytes;
  const int stages = args.stages;
  GemmCtrl* ctrl = reinterpret_cast<GemmCtrl*>(tiles + stages * stage_bytes);
  // push mode: [32 tokens][128 features] bf16 staging tile (one accumulator chunk) behind the control block;
  // fix-up mode: 512 bytes of reduction scratch first, then the staging tile
  __nv_bfloat16* stage_out = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(ctrl) +
                                                              (Fix::kind != FIX_NONE ? 1024 : 512));
  float* fix_red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctrl) + 512);

  const int acc_cols = BN * (args.gated ? 2 : 1);
  uint32_t tmem_cols = 32;
  while (tmem_cols < uint32_t(2 * acc_cols)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->tfull[i], 1);
      mbar_init(&ctrl->tempty[i], 4);
    }
    ctrl->abort = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&ctrl->tmem_base, tmem_cols);
    // a CTA that has given up its allocation permit may never allocate again: a body that runs as one stage of
    // a longer kernel (and allocates once per stage) keeps the permit
    if constexpr (!Sync::active) tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort;
  if (threadIdx.x == 0) sync.mark(1);

  const int total_work = GROUPED ? grp.num_groups * args.num_row_tiles * grp.max_col_tiles
                                 : args.num_row_tiles * args.num_col_tiles * args.splits;

  griddep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    auto issue = [&](int stage, int kb, int row0, int col0, int group, bool expect, bool do_a, bool do_b) {
      uint8_t* a_ptr = tiles + stage * stage_bytes;
      uint8_t* b_ptr = a_ptr + a_tiles * kATileBytes;
      if (expect) mbar_expect_tx(&ctrl->full[stage], stage_bytes);
      if (do_a) {
        if constexpr (GROUPED) {
          tma_load_3d(a_ptr, &tmA, &ctrl->full[stage], kb * kBlockK, row0, group);
          if (args.gated == 1)
            tma_load_3d(a_ptr + kATileBytes, &tmA, &ctrl->full[stage], kb * kBlockK, args.gate_off + row0, group);
        } else {
          tma_load_2d(a_ptr, &tmA, &ctrl->full[stage], kb * kBlockK, row0);
          if (args.gated == 1)
            tma_load_2d(a_ptr + kATileBytes, &tmA, &ctrl->full[stage], kb * kBlockK, args.gate_off + row0);
        }
      }
      if (do_b) {
        tma_load_2d(b_ptr, &tmB, &ctrl->full[stage], kb * kBlockK, col0);
        if (args.gated == 2)
          tma_load_2d(b_ptr + kBTileBytes, &tmB, &ctrl->full[stage], kb * kBlockK, args.gate_off + col0);
      }
    };
    // Weight tiles do not depend on the preceding kernel: fill the ring with them
    // before waiting for it, so the HBM stream starts during the predecessor's tail.
    int pre = 0;
    const bool w_is_a = args.weights_operand == 0;
    if (!GROUPED && args.weights_operand >= 0 && int(blockIdx.x) < total_work) {
      int rt, ct, sp;
      decode_tile(args, blockIdx.x, rt, ct, sp);
      const int kb0 = sp * args.kb_per_split;
      const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);
      pre = min(stages, kb1 - kb0);
      if (lane == 0)
        for (int i = 0; i < pre; ++i) issue(i, kb0 + i, rt * kTileRows, ct * BN, 0, true, w_is_a, !w_is_a);
      __syncwarp();
    }
    griddep_wait();
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    int arrived_group = -1;
    if constexpr (Sync::active) {
      int ok = 1;
      if (lane == 0) ok = sync.wait(abort_flag) ? 1 : 0;
      alive = __shfl_sync(0xffffffffu, ok, 0) != 0;
      if (lane == 0) sync.mark(2);
    }
    for (int w = blockIdx.x; w < total_work && alive; w += gridDim.x) {
      const WorkItem wi = decode_work<BN, GROUPED>(args, grp, w);
      if (!wi.valid) continue;
      const int sp = wi.sp;
      const int row0 = wi.rt * kTileRows, col0 = wi.col0;
      const int kb0 = sp * args.kb_per_split;
      const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);
      if constexpr (GROUPED) {
        if (grp.arrive && wi.group != arrived_group) {
          // rows of this expert come from other ranks: wait (bounded) until every source has delivered
          int ok = 1;
          if (lane == 0) {
            const unsigned int* flag = grp.arrive + wi.group;
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (int(v - grp.arrive_target) < 0) {
              const unsigned long long t0 = globaltimer_ns();
              unsigned int spins = 0;
              while (true) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if (int(v - grp.arrive_target) >= 0) break;
                if ((++spins & 255u) == 0 && (*abort_flag || globaltimer_ns() - t0 > kWaitLimitNs)) {
                  *abort_flag = 1;
                  atomicCAS(args.status, 0, ERR_WAIT_PEER_FLAG | (wi.group << 8) | (5 << 16));
                  ok = 0;
                  break;
                }
              }
            }
            // peers wrote these rows through the generic proxy; order them before the async-proxy reads
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { alive = false; break; }
          arrived_group = wi.group;
        }
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        bool ok = mbar_wait(&ctrl->empty[stage], phase ^ 1u, abort_flag, args.status, ERR_WAIT_SMEM_EMPTY);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        if (lane == 0) {
          const bool prefetched = (w == int(blockIdx.x)) && (kb - kb0 < pre);
          if (prefetched) issue(stage, kb, row0, col0, wi.group, false, !w_is_a, w_is_a);
          else issue(stage, kb, row0, col0, wi.group, true, true, true);
        }
        __syncwarp();
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if constexpr (PUSH) {
      // The kernels with the fused-collective epilogue keep the issue loop they were validated with across
      // ranks (the whole warp loops and votes, lane 0 issues); the plain kernels use the single-thread loop below.
      constexpr uint32_t idesc = make_idesc_bf16(kTileRows, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total_work && alive; w += gridDim.x) {
        const WorkItem wi = decode_work<BN, GROUPED>(args, grp, w);
        if (!wi.valid) continue;
        const int sp = wi.sp;
        const int kb0 = sp * args.kb_per_split;
        const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);
        bool ok = mbar_wait(&ctrl->tempty[acc], acc_phase ^ 1u, abort_flag, args.status, ERR_WAIT_TMEM_EMPTY);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + uint32_t(acc * acc_cols);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&ctrl->full[stage], phase, abort_flag, args.status, ERR_WAIT_SMEM_FULL);
          if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          if (lane == 0 && kb == kb0 && w == int(blockIdx.x)) sync.mark(3);
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
            const uint32_t b_addr = a_addr + a_tiles * kATileBytes;
            const uint64_t da = make_smem_desc_sw128(a_addr, 0, 1024);
            const uint64_t db = make_smem_desc_sw128(b_addr, 0, 1024);
            const uint64_t da1 = make_smem_desc_sw128(a_addr + kATileBytes, 0, 1024);
            const uint64_t db1 = make_smem_desc_sw128(b_addr + kBTileBytes, 0, 1024);
  #pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k) {
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              const uint64_t koff = uint64_t(k * 2);  // 16 bf16 = 32 bytes, >>4
              umma_f16(d0, da + koff, db + koff, idesc, accum);
              if (args.gated == 1) umma_f16(d0 + BN, da1 + koff, db + koff, idesc, accum);
              if (args.gated == 2) umma_f16(d0 + BN, da + koff, db1 + koff, idesc, accum);
            }
            umma_commit(&ctrl->empty[stage]);
          }
          __syncwarp();
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        if (lane == 0) umma_commit(&ctrl->tfull[acc]);
        if (lane == 0 && w == int(blockIdx.x)) sync.mark(4);
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    } else {
      // One elected thread runs the whole loop alone: the tensor pipe queues only a few MMAs, so warp votes,
      // reconvergence and descriptor arithmetic between two k-blocks are time in which it drains.
      constexpr uint32_t idesc = make_idesc_bf16(kTileRows, BN, 0, 0);
      if (elect_one()) {
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        const uint64_t d_tiles = make_smem_desc_sw128(smem_u32(tiles), 0, 1024);
        const uint64_t d_hi = d_tiles & 0xffffffff00000000ull;
        const uint32_t a_lo0 = uint32_t(d_tiles);
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
          const WorkItem wi = decode_work<BN, GROUPED>(args, grp, w);
          if (!wi.valid) continue;
          const int sp = wi.sp;
          const int kb0 = sp * args.kb_per_split;
          const int kb1 = min(args.kb_total, kb0 + args.kb_per_split);
          ok = mbar_wait(&ctrl->tempty[acc], acc_phase ^ 1u, abort_flag, args.status, ERR_WAIT_TMEM_EMPTY);
          if (!ok) break;
          const uint32_t d0 = tmem_base + uint32_t(acc * acc_cols);
          for (int kb = kb0; kb < kb1; ++kb) {
            ok = mbar_wait(&ctrl->full[stage], phase, abort_flag, args.status, ERR_WAIT_SMEM_FULL);
            if (!ok) break;
            if (kb == kb0 && w == int(blockIdx.x)) sync.mark(3);
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + uint32_t(stage) * uint32_t(stage_bytes >> 4);
            const uint32_t b_lo = a_lo + uint32_t(a_tiles) * uint32_t(kATileBytes >> 4);
            const uint64_t da = d_hi | a_lo, db = d_hi | b_lo;
            const uint64_t da1 = d_hi | (a_lo + uint32_t(kATileBytes >> 4)), db1 = d_hi | (b_lo + uint32_t(kBTileBytes >> 4));
  #pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k) {
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              const uint64_t koff = uint64_t(k * 2);  // 16 bf16 = 32 bytes, >>4
              umma_f16(d0, da + koff, db + koff, idesc, accum);
              if (args.gated == 1) umma_f16(d0 + BN, da1 + koff, db + koff, idesc, accum);
              if (args.gated == 2) umma_f16(d0 + BN, da + koff, db1 + koff, idesc, accum);
            }
            umma_commit(&ctrl->empty[stage]);
            if (++stage == stages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          umma_commit(&ctrl->tfull[acc]);
          if (w == int(blockIdx.x)) sync.mark(4);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may touch
    griddep_wait();  // residual / output buffers may still be in use by the preceding kernel
    int acc = 0;
    uint32_t acc_phase = 0;
    bool synced = true;
    if constexpr (Sync::active) {
      int ok = 1;
      if (lane == 0) ok = sync.wait(abort_flag) ? 1 : 0;
      synced = __shfl_sync(0xffffffffu, ok, 0) != 0;
    }
    for (int w = blockIdx.x; w < total_work && synced; w += gridDim.x) {
      const WorkItem wi = decode_work<BN, GROUPED>(args, grp, w);
      if (!wi.valid) continue;
      const int rt = wi.rt, sp = wi.sp;
      const int cols_end = wi.cols_end;
      const int row = rt * kTileRows + quad * 32 + lane;
      const int col0 = wi.col0;
      bool ok = mbar_wait(&ctrl->tfull[acc], acc_phase, abort_flag, args.status, ERR_WAIT_TMEM_FULL);
      if constexpr (PUSH) {
        // the four epilogue warps leave together: a warp left alone at the tile barrier below would hang
        if (!bar_red_and(2, 128, __all_sync(0xffffffffu, ok))) break;
      } else {
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      tc_fence_after();
      if (threadIdx.x == 64 && w == int(blockIdx.x)) sync.mark(5);
      const uint32_t t0 = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * acc_cols);
      const bool row_ok = row < args.rows;
      float* out_f = reinterpret_cast<float*>(args.out) + (args.out_fp32 ? sp * args.split_stride : 0);
      __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(args.out);
      float bias_r = 0.f, bias_u = 0.f;
      if (args.bias && args.bias_on_rows && row_ok && sp == 0) {
        const __nv_bfloat16* bp = args.bias + (GROUPED ? wi.group * grp.bias_group_stride : 0) + row;
        bias_r = __bfloat162float(bp[0]);
        if (GROUPED && args.gated) bias_u = __bfloat162float(bp[args.gate_off]);   // up-projection bias
      }

      constexpr bool kLean = Sync::lean && !GROUPED && Fix::kind == FIX_NONE && !ElemEpi::active;
      if constexpr (kLean) {
        // ---- compact epilogue (decode orientation): out[col * ldo + row], sixteen columns per iteration
        auto release_acc = [&]() {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctrl->tempty[acc]);
        };
        if constexpr (PUSH) {
          const int et = threadIdx.x - 64;  // 0..127 over the four epilogue warps
          const int row0 = rt * kTileRows;
          const long long slot = (long long)push.rank * args.splits + sp;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            const bool live = col0 + c0 < cols_end;   // CTA-uniform: the four warps take the barriers together
            if (live) {
#pragma unroll 1
              for (int c = 0; c < 32; c += 16) {
                uint32_t v[16];
                tmem_ld_32x16(t0 + c0 + c, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  stage_out[(c + j) * kTileRows + quad * 32 + lane] = __float2bfloat16(__uint_as_float(v[j]) + bias_r);
              }
            }
            if (c0 + 32 >= BN) release_acc();
            if (!live) continue;
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 1
            for (int idx = et; idx < 32 * 16; idx += 128) {
              const int tok = idx >> 4, ch = idx & 15;
              const int gtok = col0 + c0 + tok, gfeat = row0 + ch * 8;
              if (gtok < cols_end && gfeat < args.rows) {
                const uint4 val = *reinterpret_cast<const uint4*>(stage_out + tok * kTileRows + ch * 8);
                push_store_16(push, (slot * args.cols + gtok) * args.ldo + gfeat, val);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        } else {
          // transpose_out == 2 (set by the host when base, leading dimension and row count are 16-byte
          // aligned): the tile goes out through shared memory and bulk asynchronous copies, one per token row.
          // With most of the SM's memory configured as shared memory almost no L1 is left, and plain global
          // stores from these four warps then retire one L2 round trip at a time (50 ns each, 3.5 us per tile).
          const bool gated = args.gated != 0;
          const bool bulk = args.transpose_out == 2 && (gated || !args.residual);
          const int et = threadIdx.x - 64;
          const int row0 = rt * kTileRows;
          const int nrow = min(kTileRows, args.rows - row0);
          const bool as_f32 = !gated && args.out_fp32;
          const uint32_t esz = as_f32 ? 4u : 2u;
          uint8_t* stg = reinterpret_cast<uint8_t*>(stage_out);          // two buffers of 16 x 128 elements
          uint8_t* out_b = reinterpret_cast<uint8_t*>(args.out) +
                           (as_f32 ? (long long)sp * args.split_stride * 4 : 0);
#pragma unroll 1
          for (int c = 0; c < BN; c += 16) {
            const int it = c >> 4;
            float x[16];
            if (gated) {
              uint32_t g[16], u[16];
              tmem_ld_32x16(t0 + c, g);
              tmem_ld_32x16(t0 + BN + c, u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) x[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
            } else {
              uint32_t v[16];
              tmem_ld_32x16(t0 + c, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) x[j] = __uint_as_float(v[j]) + bias_r;
            }
            if (c + 16 >= BN) release_acc();
            if (col0 + c >= cols_end) continue;          // CTA-uniform
            if (bulk) {
              uint8_t* buf = stg + (it & 1) * 8192;
              // the copies that read this buffer two rounds ago (possibly for the previous tile) are done
              if (et == 0) bulk_wait_read<1>();
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (as_f32) {
                float* b = reinterpret_cast<float*>(buf) + quad * 32 + lane;
#pragma unroll
                for (int j = 0; j < 16; ++j) b[j * kTileRows] = x[j];
              } else {
                __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(buf) + quad * 32 + lane;
#pragma unroll
                for (int j = 0; j < 16; ++j) b[j * kTileRows] = __float2bfloat16(x[j]);
              }
              fence_proxy_async();
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (et == 0) {
#pragma unroll 1
                for (int j = 0; j < 16; ++j) {
                  const int col = col0 + c + j;
                  if (col < cols_end)
                    bulk_store_1d(out_b + ((long long)col * args.ldo + row0) * esz, buf + j * kTileRows * esz,
                                  uint32_t(nrow) * esz);
                }
                bulk_commit();
              }
            } else if (row_ok) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int col = col0 + c + j;
                if (col < cols_end) {
                  const long long idx = (long long)col * args.ldo + row;
                  float y = x[j];
                  if (as_f32) {
                    out_f[idx] = y;
                  } else {
                    if (!gated && args.residual) y += __bfloat162float(args.residual[idx]);
                    out_h[idx] = __float2bfloat16(y);
                  }
                }
              }
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        if (threadIdx.x == 64 && w == int(blockIdx.x) && c == 32) sync.mark(10);
        tmem_ld_32x32(t0 + c, v);
        if (args.gated) {
          uint32_t u[32];
          tmem_ld_32x32(t0 + BN + c, u);
          tmem_ld_wait();
          if (GROUPED && grp.act_limit > 0.f) {
            // clamped variant: (up + 1) * gate * sigmoid(alpha * gate), biases before the activation
            const float lim = grp.act_limit, alpha = grp.act_alpha;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gg = fminf(__uint_as_float(v[j]) + bias_r, lim);
              const float uu = fminf(fmaxf(__uint_as_float(u[j]) + bias_u, -lim), lim);
              v[j] = __float_as_uint((uu + 1.f) * gg / (1.f + __expf(-alpha * gg)));
            }
          } else if (GROUPED) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(silu_f(__uint_as_float(v[j]) + bias_r) * (__uint_as_float(u[j]) + bias_u));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(silu_f(__uint_as_float(v[j])) * __uint_as_float(u[j]));
          }
        } else {
          tmem_ld_wait();
        }
        if (threadIdx.x == 64 && w == int(blockIdx.x)) sync.mark(c == 0 ? 8 : 11);
        if (c + 32 >= BN) {
          // accumulator fully read: hand it back to the MMA warp before the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctrl->tempty[acc]);
        }
        const int cbase = col0 + c;
        if (cbase >= cols_end) continue;
        if (args.bias && sp == 0 && !args.gated) {
          if (args.bias_on_rows) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + bias_r);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cbase + j < cols_end)
                v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(args.bias[cbase + j]));
          }
        }
        if constexpr (PUSH) {
          // stage the chunk (token j, feature quad * 32 + lane), then the four warps store it to every rank as
          // 16-byte pieces, 256 contiguous bytes per token.  cbase and cols_end are CTA-uniform, so the four
          // warps reach the two barriers together.
#pragma unroll
          for (int j = 0; j < 32; ++j)
            stage_out[j * kTileRows + quad * 32 + lane] = __float2bfloat16(__uint_as_float(v[j]));
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int et = threadIdx.x - 64;  // 0..127 over the four epilogue warps
          const int row0 = rt * kTileRows;
          const long long slot = (long long)push.rank * args.splits + sp;
#pragma unroll
          for (int idx = et; idx < 32 * 16; idx += 128) {
            const int tok = idx >> 4, ch = idx & 15;
            const int gtok = cbase + tok, gfeat = row0 + ch * 8;
            if (gtok < cols_end && gfeat < args.rows) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage_out + tok * kTileRows + ch * 8);
              const long long off = (slot * args.cols + gtok) * args.ldo + gfeat;
              push_store_16(push, off, val);
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          continue;
        }
        if constexpr (ElemEpi::active) {
          if (row_ok && !args.transpose_out) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cbase + j < cols_end) v[j] = __float_as_uint(elem_epi(__uint_as_float(v[j]), row, cbase + j));
          }
        }
        if (args.transpose_out) {
          // out[col * ldo + row]: consecutive lanes hold consecutive rows -> coalesced
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = cbase + j;
              if (col < cols_end) {
                const long long idx = (long long)col * args.ldo + row;
                float x = __uint_as_float(v[j]);
                if (args.out_fp32) {
                  out_f[idx] = x;
                } else {
                  if (args.residual) x += __bfloat162float(args.residual[idx]);
                  out_h[idx] = __float2bfloat16(x);
                }
              }
            }
          }
        } else if (row_ok) {
          const long long base = (long long)row * args.ldo + cbase;
          const bool full = (cbase + 32 <= cols_end);
          if (args.out_fp32) {
            if (full && ((base & 3) == 0)) {
              float4* p = reinterpret_cast<float4*>(out_f + base);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                p[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                   __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            } else {
              for (int j = 0; j < 32; ++j)
                if (cbase + j < cols_end) out_f[base + j] = __uint_as_float(v[j]);
            }
          } else {
            if (full && ((base & 7) == 0)) {
              uint32_t pk[16];
              if (args.residual) {
                const uint4* rp = reinterpret_cast<const uint4*>(args.residual + base);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 rr = rp[q];
                  uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float2 f = unpack_bf16x2(rw[e]);
                    pk[q * 4 + e] = pack_bf16x2(__uint_as_float(v[q * 8 + 2 * e]) + f.x,
                                                __uint_as_float(v[q * 8 + 2 * e + 1]) + f.y);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  pk[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
              }
              uint4* p = reinterpret_cast<uint4*>(out_h + base);
#pragma unroll
              for (int q = 0; q < 4; ++q) p[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            } else {
              for (int j = 0; j < 32; ++j) {
                if (cbase + j < cols_end) {
                  float x = __uint_as_float(v[j]);
                  if (args.residual) x += __bfloat162float(args.residual[base + j]);
                  out_h[base + j] = __float2bfloat16(x);
                }
              }
            }
          }
        }
      }
      }  // general epilogue
      if constexpr (Fix::kind != FIX_NONE) {
        // this CTA's partial of the tile is stored: count it, and finish the tile if it was the last one
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int pairs = Fix::kind == FIX_SWIGLU ? args.num_row_tiles / 2 : args.num_row_tiles;
          unsigned int* ctr = fix.c.tile_counters + (rt % pairs);
          const unsigned int target = unsigned(args.splits) * (Fix::kind == FIX_SWIGLU ? 2u : 1u);
          const unsigned int old = atomicAdd(ctr, 1u);
          const int last = old == target - 1u;
          if (last) *ctr = 0u;   // all arrivals of this launch are in; the next launch starts from zero
          ctrl->fix_last = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ctrl->fix_last) {
          __threadfence();
          const int pairs = Fix::kind == FIX_SWIGLU ? args.num_row_tiles / 2 : args.num_row_tiles;
          run_fix<Fix>(fix, rt % pairs, Fix::kind == FIX_SWIGLU ? args.rows / 2 : args.rows, args.cols, args.splits,
                       args.split_stride, stage_out, fix_red);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if constexpr (Fix::kind == FIX_PUSH) {
      // same completion protocol as the push epilogue below: every CTA counts itself after its last tile, the
      // last CTA of the grid publishes all peer stores with one system-scope fence and bumps the peers' flags
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        __threadfence();
        const unsigned int old = atomicAdd(fix.push.done_counter, 1u);
        if (old == gridDim.x - 1) {
          *fix.push.done_counter = 0u;
          __threadfence_system();
          push_signal(fix.push);
        }
      }
    }
    if constexpr (PUSH) {
      // all peer stores of this CTA are issued: publish them, count the CTA, and let the
      // last CTA of the grid signal every peer
      // The barrier orders the four warps' stores before the publishing thread's fence.  Every CTA releases at
      // GPU scope into the grid counter; the last CTA, which has observed all of them, releases at system scope
      // into the peers' flags (causality order is transitive across the two scopes).
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        __threadfence();
        const unsigned int old = atomicAdd(push.done_counter, 1u);
        if (old == gridDim.x - 1) {
          *push.done_counter = 0u;
          __threadfence_system();
          push_signal(push);
        }
      }
    }
  }

  if constexpr (Sync::lean) {
    // bulk copies of the compact epilogue: complete (and visible) before this CTA signals anybody
    if (threadIdx.x == 64) {
      bulk_wait_all();
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  }
  if (threadIdx.x == 64) sync.mark(6);
  if (*abort_flag) {
    // let copies / MMAs that were already issued drain before shared memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  const bool all_ok = *abort_flag == 0;
  if (threadIdx.x == 0) sync.mark(7);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if constexpr (Sync::active) {
    // a stage of a longer kernel: the next stage creates its barriers in the same place.  After a time-out
    // some barrier may still have a transaction pending, so the words are left alone (the caller returns).
    if (threadIdx.x == 0 && all_ok) {
      for (int s = 0; s < stages; ++s) {
        mbar_inval(&ctrl->full[s]);
        mbar_inval(&ctrl->empty[s]);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_inval(&ctrl->tfull[i]);
        mbar_inval(&ctrl->tempty[i]);
      }
    }
    __syncthreads();
  }
  return all_ok;
}

template <int BN, int MINB, bool PUSH>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmArgs args, const PushArgs push) {
  gemm_bf16_body<BN, PUSH, false>(tmA, tmB, args, push, GroupArgs{});
}

// Decode orientation only (transposed output, bias per row): the compact epilogue.
template <int BN, int MINB, bool PUSH>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gemm_bf16_lean_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmArgs args, const PushArgs push) {
  gemm_bf16_body<BN, PUSH, false, NoFix, NoElemEpi, LeanSync>(tmA, tmB, args, push, GroupArgs{}, NoFix::Args{},
                                                              NoElemEpi{}, LeanSync{});
}

template <int BN, int MINB, class Fix>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gemm_bf16_fix_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const GemmArgs args, const typename Fix::Args fix) {
  gemm_bf16_body<BN, false, false, Fix>(tmA, tmB, args, PushArgs{}, GroupArgs{}, fix);
}

template <int BN, int MINB>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gemm_bf16_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmArgs args, const GroupArgs grp) {
  gemm_bf16_body<BN, false, true>(tmA, tmB, args, PushArgs{}, grp);
}

}  // namespace nkb
