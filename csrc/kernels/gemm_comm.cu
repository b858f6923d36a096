// Tensor-parallel GEMMs fused with their collective for prefill-sized batches:
//
//   gemm_rs  (row-parallel):    out[M/tp, N] = reduce_scatter_rows( X[M, K/tp] * W[N, K/tp]^T )
//   ag_gemm  (column-parallel): out[M, N/tp] = all_gather_rows( X[M/tp, K] ) * W[N/tp, K]^T
//
// Each is ONE kernel per rank.  The GEMM part is the persistent warp-specialised tcgen05 pipeline
// (TMA -> shared-memory ring -> tcgen05.mma into a double-buffered TMEM accumulator -> epilogue warps);
// the collective part moves data with plain peer stores over NVLink into symmetric (IPC-mapped)
// buffers and synchronises with system-scope arrival counters.  TMA only ever reads this GPU's own
// memory, and nothing here uses multicast.
//
// gemm_rs: row tiles are visited starting with the tile after this rank's own slab, so tiles owned by
//   peers are produced first.  The epilogue converts a finished tile to bf16, stages it through shared
//   memory so that every warp store covers 256 contiguous bytes of a row, and writes it into slot
//   [rank] of the OWNER's staging array [tp, M/tp, N]; after a system fence one thread adds 1 to the
//   owner's counter (src = rank, row tile).  When a CTA has no GEMM tile left its epilogue warps turn
//   into the reducer: for every (own row tile, 256-column chunk) they wait (bounded) until all tp
//   sources have delivered, sum the tp slots in fp32 and write the bf16 result.
// ag_gemm: the first `comm_ctas` CTAs only push this rank's slab, 128-row chunk by chunk, into every
//   peer's gather buffer (destination order rank-1, rank-2, ... so that every link carries one slab at a
//   time and slabs arrive in the order the consumer visits them), bumping the counter (src = rank, chunk)
//   on the destination after each chunk.  The other CTAs run the GEMM over the row tiles in the order own
//   slab, slab rank+1, ...; the TMA producer waits (bounded) for the counters of the chunks a tile needs
//   before its first load.
// Counters only grow (the host passes the call number as `epoch`), two buffers alternate between
// consecutive calls, and a rank can be at most one call ahead of a peer because it needs that peer's
// data of the current call to finish it.
//
// Reference parity: the reference shards o_proj/down row-wise and QKV/gate_up column-wise and reduces
// with all-reduce instructions inside the compiled graph (examples/models/qwen3/kernels/attention.py:
// 150-154, examples/models/qwen3/kernels/transformer_layer.py:112-115); these kernels are the NVLink
// counterpart for token counts where reduce-scatter / all-gather (sequence-parallel layout) pay off.
#include "gemm_tcgen05.cuh"
#include "api.h"
#include <stdlib.h>

namespace nkb {

constexpr int kCommMaxPeers = 8;

struct CommArgs {               // <= 128 bytes (see GemmArgs)
  int m, n, k;                  // this rank's GEMM: A [m, k], B [n, k]
  int num_row_tiles, num_col_tiles, kb_total, stages;
  int tp, rank, rows_per_rank;
  int first_tile;               // rotation of the row-tile order
  int comm_ctas;                // ag_gemm: CTAs that only push slabs
  int local_direct;             // ag_gemm: own slab is read from x_local (rows_per_rank % 128 == 0)
  unsigned int epoch;           // 1, 2, 3, ... per call on these buffers
  int flag_stride;              // counters per source rank
  int ldx;                      // ag_gemm: row stride of x_local in elements
  int gated;                    // ag_gemm on CTA pairs: B holds [gate; up], out = silu(gate) * up
  int gate_off;                 // row offset of the up half in B
  long long ldo;
  void* out;
  const __nv_bfloat16* x_local; // ag_gemm: this rank's slab [rows_per_rank, k]
  __nv_bfloat16* local_buf;     // gemm_rs: staging [tp, rows_per_rank, n]; ag_gemm: gather buffer [m, k]
  unsigned int* local_flags;    // [tp * flag_stride]
  int* status;
};
static_assert(sizeof(CommArgs) <= 128, "CommArgs grew past the fast kernel-parameter size");

struct CommPeers {
  __nv_bfloat16* buf[kCommMaxPeers];     // every rank's staging / gather buffer of this call
  unsigned int* flags[kCommMaxPeers];    // every rank's counter array
};

__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *flag >= target (wrap-safe).  false = gave up (status written).
__device__ __forceinline__ bool wait_counter(const unsigned int* flag, unsigned int target, int* status, int detail) {
  if (int(ld_acquire_sys_u32(flag) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (int(ld_acquire_sys_u32(flag) - target) < 0) {
    if ((++spins & 127u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (detail << 8));
      return false;
    }
  }
  return true;
}

struct CommShared {
  GemmCtrl ctrl;                               // <= 512 bytes
  __nv_bfloat16* peer_buf[kCommMaxPeers];
  unsigned int* peer_flags[kCommMaxPeers];
  uint64_t pub_full[2];                        // gemm_rs: a tile's peer stores are issued (4 epilogue warps arrive)
  uint64_t pub_empty[2];                       // gemm_rs: the publisher has counted that tile
};

// warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warp 6 publisher (gemm_rs: system fence + arrival counters,
// kept off the epilogue's critical path)
constexpr int kCommThreads = kGemmThreads + 32;

constexpr int kCommCtrlBytes = 1024;
constexpr int kStageOutBytes = 4 * 32 * 128 * 2;   // per epilogue warp: 32 rows x 128 columns bf16

// MODE 0 = gemm_rs, 1 = ag_gemm.  PAIR: two CTAs of a cluster share one 256 x BN tile through
// `tcgen05.mma.cta_group::2` (CTA r of the pair holds rows 128 r .. 128 r + 127 of the A tile and of the
// B tile); everything below that is keyed on 128-row tiles (owners, counters, staging, chunk waits) then
// simply applies to this CTA's half.  The first CTA of a pair issues the MMAs and owns the `full` and
// `tempty` barriers; see gemm_2cta.cu for the barrier scheme.
template <int BN, int MODE, bool PAIR>
__global__ void __launch_bounds__(kCommThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB, const CommArgs args, const CommPeers peers) {
  // shared memory: [control block 1 KB][gemm_rs: epilogue staging 32 KB][ring of stages], 1024-aligned
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  CommShared* sh = reinterpret_cast<CommShared*>(base);
  uint8_t* stage_out = base + kCommCtrlBytes;                              // gemm_rs only
  uint8_t* tiles = base + kCommCtrlBytes + (MODE == 0 ? kStageOutBytes : 0);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < kCommMaxPeers) {
    sh->peer_buf[threadIdx.x] = peers.buf[threadIdx.x];
    sh->peer_flags[threadIdx.x] = peers.flags[threadIdx.x];
  }
  __syncthreads();

  // ------------------------------------------------------------------ ag_gemm: slab pusher CTAs
  // One thread per pusher CTA streams the slab through a ring of 16 KB shared-memory buffers with bulk
  // copies (global -> shared, shared -> peer global): 128 KB of loads and up to 64 KB of peer stores in
  // flight per CTA without spending registers or issue slots on the data.
  if (MODE == 1 && int(blockIdx.x) < args.comm_ctas) {
    constexpr int kSlots = 12, kAhead = 8, kPiece = 16384;
    uint8_t* ring = base + kCommCtrlBytes;
    uint64_t* full = sh->ctrl.full;
    if (threadIdx.x == 0) {
      for (int i = 0; i < kSlots; ++i) mbar_init(&full[i], 1);
      sh->ctrl.abort = 0;
      mbar_fence_init();
      fence_proxy_async();
    }
    if (threadIdx.x != 0) return;
    griddep_wait();
    griddep_launch();
    const int nch = (args.rows_per_rank + 127) / 128;
    const int nd = args.local_direct ? args.tp - 1 : args.tp;
    const int items = nch * nd;
    const bool contiguous = args.ldx == args.k;
    const long long row_bytes = (long long)args.k * 2;
    int issued = 0, consumed = 0;   // pieces loaded / stored so far by this CTA (ring positions)
    for (int it = blockIdx.x; it < items; it += args.comm_ctas) {
      const int d = it / nch, c = it - d * nch;
      const int s = args.local_direct ? d + 1 : d;              // 0 = self copy (small batches only)
      const int dest = (args.rank - s + args.tp) % args.tp;
      const int r0 = c * 128, r1 = min(args.rows_per_rank, r0 + 128);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(args.x_local + (long long)r0 * args.ldx);
      uint8_t* dst = reinterpret_cast<uint8_t*>(sh->peer_buf[dest] +
                                                (long long)(args.rank * args.rows_per_rank + r0) * args.k);
      // spans: the whole chunk when the slab is dense, otherwise one span per row
      const int nspans = contiguous ? 1 : (r1 - r0);
      const long long span_bytes = contiguous ? (long long)(r1 - r0) * row_bytes : row_bytes;
      const int pps = int((span_bytes + kPiece - 1) / kPiece);
      const int pieces = nspans * pps;
      auto piece = [&](int i, const uint8_t*& ps, uint8_t*& pd, uint32_t& bytes) {
        const int sp = i / pps;
        const long long off = (long long)(i - sp * pps) * kPiece;
        bytes = uint32_t(min((long long)kPiece, span_bytes - off));
        ps = src + (long long)sp * args.ldx * 2 + off;
        pd = dst + (long long)sp * row_bytes + off;
      };
      auto load = [&](int i) {
        const uint8_t* ps; uint8_t* pd; uint32_t bytes;
        piece(i, ps, pd, bytes);
        const int slot = issued % kSlots;
        mbar_expect_tx(&full[slot], bytes);
        bulk_load_1d(ring + slot * kPiece, ps, bytes, &full[slot]);
        ++issued;
      };
      bool ok = true;
      const int first = issued;
      for (int i = 0; i < min(kAhead, pieces); ++i) load(i);
      for (int i = 0; i < pieces && ok; ++i) {
        const int slot = consumed % kSlots;
        ok = mbar_wait(&full[slot], uint32_t(consumed / kSlots) & 1u, &sh->ctrl.abort, args.status,
                       ERR_WAIT_SMEM_FULL);
        if (!ok) break;
        const uint8_t* ps; uint8_t* pd; uint32_t bytes;
        piece(i, ps, pd, bytes);
        bulk_store_1d(pd, ring + slot * kPiece, bytes);
        bulk_commit();
        ++consumed;
        const int j = issued - first;            // next piece of this item to load
        if (j < pieces) {
          // its slot was last read by the store issued kSlots - kAhead pieces ago
          bulk_wait_read<kSlots - kAhead>();
          load(j);
        }
      }
      bulk_wait_all();                            // every store of this chunk has landed
      if (!ok) break;
      __threadfence_system();
      atomicAdd_system(sh->peer_flags[dest] + args.rank * args.flag_stride + c, 1u);
    }
    return;
  }

  constexpr int kBTileBytes = (PAIR ? BN / 2 : BN) * kBlockK * 2;      // this CTA's rows of the B tile
  constexpr int stage_bytes = kATileBytes + kBTileBytes;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;                // 0 issues the MMAs
  const int stages = args.stages;
  GemmCtrl* ctrl = &sh->ctrl;
  constexpr uint32_t tmem_cols = 2 * BN;                                  // 256 or 512

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    if (MODE == 1) tma_prefetch_desc(&tmA2);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->tfull[i], 1);
      mbar_init(&ctrl->tempty[i], PAIR ? 8 : 4);
      mbar_init(&sh->pub_full[i], 4);
      mbar_init(&sh->pub_empty[i], 1);
    }
    ctrl->abort = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(&ctrl->tmem_base, tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&ctrl->tmem_base, tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();          // both CTAs' barriers exist before anything remote arrives
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort;

  // work items: (row tile or pair of row tiles in rotated order) x column tile
  const int units = PAIR ? 2 : 1;
  const int cta = (int(blockIdx.x) - (MODE == 1 ? args.comm_ctas : 0)) / units;
  const int ncta = (int(gridDim.x) - (MODE == 1 ? args.comm_ctas : 0)) / units;
  const int row_groups = PAIR ? (args.num_row_tiles + 1) / 2 : args.num_row_tiles;
  const int total_work = row_groups * args.num_col_tiles;
  // this CTA's 128-row tile and the column tile of work item w (the row tile may lie past the last row
  // for the second CTA of the last pair: it then loads zeros and skips its epilogue)
  auto decode = [&](int w, int& rt, int& ct) {
    const int ro = w / args.num_col_tiles;
    ct = w - ro * args.num_col_tiles;
    int g = args.first_tile + ro;
    if (g >= row_groups) g -= row_groups;
    rt = PAIR ? 2 * g + int(crank) : g;
  };
  griddep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    griddep_wait();
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int w = cta; w < total_work && alive; w += ncta) {
      int rt, ct;
      decode(w, rt, ct);
      const int r0 = rt * kTileRows, r1 = min(args.m, r0 + kTileRows);
      bool from_local = false;
      int a_row = r0;
      if (MODE == 1) {
        // rows [r0, r1) of the gathered activations: wait for the chunks that hold them
        const int rpr = args.rows_per_rank;
        const int s0 = r0 / rpr, s1 = r1 > r0 ? (r1 - 1) / rpr : s0 - 1;
        if (args.local_direct && s0 == args.rank && r1 > r0) {
          from_local = true;
          a_row = r0 - args.rank * rpr;
        } else {
          int ok = 1;
          if (lane == 0) {
            for (int src = s0; src <= s1 && ok; ++src) {
              const int lo = max(r0, src * rpr) - src * rpr, hi = min(r1, (src + 1) * rpr) - src * rpr;
              for (int c = lo / 128; c <= (hi - 1) / 128 && ok; ++c)
                ok = wait_counter(args.local_flags + src * args.flag_stride + c, args.epoch, args.status,
                                  (blockIdx.x << 8) | src)
                         ? 1 : 0;
            }
            if (!ok) *abort_flag = 1;
            // peers wrote these rows through the generic proxy; order them before the async-proxy reads
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { alive = false; break; }
        }
      }
      for (int kb = 0; kb < args.kb_total; ++kb) {
        bool ok = mbar_wait(&ctrl->empty[stage], phase ^ 1u, abort_flag, args.status, ERR_WAIT_SMEM_EMPTY);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        if (lane == 0) {
          uint8_t* a_ptr = tiles + stage * stage_bytes;
          const CUtensorMap* ma = (MODE == 1 && !from_local) ? &tmA2 : &tmA;
          if (PAIR) {
            // the first CTA announces the bytes of both; both CTAs' loads complete on its barrier
            const uint32_t full0 = map_to_cta(&ctrl->full[stage], 0);
            if (crank == 0) mbar_expect_tx(&ctrl->full[stage], 2 * stage_bytes);
            tma_load_2d_pair(a_ptr, ma, full0, kb * kBlockK, a_row);
            const int b_row = (MODE == 1 && args.gated) ? int(crank) * args.gate_off + ct * (BN / 2)
                                                        : ct * BN + int(crank) * (BN / 2);
            tma_load_2d_pair(a_ptr + kATileBytes, &tmB, full0, kb * kBlockK, b_row);
          } else {
            mbar_expect_tx(&ctrl->full[stage], stage_bytes);
            tma_load_2d(a_ptr, ma, &ctrl->full[stage], kb * kBlockK, a_row);
            tma_load_2d(a_ptr + kATileBytes, &tmB, &ctrl->full[stage], kb * kBlockK, ct * BN);
          }
        }
        __syncwarp();
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 && crank == 0) {
    // ------------------------------------------------------------------ MMA issuer (first CTA of a pair)
    constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 2 * kTileRows : kTileRows, BN, 0, 0);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    for (int w = cta; w < total_work && alive; w += ncta) {
      bool ok = mbar_wait(&ctrl->tempty[acc], acc_phase ^ 1u, abort_flag, args.status, ERR_WAIT_TMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      tc_fence_after();
      const uint32_t d0 = tmem_base + uint32_t(acc * BN);
      for (int kb = 0; kb < args.kb_total; ++kb) {
        ok = mbar_wait(&ctrl->full[stage], phase, abort_flag, args.status, ERR_WAIT_SMEM_FULL);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_addr = smem_u32(tiles + stage * stage_bytes);
          const uint64_t da = make_smem_desc_sw128(a_addr, 0, 1024);
          const uint64_t db = make_smem_desc_sw128(a_addr + kATileBytes, 0, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            if (PAIR) umma_f16_pair(d0, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16(d0, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          if (PAIR) {
            umma_commit_pair(map_to_cta(&ctrl->empty[stage], 0));
            umma_commit_pair(map_to_cta(&ctrl->empty[stage], 1));
          } else {
            umma_commit(&ctrl->empty[stage]);
          }
        }
        __syncwarp();
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
      if (!alive) break;
      if (lane == 0) {
        if (PAIR) {
          umma_commit_pair(map_to_cta(&ctrl->tfull[acc], 0));
          umma_commit_pair(map_to_cta(&ctrl->tfull[acc], 1));
        } else {
          umma_commit(&ctrl->tfull[acc]);
        }
      }
      __syncwarp();
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else if (warp == 1) {
    // second CTA of a pair: the MMAs of both CTAs are issued by the first
  } else if (warp == 6) {
    // ------------------------------------------------------------------ publisher (gemm_rs)
    // A system fence waits for every peer store this SM has in flight, which under a saturated link is
    // tens of microseconds: the counters of the tiles of one owner phase are therefore published in
    // batches (one fence per batch).  A tile that also holds rows of this rank is published at once,
    // because the same CTA then waits for its peers, who may be waiting for exactly this tile.
    if (MODE == 0 && args.tp > 1) {
      constexpr int kBatch = 8;
      const int rpr = args.rows_per_rank;
      const int own0 = args.rank * rpr, own1 = own0 + rpr;
      unsigned int* pend[kBatch];
      int npend = 0, pend_phase = -1;
      int u = 0;
      bool alive = true;
      auto flush = [&]() {
        if (lane == 0 && npend > 0) {
          // the epilogue warps' stores happen-before this point (mbarrier acquire); the fence is cumulative
          __threadfence_system();
          for (int i = 0; i < npend; ++i) atomicAdd_system(pend[i], 1u);
        }
        npend = 0;
      };
      for (int w = cta; w < total_work && alive; w += ncta) {
        int rt, ct_unused;
        decode(w, rt, ct_unused);
        const int r0 = rt * kTileRows, r1 = min(args.m, r0 + kTileRows);
        if (r0 >= args.m) continue;                // the second CTA of the last pair may have no rows
        const int phase_id = r0 / rpr;
        if (npend > 0 && phase_id != pend_phase) flush();
        if (!(r0 < own0 || r1 > own1)) continue;   // no peer rows in this tile
        const int slot = u & 1;
        bool ok = mbar_wait(&sh->pub_full[slot], (uint32_t(u) >> 1) & 1u, abort_flag, args.status, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        if (lane == 0) mbar_arrive(&sh->pub_empty[slot]);
        ++u;
        for (int o = r0 / rpr; o <= (r1 - 1) / rpr; ++o) {
          if (o == args.rank) continue;
          const int lo = max(r0, o * rpr) - o * rpr, hi = min(r1, (o + 1) * rpr) - o * rpr;
          for (int t = lo / 128; t <= (hi - 1) / 128; ++t) {
            if (npend == kBatch) flush();
            pend[npend++] = sh->peer_flags[o] + args.rank * args.flag_stride + t;
          }
        }
        pend_phase = phase_id;
        if (r0 < own1 && r1 > own0) flush();       // this CTA is about to wait for its peers
        __syncwarp();
      }
      flush();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    griddep_wait();
    int published = 0;   // gemm_rs: tiles of this CTA handed to the publisher so far
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    // hands an accumulator back to the MMA warp (of the pair's first CTA)
    auto release_acc = [&](int a) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(&ctrl->tempty[a], 0));
        else mbar_arrive(&ctrl->tempty[a]);
      }
    };
    for (int w = cta; w < total_work; w += ncta) {
      int rt, ct;
      decode(w, rt, ct);
      const int col0 = ct * BN;
      bool ok = mbar_wait(&ctrl->tfull[acc], acc_phase, abort_flag, args.status, ERR_WAIT_TMEM_FULL);
      // the four epilogue warps leave together: a warp left alone at the tile barrier below would hang
      if (!bar_red_and(2, 128, __all_sync(0xffffffffu, ok))) { alive = false; break; }
      tc_fence_after();
      const uint32_t t0 = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN);
      if (rt * kTileRows >= args.m) {              // no rows in this CTA's half: nothing to write or publish
        release_acc(acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      }
      if (MODE == 1 && PAIR && args.gated) {
        // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up (the pair's first CTA loaded gate rows, the
        // second up rows): out[:, ct * BN/2 + j] = silu(gate_j) * up_j
        const int row = rt * kTileRows + quad * 32 + lane;
        __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(args.out);
        const int gcol0 = ct * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          uint32_t v[32], u[32];
          tmem_ld_32x32(t0 + c, v);
          tmem_ld_32x32(t0 + BN / 2 + c, u);
          tmem_ld_wait();
          if (c + 32 >= BN / 2) release_acc(acc);
          const int cbase = gcol0 + c;
          if (row < args.m && cbase < args.n) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(silu_f(__uint_as_float(v[j])) * __uint_as_float(u[j]));
            const long long base = (long long)row * args.ldo + cbase;
            if (cbase + 32 <= args.n && ((base & 7) == 0)) {
              uint4* p = reinterpret_cast<uint4*>(out_h + base);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                p[q] = make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
            } else {
              for (int j = 0; j < 32; ++j)
                if (cbase + j < args.n) out_h[base + j] = __float2bfloat16(__uint_as_float(v[j]));
            }
          }
        }
      } else if (MODE == 1) {
        // local output rows, 64 contiguous bytes per lane and chunk
        const int row = rt * kTileRows + quad * 32 + lane;
        __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(args.out);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(t0 + c, v);
          tmem_ld_wait();
          if (c + 32 >= BN) release_acc(acc);
          const int cbase = col0 + c;
          if (row < args.m && cbase < args.n) {
            const long long base = (long long)row * args.ldo + cbase;
            if (cbase + 32 <= args.n && ((base & 7) == 0)) {
              uint4* p = reinterpret_cast<uint4*>(out_h + base);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                p[q] = make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                                  pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
            } else {
              for (int j = 0; j < 32; ++j)
                if (cbase + j < args.n) out_h[base + j] = __float2bfloat16(__uint_as_float(v[j]));
            }
          }
        }
      } else {
        // gemm_rs: stage 32 rows x 128 columns per warp, then hand 256-byte row segments to their owner:
        // rows of a peer are stored into slot [rank] of that peer's staging array; rows of this rank are
        // summed with the tp - 1 staged partials of the peers (which produced them early in their own
        // tile order) and written to the output.  A tile that holds rows of both kinds is read from TMEM
        // twice: the peers' rows are pushed and counted before this rank waits for anything.
        uint8_t* my_stage = stage_out + quad * (32 * 128 * 2);
        const int rpr = args.rows_per_rank;
        const int own0 = args.rank * rpr, own1 = own0 + rpr;
        const int r0 = rt * kTileRows, r1 = min(args.m, r0 + kTileRows);
        const int w0 = r0 + quad * 32, w1 = min(args.m, w0 + 32);   // this warp's rows
        const bool tile_own = r0 < own1 && r1 > own0;
        const bool tile_peer = r0 < own0 || r1 > own1;
        const bool warp_own = w0 < own1 && w1 > own0;
        const long long slot_stride = (long long)rpr * args.n;
        __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(args.out);

        auto pass = [&](bool do_peer, bool do_own, bool release) {
#pragma unroll 1
          for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
              uint32_t v[32];
              tmem_ld_32x32(t0 + half * 128 + c, v);
              tmem_ld_wait();
              if (release && half * 128 + c + 32 >= BN) release_acc(acc);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int chunk = (c >> 3) + q;   // 16-byte chunk index inside the 256-byte staged row
                *reinterpret_cast<uint4*>(my_stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) =
                    make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                               pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                               pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                               pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
              }
            }
            __syncwarp();
            const int cb = col0 + half * 128 + (lane & 15) * 8;   // first column of this lane's 16 bytes
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
              const int lr = 2 * i + (lane >> 4);
              const int row = w0 + lr;
              if (row < args.m && cb < args.n) {
                const int owner = row / rpr, lrow = row - owner * rpr;
                if (owner != args.rank ? !do_peer : !do_own) continue;
                const uint4 val =
                    *reinterpret_cast<const uint4*>(my_stage + lr * 256 + (((lane & 15) ^ (lr & 15)) << 4));
                if (owner != args.rank) {
                  __nv_bfloat16* dst = sh->peer_buf[owner] + ((long long)(args.rank * rpr + lrow) * args.n + cb);
                  *reinterpret_cast<uint4*>(dst) = val;
                } else {
                  const uint32_t vw[4] = {val.x, val.y, val.z, val.w};
                  float a[8];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack_bf16x2(vw[e]);
                    a[2 * e] = f.x;
                    a[2 * e + 1] = f.y;
                  }
                  const long long off = (long long)lrow * args.n + cb;
                  for (int s2 = 1; s2 < args.tp; ++s2) {
                    int src = args.rank + s2;
                    if (src >= args.tp) src -= args.tp;
                    // written by a peer: read from L2, never from a stale L1 line
                    const uint4 p = __ldcg(reinterpret_cast<const uint4*>(args.local_buf + src * slot_stride + off));
                    const uint32_t pw[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 f = unpack_bf16x2(pw[e]);
                      a[2 * e] += f.x;
                      a[2 * e + 1] += f.y;
                    }
                  }
                  *reinterpret_cast<uint4*>(out_h + (long long)lrow * args.ldo + cb) =
                      make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                                 pack_bf16x2(a[6], a[7]));
                }
              }
            }
            __syncwarp();
          }
        };
        // hand the tile to the publisher warp: it fences and counts while these warps go on.  The slot
        // of two tiles ago must have been published first (bounded wait; first uses pass at once).
        auto publish = [&]() {
          const int slot = published & 1;
          const bool ok2 = mbar_wait(&sh->pub_empty[slot], ((uint32_t(published) >> 1) & 1u) ^ 1u, abort_flag,
                                     args.status, ERR_WAIT_PEER_FLAG);
          __syncwarp();
          if (lane == 0 && ok2) mbar_arrive(&sh->pub_full[slot]);
          ++published;
        };
        // bounded wait (per warp) until every peer has delivered its partials of this warp's own rows
        auto wait_peers = [&]() -> bool {
          if (!warp_own || args.tp == 1) return true;
          int ok = 1;
          if (lane == 0) {
            const int lo = max(w0, own0) - own0, hi = min(w1, own1) - own0;
            for (int t = lo / 128; t <= (hi - 1) / 128 && ok; ++t) {
              const int g0 = own0 + t * 128, g1 = own0 + min(rpr, t * 128 + 128);
              const unsigned int per_call = unsigned(args.num_col_tiles) * unsigned((g1 - 1) / 128 - g0 / 128 + 1);
              for (int src = 0; src < args.tp && ok; ++src)
                if (src != args.rank)
                  ok = wait_counter(args.local_flags + src * args.flag_stride + t, per_call * args.epoch,
                                    args.status, (blockIdx.x << 8) | src)
                           ? 1 : 0;
            }
            if (!ok) *abort_flag = 1;
          }
          return __shfl_sync(0xffffffffu, ok, 0) != 0;
        };
        if (tile_peer && tile_own) {
          pass(true, false, !warp_own);
          publish();
          if (wait_peers()) { if (warp_own) pass(false, true, true); }
          else if (warp_own) release_acc(acc);
        } else if (tile_own) {
          if (wait_peers()) pass(false, true, true);
          else release_acc(acc);
        } else {
          pass(true, false, true);
          publish();
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
  if (PAIR) cluster_sync_all();   // neither CTA frees shared / tensor memory while its peer still works
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, tmem_cols);
    else tmem_dealloc(tmem_base, tmem_cols);
  }
}

template <int BN, int MODE, bool PAIR>
static int launch_comm(const CUtensorMap& ta, const CUtensorMap& ta2, const CUtensorMap& tb, CommArgs& args,
                       const CommPeers& peers, cudaStream_t stream) {
  constexpr int stage_bytes = kATileBytes + (PAIR ? BN / 2 : BN) * kBlockK * 2;
  const int extra = kCommCtrlBytes + (MODE == 0 ? kStageOutBytes : 0);
  int stages = (232448 - 1024 - extra) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return -3;
  args.stages = stages;
  static_assert(sizeof(CommShared) <= kCommCtrlBytes, "control block grew");
  const int smem = stages * stage_bytes + 1024 + extra;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(gemm_comm_kernel<BN, MODE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return int(e);
    attr_set = true;
  }
  // The work loops stride by the grid (or the number of pairs), so every CTA must be resident at once; the
  // pushers of ag_gemm must run beside the consumers in any case.
  if (!PAIR)
    return launch_pdl(gemm_comm_kernel<BN, MODE, PAIR>, dim3(num_sms()), dim3(kCommThreads), size_t(smem), stream, ta,
                      ta2, tb, args, peers);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (num_sms() / 2));
  cfg.blockDim = dim3(kCommThreads);
  cfg.dynamicSmemBytes = size_t(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static int max_pairs = 0;      // pairs need two SMs of one GPC; not every SM can be paired
  if (max_pairs == 0) {
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_comm_kernel<BN, MODE, PAIR>, &cfg);
    max_pairs = (e == cudaSuccess && n > 0) ? n : num_sms() / 4;
  }
  cfg.gridDim = dim3(2 * max_pairs);
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return int(cudaLaunchKernelEx(&cfg, gemm_comm_kernel<BN, MODE, PAIR>, ta, ta2, tb, args, peers));
}

static bool comm_pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("NKIPY_B200_COMM_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace nkb

using namespace nkb;

// Row-parallel GEMM + reduce-scatter over rows.  x [m, k] (this rank's K shard), w [n, k]; out [m / tp, n] bf16.
// peer_stage[r] / peer_flags[r]: rank r's staging array [tp, m / tp, n] bf16 of this call and its counter
// array (tp * flag_stride u32, flag_stride >= ceil(m / tp / 128)), own entries included.  epoch = 1, 2, ...
extern "C" int nkb_gemm_rs(const void* x, const void* w, void* out, int m, int n, int k, long long ldx, long long ldw,
                           long long ldo, void* const* peer_stage, void* const* peer_flags, int flag_stride, int tp,
                           int rank, unsigned int epoch, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (m <= 0 || n <= 0 || k <= 0 || tp < 1 || tp > kCommMaxPeers || rank < 0 || rank >= tp) return -2;
  if ((m % tp) || (k & 7) || (n & 7) || (ldx & 7) || (ldw & 7) || (ldo & 7)) return -2;
  const int rpr = m / tp;
  if (flag_stride < (rpr + 127) / 128) return -2;
  CommArgs a{};
  a.m = m; a.n = n; a.k = k;
  a.num_row_tiles = (m + kTileRows - 1) / kTileRows;
  a.kb_total = (k + kBlockK - 1) / kBlockK;
  a.tp = tp; a.rank = rank; a.rows_per_rank = rpr;
  a.first_tile = (((rank + 1) * rpr + kTileRows - 1) / kTileRows) % a.num_row_tiles;
  a.epoch = epoch;
  a.flag_stride = flag_stride;
  a.ldo = ldo;
  a.out = out;
  a.local_buf = reinterpret_cast<__nv_bfloat16*>(peer_stage[rank]);
  a.local_flags = reinterpret_cast<unsigned int*>(peer_flags[rank]);
  a.status = status_word();
  CommPeers p{};
  for (int i = 0; i < tp; ++i) {
    p.buf[i] = reinterpret_cast<__nv_bfloat16*>(peer_stage[i]);
    p.flags[i] = reinterpret_cast<unsigned int*>(peer_flags[i]);
  }
  const int bn = n >= 256 ? 256 : 128;
  const bool pair = bn == 256 && m >= 256 && comm_pair_enabled();
  a.num_col_tiles = (n + bn - 1) / bn;
  if (pair) {
    // rotation in units of 256-row pairs: start with the pair after the one that holds this rank's last row
    const int groups = (a.num_row_tiles + 1) / 2;
    a.first_tile = ((((rank + 1) * rpr + 2 * kTileRows - 1) / (2 * kTileRows))) % groups;
  }
  CUtensorMap ta, tb;
  if (encode_tmap_bf16_2d(&ta, x, k, m, ldx, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, w, k, n, ldw, kBlockK, pair ? bn / 2 : bn)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (pair) return launch_comm<256, 0, true>(ta, ta, tb, a, p, s);
  return bn == 256 ? launch_comm<256, 0, false>(ta, ta, tb, a, p, s) : launch_comm<128, 0, false>(ta, ta, tb, a, p, s);
}

// All-gather + column-parallel GEMM.  x_local [m / tp, k] (this rank's row slab), w [n, k] (this rank's
// column shard); out [m, n] bf16.  peer_gather[r]: rank r's gather buffer [m, k] bf16 of this call,
// peer_flags[r]: its counter array (tp * flag_stride u32, flag_stride >= ceil(m / tp / 128)).
extern "C" int nkb_ag_gemm(const void* x_local, const void* w, void* out, int m, int n, int k, long long ldx,
                           long long ldw, long long ldo, void* const* peer_gather, void* const* peer_flags,
                           int flag_stride, int tp, int rank, unsigned int epoch, int comm_ctas, int gated, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (m <= 0 || n <= 0 || k <= 0 || tp < 1 || tp > kCommMaxPeers || rank < 0 || rank >= tp) return -2;
  if ((m % tp) || (k & 7) || (ldx & 7) || (ldw & 7) || (ldo & 7)) return -2;
  if (reinterpret_cast<uintptr_t>(x_local) & 15) return -2;   // bulk copies need 16-byte aligned rows
  const int rpr = m / tp;
  if (flag_stride < (rpr + 127) / 128) return -2;
  CommArgs a{};
  a.m = m; a.n = n; a.k = k;
  a.num_row_tiles = (m + kTileRows - 1) / kTileRows;
  a.kb_total = (k + kBlockK - 1) / kBlockK;
  a.tp = tp; a.rank = rank; a.rows_per_rank = rpr;
  a.local_direct = (rpr % kTileRows) == 0 ? 1 : 0;
  a.first_tile = (rank * rpr) / kTileRows;
  if (comm_ctas < 1) {
    // enough pusher CTAs (about 45 GB/s each) to deliver the peers' slabs well inside the time the GEMM
    // spends on the slabs it already has; every pusher costs 1/148 of the GEMM's throughput
    const double gemm_us = 2.0 * m * double(n) * k / 1.3e9;
    const double push_bytes = double(tp - 1) * rpr * double(k) * 2.0;
    const double window_us = gemm_us * (tp - 1) / tp * 0.6 + 1.0;
    const double want = push_bytes / window_us / 1e3 / 45.0;
    comm_ctas = int(want) + 1;
    if (comm_ctas < 2) comm_ctas = 2;
    if (comm_ctas > 32) comm_ctas = 32;
  }
  if (tp == 1) comm_ctas = a.local_direct ? 0 : 1;
  if (comm_ctas > num_sms() / 2) comm_ctas = num_sms() / 2;
  a.comm_ctas = comm_ctas;
  a.epoch = epoch;
  a.flag_stride = flag_stride;
  a.ldx = int(ldx);
  a.ldo = ldo;
  a.out = out;
  a.x_local = reinterpret_cast<const __nv_bfloat16*>(x_local);
  a.local_buf = reinterpret_cast<__nv_bfloat16*>(peer_gather[rank]);
  a.local_flags = reinterpret_cast<unsigned int*>(peer_flags[rank]);
  a.status = status_word();
  CommPeers p{};
  for (int i = 0; i < tp; ++i) {
    p.buf[i] = reinterpret_cast<__nv_bfloat16*>(peer_gather[i]);
    p.flags[i] = reinterpret_cast<unsigned int*>(peer_flags[i]);
  }
  const int bn = (gated || n >= 256) ? 256 : 128;
  const bool pair = bn == 256 && m >= 256 && comm_pair_enabled();
  if (gated && !pair) return -5;       // SwiGLU epilogue exists on CTA pairs only: callers gate separately
  a.gated = gated ? 1 : 0;
  a.gate_off = n;                      // w holds n gate rows followed by n up rows
  a.num_col_tiles = gated ? (n + 127) / 128 : (n + bn - 1) / bn;
  if (pair) {
    a.first_tile = (rank * rpr) / (2 * kTileRows);
    a.comm_ctas = (a.comm_ctas + 1) & ~1;          // whole pairs push
  }
  CUtensorMap ta, tg, tb;
  if (encode_tmap_bf16_2d(&ta, x_local, k, rpr, ldx, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tg, peer_gather[rank], k, m, k, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, w, k, gated ? 2 * uint64_t(n) : uint64_t(n), ldw, kBlockK, pair ? bn / 2 : bn))
    return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (pair) return launch_comm<256, 1, true>(ta, tg, tb, a, p, s);
  return bn == 256 ? launch_comm<256, 1, false>(ta, tg, tb, a, p, s) : launch_comm<128, 1, false>(ta, tg, tb, a, p, s);
}
