// Decode-sized GEMM with the split-K reduction folded into the kernel (sm_100a).
//
//   y[t, f] = sum_k x[t, k] * w[f, k]        tokens t <= 128, features f on the 128-row MMA side
//
// A decode step multiplies a handful of tokens with weight matrices that are far too
// small (per tensor-parallel rank) to fill 148 SMs with one 128-row tile each, so the
// contraction has to be split.  Instead of writing fp32 partials to global memory for
// the next kernel to sum, the S CTAs that share one row tile form a thread-block
// cluster: each accumulates its K slice in TMEM (tcgen05.mma fed by TMA), then sends
// every peer the token columns that peer owns as asynchronous distributed-shared-memory
// stores (st.async, completion counted in bytes on the receiver's mbarrier), and sums
// the S partials of its own BN / S token columns.  The owner then runs the epilogue on
// finished values, which is what allows fusing work that needs the complete sum:
//
//   STORE  bf16 output (+ bias, + residual)
//   SWIGLU the gate / up projection: a tile takes 64 gate rows and the 64 matching up rows of the
//          [gate; up] weight (two half-height TMA boxes), so silu(gate) * up is formed in the epilogue
//   PUSH   one bf16 partial per rank stored into every tensor-parallel peer's symmetric
//          buffer (plain peer stores over NVLink) + arrival counters: the producer half
//          of the fused all-reduce (consumer: tp_reduce_rmsnorm in comm.cu)
//   ROPE   the fused QKV projection: bias, per-head QK-RMSNorm, rotate-halves RoPE and
//          the write of K / V into the paged cache, Q into its buffer
//
// No multicast load is used anywhere; peer GPU memory is touched only by plain stores.
// Every wait is bounded (1 s) and reports into the library's status word.
//
// Reference parity: the projections of examples/models/qwen3/kernels/attention.py:72-106
// (QKV + QK-norm + RoPE + cache write), :146-154 (o_proj + all-reduce) and
// kernels/feedforward.py:4-18 (SwiGLU), which the reference compiles into one device program.
#include "common.cuh"
#include "gemm_args.h"
#include "api.h"

namespace nkb {

enum : int { EPI_STORE = 0, EPI_PUSH = 1, EPI_ROPE = 2, EPI_SWIGLU = 3 };

struct DGemmArgs {
  int features, tokens;
  int kb_total, splits;
  int gate_off;   // SWIGLU: row offset of the "up" half inside the weight matrix
  int stages;
  long long ldo;
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int* status;
};

struct StoreEpi {
  static constexpr int kind = EPI_STORE;
  struct Args {};
};
struct PushEpi {
  static constexpr int kind = EPI_PUSH;
  using Args = PushArgs;
};
struct RopeArgs {
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
struct RopeEpi {
  static constexpr int kind = EPI_ROPE;
  using Args = RopeArgs;
};

struct SwigluArgs {
  float act_limit;   // > 0: clamped form (up + 1) * gate * sigmoid(act_alpha * gate)
  float act_alpha;
};
struct SwigluEpi {
  static constexpr int kind = EPI_SWIGLU;
  using Args = SwigluArgs;
};

struct DGemmCtrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tfull;
  uint64_t recv_bar;
  uint32_t tmem_base;
  int abort;
  float red[4][32];
};
constexpr int kDCtrlBytes = 1024;
static_assert(sizeof(DGemmCtrl) <= kDCtrlBytes, "control block grew");

__host__ __device__ constexpr int dgemm_stage_bytes(int bn) { return kATileBytes + bn * kBlockK * 2; }
__host__ __device__ constexpr int dgemm_recv_bytes(int bn) { return kTileRows * bn * 4; }

__device__ __forceinline__ void st_async_v4(uint32_t remote_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(remote_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
               : "memory");
}

__device__ __forceinline__ float dsilu(float g) { return g / (1.f + __expf(-g)); }

template <int BN, class Epi>
__global__ void __launch_bounds__(kGemmThreads)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const DGemmArgs args, const typename Epi::Args epi) {
  constexpr bool kHalf = Epi::kind == EPI_SWIGLU;   // a tile = 64 gate rows + the 64 matching up rows
  constexpr int kStageBytes = dgemm_stage_bytes(BN);
  constexpr int kRecvBytes = dgemm_recv_bytes(BN);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = args.stages;
  float* recv = reinterpret_cast<float*>(tiles + stages * kStageBytes);
  DGemmCtrl* ctrl = reinterpret_cast<DGemmCtrl*>(reinterpret_cast<uint8_t*>(recv) + kRecvBytes);
  // Epilogue staging (at most 32 tokens x 128 features x 4 bytes) reuses the first ring stage: when the
  // epilogue runs every load has landed and every MMA has retired, and peers never write into the ring.
  static_assert(2 * kStageBytes >= 32 * kTileRows * 4, "epilogue staging must fit in the ring");
  uint8_t* extra = tiles;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = args.splits;
  const int crank = int(cluster_ctarank());
  const int rt = blockIdx.x / S;
  const int row0 = rt * (kHalf ? kTileRows / 2 : kTileRows);   // first weight row (SWIGLU: of the gate half)
  const int kb0 = int((long long)crank * args.kb_total / S);
  const int kb1 = int((long long)(crank + 1) * args.kb_total / S);
  const int CW = BN / S;   // token columns owned by each CTA of the cluster (a power of two >= 4)

  uint32_t tmem_cols = 32;
  while (tmem_cols < uint32_t(BN)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctrl->full[s], 1);
      mbar_init(&ctrl->empty[s], 1);
    }
    mbar_init(&ctrl->tfull, 1);
    mbar_init(&ctrl->recv_bar, 1);
    ctrl->abort = 0;
    mbar_fence_init();
    fence_proxy_async();
    // every CTA of the cluster (this one included) delivers its partial of this CTA's columns
    mbar_expect_tx(&ctrl->recv_bar, uint32_t(kRecvBytes));
  }
  if (warp == 1) {
    tmem_alloc(&ctrl->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // peers must not signal a barrier that is not initialised yet
  cluster_sync_all();
  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort;

  griddep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // weight tiles do not depend on the preceding kernel: the first ring fill starts before the wait
    const int nkb = kb1 - kb0;
    const int pre = min(stages, nkb);
    if (lane == 0) {
      for (int i = 0; i < pre; ++i) {
        uint8_t* a_ptr = tiles + i * kStageBytes;
        mbar_expect_tx(&ctrl->full[i], kStageBytes);
        tma_load_2d(a_ptr, &tmA, &ctrl->full[i], (kb0 + i) * kBlockK, row0);
        if (kHalf) tma_load_2d(a_ptr + kATileBytes / 2, &tmA, &ctrl->full[i], (kb0 + i) * kBlockK, args.gate_off + row0);
      }
    }
    __syncwarp();
    griddep_wait();
    int stage = 0;
    uint32_t phase = 0;
    for (int i = 0; i < nkb; ++i) {
      const int kb = kb0 + i;
      if (i >= pre) {
        bool ok = mbar_wait(&ctrl->empty[stage], phase ^ 1u, abort_flag, args.status, ERR_WAIT_SMEM_EMPTY);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      if (lane == 0) {
        uint8_t* a_ptr = tiles + stage * kStageBytes;
        uint8_t* b_ptr = a_ptr + kATileBytes;
        if (i >= pre) {
          mbar_expect_tx(&ctrl->full[stage], kStageBytes);
          tma_load_2d(a_ptr, &tmA, &ctrl->full[stage], kb * kBlockK, row0);
          if (kHalf) tma_load_2d(a_ptr + kATileBytes / 2, &tmA, &ctrl->full[stage], kb * kBlockK, args.gate_off + row0);
        }
        tma_load_2d(b_ptr, &tmB, &ctrl->full[stage], kb * kBlockK, 0);
      }
      __syncwarp();
      if (++stage == stages) { stage = 0; phase ^= 1u; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(kTileRows, BN, 0, 0);
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int kb = kb0; kb < kb1 && alive; ++kb) {
      bool ok = mbar_wait(&ctrl->full[stage], phase, abort_flag, args.status, ERR_WAIT_SMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(tiles + stage * kStageBytes);
        const uint32_t b_addr = a_addr + kATileBytes;
        const uint64_t da = make_smem_desc_sw128(a_addr, 0, 1024);
        const uint64_t db = make_smem_desc_sw128(b_addr, 0, 1024);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) {
          const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
          const uint64_t koff = uint64_t(k * 2);
          umma_f16(tmem_base, da + koff, db + koff, idesc, accum);
        }
        umma_commit(&ctrl->empty[stage]);
      }
      __syncwarp();
      if (++stage == stages) { stage = 0; phase ^= 1u; }
    }
    if (alive && lane == 0) umma_commit(&ctrl->tfull);
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ exchange + epilogue (warps 2..5)
    const int quad = warp & 3;
    const int f = quad * 32 + lane;          // feature row of this thread inside the tile
    const int et = threadIdx.x - 64;         // 0..127 over the four epilogue warps
    griddep_wait();                          // outputs / residual may still be in use by the preceding kernel
    bool ok = mbar_wait(&ctrl->tfull, 0, abort_flag, args.status, ERR_WAIT_TMEM_FULL);
    ok = bar_red_and(2, 128, __all_sync(0xffffffffu, ok));
    if (ok) {
      tc_fence_after();
      const uint32_t t0 = tmem_base + (uint32_t(quad * 32) << 16);
      const int cw_shift = __ffs(CW) - 1;
      // ---- send: columns [d * CW, (d + 1) * CW) of this partial go to CTA d of the cluster
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int col = c + 4 * q;
          const int dest = col >> cw_shift, within = col & (CW - 1);
          const float* slot = recv + (crank * kTileRows + f) * CW + within;
          const uint32_t raddr = map_to_cta(slot, uint32_t(dest));
          const uint32_t rbar = map_to_cta(&ctrl->recv_bar, uint32_t(dest));
          st_async_v4(raddr, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3], rbar);
        }
      }
      tc_fence_before();
      // ---- receive: all S partials of this CTA's CW token columns
      ok = mbar_wait_cluster(&ctrl->recv_bar, 0, abort_flag, args.status, ERR_WAIT_PEER_FLAG);
      ok = bar_red_and(2, 128, __all_sync(0xffffffffu, ok));
    }
    if (ok) {
      // SWIGLU: lanes 0..63 hold the gate rows of output features row0 .. row0 + 63, lanes 64..127 the up rows
      const int feat = kHalf ? row0 + (f & 63) : row0 + f;
      const bool feat_ok = feat < args.features;
      const int tok_base = crank * CW;
      float bias_f = 0.f;
      if (args.bias && feat_ok) bias_f = __bfloat162float(args.bias[(kHalf && f >= 64) ? args.gate_off + feat : feat]);
#pragma unroll 1
      for (int c0 = 0; c0 < CW; c0 += 32) {
        const int n = min(32, CW - c0);
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = bias_f;
        for (int s = 0; s < S; ++s) {
          const float* src = recv + (s * kTileRows + f) * CW + c0;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (4 * q < n) {
              const float4 t = *reinterpret_cast<const float4*>(src + 4 * q);
              acc[4 * q] += t.x; acc[4 * q + 1] += t.y; acc[4 * q + 2] += t.z; acc[4 * q + 3] += t.w;
            }
          }
        }

        if constexpr (Epi::kind == EPI_STORE) {
          if (feat_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = tok_base + c0 + j;
              if (j < n && tok < args.tokens) {
                const long long idx = (long long)tok * args.ldo + feat;
                float x = acc[j];
                if (args.residual) x += __bfloat162float(args.residual[idx]);
                args.out[idx] = __float2bfloat16(x);
              }
            }
          }
        } else if constexpr (Epi::kind == EPI_SWIGLU) {
          float* xch = reinterpret_cast<float*>(extra);   // [token j][lane]
          if (f >= 64) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < n) xch[j * kTileRows + f] = acc[j];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (f < 64 && feat_ok) {
            const float lim = epi.act_limit, alpha = epi.act_alpha;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = tok_base + c0 + j;
              if (j < n && tok < args.tokens) {
                float g = acc[j], u = xch[j * kTileRows + f + 64];
                float y;
                if (lim > 0.f) {
                  g = fminf(g, lim);
                  u = fminf(fmaxf(u, -lim), lim);
                  y = (u + 1.f) * g / (1.f + __expf(-alpha * g));
                } else {
                  y = dsilu(g) * u;
                }
                args.out[(long long)tok * args.ldo + feat] = __float2bfloat16(y);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        } else if constexpr (Epi::kind == EPI_PUSH) {
          // stage [token][feature] bf16, then the four warps store 16-byte pieces to every rank: each token row
          // is one contiguous 256-byte run in the destination's slot [rank][token][feature]
          __nv_bfloat16* stage_out = reinterpret_cast<__nv_bfloat16*>(extra);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < n) stage_out[j * kTileRows + f] = __float2bfloat16(acc[j]);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int idx = et; idx < n * 16; idx += 128) {
            const int tl = idx >> 4, ch = idx & 15;
            const int gtok = tok_base + c0 + tl, gfeat = row0 + ch * 8;
            if (gtok < args.tokens && gfeat < args.features) {
              const uint4 val = *reinterpret_cast<const uint4*>(stage_out + tl * kTileRows + ch * 8);
              const long long off = ((long long)epi.rank * args.tokens + gtok) * args.ldo + gfeat;
              push_store_16(epi, off, val);
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        } else {
          // ---- fused QKV epilogue: (QK-norm) -> RoPE -> Q buffer / paged K, V cache
          const int D = epi.head_dim;                 // 64 or 128: heads never straddle a tile
          const int head = feat / D, i = feat - head * D;
          const bool is_q = head < epi.nq, is_k = !is_q && head < epi.nq + epi.nkv;
          const __nv_bfloat16* nw = is_q ? epi.q_norm_w : (is_k ? epi.k_norm_w : nullptr);
          if (epi.q_norm_w || epi.k_norm_w) {
            // sum of squares over the head: warp shuffle, then the warps of the head through shared memory
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < n) {
                const float ss = warp_sum(acc[j] * acc[j]);
                if (lane == 0) ctrl->red[quad][j] = ss;
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (nw && feat_ok) {
              const float wgt = __bfloat162float(nw[i]);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (j < n) {
                  float tot;
                  if (D == 128) tot = ctrl->red[0][j] + ctrl->red[1][j] + ctrl->red[2][j] + ctrl->red[3][j];
                  else tot = ctrl->red[quad & 2][j] + ctrl->red[(quad & 2) + 1][j];
                  const float inv = rsqrtf(tot / float(D) + epi.norm_eps);
                  // round to bf16 after the norm like an unfused implementation would
                  acc[j] = __bfloat162float(__float2bfloat16(acc[j] * inv * wgt));
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
          if (epi.cos_sin) {
            float* xch = reinterpret_cast<float*>(extra);   // [token j][feature]
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < n) xch[j * kTileRows + f] = acc[j];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (is_q || is_k) {
              const int half = D >> 1;
              const int ih = i < half ? i : i - half;
              const int fp = i < half ? f + half : f - half;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int tok = tok_base + c0 + j;
                if (j < n && tok < args.tokens) {
                  int pos = epi.positions[tok];
                  pos = pos < 0 ? 0 : (pos >= epi.max_pos ? epi.max_pos - 1 : pos);
                  const float* cs = epi.cos_sin + (long long)pos * D;
                  const float cc = cs[ih], sn = cs[half + ih];
                  const float other = xch[j * kTileRows + fp];
                  acc[j] = i < half ? acc[j] * cc - other * sn : acc[j] * cc + other * sn;
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
          if (feat_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = tok_base + c0 + j;
              if (j < n && tok < args.tokens) {
                __nv_bfloat16* dst = nullptr;
                if (is_q) {
                  dst = epi.q_out + ((long long)tok * epi.nq + head) * D + i;
                } else {
                  const int slot = epi.slots ? epi.slots[tok] : -1;
                  if (slot >= 0) {
                    const int kh = is_k ? head - epi.nq : head - epi.nq - epi.nkv;
                    const long long blk = slot / epi.block_size, off = slot % epi.block_size;
                    dst = (is_k ? epi.k_cache : epi.v_cache) + ((blk * epi.nkv + kh) * epi.block_size + off) * D + i;
                  }
                }
                if (dst) *dst = __float2bfloat16(acc[j]);
              }
            }
          }
        }
      }
    }
    if constexpr (Epi::kind == EPI_PUSH) {
      // all peer stores of this CTA are issued: release at GPU scope into the grid counter; the last CTA, which
      // has observed every other CTA's release, publishes them with one system-scope fence and bumps the peers' flags
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        __threadfence();
        const unsigned int old = atomicAdd(epi.done_counter, 1u);
        if (old == gridDim.x - 1) {
          *epi.done_counter = 0u;
          __threadfence_system();
          if (ok)
            push_signal(epi);
        }
      }
    }
  }

  if (*abort_flag) {
    // let copies / MMAs / remote stores that were already issued drain before shared memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
template <int BN, class Epi>
static int launch_decode_gemm(const CUtensorMap& ta, const CUtensorMap& tb, DGemmArgs& args, int ctas_per_sm,
                              const typename Epi::Args& epi, cudaStream_t stream) {
  constexpr int kStage = dgemm_stage_bytes(BN);
  constexpr int kFixed = 1024 + dgemm_recv_bytes(BN) + kDCtrlBytes;
  const int nkb = (args.kb_total + args.splits - 1) / args.splits;
  int budget = ctas_per_sm == 2 ? 113 * 1024 : 232448;
  int stages = (budget - kFixed) / kStage;
  if (stages < 3 && ctas_per_sm == 2) {   // not enough ring for two CTAs per SM: take the whole SM
    budget = 232448;
    stages = (budget - kFixed) / kStage;
  }
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > nkb) stages = nkb < 2 ? 2 : nkb;
  if (stages < 2) return -3;
  args.stages = stages;
  const int smem = kFixed + stages * kStage;
  auto kernel = decode_gemm_kernel<BN, Epi>;
  static int attr_dev_mask[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_dev_mask[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return int(e);
    attr_dev_mask[dev] = 1;
  }
  constexpr int kRowsPerTile = Epi::kind == EPI_SWIGLU ? kTileRows / 2 : kTileRows;
  const int row_tiles = (args.features + kRowsPerTile - 1) / kRowsPerTile;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(row_tiles * args.splits));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = size_t(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(args.splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return int(cudaLaunchKernelEx(&cfg, kernel, ta, tb, args, epi));
}

// splits must be a power of two <= 8 that divides block_n into columns of at least 4 and does not exceed the
// number of 64-wide k-blocks
static int normalize_splits(int splits, int block_n, int kb_total) {
  int s = 1;
  while (s * 2 <= splits && s * 2 <= 8 && block_n / (s * 2) >= 4 && s * 2 <= kb_total) s *= 2;
  return s;
}

static int fill_args(DGemmArgs& a, int features, int tokens, int k, int splits, int block_n, long long ldo) {
  if (features <= 0 || tokens <= 0 || k <= 0 || (k & 7)) return -2;
  if (block_n != 32 && block_n != 64 && block_n != 128) return -2;
  if (tokens > block_n) return -2;
  a.features = features;
  a.tokens = tokens;
  a.kb_total = (k + kBlockK - 1) / kBlockK;
  a.splits = normalize_splits(splits, block_n, a.kb_total);
  a.ldo = ldo;
  a.status = status_word();
  return 0;
}

}  // namespace nkb

using namespace nkb;

extern "C" int nkb_decode_gemm_splits(int splits, int block_n, int k) {
  return normalize_splits(splits, block_n, (k + kBlockK - 1) / kBlockK);
}

// out[tokens, features] = x[tokens, k] @ w[features, k]^T (+ bias[features]) (+ residual[tokens, ldo]).
// gated: w holds [gate; up] rows (up half at row gate_off, features rows each) and
// out = silu(x @ gate^T + bias_g) * (x @ up^T + bias_u); act_limit > 0 selects the clamped form.
extern "C" int nkb_decode_gemm(const void* w, const void* x, void* out, int features, int tokens, int k,
                               long long ldw, long long ldx, long long ldo, int splits, int gated, int gate_off,
                               const void* bias, const void* residual, float act_limit, float act_alpha, int block_n,
                               int ctas_per_sm, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if ((ldw & 7) || (ldx & 7)) return -2;
  if (gated && residual) return -2;
  DGemmArgs a{};
  if (int rc = fill_args(a, features, tokens, k, splits, block_n, ldo)) return rc;
  a.gate_off = gate_off;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  CUtensorMap ta, tb;
  if (encode_tmap_bf16_2d(&tb, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gated) {
    // half-height boxes: a tile is 64 gate rows followed by the 64 up rows of the same output features
    if (encode_tmap_bf16_2d(&ta, w, k, uint64_t(gate_off) + features, ldw, kBlockK, kTileRows / 2)) return -4;
    SwigluArgs e{act_limit, act_alpha};
    switch (block_n) {
      case 32: return launch_decode_gemm<32, SwigluEpi>(ta, tb, a, ctas_per_sm, e, s);
      case 64: return launch_decode_gemm<64, SwigluEpi>(ta, tb, a, ctas_per_sm, e, s);
      default: return launch_decode_gemm<128, SwigluEpi>(ta, tb, a, ctas_per_sm, e, s);
    }
  }
  if (encode_tmap_bf16_2d(&ta, w, k, features, ldw, kBlockK, kTileRows)) return -4;
  StoreEpi::Args e{};
  switch (block_n) {
    case 32: return launch_decode_gemm<32, StoreEpi>(ta, tb, a, ctas_per_sm, e, s);
    case 64: return launch_decode_gemm<64, StoreEpi>(ta, tb, a, ctas_per_sm, e, s);
    default: return launch_decode_gemm<128, StoreEpi>(ta, tb, a, ctas_per_sm, e, s);
  }
}

// Row-parallel projection whose finished bf16 partial [tokens, features] is stored into slot [rank] of every
// peer's partial array [n_peers, tokens, ldo]; the last CTA bumps this rank's arrival counter on every peer.
extern "C" int nkb_decode_gemm_push(const void* w, const void* x, int features, int tokens, int k, long long ldw,
                                    long long ldx, long long ldo, int splits, const void* bias, int block_n,
                                    void* const* peer_out, void* const* peer_flag, int n_peers, int rank,
                                    void* done_counter, void* mc_out, void* mc_flag, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if ((ldw & 7) || (ldx & 7) || (ldo & 7) || (features & 7)) return -2;
  if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return -2;
  DGemmArgs a{};
  if (int rc = fill_args(a, features, tokens, k, splits, block_n, ldo)) return rc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  PushArgs pa{};
  pa.n_peers = n_peers;
  pa.rank = rank;
  for (int i = 0; i < n_peers; ++i) {
    pa.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(peer_out[i]);
    pa.peer_flag[i] = reinterpret_cast<unsigned int*>(peer_flag[i]);
  }
  pa.done_counter = reinterpret_cast<unsigned int*>(done_counter);
  pa.mc_out = reinterpret_cast<__nv_bfloat16*>(mc_out);
  pa.mc_flag = reinterpret_cast<unsigned int*>(mc_flag);
  CUtensorMap ta, tb;
  if (encode_tmap_bf16_2d(&ta, w, k, features, ldw, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (block_n) {
    case 32: return launch_decode_gemm<32, PushEpi>(ta, tb, a, 2, pa, s);
    case 64: return launch_decode_gemm<64, PushEpi>(ta, tb, a, 2, pa, s);
    default: return launch_decode_gemm<128, PushEpi>(ta, tb, a, 2, pa, s);
  }
}

// Fused QKV projection of a decode step: w [(nq + 2 nkv) * head_dim, k]; Q rows go to q_out [tokens, nq * head_dim],
// K / V rows to the paged cache [blocks, nkv, block_size, head_dim] at slots[token] (negative = not stored).
extern "C" int nkb_decode_gemm_rope(const void* w, const void* x, int tokens, int k, long long ldw, long long ldx,
                                    int splits, const void* bias, const int* positions, const int* slots,
                                    const float* cos_sin, const void* q_norm_w, const void* k_norm_w, float norm_eps,
                                    void* q_out, void* k_cache, void* v_cache, int nq, int nkv, int head_dim,
                                    int max_pos, int block_size, int block_n, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if ((ldw & 7) || (ldx & 7)) return -2;
  if (head_dim != 64 && head_dim != 128) return -2;
  if (cos_sin && !positions) return -2;
  const int features = (nq + 2 * nkv) * head_dim;
  DGemmArgs a{};
  if (int rc = fill_args(a, features, tokens, k, splits, block_n, 0)) return rc;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  RopeArgs r{};
  r.positions = positions;
  r.slots = slots;
  r.cos_sin = cos_sin;
  r.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  r.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  r.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  r.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  r.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  r.norm_eps = norm_eps;
  r.nq = nq; r.nkv = nkv; r.head_dim = head_dim; r.max_pos = max_pos; r.block_size = block_size;
  CUtensorMap ta, tb;
  if (encode_tmap_bf16_2d(&ta, w, k, features, ldw, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (block_n) {
    case 32: return launch_decode_gemm<32, RopeEpi>(ta, tb, a, 2, r, s);
    case 64: return launch_decode_gemm<64, RopeEpi>(ta, tb, a, 2, r, s);
    default: return launch_decode_gemm<128, RopeEpi>(ta, tb, a, 2, r, s);
  }
}
