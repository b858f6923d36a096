// One persistent kernel for everything between two attention calls of a decode step.
//
// A decode step of a transformer layer is a chain of tiny dependent operations -- at batch 64 each of them
// moves a few megabytes at most -- so launched one by one they cost a launch and a drain each and the
// GPU idles most of the time.  This kernel runs the whole chain
//
//   o_proj GEMM (-> peers)   sum over ranks / split-K partials + residual + RMSNorm
//   gate/up GEMM             SwiGLU (in the GEMM epilogue, or from split-K partials)
//   down GEMM (-> peers)     sum over ranks / split-K partials + residual + RMSNorm
//   QKV GEMM of the next layer      bias + QK-norm + RoPE + paged KV-cache append
//
// on one CTA per SM; the CTAs meet at a grid-wide barrier in global memory between dependent stages (a
// generation counter, bounded spin).  The GEMM stages are the library's tcgen05 / TMA body
// (gemm_tcgen05.cuh) run over all CTAs; with tensor parallelism the two row-parallel GEMMs push their bf16
// partial tiles straight into every rank's symmetric buffer (peer stores or one NVLink-multicast store)
// and the reducing stage waits for the ranks' arrival counters, exactly like the stand-alone kernels in
// gemm_tcgen05.cu / comm.cu whose protocol (slots, counters, two alternating buffers) it shares.
// A stage mask selects a sub-chain: the first layer of a step runs only the last two stages, the last
// layer stops after the second reduction, MoE layers run the two ends around their expert kernels.
//
// Every wait is bounded: a barrier or flag that does not complete within the limit records a code in the
// library's status word; every other CTA sees the word in its own wait loop and leaves too.
//
// Reference parity: the reference compiles a whole transformer layer into one device program
// (examples/models/qwen3/kernels/transformer_layer.py:17-115); this is the decode-time counterpart.
#include "gemm_tcgen05.cuh"
#include "api.h"

namespace nkb {

enum : int {
  ST_O = 1, ST_RED1 = 2, ST_GU = 4, ST_SILU = 8, ST_DOWN = 16, ST_RED2 = 32, ST_QKV = 64, ST_ROPE = 128
};

struct StageGemm {
  CUtensorMap tmA, tmB;
  GemmArgs args;
};

// Sum of bf16 slabs pushed by the ranks (flags != nullptr) or of fp32 split-K partials, + bias + residual,
// then RMSNorm.  One CTA per token row.
struct ReduceArgs {
  const __nv_bfloat16* slabs;      // [slots][tokens][hidden] bf16, local symmetric buffer
  const unsigned int* flags;       // [n_src] arrival counters (nullptr: local partials)
  unsigned int* seen;              // uses of this buffer consumed so far
  const float* partials;           // [splits][tokens][hidden] fp32
  long long split_stride;
  const __nv_bfloat16* bias;       // [hidden] or nullptr (local partials only; pushed slabs carry the bias)
  const __nv_bfloat16* x;          // [tokens][hidden] bf16 addend or nullptr (a block output computed elsewhere)
  const __nv_bfloat16* residual_in;
  const __nv_bfloat16* w;          // norm weight; nullptr: no norm output
  __nv_bfloat16* residual_out;
  __nv_bfloat16* normed_out;
  int slots, n_src, splits;
};

struct SiluArgs {
  const float* parts;              // [splits][tokens][2 * inter]
  long long stride;
  const __nv_bfloat16* bias;       // [2 * inter] or nullptr
  __nv_bfloat16* out;              // [tokens][inter]
  int splits, inter;
  float limit, alpha;
};

struct RopeArgs {
  const float* partials;           // [splits][tokens][(nq + 2 nkv) * D]
  long long split_stride;
  const __nv_bfloat16* bias;
  const int* positions;
  const int* slots;
  const float* cos_sin;
  const __nv_bfloat16* q_norm_w;
  const __nv_bfloat16* k_norm_w;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  float norm_eps;
  int splits, nq, nkv, head_dim, max_pos, block_size;
};

struct DecodeLayerArgs {
  StageGemm o, gu, down, qkv;
  PushArgs push_o, push_down;
  ReduceArgs red1, red2;
  SiluArgs silu;
  RopeArgs rope;
  unsigned int* grid_bar;          // [0] arrivals of the current barrier, [1] generation
  unsigned long long* timing;      // optional [80]: CTA 0 records the global timer after every stage, [16 + 16 g + p]: phase p of GEMM stage g (ns)
  int* status;
  int mask, tokens, hidden;
  float eps;
};
static_assert(sizeof(DecodeLayerArgs) <= 4000, "kernel parameter block");

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_system(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Grid-wide barrier in two halves.  `grid_arrive` (all threads of the CTA) publishes this CTA's writes and
// counts it; the CTA that completes the count opens the next generation.  `grid_wait` spins (bounded) until
// the generation read at arrival has passed.  Writes made before a CTA's arrival are visible after another
// CTA's wait to generic loads and, through the proxy fence, to TMA loads.  A GEMM stage that follows takes the
// wait inside (GridSync): its producer warp first fills the ring with weight tiles.
__device__ __forceinline__ unsigned int grid_arrive(unsigned int* bar) {
  __shared__ unsigned int gen_s;
  asm volatile("fence.proxy.async;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int gen = ld_acquire_gpu(bar + 1);   // cannot advance before this CTA has arrived
    __threadfence();
    const unsigned int prev = atomicAdd(bar, 1u);
    if (prev == gridDim.x - 1) {
      bar[0] = 0u;
      __threadfence();
      st_release_gpu(bar + 1, gen + 1u);
    }
    gen_s = gen;
  }
  __syncthreads();
  return gen_s;
}

// One thread's wait.  Returns false when the limit ran out or another CTA already reported an error.
__device__ __forceinline__ bool grid_wait_thread(const unsigned int* bar, unsigned int gen, int* status, int where) {
  if (ld_acquire_gpu(bar + 1) != gen) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (ld_acquire_gpu(bar + 1) == gen) {
    // polite polling: CTAs that arrive early (or have no work in a stage) would otherwise hammer the L2 slice
    // that holds this word and slow down the stores of the CTAs still working
    __nanosleep(100);
    if ((++spins & 127u) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (where << 8) | (int(blockIdx.x) << 16));
        return false;
      }
    }
  }
  return true;
}

// The whole CTA waits.
__device__ __forceinline__ bool grid_wait(const unsigned int* bar, unsigned int gen, int* status, int where) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = grid_wait_thread(bar, gen, status, where) ? 1 : 0;
  __syncthreads();
  asm volatile("fence.proxy.async;" ::: "memory");
  return ok_s != 0;
}

struct GridSync {
  static constexpr bool active = true;
  static constexpr bool lean = true;
  const unsigned int* bar;
  unsigned int gen;
  int* status;
  int where;
  bool pending;     // false: nothing to wait for (first stage of a launch)
  unsigned long long* marks;   // optional [16]: CTA 0 stores the global timer at the phases of the GEMM body
  __device__ __forceinline__ void mark(int slot) const {
    if (marks && blockIdx.x == 0) marks[slot] = globaltimer_ns();
  }
  __device__ __forceinline__ bool wait(volatile int* abort_flag) const {
    if (!pending) return true;
    const bool ok = grid_wait_thread(bar, gen, status, where);
    if (!ok) *abort_flag = 1;
    asm volatile("fence.proxy.async;" ::: "memory");
    return ok;
  }
};

// One copy of the GEMM body per (BN, PUSH) serves every GEMM stage of the kernel, so its instructions stay in
// the instruction cache from stage to stage and from layer to layer.  The argument block and the barrier state
// are passed by value (registers); behind a reference they would be re-read from the kernel's parameter
// space through generic loads after every memory clobber.
template <int BN, bool PUSH>
__device__ __noinline__ bool gemm_stage(const CUtensorMap* tmA, const CUtensorMap* tmB, const GemmArgs args,
                                        const PushArgs* push, const GridSync sync) {
  return gemm_bf16_body<BN, PUSH, false, NoFix, NoElemEpi, GridSync>(*tmA, *tmB, args, *push, GroupArgs{},
                                                                     NoFix::Args{}, NoElemEpi{}, sync);
}

constexpr int kRedIters = 4;   // 8 elements per thread per iteration: hidden <= 192 * 8 * 4

__device__ __forceinline__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kGemmThreads / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ void add_bf16x8(float (&a)[8], uint4 r) {
  const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16x2(rw[e]);
    a[2 * e] += f.x;
    a[2 * e + 1] += f.y;
  }
}

// Returns false when the wait for the ranks' partials ran out.
__device__ __noinline__ bool reduce_stage(const ReduceArgs r, int tokens, int hidden, float eps, int* status) {
  __shared__ float red[32];
  __shared__ int ok_s;
  if (int(blockIdx.x) >= tokens) return true;
  if (r.flags) {
    if (threadIdx.x == 0) {
      const unsigned int target = *reinterpret_cast<volatile unsigned int*>(r.seen) + 1u;
      int ok = 1;
      const unsigned long long t0 = globaltimer_ns();
      for (int s = 0; s < r.n_src && ok; ++s) {
        unsigned int spins = 0;
        while (int(ld_acquire_system(r.flags + s) - target) < 0) {
          __nanosleep(100);
          if ((++spins & 127u) == 0) {
            if (*reinterpret_cast<volatile int*>(status) != 0) { ok = 0; break; }
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
              atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (s << 8) | (int(blockIdx.x) << 16));
              ok = 0;
              break;
            }
          }
        }
      }
      ok_s = ok;
    }
    __syncthreads();
    if (!ok_s) return false;
  }
  const int nvec = hidden >> 3;
  for (long long row = blockIdx.x; row < tokens; row += gridDim.x) {
    float h[kRedIters][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kRedIters; ++it) {
      const int v = threadIdx.x + it * kGemmThreads;
      if (v < nvec) {
        const long long off = row * hidden + (long long)v * 8;
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = 0.f;
        if (r.flags) {
          // other ranks wrote these lines: read them from L2.  Eight slabs per batch keep 128 bytes per
          // thread in flight instead of a chain of dependent round trips.
          constexpr int kBatch = 8;
          const long long slot_stride = (long long)tokens * hidden;
          for (int s0 = 0; s0 < r.slots; s0 += kBatch) {
            uint4 q[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              q[u] = (s0 + u < r.slots) ? __ldcg(reinterpret_cast<const uint4*>(r.slabs + (s0 + u) * slot_stride + off))
                                        : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int u = 0; u < kBatch; ++u) add_bf16x8(a, q[u]);
          }
        } else {
          for (int s0 = 0; s0 < r.splits; s0 += 4) {
            float4 p[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (s0 + u < r.splits) {
                const float4* src = reinterpret_cast<const float4*>(r.partials + (s0 + u) * r.split_stride + off);
                p[u][0] = __ldcg(src);
                p[u][1] = __ldcg(src + 1);
              } else {
                p[u][0] = p[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              a[0] += p[u][0].x; a[1] += p[u][0].y; a[2] += p[u][0].z; a[3] += p[u][0].w;
              a[4] += p[u][1].x; a[5] += p[u][1].y; a[6] += p[u][1].z; a[7] += p[u][1].w;
            }
          }
          if (r.bias) add_bf16x8(a, *reinterpret_cast<const uint4*>(r.bias + (long long)v * 8));
        }
        if (r.x) add_bf16x8(a, __ldcg(reinterpret_cast<const uint4*>(r.x + off)));
        if (r.residual_in) add_bf16x8(a, __ldcg(reinterpret_cast<const uint4*>(r.residual_in + off)));
        uint4 o;
        o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
        o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
        if (r.residual_out) *reinterpret_cast<uint4*>(r.residual_out + off) = o;
        // statistics from the bf16-rounded stream: what an unfused norm reading the stored residual would see
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(ow[e]);
          h[it][2 * e] = f.x;
          h[it][2 * e + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    if (r.w) {
      const float tot = cta_sum(ss, red);
      const float inv = rsqrtf(tot / float(hidden) + eps);
#pragma unroll
      for (int it = 0; it < kRedIters; ++it) {
        const int v = threadIdx.x + it * kGemmThreads;
        if (v < nvec) {
          const long long off = row * hidden + (long long)v * 8;
          const uint4 wr = *reinterpret_cast<const uint4*>(r.w + (long long)v * 8);
          const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(ww[e]);
            o[e] = pack_bf16x2(h[it][2 * e] * inv * f.x, h[it][2 * e + 1] * inv * f.y);
          }
          *reinterpret_cast<uint4*>(r.normed_out + off) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
  return true;
}

__device__ __forceinline__ void silu_stage(const SiluArgs& s, int tokens) {
  const int per_row = s.inter >> 2;
  const long long nvec = (long long)tokens * per_row;
  for (long long i = blockIdx.x * (long long)kGemmThreads + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * kGemmThreads) {
    const long long r = i / per_row;
    const int c = int(i % per_row) * 4;
    float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
    // four splits per batch: eight independent 16-byte loads in flight instead of a chain of round trips
    for (int s0 = 0; s0 < s.splits; s0 += 4) {
      float4 gv[4], uv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (s0 + q < s.splits) {
          const float* base = s.parts + (s0 + q) * s.stride + r * 2 * s.inter + c;
          gv[q] = __ldcg(reinterpret_cast<const float4*>(base));
          uv[q] = __ldcg(reinterpret_cast<const float4*>(base + s.inter));
        } else {
          gv[q] = uv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        g[0] += gv[q].x; g[1] += gv[q].y; g[2] += gv[q].z; g[3] += gv[q].w;
        u[0] += uv[q].x; u[1] += uv[q].y; u[2] += uv[q].z; u[3] += uv[q].w;
      }
    }
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float gg = g[e], uu = u[e];
      if (s.bias) {
        gg += __bfloat162float(s.bias[c + e]);
        uu += __bfloat162float(s.bias[s.inter + c + e]);
      }
      if (s.limit > 0.f) {
        gg = fminf(gg, s.limit);
        uu = fminf(fmaxf(uu, -s.limit), s.limit);
        o[e] = (uu + 1.f) * gg / (1.f + __expf(-s.alpha * gg));
      } else {
        o[e] = gg / (1.f + __expf(-gg)) * uu;
      }
    }
    uint2 pk;
    pk.x = pack_bf16x2(o[0], o[1]);
    pk.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(s.out + r * s.inter + c) = pk;
  }
}

// One warp per (token, head): sum of the QKV partials, bias, per-head RMSNorm of queries and keys, the
// rotate-halves rotation, queries to q_out, keys and values to their slot of the paged cache
// [block, kv_head, token_in_block, D].
template <int D>
__device__ __forceinline__ void rope_stage(const RopeArgs& a, int tokens) {
  constexpr int PER = D / 64;
  const int heads = a.nq + 2 * a.nkv;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)tokens * heads;
  const int width = heads * D;
  for (long long gw = blockIdx.x * (kGemmThreads / 32) + (threadIdx.x >> 5); gw < total;
       gw += (long long)gridDim.x * (kGemmThreads / 32)) {
    const int t = int(gw / heads), h = int(gw % heads);
    const long long base = (long long)t * width + (long long)h * D;
    float lo[PER], hi[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) lo[j] = hi[j] = 0.f;
    // four splits per batch: all loads of a batch are issued before the first sum needs one
    for (int s0 = 0; s0 < a.splits; s0 += 4) {
      float xv[4][PER], yv[4][PER];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int i = lane * PER + j;
          const bool on = s0 + q < a.splits;
          const float* src = a.partials + (long long)(s0 + q) * a.split_stride + base + i;
          xv[q][j] = on ? __ldcg(src) : 0.f;
          yv[q][j] = on ? __ldcg(src + D / 2) : 0.f;
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          lo[j] += xv[q][j];
          hi[j] += yv[q][j];
        }
      }
    }
    if (a.bias) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane * PER + j;
        lo[j] += __bfloat162float(a.bias[h * D + i]);
        hi[j] += __bfloat162float(a.bias[h * D + D / 2 + i]);
      }
    }
    const bool is_q = h < a.nq, is_k = !is_q && h < a.nq + a.nkv;
    const int slot = a.slots ? a.slots[t] : -1;
    if (is_q || is_k) {
      const __nv_bfloat16* nw = is_q ? a.q_norm_w : a.k_norm_w;
      if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < PER; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / float(D) + a.norm_eps);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int i = lane * PER + j;
          lo[j] = __bfloat162float(__float2bfloat16(lo[j] * inv * __bfloat162float(nw[i])));
          hi[j] = __bfloat162float(__float2bfloat16(hi[j] * inv * __bfloat162float(nw[D / 2 + i])));
        }
      }
      if (a.cos_sin) {
        int pos = a.positions[t];
        pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
        const float* cs = a.cos_sin + (long long)pos * D;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int i = lane * PER + j;
          const float c = cs[i], s = cs[D / 2 + i];
          const float x = lo[j], y = hi[j];
          lo[j] = x * c - y * s;
          hi[j] = y * c + x * s;
        }
      }
    }
    __nv_bfloat16* dst;
    if (is_q) {
      dst = a.q_out + (long long)t * a.nq * D + (long long)h * D;
    } else {
      if (slot < 0) continue;
      const int kh = is_k ? h - a.nq : h - a.nq - a.nkv;
      const long long blk = slot / a.block_size, off = slot % a.block_size;
      dst = (is_k ? a.k_cache : a.v_cache) + ((blk * a.nkv + kh) * a.block_size + off) * D;
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane * PER + j;
      dst[i] = __float2bfloat16(lo[j]);
      dst[D / 2 + i] = __float2bfloat16(hi[j]);
    }
  }
}

template <int BN, bool TP>
__global__ void __launch_bounds__(kGemmThreads, 1) decode_layer_kernel(const __grid_constant__ DecodeLayerArgs L) {
  const int mask = L.mask;
  int* status = L.status;
  // a kernel of an earlier, failed step left its error: do nothing (the host reads and clears the word)
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  if (!(mask & ST_O)) griddep_wait();     // the GEMM body orders itself against the preceding kernel
  unsigned int* bar = L.grid_bar;
  int nbar = 0, ntick = 0;
  auto tick = [&]() {
    if (L.timing && blockIdx.x == 0 && threadIdx.x == 0) L.timing[ntick] = globaltimer_ns();
    ++ntick;
  };
  tick();
  GridSync sync{bar, 0u, status, 0, false, nullptr};
  int ngemm = 0;
  auto marks = [&]() { sync.marks = L.timing ? L.timing + 16 + 16 * ngemm++ : nullptr; };
  // arrive now, wait later: the next stage (or `settle`) completes the barrier
  auto arrive = [&]() {
    sync.gen = grid_arrive(bar);
    sync.where = 32 + nbar++;
    sync.pending = true;
  };
  auto settle = [&]() -> bool {
    if (!sync.pending) return true;
    sync.pending = false;
    return grid_wait(bar, sync.gen, status, sync.where);
  };
  // which reduction still has to advance its "uses consumed" counter once every CTA has read it
  unsigned int* bump = nullptr;
  auto bump_seen = [&]() {
    if (TP && bump && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(bump, 1u);
    bump = nullptr;
  };

  if (mask & ST_O) {
    marks();
    if (!gemm_stage<BN, TP>(&L.o.tmA, &L.o.tmB, L.o.args, &L.push_o, sync)) return;
    if (!TP) arrive();                    // pushed partials are ordered by the ranks' arrival counters instead
    tick();
  }
  if (mask & ST_RED1) {
    if (!settle()) return;
    if (!reduce_stage(L.red1, L.tokens, L.hidden, L.eps, status)) return;
    arrive();
    bump = L.red1.seen;
    tick();
  }
  if (mask & ST_GU) {
    marks();
    if (!gemm_stage<BN, false>(&L.gu.tmA, &L.gu.tmB, L.gu.args, &L.push_o, sync)) return;
    sync.pending = false;
    bump_seen();
    arrive();
    tick();
  }
  if (mask & ST_SILU) {
    if (!settle()) return;
    silu_stage(L.silu, L.tokens);
    arrive();
    tick();
  }
  if (mask & ST_DOWN) {
    marks();
    if (!gemm_stage<BN, TP>(&L.down.tmA, &L.down.tmB, L.down.args, &L.push_down, sync)) return;
    sync.pending = false;
    bump_seen();
    if (!TP) arrive();
    tick();
  }
  if (mask & ST_RED2) {
    if (!settle()) return;
    bump_seen();
    if (!reduce_stage(L.red2, L.tokens, L.hidden, L.eps, status)) return;
    arrive();
    bump = L.red2.seen;
    tick();
  }
  if (mask & ST_QKV) {
    marks();
    if (!gemm_stage<BN, false>(&L.qkv.tmA, &L.qkv.tmB, L.qkv.args, &L.push_o, sync)) return;
    sync.pending = false;
    bump_seen();
    arrive();
    tick();
  }
  if (mask & ST_ROPE) {
    if (!settle()) return;
    switch (L.rope.head_dim) {
      case 64: rope_stage<64>(L.rope, L.tokens); break;
      case 128: rope_stage<128>(L.rope, L.tokens); break;
      default: rope_stage<256>(L.rope, L.tokens); break;
    }
  }
  // a barrier that is still open (the launch ends with a reduction): complete it, the counter needs it
  if (!settle()) return;
  bump_seen();
  tick();
}

}  // namespace nkb

using namespace nkb;

// Flat description of one launch, filled by the Python layer (ctypes structure with the same field order).
// Pointers may be null where the text says so; all leading dimensions are in elements.
extern "C" struct NkbDecodeLayer {
  int mask, tokens, hidden, block_n;
  int n_ranks, rank;                // n_ranks == 0: no tensor-parallel push (split-K partials are summed locally)
  float eps;
  int _pad0;
  // o_proj: w_o [hidden, k_o], attn [tokens, k_o]
  const void* w_o; const void* attn; long long ld_wo, ld_attn; int k_o, splits_o; const void* bias_o;
  // post-attention reduction
  const void* resid_in; const void* norm1_w; void* resid_mid; void* normed_mid;
  // gate / up: w_gu [2 * inter, hidden]; fused_gate != 0: SwiGLU inside the GEMM (splits_gu ignored)
  const void* w_gu; long long ld_wgu; int inter, splits_gu, fused_gate, _pad1; const void* bias_gu;
  float act_limit, act_alpha; void* act;     // [tokens, inter]
  // down: w_down [hidden, inter]
  const void* w_down; long long ld_wdown; int splits_down, _pad2; const void* bias_down;
  // second reduction
  const void* norm2_w; void* resid_out; void* normed_out;
  // QKV of the next layer: w_qkv [(nq + 2 nkv) * head_dim, hidden]
  const void* w_qkv; long long ld_wqkv; int splits_qkv, nq, nkv, head_dim; const void* bias_qkv;
  const int* positions; const int* slots; const float* cos_sin; const void* q_norm_w; const void* k_norm_w;
  void* q_out; void* k_cache; void* v_cache; int max_pos, block_size;
  // scratch: fp32 partials (floats), the grid barrier words [2]
  float* scratch; long long scratch_floats; unsigned int* grid_bar;
  // tensor-parallel push (n_ranks > 0): two alternating symmetric buffers, the o_proj uses buffer buf_o and the
  // down projection buffer buf_down; *_local are this rank's views, peer_* the same locations on every rank
  void* const* peer_out_o; void* const* peer_flag_o; void* mc_out_o; void* mc_flag_o;
  const void* slabs_o; const void* flags_o; void* seen_o; void* done_o;
  void* const* peer_out_d; void* const* peer_flag_d; void* mc_out_d; void* mc_flag_d;
  const void* slabs_d; const void* flags_d; void* seen_d; void* done_d;
  int max_slots, _pad3;
  // second reduction without the down stage (the block between the two ends ran elsewhere, e.g. MoE experts):
  // with ranks the pushed slabs of buffer "d" (red2_slots of them) are summed, else red2_x [tokens, hidden] bf16
  const void* red2_x; int red2_slots, _pad4;
  // optional: 80 unsigned 64-bit words; CTA 0 stores the global timer (ns) at kernel start and after every stage
  // ([0..15]) and at eight phases of each GEMM stage ([16 + 16 * stage + phase], ten phases)
  void* timing;
};

namespace {

int setup_gemm(StageGemm& g, const void* w, const void* x, int rows, int tokens, int k, long long ldw, long long ldx,
               int splits, int block_n, int gated, int gate_off) {
  if (rows <= 0 || k <= 0 || (k & 7) || (ldw & 7) || (ldx & 7)) return -2;
  GemmArgs& a = g.args;
  a = GemmArgs{};
  a.rows = rows;
  a.cols = tokens;
  a.k = k;
  a.kb_total = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > a.kb_total) splits = a.kb_total;
  a.kb_per_split = (a.kb_total + splits - 1) / splits;
  a.splits = (a.kb_total + a.kb_per_split - 1) / a.kb_per_split;
  a.num_row_tiles = (rows + kTileRows - 1) / kTileRows;
  a.num_col_tiles = 1;
  a.gated = gated;
  a.gate_off = gate_off;
  a.transpose_out = 1;
  a.bias_on_rows = 1;
  a.status = status_word();
  a.weights_operand = 0;
  const uint64_t a_rows = gated ? uint64_t(gate_off) + rows : rows;
  if (encode_tmap_bf16_2d(&g.tmA, w, k, a_rows, ldw, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&g.tmB, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  return 0;
}

// Dynamic shared memory of the layer kernel: an SM's 227 KB minus room for the kernel's static variables
// (reduction scratch, barrier hand-over words).
constexpr int kLayerDynSmem = 232448 - 2048;

// Ring depth for one CTA per SM; returns the dynamic shared memory the stage needs.
int ring(GemmArgs& a, int block_n, bool push) {
  if (!push) mark_bulk(a);
  const int a_tiles = a.gated == 1 ? 2 : 1;
  const int stage_bytes = a_tiles * kATileBytes + block_n * kBlockK * 2;
  const int extra = 512 + (push ? 32 * kTileRows * 2 : 2 * 16 * kTileRows * 4);
  const int budget = kLayerDynSmem - 1024 - extra - 64;
  int stages = budget / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  return stages * stage_bytes + 1024 + extra + 64;
}

void fill_push(PushArgs& p, int n, int rank, void* const* out, void* const* flag, void* mc_out, void* mc_flag,
               void* done) {
  p = PushArgs{};
  p.n_peers = n;
  p.rank = rank;
  for (int i = 0; i < n; ++i) {
    p.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(out[i]);
    p.peer_flag[i] = reinterpret_cast<unsigned int*>(flag[i]);
  }
  p.done_counter = reinterpret_cast<unsigned int*>(done);
  p.mc_out = reinterpret_cast<__nv_bfloat16*>(mc_out);
  p.mc_flag = reinterpret_cast<unsigned int*>(mc_flag);
}

template <int BN, bool TP>
int launch_layer(const DecodeLayerArgs& L, int smem, cudaStream_t stream) {
  auto kernel = decode_layer_kernel<BN, TP>;
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLayerDynSmem);
    if (e != cudaSuccess) return int(e);
    attr_set[dev] = true;
  }
  return launch_pdl(kernel, dim3(num_sms()), dim3(kGemmThreads), size_t(smem), stream, L);
}

}  // namespace

extern "C" int nkb_decode_layer(const NkbDecodeLayer* d, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (!d || d->tokens <= 0 || d->hidden <= 0 || (d->hidden & 7)) return -2;
  const int T = d->tokens, H = d->hidden, bn = d->block_n;
  if ((bn != 32 && bn != 64 && bn != 128) || T > bn) return -2;
  if (H > kGemmThreads * 8 * kRedIters) return -2;
  if (!d->grid_bar || !d->scratch) return -2;
  const bool tp = d->n_ranks > 0;
  if (tp && (d->n_ranks > kMaxPeers || d->rank < 0 || d->rank >= d->n_ranks)) return -2;
  const int mask = d->mask;
  DecodeLayerArgs L{};
  L.mask = mask;
  L.tokens = T;
  L.hidden = H;
  L.eps = d->eps;
  L.grid_bar = d->grid_bar;
  L.timing = reinterpret_cast<unsigned long long*>(d->timing);
  L.status = status_word();
  int smem = 4096;
  auto bf = [](const void* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
  auto bfm = [](void* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
  int rc;

  if (mask & ST_O) {
    if ((rc = setup_gemm(L.o, d->w_o, d->attn, H, T, d->k_o, d->ld_wo, d->ld_attn, d->splits_o, bn, 0, 0))) return rc;
    GemmArgs& a = L.o.args;
    a.bias = bf(d->bias_o);
    if (tp) {
      if (d->n_ranks * a.splits > d->max_slots) return -2;
      a.ldo = H;
      fill_push(L.push_o, d->n_ranks, d->rank, d->peer_out_o, d->peer_flag_o, d->mc_out_o, d->mc_flag_o, d->done_o);
    } else {
      if ((long long)a.splits * T * H > d->scratch_floats) return -2;
      a.out_fp32 = 1;
      a.ldo = H;
      a.split_stride = (long long)T * H;
      a.out = d->scratch;
    }
    const int s = ring(a, bn, tp);
    if (a.stages < 2) return -3;
    if (s > smem) smem = s;
  }
  auto fill_reduce = [&](ReduceArgs& r, const GemmArgs& g, const void* slabs, const void* flags, void* seen,
                         const void* resid_in, const void* w, void* resid_out, void* normed_out) {
    r = ReduceArgs{};
    if (tp) {
      r.slabs = bf(slabs);
      r.flags = reinterpret_cast<const unsigned int*>(flags);
      r.seen = reinterpret_cast<unsigned int*>(seen);
      r.slots = d->n_ranks * g.splits;
      r.n_src = d->n_ranks;
    } else {
      r.partials = d->scratch;
      r.splits = g.splits;
      r.split_stride = (long long)T * H;
    }
    r.residual_in = bf(resid_in);
    r.w = bf(w);
    r.residual_out = bfm(resid_out);
    r.normed_out = bfm(normed_out);
  };
  if (mask & ST_RED1) {
    if (!(mask & ST_O)) return -2;
    if (!d->resid_mid || (d->norm1_w && !d->normed_mid)) return -2;
    fill_reduce(L.red1, L.o.args, d->slabs_o, d->flags_o, d->seen_o, d->resid_in, d->norm1_w, d->resid_mid,
                d->normed_mid);
  }
  if (mask & ST_GU) {
    const int I = d->inter;
    if (I <= 0 || (I & 7) || !d->normed_mid || !d->act) return -2;
    if (d->fused_gate) {
      if ((mask & ST_SILU) || d->bias_gu || d->act_limit > 0.f) return -2;
      if ((rc = setup_gemm(L.gu, d->w_gu, d->normed_mid, I, T, H, d->ld_wgu, H, 1, bn, 1, I))) return rc;
      L.gu.args.ldo = I;
      L.gu.args.out = d->act;
    } else {
      if (!(mask & ST_SILU)) return -2;
      if ((rc = setup_gemm(L.gu, d->w_gu, d->normed_mid, 2 * I, T, H, d->ld_wgu, H, d->splits_gu, bn, 0, 0))) return rc;
      GemmArgs& a = L.gu.args;
      if ((long long)a.splits * T * 2 * I > d->scratch_floats) return -2;
      a.out_fp32 = 1;
      a.ldo = 2 * I;
      a.split_stride = (long long)T * 2 * I;
      a.out = d->scratch;
      L.silu = SiluArgs{};
      L.silu.parts = d->scratch;
      L.silu.stride = a.split_stride;
      L.silu.bias = bf(d->bias_gu);
      L.silu.out = bfm(d->act);
      L.silu.splits = a.splits;
      L.silu.inter = I;
      L.silu.limit = d->act_limit;
      L.silu.alpha = d->act_alpha;
    }
    const int s = ring(L.gu.args, bn, false);
    if (L.gu.args.stages < 2) return -3;
    if (s > smem) smem = s;
  }
  if (mask & ST_DOWN) {
    if ((rc = setup_gemm(L.down, d->w_down, d->act, H, T, d->inter, d->ld_wdown, d->inter, d->splits_down, bn, 0, 0)))
      return rc;
    GemmArgs& a = L.down.args;
    a.bias = bf(d->bias_down);
    if (tp) {
      if (d->n_ranks * a.splits > d->max_slots) return -2;
      a.ldo = H;
      fill_push(L.push_down, d->n_ranks, d->rank, d->peer_out_d, d->peer_flag_d, d->mc_out_d, d->mc_flag_d, d->done_d);
    } else {
      if ((long long)a.splits * T * H > d->scratch_floats) return -2;
      a.out_fp32 = 1;
      a.ldo = H;
      a.split_stride = (long long)T * H;
      a.out = d->scratch;
    }
    const int s = ring(a, bn, tp);
    if (a.stages < 2) return -3;
    if (s > smem) smem = s;
  }
  if (mask & ST_RED2) {
    if (!d->resid_out || (d->norm2_w && !d->normed_out)) return -2;
    if (mask & ST_DOWN) {
      fill_reduce(L.red2, L.down.args, d->slabs_d, d->flags_d, d->seen_d, d->resid_mid, d->norm2_w, d->resid_out,
                  d->normed_out);
    } else {
      // the block output comes from other kernels: pushed slabs (ranks) or one bf16 tensor
      GemmArgs none{};
      none.splits = 0;
      fill_reduce(L.red2, none, d->slabs_d, d->flags_d, d->seen_d, d->resid_mid, d->norm2_w, d->resid_out,
                  d->normed_out);
      if (tp) {
        if (d->red2_slots < 1 || d->red2_slots > d->max_slots) return -2;
        L.red2.slots = d->red2_slots;
      } else {
        if (!d->red2_x) return -2;
        L.red2.x = bf(d->red2_x);
      }
    }
  }
  if (mask & ST_QKV) {
    const int width = (d->nq + 2 * d->nkv) * d->head_dim;
    if (!(mask & ST_ROPE) || !d->normed_out) return -2;
    if (d->head_dim != 64 && d->head_dim != 128 && d->head_dim != 256) return -2;
    if ((rc = setup_gemm(L.qkv, d->w_qkv, d->normed_out, width, T, H, d->ld_wqkv, H, d->splits_qkv, bn, 0, 0)))
      return rc;
    GemmArgs& a = L.qkv.args;
    if ((long long)a.splits * T * width > d->scratch_floats) return -2;
    a.out_fp32 = 1;
    a.ldo = width;
    a.split_stride = (long long)T * width;
    a.out = d->scratch;
    const int s = ring(a, bn, false);
    if (a.stages < 2) return -3;
    if (s > smem) smem = s;
    RopeArgs& r = L.rope;
    r = RopeArgs{};
    r.partials = d->scratch;
    r.split_stride = a.split_stride;
    r.splits = a.splits;
    r.bias = bf(d->bias_qkv);
    r.positions = d->positions;
    r.slots = d->slots;
    r.cos_sin = d->cos_sin;
    r.q_norm_w = bf(d->q_norm_w);
    r.k_norm_w = bf(d->k_norm_w);
    r.q_out = bfm(d->q_out);
    r.k_cache = bfm(d->k_cache);
    r.v_cache = bfm(d->v_cache);
    r.norm_eps = d->eps;
    r.nq = d->nq;
    r.nkv = d->nkv;
    r.head_dim = d->head_dim;
    r.max_pos = d->max_pos;
    r.block_size = d->block_size;
    if (!r.q_out || !r.k_cache || !r.v_cache || (r.cos_sin && !r.positions)) return -2;
  } else if (mask & ST_ROPE) {
    return -2;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define NKB_LAYER(BNV)                                               \
  return tp ? launch_layer<BNV, true>(L, smem, s) : launch_layer<BNV, false>(L, smem, s)
  switch (bn) {
    case 32: NKB_LAYER(32);
    case 64: NKB_LAYER(64);
    default: NKB_LAYER(128);
  }
#undef NKB_LAYER
}

// Size of the descriptor as this library was compiled: the Python binding compares it with its own layout.
extern "C" int nkb_decode_layer_desc_size() { return int(sizeof(NkbDecodeLayer)); }
