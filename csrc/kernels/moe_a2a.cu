// Expert-parallel token all-to-all around the grouped expert GEMM (sm_100a, NVLink peer memory).
//
// Tokens are sharded over the ranks (sequence-parallel prefill, or data-parallel attention); experts are
// sharded too: rank d owns experts [d * E_l, (d + 1) * E_l).  One MoE block of one rank is
//
//   count     histogram of this rank's (token, expert) pairs; the row of counts is stored into every peer's
//             count matrix [source][expert] with plain peer stores, then a per-source arrival flag.  The same
//             (single-CTA) kernel waits for all sources and builds, from the full matrix, the schedule of
//             this rank's grouped GEMMs: group offsets, compact tile lists, total rows, overflow check.
//   dispatch  every pair's 4 KB activation row is stored straight into its expert owner's receive buffer,
//             at the row that the (identical on every rank) count matrix assigns to (source, expert);
//             when the last row of a (source, expert) segment is out, the source bumps that expert's
//             arrival counter on the owner.
//   GEMMs     the grouped tcgen05 GEMM (gemm_tcgen05.cuh) waits per expert, bounded, until all sources
//             have arrived, so the first experts multiply while later rows are still in flight.
//   combine   every rank announces "my expert outputs are complete", waits for the ranks it needs, and
//             pulls the k output rows of each of its tokens with plain peer loads, weighting and summing them.
//
// All counters only grow (targets are multiples of a call counter kept by the host), all waits are bounded
// and report into the library's status word.  No TMA and no multicast load ever touches peer memory: rows
// land in the owner's HBM before its TMA reads them, outputs are fetched with ordinary loads.
//
// Reference parity: the reference replicates all experts on every rank and all-reduces the block output
// (examples/models/qwen3/kernels/transformer_layer.py:70-115); expert parallelism with a token
// all-to-all is the NVSwitch-native alternative to it.
#include "common.cuh"
#include "api.h"

namespace nkb {

constexpr int kA2AMaxExperts = 1024;
constexpr int kA2AMaxRanks = 8;

__device__ __forceinline__ unsigned int a2a_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *p >= target (wrap-safe).  One thread calls it.
__device__ __forceinline__ bool a2a_wait_ge(const unsigned int* p, unsigned int target, int* status, int code) {
  if (int(a2a_ld_acquire(p) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (int(a2a_ld_acquire(p) - target) < 0) {
    if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

struct A2APeers {
  int* cnt[kA2AMaxRanks];                 // count matrix [n_ranks][experts] of every rank
  unsigned int* cnt_flag[kA2AMaxRanks];   // [n_ranks] per-source arrival counters of every rank
  unsigned int* arrive[kA2AMaxRanks];     // [experts_local] per-expert arrival counters of every rank
  unsigned int* ready[kA2AMaxRanks];      // [n_ranks] "expert outputs complete" counters of every rank
  __nv_bfloat16* x_recv[kA2AMaxRanks];    // receive buffer of every rank
  const __nv_bfloat16* y[kA2AMaxRanks];   // expert output buffer of every rank
};

// ---------------------------------------------------------------------------
// count + exchange + plan (one CTA of 1024 threads)
// ---------------------------------------------------------------------------
__global__ void moe_a2a_count_plan_kernel(const int* __restrict__ experts, int pairs, int num_experts, int n_ranks,
                                          int rank, unsigned int epoch, const A2APeers peers,
                                          int* __restrict__ cursors, int* __restrict__ sent,
                                          int* __restrict__ offsets, int capacity_rows, int bn_a,
                                          int* __restrict__ tiles_a, int* __restrict__ ntiles_a, int bn_b,
                                          int* __restrict__ tiles_b, int* __restrict__ ntiles_b,
                                          int* __restrict__ total_rows, int* __restrict__ status) {
  __shared__ int cnt[kA2AMaxExperts], off[kA2AMaxExperts + 1], sa[kA2AMaxExperts], sb[kA2AMaxExperts];
  __shared__ int ok_flag;
  griddep_wait();
  griddep_launch();
  const int t = threadIdx.x;
  cnt[t] = 0;
  __syncthreads();
  for (int i = t; i < pairs; i += 1024) {
    const int e = experts[i];
    if (e >= 0 && e < num_experts) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  // this rank's row of the count matrix goes to every rank (this one included); local cursors start at zero
  if (t < num_experts) {
    for (int pr = 0; pr < n_ranks; ++pr) peers.cnt[pr][rank * num_experts + t] = cnt[t];
    cursors[t] = 0;
    sent[t] = 0;
  }
  __syncthreads();
  if (t == 0) {
    __threadfence_system();
    for (int pr = 0; pr < n_ranks; ++pr) atomicAdd_system(peers.cnt_flag[pr] + rank, 1u);
    int ok = 1;
    for (int s = 0; s < n_ranks && ok; ++s)
      ok = a2a_wait_ge(peers.cnt_flag[rank] + s, epoch, status, ERR_WAIT_PEER_FLAG | (s << 8) | (1 << 16));
    ok_flag = ok;
  }
  __syncthreads();
  if (!ok_flag) return;
  // plan of this rank's grouped GEMMs: local expert el receives sum over sources of cnt[s][rank * E_l + el]
  const int e_local = num_experts / n_ranks;
  int n = 0;
  if (t < e_local)
    for (int s = 0; s < n_ranks; ++s) n += __ldcg(peers.cnt[rank] + s * num_experts + rank * e_local + t);
  const int ca = (n + bn_a - 1) / bn_a, cb = (n + bn_b - 1) / bn_b;
  off[t + 1] = n;
  sa[t] = ca;
  sb[t] = cb;
  if (t == 0) off[0] = 0;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = t >= o ? off[t + 1 - o] : 0, va = t >= o ? sa[t - o] : 0, vb = t >= o ? sb[t - o] : 0;
    __syncthreads();
    off[t + 1] += v;
    sa[t] += va;
    sb[t] += vb;
    __syncthreads();
  }
  if (t <= e_local) offsets[t] = off[t];
  if (t < e_local) {
    int base = sa[t] - ca;
    for (int i = 0; i < ca; ++i) { tiles_a[2 * (base + i)] = t; tiles_a[2 * (base + i) + 1] = i; }
    base = sb[t] - cb;
    for (int i = 0; i < cb; ++i) { tiles_b[2 * (base + i)] = t; tiles_b[2 * (base + i) + 1] = i; }
  }
  if (t == 1023) {
    *ntiles_a = sa[1023];
    *ntiles_b = sb[1023];
    *total_rows = off[e_local];
    if (off[e_local] > capacity_rows) atomicCAS(status, 0, ERR_BAD_ARGUMENT | (2 << 16));
  }
}

// ---------------------------------------------------------------------------
// dispatch: one warp per (token, expert) pair
// ---------------------------------------------------------------------------
__global__ void moe_a2a_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ experts,
                                        int pairs, int top_k, int hidden, int num_experts, int n_ranks, int rank,
                                        unsigned int epoch, const A2APeers peers, int* __restrict__ cursors,
                                        int* __restrict__ sent, int* __restrict__ pair_dest, int capacity_rows,
                                        int* __restrict__ status) {
  __shared__ int base[kA2AMaxExperts];   // first receive row of (this source, expert) on the expert's owner
  __shared__ int mine[kA2AMaxExperts];   // pairs this rank sends to the expert
  __shared__ int ok_flag;
  griddep_wait();
  griddep_launch();
  const int e_local = num_experts / n_ranks;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < n_ranks && ok; ++s)
      ok = a2a_wait_ge(peers.cnt_flag[rank] + s, epoch, status, ERR_WAIT_PEER_FLAG | (s << 8) | (3 << 16));
    ok_flag = ok;
  }
  __syncthreads();
  if (!ok_flag) return;
  const int* cm = peers.cnt[rank];       // the matrix is identical on every rank
  // group offset of expert e on its owner = rows of the owner's earlier local experts (all sources);
  // inside the group the sources follow each other in rank order
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int owner = e / e_local;
    int b = 0;
    for (int e2 = owner * e_local; e2 < e; ++e2)
      for (int s = 0; s < n_ranks; ++s) b += __ldcg(cm + s * num_experts + e2);
    for (int s = 0; s < rank; ++s) b += __ldcg(cm + s * num_experts + e);
    base[e] = b;
    mine[e] = __ldcg(cm + rank * num_experts + e);
  }
  __syncthreads();
  // experts this rank sends nothing to still have to hear from it
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
      if (mine[e] == 0) atomicAdd_system(peers.arrive[e / e_local] + (e % e_local), 1u);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  for (int p = blockIdx.x * warps + warp; p < pairs; p += gridDim.x * warps) {
    const int e = experts[p];
    if (e < 0 || e >= num_experts) {
      if (lane == 0) pair_dest[p] = -1;
      continue;
    }
    const int owner = e / e_local;
    int row = 0;
    if (lane == 0) row = base[e] + atomicAdd(&cursors[e], 1);
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row >= capacity_rows) {          // overflow was reported by the plan kernel; never write out of bounds
      if (lane == 0) pair_dest[p] = -1;
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(p / top_k) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(peers.x_recv[owner] + (long long)row * hidden);
    for (int v = lane; v < (hidden >> 3); v += 32) dst[v] = src[v];
    __syncwarp();
    if (lane == 0) {
      pair_dest[p] = (owner << 24) | row;
      __threadfence_system();            // the row is visible to the owner before it is counted
      const int done = atomicAdd(&sent[e], 1) + 1;
      if (done == mine[e]) {
        __threadfence_system();          // ... and so are the rows counted by the other warps before this one
        atomicAdd_system(peers.arrive[owner] + (e % e_local), 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// combine: one CTA per local token
// ---------------------------------------------------------------------------
__global__ void moe_a2a_combine_kernel(const int* __restrict__ pair_dest, const float* __restrict__ weights,
                                       int tokens, int top_k, int hidden, int n_ranks, int rank,
                                       unsigned int epoch, const A2APeers peers, __nv_bfloat16* __restrict__ out,
                                       int* __restrict__ status) {
  __shared__ int ok_flag;
  griddep_wait();          // the preceding kernel on this stream is this rank's last expert GEMM
  griddep_launch();
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int pr = 0; pr < n_ranks; ++pr) atomicAdd_system(peers.ready[pr] + rank, 1u);
    }
    int ok = 1;
    for (int s = 0; s < n_ranks && ok; ++s)
      ok = a2a_wait_ge(peers.ready[rank] + s, epoch, status, ERR_WAIT_PEER_FLAG | (s << 8) | (4 << 16));
    ok_flag = ok;
  }
  __syncthreads();
  if (!ok_flag) return;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top_k; ++j) {
        const int pd = pair_dest[t * top_k + j];
        if (pd < 0) continue;
        const float w = weights[t * top_k + j];
        const __nv_bfloat16* row = peers.y[pd >> 24] + (long long)(pd & 0xFFFFFF) * hidden;
        // written by another GPU's kernel: read it from L2 / the link, never from a stale L1 line
        const uint4 r = __ldcg(reinterpret_cast<const uint4*>(row) + v);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(rw[e]);
          acc[2 * e] += w * f.x;
          acc[2 * e + 1] += w * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + (long long)t * hidden + v * 8) = o;
    }
  }
}

static int fill_peers(A2APeers& p, int n_ranks, void* const* cnt, void* const* cnt_flag, void* const* arrive,
                      void* const* ready, void* const* x_recv, void* const* y) {
  if (n_ranks < 1 || n_ranks > kA2AMaxRanks) return -2;
  for (int i = 0; i < n_ranks; ++i) {
    p.cnt[i] = reinterpret_cast<int*>(cnt[i]);
    p.cnt_flag[i] = reinterpret_cast<unsigned int*>(cnt_flag[i]);
    p.arrive[i] = reinterpret_cast<unsigned int*>(arrive[i]);
    p.ready[i] = reinterpret_cast<unsigned int*>(ready[i]);
    p.x_recv[i] = reinterpret_cast<__nv_bfloat16*>(x_recv[i]);
    p.y[i] = reinterpret_cast<const __nv_bfloat16*>(y[i]);
  }
  return 0;
}

}  // namespace nkb

using namespace nkb;

// Pointer tables (one entry per rank) address the same regions of every rank's symmetric buffer:
// cnt int[n_ranks * experts], cnt_flag / ready unsigned[n_ranks], arrive unsigned[experts / n_ranks],
// x_recv / y bf16[capacity_rows * hidden].  epoch = number of this call (1, 2, ...), the same on every rank.
// Workspace (local, int32): cursors[experts], sent[experts], offsets[experts_local + 1], pair_dest[pairs],
// tiles_a / tiles_b [2 * max tiles], ntiles_a / ntiles_b / total_rows [1].
extern "C" int nkb_moe_a2a_dispatch(const void* x, const int* experts, int tokens, int top_k, int hidden,
                                    int num_experts, int n_ranks, int rank, unsigned int epoch, void* const* cnt,
                                    void* const* cnt_flag, void* const* arrive, void* const* ready,
                                    void* const* x_recv, void* const* y, int* cursors, int* sent, int* offsets,
                                    int* pair_dest, int capacity_rows, int bn_a, int* tiles_a, int* ntiles_a, int bn_b,
                                    int* tiles_b, int* ntiles_b, int* total_rows, void* stream) {
  if (tokens < 0 || top_k <= 0) return -2;
  if (num_experts <= 0 || num_experts > kA2AMaxExperts || num_experts % n_ranks || (hidden & 7)) return -2;
  if (capacity_rows <= 0 || capacity_rows >= (1 << 24) || rank < 0 || rank >= n_ranks) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  A2APeers p{};
  if (int rc = fill_peers(p, n_ranks, cnt, cnt_flag, arrive, ready, x_recv, y)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int pairs = tokens * top_k;
  int rc = launch_pdl(moe_a2a_count_plan_kernel, dim3(1), dim3(1024), 0, s, experts, pairs, num_experts, n_ranks, rank,
                      epoch, p, cursors, sent, offsets, capacity_rows, bn_a, tiles_a, ntiles_a, bn_b, tiles_b,
                      ntiles_b, total_rows, status_word());
  if (rc) return rc;
  int grid = (pairs + 7) / 8;
  const int cap = 4 * num_sms();
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return launch_pdl(moe_a2a_dispatch_kernel, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)x, experts, pairs,
                    top_k, hidden, num_experts, n_ranks, rank, epoch, p, cursors, sent, pair_dest, capacity_rows,
                    status_word());
}

extern "C" int nkb_moe_a2a_combine(const int* pair_dest, const float* weights, int tokens, int top_k, int hidden,
                                   int n_ranks, int rank, unsigned int epoch, void* const* cnt,
                                   void* const* cnt_flag, void* const* arrive, void* const* ready,
                                   void* const* x_recv, void* const* y, void* out, void* stream) {
  if (tokens < 0 || (hidden & 7) || rank < 0 || rank >= n_ranks) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  A2APeers p{};
  if (int rc = fill_peers(p, n_ranks, cnt, cnt_flag, arrive, ready, x_recv, y)) return rc;
  int grid = tokens < 1 ? 1 : tokens;
  const int cap = 8 * num_sms();
  if (grid > cap) grid = cap;
  return launch_pdl(moe_a2a_combine_kernel, dim3(grid), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    pair_dest, weights, tokens, top_k, hidden, n_ranks, rank, epoch, p, (__nv_bfloat16*)out,
                    status_word());
}
