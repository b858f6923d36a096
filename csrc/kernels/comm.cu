// Symmetric (peer-mapped) memory and the consumer side of the fused
// GEMM + all-reduce used by tensor-parallel decode.
//
// Every rank allocates the same buffers with cudaMalloc, exports them with CUDA
// IPC handles (exchanged by the Python layer over the process group) and maps its
// peers' buffers; kernels then address peer memory with plain loads / stores over
// NVLink.  No TMA (and no multicast) ever touches peer memory here.
//
// Protocol of one row-parallel GEMM + sum over ranks (one "use" of a buffer):
//   producer (gemm_tcgen05.cu, push mode)  stores its bf16 partial tiles into slot
//       (rank * splits + split) of every peer's partial array, then its last CTA
//       adds 1 to flags[rank] on every peer (system-scope atomic after a fence);
//   consumer (tp_reduce_rmsnorm below)     waits until flags[src] >= seen + 1 for
//       every source rank (bounded spin, error status on expiry), sums the slots with
//       L1-bypassing loads, adds residual / bias, applies RMSNorm, and its last CTA
//       advances `seen`.
// Counters only ever grow, so a captured CUDA graph can be replayed without any
// host-side reset.  Two buffers are used alternately by consecutive operations; a
// rank can be at most one operation ahead of a peer (it needs that peer's partial
// of the previous operation first), so a buffer is never overwritten while a peer
// still reads it.
//
// Reference parity: the reference reduces with an HLO all-reduce executed by the
// Neuron runtime (examples/models/qwen3/kernels/attention.py:150-154,
// examples/models/qwen3/kernels/transformer_layer.py:112-115).
#include "common.cuh"
#include "gemm_args.h"
#include "api.h"
#include <string.h>

namespace nkb {

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int kTpMaxIters = 4;

// One CTA per token row.  partials: [slots, rows, hidden] bf16 (local memory, written by
// all ranks).  flags: [n_src] arrival counters, seen: uses completed so far.
__global__ void tp_reduce_rmsnorm_kernel(const __nv_bfloat16* __restrict__ partials, int slots,
                                         const unsigned int* __restrict__ flags, int n_src,
                                         unsigned int* __restrict__ seen, unsigned int* __restrict__ done_counter,
                                         const __nv_bfloat16* __restrict__ residual_in,
                                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ residual_out,
                                         __nv_bfloat16* __restrict__ normed_out, int rows, int hidden, float eps,
                                         int* __restrict__ status) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  griddep_wait();
  griddep_launch();
  if (threadIdx.x == 0) {
    const unsigned int target = *reinterpret_cast<volatile unsigned int*>(seen) + 1u;
    int ok = 1;
    const unsigned long long t0 = globaltimer_ns();
    for (int s = 0; s < n_src && ok; ++s) {
      unsigned int spins = 0;
      while (int(ld_acquire_sys(flags + s) - target) < 0) {
        if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
          atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (s << 8) | (blockIdx.x << 16));
          ok = 0;
          break;
        }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  const long long row = blockIdx.x;
  const int nvec = hidden >> 3;
  float h[kTpMaxIters][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kTpMaxIters; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      const long long off = row * hidden + (long long)v * 8;
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      // remote ranks wrote these lines: read them from L2, never from a stale L1 line.  Eight slots are
      // fetched per batch so that a thread keeps 128 bytes in flight (one row per CTA leaves most SMs idle,
      // and with 8 ranks x 3 splits a slot-by-slot loop was a chain of 24 L2 round trips).
      constexpr int kBatch = 8;
      const long long slot_stride = (long long)rows * hidden;
      for (int s0 = 0; s0 < slots; s0 += kBatch) {
        uint4 r[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          r[u] = (s0 + u < slots) ? __ldcg(reinterpret_cast<const uint4*>(partials + (s0 + u) * slot_stride + off))
                                  : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const uint32_t rw[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16x2(rw[e]);
            a[2 * e] += f.x;
            a[2 * e + 1] += f.y;
          }
        }
      }
      if (residual_in) {
        const uint4 r = *reinterpret_cast<const uint4*>(residual_in + off);
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(rw[e]);
          a[2 * e] += f.x;
          a[2 * e + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
      o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
      if (residual_out) *reinterpret_cast<uint4*>(residual_out + off) = o;
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
  if (w) {
    ss = warp_sum(ss);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    const float inv = rsqrtf(t / float(hidden) + eps);
#pragma unroll
    for (int it = 0; it < kTpMaxIters; ++it) {
      const int v = threadIdx.x + it * blockDim.x;
      if (v < nvec) {
        const long long off = row * hidden + (long long)v * 8;
        const uint4 wr = *reinterpret_cast<const uint4*>(w + (long long)v * 8);
        const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(ww[e]);
          o[e] = pack_bf16x2(h[it][2 * e] * inv * f.x, h[it][2 * e + 1] * inv * f.y);
        }
        *reinterpret_cast<uint4*>(normed_out + off) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  // the last CTA to finish marks this use of the buffer as consumed
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(done_counter, 1u);
    if (old == gridDim.x - 1) {
      *done_counter = 0u;
      if (ok_flag) atomicAdd(seen, 1u);
      __threadfence();
    }
  }
}

// Split-K sum, exchange over NVLink, sum over ranks, residual and RMSNorm in ONE launch, one CTA per token row.
// The producing GEMM leaves its fp32 split-K partials in local memory; this kernel adds them up first, so one
// bf16 row per rank crosses NVLink instead of one per split (with seven splits at four ranks that is 2 MB
// instead of 14.7 MB per operation and rank, in both directions), and the consumer sums n slots instead of
// n x splits.  Protocol per row r:  push the pre-summed row into slot [rank] of every rank's slot array (plain
// peer stores, or one multimem store through the NVLink multicast mapping); fence at system scope; add 1 to
// this rank's counter for row r on every rank; wait (bounded) until all ranks' counters for row r reach
// seen + 1; sum the slots.  Counters only grow and two buffers alternate, exactly like the push protocol above.
// push.peer_out[p]: slot array [n][rows][hidden] of rank p; push.peer_flag[p]: row counters [n][kRowFlags] of
// rank p; push.mc_out / push.mc_flag: the same arrays through the multicast mapping, or nullptr.
constexpr int kRowFlags = 128;
__global__ void __launch_bounds__(512) tp_exchange_reduce_rmsnorm_kernel(const float* __restrict__ partials, int splits,
                                                  long long split_stride, const __nv_bfloat16* __restrict__ y,
                                                  const PushArgs push, const __nv_bfloat16* __restrict__ slots,
                                                  const unsigned int* __restrict__ rowflags,
                                                  unsigned int* __restrict__ seen,
                                                  unsigned int* __restrict__ done_counter,
                                                  const __nv_bfloat16* __restrict__ residual_in,
                                                  const __nv_bfloat16* __restrict__ w,
                                                  __nv_bfloat16* __restrict__ residual_out,
                                                  __nv_bfloat16* __restrict__ normed_out, int rows, int hidden,
                                                  float eps, int* __restrict__ status) {
  __shared__ float red[32];
  __shared__ int ok_flag;
  griddep_wait();
  griddep_launch();
  const long long row = blockIdx.x;
  const int nvec = hidden >> 3;
  const int n = push.n_peers;
  const long long slot_stride = (long long)rows * hidden;
  const unsigned int target = *reinterpret_cast<volatile unsigned int*>(seen) + 1u;
  // ---- phase 1: this rank's contribution for the row, summed over its split-K partials, to every rank
#pragma unroll 1
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const long long off = row * hidden + (long long)v * 8;
    uint4 o;
    if (partials) {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < splits; s0 += 4) {
        float4 p[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (s0 + u < splits) {
            const float4* src = reinterpret_cast<const float4*>(partials + (s0 + u) * split_stride + off);
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
      o = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                     pack_bf16x2(a[6], a[7]));
    } else {
      o = __ldcg(reinterpret_cast<const uint4*>(y + off));
    }
    push_store_16(push, (long long)push.rank * slot_stride + off, o);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const long long fidx = (long long)push.rank * kRowFlags + row;
    if (push.mc_flag) {
      multimem_add_release_u32(push.mc_flag + fidx, 1u);
    } else {
      for (int pr = 0; pr < n; ++pr)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(push.peer_flag[pr] + fidx), "r"(1u) : "memory");
    }
    int ok = 1;
    const unsigned long long t0 = globaltimer_ns();
    for (int s = 0; s < n && ok; ++s) {
      unsigned int spins = 0;
      while (int(ld_acquire_sys(rowflags + s * kRowFlags + row) - target) < 0) {
        if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
          atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (s << 8) | (blockIdx.x << 16));
          ok = 0;
          break;
        }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  // ---- phase 2: sum over ranks, residual, norm
  float h[kTpMaxIters][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < kTpMaxIters; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      const long long off = row * hidden + (long long)v * 8;
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 r[kMaxPeers];
#pragma unroll
      for (int u = 0; u < kMaxPeers; ++u)
        r[u] = u < n ? __ldcg(reinterpret_cast<const uint4*>(slots + u * slot_stride + off)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < kMaxPeers; ++u) {
        const uint32_t rw[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(rw[e]);
          a[2 * e] += f.x;
          a[2 * e + 1] += f.y;
        }
      }
      if (residual_in) {
        const uint4 q = *reinterpret_cast<const uint4*>(residual_in + off);
        const uint32_t rw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(rw[e]);
          a[2 * e] += f.x;
          a[2 * e + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
      o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
      if (residual_out) *reinterpret_cast<uint4*>(residual_out + off) = o;
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
  if (w) {
    ss = warp_sum(ss);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    const float inv = rsqrtf(t / float(hidden) + eps);
#pragma unroll
    for (int it = 0; it < kTpMaxIters; ++it) {
      const int v = threadIdx.x + it * blockDim.x;
      if (v < nvec) {
        const long long off = row * hidden + (long long)v * 8;
        const uint4 wr = *reinterpret_cast<const uint4*>(w + (long long)v * 8);
        const uint32_t ww[4] = {wr.x, wr.y, wr.z, wr.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(ww[e]);
          o[e] = pack_bf16x2(h[it][2 * e] * inv * f.x, h[it][2 * e + 1] * inv * f.y);
        }
        *reinterpret_cast<uint4*>(normed_out + off) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(done_counter, 1u);
    if (old == gridDim.x - 1) {
      *done_counter = 0u;
      if (ok_flag) atomicAdd(seen, 1u);
      __threadfence();
    }
  }
}

// MoE combine fused with the push half of the all-reduce: out[t] = sum_j w[t, j] * y_sorted[pair_pos[t, j]]
// over the pairs handled by this rank's experts, stored as a bf16 partial row into slot [rank] of every
// peer's partial array (rows without local pairs are stored as zeros: the consumer sums all slots).
// The last CTA signals every peer exactly like the GEMM push epilogue does.
__global__ void moe_combine_push_kernel(const __nv_bfloat16* __restrict__ y_sorted, const int* __restrict__ pair_pos,
                                        const float* __restrict__ weights, int tokens, int top_k, int hidden,
                                        const PushArgs push) {
  griddep_wait();
  griddep_launch();
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int pos = pair_pos[t * top_k + j];
      if (pos < 0) continue;
      const float w = weights[t * top_k + j];
      const uint4 r = *reinterpret_cast<const uint4*>(y_sorted + (long long)pos * hidden + v * 8);
      const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(rw[e]);
        acc[2 * e] += w * f.x;
        acc[2 * e + 1] += w * f.y;
      }
    }
    const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                               pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    const long long off = ((long long)push.rank * tokens + t) * hidden + v * 8;
    push_store_16(push, off, o);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // release at GPU scope into the grid counter; the last CTA has observed every other CTA's release and
    // publishes all of them with one system-scope fence before it bumps the peers' flags
    __threadfence();
    const unsigned int old = atomicAdd(push.done_counter, 1u);
    if (old == gridDim.x - 1) {
      *push.done_counter = 0u;
      __threadfence_system();
      push_signal(push);
    }
  }
}

// Cross-rank arg-max of a vocabulary-parallel head in one launch of one CTA: every rank stores its
// (value, global id) pair per row into all peers' pair arrays [2][n_peers][max_rows] (the half is chosen
// by the parity of `seen`, which all ranks advance in step), bumps its arrival counter on every peer,
// waits (bounded) for all counters and picks the best pair per row (the lowest rank wins ties, i.e. the
// lowest vocabulary index).  Replaces an all-gather plus a handful of tiny kernels
// (examples/models/qwen3/kernels/sampling.py:130-135 in the reference gathers values and ids).
struct ArgmaxPeers {
  float2* pairs[kMaxPeers];
  unsigned int* flag[kMaxPeers];   // this rank's counter inside each peer's flag array
};
__global__ void argmax_exchange_kernel(const float* __restrict__ vals, const int* __restrict__ ids, int rows,
                                       int max_rows, int id_offset, int rank, int n_peers, const ArgmaxPeers peers,
                                       const float2* __restrict__ local_pairs, const unsigned int* __restrict__ flags,
                                       unsigned int* __restrict__ seen, int* __restrict__ out_ids,
                                       int* __restrict__ status) {
  __shared__ int ok_flag;
  griddep_wait();
  griddep_launch();
  const unsigned int use = *reinterpret_cast<volatile unsigned int*>(seen);
  const long long half = (long long)(use & 1u) * n_peers * max_rows;
  for (int i = threadIdx.x; i < rows * n_peers; i += blockDim.x) {
    const int pr = i / rows, r = i - pr * rows;
    peers.pairs[pr][half + (long long)rank * max_rows + r] = make_float2(vals[r], __int_as_float(ids[r] + id_offset));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int pr = 0; pr < n_peers; ++pr) atomicAdd_system(peers.flag[pr], 1u);
    int ok = 1;
    const unsigned long long t0 = globaltimer_ns();
    for (int s = 0; s < n_peers && ok; ++s) {
      unsigned int spins = 0;
      while (int(ld_acquire_sys(flags + s) - (use + 1u)) < 0) {
        if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
          atomicCAS(status, 0, ERR_WAIT_PEER_FLAG | (s << 8));
          ok = 0;
          break;
        }
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  if (ok_flag) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      float best = -INFINITY;
      int best_id = 0;
      for (int s = 0; s < n_peers; ++s) {
        const float2 p = __ldcg(local_pairs + half + (long long)s * max_rows + r);
        if (s == 0 || p.x > best) {
          best = p.x;
          best_id = __float_as_int(p.y);
        }
      }
      out_ids[r] = best_id;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && ok_flag) {
    __threadfence();
    *seen = use + 1u;
  }
}

}  // namespace nkb

using namespace nkb;

// ---- symmetric memory over CUDA IPC (host side) ----------------------------------
extern "C" int nkb_symm_alloc(void** out, long long bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaMemset(p, 0, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaDeviceSynchronize();
  *out = p;
  return int(e);
}
extern "C" int nkb_symm_free(void* p) { return int(cudaFree(p)); }
// handle_out must have room for 64 bytes
extern "C" int nkb_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return int(e);
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int nkb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return int(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int nkb_ipc_close(void* p) { return int(cudaIpcCloseMemHandle(p)); }

extern "C" int nkb_tp_reduce_rmsnorm(const void* partials, int slots, const void* flags, int n_src, void* seen,
                                     void* done_counter, const void* residual_in, const void* w, void* residual_out,
                                     void* normed_out, int rows, int hidden, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (hidden & 7) return -2;
  const int nvec = hidden >> 3;
  if (nvec > 1024 * kTpMaxIters) return -2;
  int threads = nvec <= 1024 ? (nvec + 31) / 32 * 32 : ((nvec + kTpMaxIters - 1) / kTpMaxIters + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (!status_word() && nkb_init() != 0) return -1;
  return launch_pdl(tp_reduce_rmsnorm_kernel, dim3(rows), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
                    (const __nv_bfloat16*)partials, slots, (const unsigned int*)flags, n_src, (unsigned int*)seen,
                    (unsigned int*)done_counter, (const __nv_bfloat16*)residual_in, (const __nv_bfloat16*)w,
                    (__nv_bfloat16*)residual_out, (__nv_bfloat16*)normed_out, rows, hidden, eps, status_word());
}

// partials [splits][rows][hidden] fp32 (or y [rows][hidden] bf16 when partials is null): this rank's output
// of the row-parallel GEMM.  peer_slots[r] / peer_rowflags[r]: slot array and row counters of rank r for this
// buffer; local_*: this rank's own.  rows <= 128.
extern "C" int nkb_tp_exchange_reduce_rmsnorm(const float* partials, int splits, long long split_stride, const void* y,
                                              void* const* peer_slots, void* const* peer_rowflags, void* mc_slots,
                                              void* mc_rowflags, int n_peers, int rank, const void* local_slots,
                                              const void* local_rowflags, void* seen, void* done_counter,
                                              const void* residual_in, const void* w, void* residual_out,
                                              void* normed_out, int rows, int hidden, float eps, void* stream) {
  if (rows <= 0) return 0;
  if ((hidden & 7) || rows > kRowFlags || n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return -2;
  if ((!partials && !y) || (partials && splits < 1) || (w && !normed_out)) return -2;
  const int nvec = hidden >> 3;
  if (nvec > 512 * kTpMaxIters) return -2;
  int threads = nvec <= 512 ? (nvec + 31) / 32 * 32 : ((nvec + kTpMaxIters - 1) / kTpMaxIters + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  if (!status_word() && nkb_init() != 0) return -1;
  PushArgs pa{};
  pa.n_peers = n_peers;
  pa.rank = rank;
  for (int i = 0; i < n_peers; ++i) {
    pa.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(peer_slots[i]);
    pa.peer_flag[i] = reinterpret_cast<unsigned int*>(peer_rowflags[i]);
  }
  pa.mc_out = reinterpret_cast<__nv_bfloat16*>(mc_slots);
  pa.mc_flag = reinterpret_cast<unsigned int*>(mc_rowflags);
  return launch_pdl(tp_exchange_reduce_rmsnorm_kernel, dim3(rows), dim3(threads), 0,
                    reinterpret_cast<cudaStream_t>(stream), partials, splits, split_stride,
                    (const __nv_bfloat16*)y, pa, (const __nv_bfloat16*)local_slots,
                    (const unsigned int*)local_rowflags, (unsigned int*)seen, (unsigned int*)done_counter,
                    (const __nv_bfloat16*)residual_in, (const __nv_bfloat16*)w, (__nv_bfloat16*)residual_out,
                    (__nv_bfloat16*)normed_out, rows, hidden, eps, status_word());
}

// y_sorted [pairs, hidden] bf16, pair_pos [tokens * top_k], weights [tokens, top_k] fp32.  peer_out[r] is
// rank r's partial array [n_peers, tokens, hidden] bf16, peer_flag[r] this rank's counter on rank r.
extern "C" int nkb_moe_combine_push(const void* y_sorted, const int* pair_pos, const float* weights, int tokens,
                                    int top_k, int hidden, void* const* peer_out, void* const* peer_flag, int n_peers,
                                    int rank, void* done_counter, void* mc_out, void* mc_flag, void* stream) {
  if (tokens <= 0) return 0;
  if ((hidden & 7) || n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
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
  return launch_pdl(moe_combine_push_kernel, dim3(tokens), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                    (const __nv_bfloat16*)y_sorted, pair_pos, weights, tokens, top_k, hidden, pa);
}

// vals / ids [rows]: this rank's per-row maximum and local index; id_offset is added to make the index
// global.  peer_pairs[r]: rank r's pair array (2 * n_peers * max_rows float2), peer_flag[r]: this rank's
// counter on rank r; local_pairs / local_flags: this rank's own arrays; seen: device counter of completed
// exchanges (selects the half of the pair array).
extern "C" int nkb_argmax_exchange(const float* vals, const int* ids, int rows, int max_rows, int id_offset,
                                   void* const* peer_pairs, void* const* peer_flag, int n_peers, int rank,
                                   const void* local_pairs, const void* local_flags, void* seen, int* out_ids,
                                   void* stream) {
  if (rows <= 0) return 0;
  if (rows > max_rows || n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return -2;
  if (!status_word() && nkb_init() != 0) return -1;
  ArgmaxPeers ap{};
  for (int i = 0; i < n_peers; ++i) {
    ap.pairs[i] = reinterpret_cast<float2*>(peer_pairs[i]);
    ap.flag[i] = reinterpret_cast<unsigned int*>(peer_flag[i]);
  }
  return launch_pdl(argmax_exchange_kernel, dim3(1), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), vals, ids,
                    rows, max_rows, id_offset, rank, n_peers, ap, (const float2*)local_pairs,
                    (const unsigned int*)local_flags, (unsigned int*)seen, out_ids, status_word());
}
