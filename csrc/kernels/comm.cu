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
      for (int s = 0; s < slots; ++s) {
        // remote ranks wrote these lines: read them from L2, never from a stale L1 line
        const uint4 r = __ldcg(reinterpret_cast<const uint4*>(partials + (long long)s * rows * hidden + off));
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(rw[e]);
          a[2 * e] += f.x;
          a[2 * e + 1] += f.y;
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
