// Blockwise (flash) prefill attention on tcgen05 for sm_100a, reading K/V from
// the paged cache through the per-sequence block table.
//
// One CTA per (128-row query tile, query head, sequence):
//   warp 0   TMA producer: Q tile once, then a 2-stage ring of 128-token K and V
//            tiles (four 32-token pages each, 128-byte swizzle, non-multicast)
//   warp 1   issues tcgen05.mma:  S = Q K^T  (M=128, N=128, fp32 in TMEM, two S
//            buffers so QK^T of tile j+1 overlaps the softmax of tile j), then
//            O_tile = P V with V as an MN-major B operand
//   warps 2-5 one thread per query row: online softmax straight out of TMEM
//            (row max / sum need no cross-thread reduction), P written to shared
//            memory in the swizzled K-major layout the MMA reads, O accumulated
//            in registers.
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

constexpr int kQTile = 128;
constexpr int kKVTile = 128;
constexpr int kPfPage = 32;
constexpr int kPfThreads = 192;

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
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, o_full, o_empty;
  uint32_t tmem_base;
  int abort;
};

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
flash_attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const PrefillParams p) {
  constexpr int NH = D / 64;
  constexpr int kHalf = 128 * 128;          // [128 rows][64 bf16] swizzled slab = 16 KB
  constexpr int kQBytes = NH * kHalf;
  constexpr int kKVBytes = NH * kHalf;
  constexpr int kPBytes = 2 * kHalf;        // [128 rows][128 tokens]
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSCol0 = 0, kSCol1 = 128, kOCol = 256;

  const int qt = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  griddep_wait();
  griddep_launch();
  const int q_len = p.q_lens[b];
  if (qt * kQTile >= q_len) return;
  const int ctx = p.context_lens[b];
  const int q_row0 = p.q_start[b] + qt * kQTile;        // row in the packed q / out arrays
  const int pos0 = ctx - q_len + qt * kQTile;           // kv position of the tile's first query
  const int rows_here = min(kQTile, q_len - qt * kQTile);
  const int kvh = head / (p.nq / p.nkv);

  // kv tile range
  int j_hi = (ctx + kKVTile - 1) / kKVTile;
  if (p.causal) j_hi = min(j_hi, (pos0 + rows_here - 1) / kKVTile + 1);
  int j_lo = 0;
  if (p.window > 0) j_lo = max(0, pos0 - p.window + 1) / kKVTile;
  const int n_tiles = j_hi - j_lo;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + kQBytes;              // 2 stages
  uint8_t* v_s = k_s + 2 * kKVBytes;         // 2 stages
  uint8_t* p_s = v_s + 2 * kKVBytes;
  PrefillCtrl* ctrl = reinterpret_cast<PrefillCtrl*>(p_s + kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(&ctrl->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctrl->k_full[i], 1);
      mbar_init(&ctrl->k_empty[i], 1);
      mbar_init(&ctrl->v_full[i], 1);
      mbar_init(&ctrl->v_empty[i], 1);
      mbar_init(&ctrl->s_full[i], 1);
      mbar_init(&ctrl->s_empty[i], 4);
    }
    mbar_init(&ctrl->p_full, 4);
    mbar_init(&ctrl->o_full, 1);
    mbar_init(&ctrl->o_empty, 4);
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
      mbar_expect_tx(&ctrl->q_full, kQBytes);
#pragma unroll
      for (int h = 0; h < NH; ++h) tma_load_3d(q_s + h * kHalf, &tmQ, &ctrl->q_full, h * 64, head, q_row0);
    }
    __syncwarp();
    const int* table = p.block_table + (long long)b * p.max_blocks;
    const int last_page = max((ctx + kPfPage - 1) / kPfPage - 1, 0);
    for (int it = 0; it < n_tiles; ++it) {
      const int j = j_lo + it;
      const int st = it & 1;
      const uint32_t ph = (uint32_t(it) >> 1) & 1u;
      bool ok = mbar_wait(&ctrl->k_empty[st], ph ^ 1u, abort_flag, p.status, ERR_WAIT_SMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) break;
      int blk[4];
#pragma unroll
      for (int pi = 0; pi < 4; ++pi) blk[pi] = table[min(j * 4 + pi, last_page)];
      if (lane == 0) {
        mbar_expect_tx(&ctrl->k_full[st], kKVBytes);
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_4d(k_s + st * kKVBytes + h * kHalf + pi * (kPfPage * 128), &tmK, &ctrl->k_full[st], h * 64, 0,
                        kvh, blk[pi]);
      }
      __syncwarp();
      ok = mbar_wait(&ctrl->v_empty[st], ph ^ 1u, abort_flag, p.status, ERR_WAIT_SMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) break;
      if (lane == 0) {
        mbar_expect_tx(&ctrl->v_full[st], kKVBytes);
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma_load_4d(v_s + st * kKVBytes + h * kHalf + pi * (kPfPage * 128), &tmV, &ctrl->v_full[st], h * 64, 0,
                        kvh, blk[pi]);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, kKVTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);  // B = V is MN-major
    bool alive = true;
    bool ok = mbar_wait(&ctrl->q_full, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
    if (!__all_sync(0xffffffffu, ok)) alive = false;
    auto issue_qk = [&](int it) -> bool {
      const int st = it & 1;
      const uint32_t ph = (uint32_t(it) >> 1) & 1u;
      bool ok2 = mbar_wait(&ctrl->k_full[st], ph, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      if (!__all_sync(0xffffffffu, ok2)) return false;
      ok2 = mbar_wait(&ctrl->s_empty[st], ph ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok2)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + st * kKVBytes);
        const uint32_t d = tmem_base + (st ? kSCol1 : kSCol0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 32;
          umma_f16(d, make_smem_desc_sw128(qa + off, 0, 1024), make_smem_desc_sw128(ka + off, 0, 1024), idesc_qk,
                   ks > 0 ? 1u : 0u);
        }
        umma_commit(&ctrl->s_full[st]);
        umma_commit(&ctrl->k_empty[st]);
      }
      __syncwarp();
      return true;
    };
    if (alive && n_tiles > 0) alive = issue_qk(0);
    for (int it = 0; it < n_tiles && alive; ++it) {
      if (it + 1 < n_tiles) {
        alive = issue_qk(it + 1);
        if (!alive) break;
      }
      const int st = it & 1;
      const uint32_t ph = (uint32_t(it) >> 1) & 1u;
      ok = mbar_wait(&ctrl->p_full, uint32_t(it) & 1u, abort_flag, p.status, ERR_WAIT_SOFTMAX);
      if (!__all_sync(0xffffffffu, ok)) break;
      ok = mbar_wait(&ctrl->v_full[st], ph, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) break;
      ok = mbar_wait(&ctrl->o_empty, (uint32_t(it) & 1u) ^ 1u, abort_flag, p.status, ERR_WAIT_TMEM_EMPTY);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(p_s), va = smem_u32(v_s + st * kKVBytes);
        const uint32_t d = tmem_base + kOCol;
#pragma unroll
        for (int ks = 0; ks < kKVTile / 16; ++ks) {
          const uint64_t da = make_smem_desc_sw128(pa + (ks >> 2) * kHalf + (ks & 3) * 32, 0, 1024);
          // V tile: [token][64 dims] rows of 128 B; 16 tokens per step = 2 KB; next 64 dims one slab on
          const uint64_t db = make_smem_desc_sw128(va + ks * 2048, kHalf, 1024);
          umma_f16(d, da, db, idesc_pv, ks > 0 ? 1u : 0u);
        }
        umma_commit(&ctrl->o_full);
        umma_commit(&ctrl->v_empty[st]);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- softmax / accumulate
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // row of the query tile
    const int q_pos = pos0 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    int hi_pos = ctx - 1;
    if (p.causal) hi_pos = min(hi_pos, q_pos);
    const int lo_pos = p.window > 0 ? q_pos - p.window + 1 : 0;
    bool alive = true;

    auto accumulate_o = [&](float alpha) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + kOCol + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
    };

    for (int it = 0; it < n_tiles; ++it) {
      const int j = j_lo + it;
      const int st = it & 1;
      const uint32_t ph = (uint32_t(it) >> 1) & 1u;
      bool ok = mbar_wait(&ctrl->s_full[st], ph, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_off + (st ? kSCol1 : kSCol0);
      const int kv0 = j * kKVTile;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kKVTile / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + c * 32 + i;
          const float x = (kv <= hi_pos && kv >= lo_pos) ? __uint_as_float(v[i]) * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m - base);
      m = m_new;
      // previous tile's P.V result: fold into the register accumulator, free P and the O tile
      if (it > 0) {
        ok = mbar_wait(&ctrl->o_full, uint32_t(it - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        tc_fence_after();
        accumulate_o(alpha_prev);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctrl->o_empty);
      }
      alpha_prev = alpha;
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < kKVTile / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int kv = kv0 + c * 32 + i;
          const float x0 = (kv <= hi_pos && kv >= lo_pos) ? __uint_as_float(v[i]) * p.scale_log2 : -INFINITY;
          const float x1 =
              (kv + 1 <= hi_pos && kv + 1 >= lo_pos) ? __uint_as_float(v[i + 1]) * p.scale_log2 : -INFINITY;
          const float e0 = exp2f(x0 - base), e1 = exp2f(x1 - base);
          // the row sum uses the rounded values the MMA will see
          const uint32_t pr = pack_bf16x2(e0, e1);
          const float2 back = unpack_bf16x2(pr);
          sum += back.x + back.y;
          pk[i >> 1] = pr;
        }
        // 32 tokens = four 16-byte chunks; chunk index within the 128-token row = c*4 + q
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q;
          uint8_t* dst = p_s + (chunk >> 3) * kHalf + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      l = l * alpha + sum;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&ctrl->p_full);
        mbar_arrive(&ctrl->s_empty[st]);
      }
    }
    if (alive && n_tiles > 0) {
      bool ok = mbar_wait(&ctrl->o_full, uint32_t(n_tiles - 1) & 1u, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
      if (__all_sync(0xffffffffu, ok)) {
        tc_fence_after();
        accumulate_o(alpha_prev);
      }
    }
    if (p.sinks) {
      const float sk = p.sinks[head] * 1.4426950408889634f;
      const float m2 = fmaxf(m, sk);
      const float sc = (m == -INFINITY) ? 0.f : exp2f(m - m2);
      l = l * sc + exp2f(sk - m2);
#pragma unroll
      for (int i = 0; i < D; ++i) o_acc[i] *= sc;
    }
    if (r < rows_here && !*abort_flag) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((long long)(q_row0 + r) * p.nq + head) * D;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        uint4 o;
        o.x = pack_bf16x2(o_acc[i] * inv, o_acc[i + 1] * inv);
        o.y = pack_bf16x2(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
        o.z = pack_bf16x2(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
        o.w = pack_bf16x2(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
        *reinterpret_cast<uint4*>(dst + i) = o;
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
  constexpr int smem = NH * 16384 * 5 + 2 * 16384 + int(sizeof(PrefillCtrl)) + 1024 + 64;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(flash_attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    attr_set = true;
  }
  dim3 grid((max_q_len + kQTile - 1) / kQTile, p.nq, batch);
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
