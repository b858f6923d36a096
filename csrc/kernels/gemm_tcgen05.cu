// Host launchers of the tcgen05 GEMM (device code in gemm_tcgen05.cuh).
#include "gemm_tcgen05.cuh"
#include "api.h"
#include <cstdlib>

namespace nkb {

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// ctas_per_sm = 2 caps the ring so that two CTAs (of this or of the next GEMM in
// the stream, started early by programmatic dependent launch) fit on one SM: the
// successor then prefetches its weight tiles while this kernel drains.
template <int BN, int MINB, bool PUSH, bool GROUPED>
static int ring_stages(const GemmArgs& args, int& smem, bool lean = false) {
  const int a_tiles = args.gated == 1 ? 2 : 1, b_tiles = args.gated == 2 ? 2 : 1;
  const int stage_bytes = a_tiles * kATileBytes + b_tiles * BN * kBlockK * 2;
  // control block + staging: the push tile (32 tokens x 128 features bf16), or the compact epilogue's two
  // 16-column buffers of fp32
  const int extra = 512 + (PUSH ? 32 * kTileRows * 2 : (lean ? 2 * 16 * kTileRows * 4 : 0));
  const int budget = (MINB == 2 ? 113 * 1024 : 232448) - 1024 - extra - 64;
  int stages = budget / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  static_assert(sizeof(GemmCtrl) <= 512, "control block grew");
  smem = stages * stage_bytes + 1024 + extra + 64;
  return stages;
}

// The decode orientation (transposed output, bias per row or none) runs the kernel with the compact epilogue.
static bool lean_ok(const GemmArgs& a) {
  static const bool off = getenv("NKIPY_B200_GENERAL_EPILOGUE") != nullptr;
  return !off && a.transpose_out && (!a.bias || a.bias_on_rows);
}

// transpose_out = 2 tells the compact epilogue that every token row of the output may go out as one bulk
// copy: base, leading dimension, split stride and row count all on 16-byte boundaries.
void mark_bulk(GemmArgs& a) {
  // measured slower than plain stores for these 16-column chunks (sixteen 512-byte copies per chunk keep the
  // copy engine busy for 1.7 us): opt-in only
  static const bool on = getenv("NKIPY_B200_BULK_EPILOGUE") != nullptr;
  if (!a.transpose_out || !on) return;
  const long long esz = (a.out_fp32 && !a.gated) ? 4 : 2;
  const bool ok = (reinterpret_cast<uintptr_t>(a.out) % 16 == 0) && (a.ldo * esz) % 16 == 0 &&
                  (a.rows * esz) % 16 == 0 && (a.split_stride * 4) % 16 == 0;
  a.transpose_out = ok ? 2 : 1;
}

template <int BN, int MINB, bool PUSH = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs& args, int max_ctas,
                       cudaStream_t stream, const PushArgs* push = nullptr) {
  int smem = 0;
  const bool lean = BN <= 128 && lean_ok(args);
  if (lean && !PUSH) mark_bulk(args);
  args.stages = ring_stages<BN, MINB, PUSH, false>(args, smem, lean);
  if (args.stages < 2) return -3;
  auto kernel = lean ? gemm_bf16_lean_kernel<(BN <= 128 ? BN : 128), MINB, PUSH> : gemm_bf16_kernel<BN, MINB, PUSH>;
  static bool attr_set[2] = {false, false};
  if (!attr_set[lean]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         MINB == 2 ? 113 * 1024 : 232448);
    if (e != cudaSuccess) return int(e);
    attr_set[lean] = true;
  }
  const int total = args.num_row_tiles * args.num_col_tiles * args.splits;
  const int grid = total < max_ctas ? total : max_ctas;
  PushArgs pa{};
  if (push) pa = *push;
  return launch_pdl(kernel, dim3(grid), dim3(kGemmThreads), size_t(smem), stream, ta, tb, args, pa);
}

// Split-K with the fix-up epilogue (splitk_fix.cuh), decode orientation, two CTAs per SM.
template <int BN, class Fix>
static int launch_fix(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs& args, const typename Fix::Args& fix,
                      cudaStream_t stream) {
  const int stage_bytes = kATileBytes + BN * kBlockK * 2;
  const int extra = 1024 + (Fix::kind == FIX_PUSH ? 32 * kTileRows * 2 : 0);   // control + reduction scratch (+ staging)
  const int budget = 113 * 1024 - 1024 - extra - 64;
  int stages = budget / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return -3;
  args.stages = stages;
  const int smem = stages * stage_bytes + 1024 + extra + 64;
  auto kernel = gemm_bf16_fix_kernel<BN, 2, Fix>;
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 113 * 1024);
    if (e != cudaSuccess) return int(e);
    attr_set[dev] = true;
  }
  const int total = args.num_row_tiles * args.splits;
  const int cap = 2 * num_sms();
  const int grid = total < cap ? total : cap;
  return launch_pdl(kernel, dim3(grid), dim3(kGemmThreads), size_t(smem), stream, ta, tb, args, fix);
}

// Common argument set-up of the fix-up launches: weights [rows, k] on the MMA row side, x [tokens, k].
static int fix_setup(GemmArgs& args, FixCommon& c, CUtensorMap& ta, CUtensorMap& tb, const void* w, const void* x,
                     int rows, int tokens, int k, long long ldw, long long ldx, int splits, int block_n,
                     float* partials, unsigned int* counters, const void* bias) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (rows <= 0 || tokens <= 0 || k <= 0 || (k & 7) || (ldw & 7) || (ldx & 7)) return -2;
  if (tokens > block_n || !partials || !counters) return -2;
  if (block_n != 32 && block_n != 64 && block_n != 128) return -2;
  args = GemmArgs{};
  args.rows = rows;
  args.cols = tokens;
  args.k = k;
  args.kb_total = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > args.kb_total) splits = args.kb_total;
  args.kb_per_split = (args.kb_total + splits - 1) / splits;
  args.splits = (args.kb_total + args.kb_per_split - 1) / args.kb_per_split;
  args.num_row_tiles = (rows + kTileRows - 1) / kTileRows;
  args.num_col_tiles = 1;
  args.transpose_out = 1;
  args.out_fp32 = 1;
  args.ldo = rows;
  args.split_stride = (long long)tokens * rows;
  args.out = partials;
  args.status = status_word();
  args.weights_operand = 0;
  c.partials = partials;
  c.tile_counters = counters;
  c.ld = rows;
  c.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  if (encode_tmap_bf16_2d(&ta, w, k, rows, ldw, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  return 0;
}

#define NKB_FIX_DISPATCH(FixT, fixargs)                                                   \
  switch (block_n) {                                                                      \
    case 32: return launch_fix<32, FixT>(ta, tb, args, fixargs, s);                       \
    case 64: return launch_fix<64, FixT>(ta, tb, args, fixargs, s);                       \
    default: return launch_fix<128, FixT>(ta, tb, args, fixargs, s);                      \
  }

template <int BN, int MINB>
static int launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs& args, const GroupArgs& grp,
                          int max_ctas, cudaStream_t stream) {
  int smem = 0;
  args.stages = ring_stages<BN, MINB, false, true>(args, smem);
  if (args.stages < 2) return -3;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_grouped_kernel<BN, MINB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, MINB == 2 ? 113 * 1024 : 232448);
    if (e != cudaSuccess) return int(e);
    attr_set = true;
  }
  const int total = grp.num_groups * args.num_row_tiles * grp.max_col_tiles;
  const int grid = total < max_ctas ? total : max_ctas;
  return launch_pdl(gemm_bf16_grouped_kernel<BN, MINB>, dim3(grid), dim3(kGemmThreads), size_t(smem), stream, ta, tb,
                    args, grp);
}

}  // namespace nkb

using namespace nkb;

// D[rows, cols] = A[rows(+gate), k] * B[cols(+gate), k]^T with the fusions described above.
//   transpose_out: element (r, c) is stored at out[c * ldo + r] instead of out[r * ldo + c]
//   out_fp32 + splits > 1: partial sums go to out[s * split_stride + ...] as fp32
extern "C" int nkb_gemm_bf16(const void* A, const void* B, void* out, int rows, int cols, int k, long long lda,
                             long long ldb, long long ldo, int transpose_out, int out_fp32, int splits,
                             long long split_stride, int gated, int gate_off, const void* bias, int bias_on_rows,
                             const void* residual, int block_n, int max_ctas, int weights_operand, int ctas_per_sm, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (rows <= 0 || cols <= 0 || k <= 0) return -2;
  if ((k & 7) || (lda & 7) || (ldb & 7)) return -2;
  if (splits > 1 && !out_fp32) return -2;
  if (gated && (splits > 1 || out_fp32)) return -2;
  if (gated && block_n > 128) return -2;
  GemmArgs args{};
  args.rows = rows;
  args.cols = cols;
  args.k = k;
  args.kb_total = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > args.kb_total) splits = args.kb_total;
  args.kb_per_split = (args.kb_total + splits - 1) / splits;
  args.splits = (args.kb_total + args.kb_per_split - 1) / args.kb_per_split;
  args.num_row_tiles = (rows + kTileRows - 1) / kTileRows;
  args.num_col_tiles = (cols + block_n - 1) / block_n;
  args.gated = gated;
  args.gate_off = gate_off;
  args.transpose_out = transpose_out;
  args.out_fp32 = out_fp32;
  args.bias_on_rows = bias_on_rows;
  args.ldo = ldo;
  args.split_stride = split_stride;
  args.out = out;
  args.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  args.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  args.status = status_word();
  args.weights_operand = weights_operand;
  const int cap = num_sms() * (ctas_per_sm == 2 ? 2 : 1);
  if (max_ctas <= 0 || max_ctas > cap) max_ctas = cap;

  CUtensorMap ta, tb;
  const uint64_t a_rows = gated == 1 ? uint64_t(gate_off) + rows : rows;
  const uint64_t b_rows = gated == 2 ? uint64_t(gate_off) + cols : cols;
  if (encode_tmap_bf16_2d(&ta, A, k, a_rows, lda, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, B, k, b_rows, ldb, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (ctas_per_sm == 2 && block_n <= 128 && !(gated && block_n > 64)) {
    switch (block_n) {
      case 32: return launch_gemm<32, 2>(ta, tb, args, max_ctas, s);
      case 64: return launch_gemm<64, 2>(ta, tb, args, max_ctas, s);
      case 128: return launch_gemm<128, 2>(ta, tb, args, max_ctas, s);
      default: return -2;
    }
  }
  if (max_ctas > num_sms()) max_ctas = num_sms();
  switch (block_n) {
    case 32: return launch_gemm<32, 1>(ta, tb, args, max_ctas, s);
    case 64: return launch_gemm<64, 1>(ta, tb, args, max_ctas, s);
    case 128: return launch_gemm<128, 1>(ta, tb, args, max_ctas, s);
    case 256: return launch_gemm<256, 1>(ta, tb, args, max_ctas, s);
    default: return -2;
  }
}

// Reports the number of split partials the launcher will really produce for a
// requested split count (k-blocks are distributed in whole 64-wide slabs).
extern "C" int nkb_gemm_effective_splits(int k, int splits) {
  int kb_total = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  int per = (kb_total + splits - 1) / splits;
  return (kb_total + per - 1) / per;
}


// Decode-orientation GEMM whose epilogue pushes bf16 partial tiles into every peer's
// symmetric partial buffer (see PushArgs).  weights [features, k], x [tokens, k]; the
// destination on every peer is [n_peers * splits, tokens, ldo] bf16.
extern "C" int nkb_gemm_bf16_push(const void* weights, const void* x, int features, int tokens, int k, long long ldw,
                                  long long ldx, long long ldo, int splits, const void* bias, int block_n,
                                  void* const* peer_out, void* const* peer_flag, int n_peers, int rank,
                                  void* done_counter, void* mc_out, void* mc_flag, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (features <= 0 || tokens <= 0 || k <= 0 || (k & 7) || (ldw & 7) || (ldx & 7) || (ldo & 7) || (features & 7))
    return -2;
  if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers || tokens > block_n) return -2;
  GemmArgs args{};
  args.rows = features;
  args.cols = tokens;
  args.k = k;
  args.kb_total = (k + kBlockK - 1) / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > args.kb_total) splits = args.kb_total;
  args.kb_per_split = (args.kb_total + splits - 1) / splits;
  args.splits = (args.kb_total + args.kb_per_split - 1) / args.kb_per_split;
  args.num_row_tiles = (features + kTileRows - 1) / kTileRows;
  args.num_col_tiles = 1;
  args.transpose_out = 1;
  args.bias_on_rows = 1;
  args.ldo = ldo;
  args.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  args.status = status_word();
  args.weights_operand = 0;
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
  if (encode_tmap_bf16_2d(&ta, weights, k, features, ldw, kBlockK, kTileRows)) return -4;
  if (encode_tmap_bf16_2d(&tb, x, k, tokens, ldx, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int max_ctas = 2 * num_sms();
  switch (block_n) {
    case 32: return launch_gemm<32, 2, true>(ta, tb, args, max_ctas, s, &pa);
    case 64: return launch_gemm<64, 2, true>(ta, tb, args, max_ctas, s, &pa);
    case 128: return launch_gemm<128, 2, true>(ta, tb, args, max_ctas, s, &pa);
    default: return -2;
  }
}

// Grouped (per-expert) GEMM in the decode orientation:
//   out[r, f] = sum_k x_sorted[r, k] * weights[g(r), f, k]     for the rows r of group g,
// rows sorted by group, group g = rows [group_offsets[g], group_offsets[g + 1]).
// gated: weights hold [gate; up] per group (2 * features rows, up half at gate_off) and the
// epilogue applies the (optionally clamped) SwiGLU.  bias: [groups, bias_group_stride].
extern "C" int nkb_gemm_bf16_grouped(const void* weights, const void* x_sorted, void* out, const int* group_offsets,
                                     int num_groups, int features, int k, int total_rows, int max_rows_per_group,
                                     long long ldx, long long ldo, int gated, int gate_off, const void* bias,
                                     long long bias_group_stride, float act_limit, float act_alpha, int block_n,
                                     const int* tile_list, const int* tile_count, int max_tiles, const void* arrive,
                                     unsigned int arrive_target, void* stream) {
  if (!status_word() && nkb_init() != 0) return -1;
  if (num_groups <= 0 || features <= 0 || k <= 0 || total_rows <= 0) return 0;
  if ((k & 7) || (ldx & 7)) return -2;
  if (gated && block_n > 64) return -2;
  GemmArgs args{};
  args.rows = features;
  args.cols = total_rows;
  args.k = k;
  args.kb_total = (k + kBlockK - 1) / kBlockK;
  args.splits = 1;
  args.kb_per_split = args.kb_total;
  args.num_row_tiles = (features + kTileRows - 1) / kTileRows;
  args.num_col_tiles = 1;
  args.gated = gated ? 1 : 0;
  args.gate_off = gate_off;
  args.transpose_out = 1;
  args.bias_on_rows = 1;
  args.ldo = ldo;
  args.out = out;
  args.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  GroupArgs grp{};
  grp.bias_group_stride = bias_group_stride;
  args.status = status_word();
  args.weights_operand = -1;
  grp.num_groups = num_groups;
  grp.max_col_tiles = (max_rows_per_group + block_n - 1) / block_n;
  if (grp.max_col_tiles < 1) grp.max_col_tiles = 1;
  grp.group_offsets = group_offsets;
  if (tile_list && tile_count && max_tiles > 0) {
    grp.tile_list = tile_list;
    grp.tile_count = tile_count;
    // work items = tiles x row tiles; express the bound through max_col_tiles for the grid size
    grp.max_col_tiles = (max_tiles + num_groups - 1) / num_groups;
  }
  grp.act_limit = act_limit;
  grp.act_alpha = act_alpha;
  grp.arrive = reinterpret_cast<const unsigned int*>(arrive);
  grp.arrive_target = arrive_target;
  const long long rows_per_group = gated ? (long long)gate_off + features : features;
  CUtensorMap ta, tb;
  {
    const uint64_t dims[3] = {uint64_t(k), uint64_t(rows_per_group), uint64_t(num_groups)};
    const uint64_t strides[2] = {uint64_t(k) * 2, uint64_t(k) * 2 * uint64_t(rows_per_group)};
    const uint32_t box[3] = {kBlockK, kTileRows, 1};
    if (encode_tmap_bf16(&ta, weights, 3, dims, strides, box)) return -4;
  }
  if (encode_tmap_bf16_2d(&tb, x_sorted, k, total_rows, ldx, kBlockK, block_n)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int max_ctas = 2 * num_sms();
  const bool two = !gated || block_n <= 32;
  switch (block_n) {
    case 32:
      return two ? launch_grouped<32, 2>(ta, tb, args, grp, max_ctas, s) : launch_grouped<32, 1>(ta, tb, args, grp, num_sms(), s);
    case 64:
      return two ? launch_grouped<64, 2>(ta, tb, args, grp, max_ctas, s) : launch_grouped<64, 1>(ta, tb, args, grp, num_sms(), s);
    case 128: return launch_grouped<128, 1>(ta, tb, args, grp, num_sms(), s);
    default: return -2;
  }
}


// ---------------------------------------------------------------------------
// Decode projections whose split-K sum and epilogue run inside the GEMM kernel (splitk_fix.cuh).
// partials: fp32 scratch with room for splits * tokens * rows floats; counters: one zero-initialised
// unsigned int per 128-row tile (they are left at zero).  Both may be shared by consecutive launches
// of one stream.
// ---------------------------------------------------------------------------
extern "C" long long nkb_gemm_fix_scratch_floats(int rows, int tokens, int k, int splits) {
  return (long long)nkb_gemm_effective_splits(k, splits) * tokens * rows;
}

// out[tokens, rows] = x @ w^T (+ bias) (+ residual)
extern "C" int nkb_gemm_fix_store(const void* w, const void* x, void* out, int rows, int tokens, int k, long long ldw,
                                  long long ldx, long long ldo, int splits, const void* bias, const void* residual,
                                  float* partials, unsigned int* counters, int block_n, void* stream) {
  GemmArgs args;
  StoreFix::Args fx{};
  CUtensorMap ta, tb;
  if (int rc = fix_setup(args, fx.c, ta, tb, w, x, rows, tokens, k, ldw, ldx, splits, block_n, partials, counters, bias))
    return rc;
  fx.out = reinterpret_cast<__nv_bfloat16*>(out);
  fx.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  fx.ldo = ldo;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  NKB_FIX_DISPATCH(StoreFix, fx)
}

// out[tokens, inter] = silu(x @ gate^T) * (x @ up^T), w = [gate; up] with inter rows each (inter % 128 == 0);
// act_limit > 0 selects the clamped form; bias = [gate bias; up bias] or null.
extern "C" int nkb_gemm_fix_swiglu(const void* w, const void* x, void* out, int inter, int tokens, int k,
                                   long long ldw, long long ldx, long long ldo, int splits, const void* bias,
                                   float act_limit, float act_alpha, float* partials, unsigned int* counters,
                                   int block_n, void* stream) {
  if (inter <= 0 || (inter % kTileRows)) return -2;
  GemmArgs args;
  SwigluFix::Args fx{};
  CUtensorMap ta, tb;
  if (int rc = fix_setup(args, fx.c, ta, tb, w, x, 2 * inter, tokens, k, ldw, ldx, splits, block_n, partials, counters,
                         bias))
    return rc;
  fx.out = reinterpret_cast<__nv_bfloat16*>(out);
  fx.ldo = ldo;
  fx.inter = inter;
  fx.act_limit = act_limit;
  fx.act_alpha = act_alpha;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  NKB_FIX_DISPATCH(SwigluFix, fx)
}

// Fused QKV projection of a decode step: w [(nq + 2 nkv) * head_dim, k], head_dim 64 or 128.
extern "C" int nkb_gemm_fix_rope(const void* w, const void* x, int tokens, int k, long long ldw, long long ldx,
                                 int splits, const void* bias, const int* positions, const int* slots,
                                 const float* cos_sin, const void* q_norm_w, const void* k_norm_w, float norm_eps,
                                 void* q_out, void* k_cache, void* v_cache, int nq, int nkv, int head_dim, int max_pos,
                                 int block_size, float* partials, unsigned int* counters, int block_n, void* stream) {
  if (head_dim != 64 && head_dim != 128) return -2;
  if (cos_sin && !positions) return -2;
  GemmArgs args;
  RopeFix::Args fx{};
  CUtensorMap ta, tb;
  if (int rc = fix_setup(args, fx.c, ta, tb, w, x, (nq + 2 * nkv) * head_dim, tokens, k, ldw, ldx, splits, block_n,
                         partials, counters, bias))
    return rc;
  fx.positions = positions;
  fx.slots = slots;
  fx.cos_sin = cos_sin;
  fx.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w);
  fx.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w);
  fx.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  fx.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  fx.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  fx.norm_eps = norm_eps;
  fx.nq = nq; fx.nkv = nkv; fx.head_dim = head_dim; fx.max_pos = max_pos; fx.block_size = block_size;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  NKB_FIX_DISPATCH(RopeFix, fx)
}

// Row-parallel projection: the finished bf16 partial [tokens, rows] of this rank goes into slot [rank] of every
// peer's partial array [n_peers, tokens, rows]; the last CTA bumps this rank's arrival counter on every peer.
extern "C" int nkb_gemm_fix_push(const void* w, const void* x, int rows, int tokens, int k, long long ldw,
                                 long long ldx, int splits, const void* bias, void* const* peer_out,
                                 void* const* peer_flag, int n_peers, int rank, void* done_counter, void* mc_out,
                                 void* mc_flag, float* partials, unsigned int* counters, int block_n, void* stream) {
  if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers || (rows & 7)) return -2;
  GemmArgs args;
  PushFix::Args fx{};
  CUtensorMap ta, tb;
  if (int rc = fix_setup(args, fx.c, ta, tb, w, x, rows, tokens, k, ldw, ldx, splits, block_n, partials, counters, bias))
    return rc;
  fx.push.n_peers = n_peers;
  fx.push.rank = rank;
  for (int i = 0; i < n_peers; ++i) {
    fx.push.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(peer_out[i]);
    fx.push.peer_flag[i] = reinterpret_cast<unsigned int*>(peer_flag[i]);
  }
  fx.push.done_counter = reinterpret_cast<unsigned int*>(done_counter);
  fx.push.mc_out = reinterpret_cast<__nv_bfloat16*>(mc_out);
  fx.push.mc_flag = reinterpret_cast<unsigned int*>(mc_flag);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  NKB_FIX_DISPATCH(PushFix, fx)
}
