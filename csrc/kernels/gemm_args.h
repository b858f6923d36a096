// Argument blocks of the tcgen05 GEMM kernel, shared by the device code, the library
// launcher and the C++ runtime that launches generated kernels from a plan.
#pragma once
#include <cuda_bf16.h>

namespace nkb {

constexpr int kBlockK = 64;           // bf16 elements per K slab = one 128B swizzle row
constexpr int kTileRows = 128;        // UMMA M
constexpr int kATileBytes = kTileRows * kBlockK * 2;
constexpr int kMaxStages = 12;
constexpr int kGemmThreads = 192;     // warp0 TMA, warp1 MMA, warps2-5 epilogue

// Keep this block at or below 128 bytes: with a larger by-value struct parameter nvcc 12.9 emitted a
// kernel that ran the 128256 x 4096 decode projection 40 % slower (280 vs 200 us) from identical source.
struct GemmArgs {
  int rows, cols, k;
  int splits, kb_per_split, kb_total;
  int num_row_tiles, num_col_tiles;
  int gated;        // 0 none, 1 = A operand holds [gate; up], 2 = B operand holds [gate; up]
  int gate_off;     // row offset of the "up" half inside the gated operand
  int transpose_out;
  int out_fp32;
  int bias_on_rows;
  int stages;
  int weights_operand;  // 0 = A, 1 = B holds immutable weights (may be fetched before the dependency wait), -1 none
  long long ldo;
  long long split_stride;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int* status;
};
static_assert(sizeof(GemmArgs) <= 128, "GemmArgs grew past the fast kernel-parameter size");

// Grouped mode (MoE experts): A is [num_groups, rows(+gate), k] (3-D tensor map), B and the output
// are row-sorted by group; group g owns B rows / output columns [group_offsets[g], group_offsets[g + 1]).
// Kept apart from GemmArgs: the plain kernels do not take it.
struct GroupArgs {
  int num_groups;
  int max_col_tiles;       // upper bound of column tiles per group (work items beyond a group's count are skipped)
  const int* group_offsets;
  // optional compact schedule: tile_list[2 * t] = group, tile_list[2 * t + 1] = column tile, for
  // t < *tile_count (built on the device by the MoE dispatch); replaces the max_col_tiles enumeration
  const int* tile_list;
  const int* tile_count;
  long long bias_group_stride;
  float act_limit;         // > 0: clamped SwiGLU (up + 1) * gate * sigmoid(act_alpha * gate)
  float act_alpha;
  // expert-parallel all-to-all (moe_a2a.cu): the rows of group g are complete once arrive[g] reaches
  // arrive_target (every source rank has delivered its rows); nullptr = rows are local, no wait
  const unsigned int* arrive;
  unsigned int arrive_target;
};

// Fused collective epilogue ("push" mode, decode orientation only): every finished
// output tile is stored as a bf16 partial straight into the symmetric buffer of every
// tensor-parallel peer (plain peer stores over NVLink, 16 bytes per thread, staged
// through shared memory so that each token row is one contiguous 256-byte run), into
// slot (rank * splits + split) of the destination's [slots, M, N] partial array.  The
// last CTA of the grid then bumps this rank's arrival counter on every peer; the
// consumer (tp_reduce_rmsnorm in comm.cu) waits on those counters with a bounded spin.
constexpr int kMaxPeers = 8;
struct PushArgs {
  int n_peers;
  int rank;
  __nv_bfloat16* peer_out[kMaxPeers];
  unsigned int* peer_flag[kMaxPeers];   // this rank's arrival counter inside each peer's flag array
  unsigned int* done_counter;           // local: CTAs of this grid that finished their stores
  // NVLink multicast view of the same symmetric buffers (nullptr = none): one multimem store through mc_out
  // lands in every rank's partial array, one multimem reduction on mc_flag bumps this rank's arrival counter
  // on every rank, so a partial leaves the GPU once instead of once per peer.
  __nv_bfloat16* mc_out;
  unsigned int* mc_flag;
};

}  // namespace nkb
