// Pass registry and pipeline driver of the native compiler.
//
// The pipeline plays the role of the reference's nkipy-opt stage list
// (nkigen/nkigen/transforms/nkipy_opt.py:233-311, passes declared in
// nkigen/mlir/include/nkipy/Transforms/Passes.td): every pass is runnable on its own by
// name, the default pipeline can be stopped after a pass (by index, name, `name:N` or
// group) and can dump the IR after each stage as NN_<pass>.ir.  Pass names are kept where
// a pass has a GPU counterpart; what each one does on this target:
//
//   canonicalize group
//     remove-redundant-zero-fill      x + 0-splat / 0-splat + x -> x (accumulators start from the first MMA)
//     prepare-arithmetic              pow(x, 2) -> x * x; with fast-math, x / c -> x * (1 / c)
//     decompose-batch-matmul          mark batched dots for grid.z batching
//     canonicalize-partition-dim      fold a transposed dot operand into the dot (K-major vs MN-major operand)
//     canonicalize-reshape            reshape(reshape(x)) -> reshape(x); identity reshapes removed
//     simplify-linalg                 transpose chains composed, identity transposes removed
//     eliminate-uninitialized-copies  copies of freshly created values removed
//     eliminate-same-memspace-copy    copies whose source has no other reader removed
//     cse, canonicalize               common subexpressions, x*1, convert-to-same, dead code
//   layout group
//     infer-layout                    tile shapes and placement (Global / Shared / Tensor / Register) from dot seeds
//     assign-linalg-op-ids            stable ids for compute ops
//     knob-driven-tiling              CTA tile, k-block, stage count, split-K and grid per op (user knobs win)
//     knob-driven-fusion              elementwise fusion groups, GEMM epilogue candidates
//     apply-and-strip-transforms      consume user knob annotations
//     canonicalize-loop-step          no work on this target (kept for pipeline parity)
//   memory group
//     annotate-memory-space           memory space of every value
//     legalize-layout                 TMA box / swizzle / TMEM-column legality, tcgen05 vs SIMT path
//     insert-spill-reload             shared-memory / TMEM budget: fewer stages or smaller tiles, error if impossible
//     one-shot-bufferize              buffer assignment with reuse after last use and in-place elementwise
//     insert-memref-dealloc           last-use lists for the runtime's arena
//     inline-nkipy-reference          inline reference graphs of custom calls (CPU-oracle pipelines)
#pragma once
#include <string>
#include <vector>

#include "ir.h"

namespace b200c {

struct PassOptions {
  std::string target = "sm_100a";
  long long smem_capacity = 232448;   // bytes per CTA
  long long tmem_columns = 512;
  int sm_count = 148;
  bool fast_math = false;
};

using PassFn = void (*)(Graph&, const PassOptions&);

struct PassInfo {
  std::string name;
  std::string group;
  std::string description;
  PassFn fn;
};

const std::vector<PassInfo>& default_pipeline();
const PassInfo* find_pass(const std::string& name);
void run_pass(Graph& g, const std::string& name, const PassOptions& opts);

// Runs the default pipeline on IR text.  stop_after: "" (all), an index ("7"), a pass name,
// "name:N" (N-th occurrence) or a group name.  dump_dir: when non-empty the IR after every
// stage is written to <dump_dir>/NN_<pass>.ir (numbering starts at `dump_start`).
std::string run_pipeline(const std::string& ir_text, const std::string& stop_after, const std::string& dump_dir,
                         const PassOptions& opts, int dump_start = 1);
std::string apply_passes(const std::string& ir_text, const std::vector<std::string>& passes, const PassOptions& opts);

}  // namespace b200c
