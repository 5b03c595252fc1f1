// Internal (non-ABI) rulebook entry points for callers inside the library that chain rulebooks.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace spc {

// The strided / transposed layer whose OUTPUT rows, all of them and in its order, are the input rows
// of the rulebook being generated.  When that layer numbered its outputs through a bitmap of its
// output grid, the bitmap and its prefix sums are still in its workspace and are exactly the input
// occupancy bitmap the new rulebook would otherwise build (clear, mark, count, scan) -- and the
// input hash table is not needed either, because the rows are the ranks of the bits.
struct RulebookProducer {
  const spc_geometry* geom;
  const void* workspace;  // as spc_rulebook_prepare left it
  int64_t n_in;           // the n_in that workspace was laid out for
};

// spc_rulebook_prepare / spc_rulebook_igemm with an optional producer (nullptr = the plain calls).
int rulebook_prepare_chained(const spc_geometry* g, const int32_t* indices, int64_t n_in, void* workspace,
                             size_t workspace_bytes, int64_t* n_out_host, const RulebookProducer* producer,
                             cudaStream_t stream);
int rulebook_igemm_chained(const spc_geometry* g, const int32_t* indices, int64_t n_in, int64_t n_out,
                           void* workspace, size_t workspace_bytes, int32_t* out_indices, int32_t* pair_fwd,
                           int32_t* pair_bwd, int32_t* mask_fwd, int32_t* argsort_fwd, int32_t* mask_bwd,
                           int32_t* argsort_bwd, const uint32_t* split_masks, int n_split, int do_sort,
                           int32_t* pair_fwd_rowmajor, int32_t* pair_bwd_rowmajor,
                           const RulebookProducer* producer, cudaStream_t stream);
// do_sort == 2 in rulebook_igemm_chained asks for the tile-key order (rows grouped so that the 128
// rows of a gather-GEMM tile share kernel offsets; mask_fwd then holds sorted keys, not sorted mask
// words).  It applies to single-word masks, one split that keeps every bit and no input-side tables;
// otherwise 2 means 1.  This tells a caller in advance which of the two it will get.
bool rulebook_tile_key_applies(const spc_geometry* g, bool with_backward, const uint32_t* split_masks, int n_split);

}  // namespace spc
