// Internal interface between the prefill entry point and its tcgen05 kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/b200mops.h"

namespace b200mops {

// Capacity of the tcgen05 kernel's in-kernel schedule tables.
constexpr int kTc5MaxBatch = 1024;    // sequences per launch (longer batches are sliced)
constexpr int kTc5MaxLevels = 512;    // 128-row query tiles per sequence (max_seqlen_q <= 65536)

// Launches the tcgen05/TMEM kernel.  Requirements checked by the caller: head_dim 128,
// batch <= kTc5MaxBatch, max_seqlen_q <= 128 * kTc5MaxLevels, and for paged K/V a page size
// that is a multiple of 128; the Q, K and V tensor maps carry 128-row boxes.
int launch_varlen_prefill_tc5(const b200mops_varlen_prefill_args* a, const CUtensorMap& tm_q,
                              const CUtensorMap& tm_k, const CUtensorMap& tm_v, cudaStream_t st);

}  // namespace b200mops
