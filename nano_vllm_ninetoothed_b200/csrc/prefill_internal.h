// Internal interface between the prefill entry point and its tcgen05 kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/b200mops.h"

namespace b200mops {

// Launches the tcgen05/TMEM kernel.  Requirements checked by the caller: packed (non-paged)
// K/V, head_dim 128, an even number of query heads per KV head; the Q, K and V tensor maps
// carry 128-row boxes.
int launch_varlen_prefill_tc5(const b200mops_varlen_prefill_args* a, const CUtensorMap& tm_q,
                              const CUtensorMap& tm_k, const CUtensorMap& tm_v, cudaStream_t st);

}  // namespace b200mops
