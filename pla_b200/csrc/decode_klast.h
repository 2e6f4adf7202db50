// Internal launchers shared between the k-last translation units.
#pragma once

#include <cuda_runtime.h>

#include "../../include/pla_b200.h"

namespace pla {

// Persistent streaming kernel for plain single-token decode (no snapshots, no
// 2-D slot table, fp32 pool, 8-byte aligned v / o rows).
bool klast_stream_eligible(const pla_b200_klast_args& a);
int launch_klast_stream(const pla_b200_klast_args& a, cudaStream_t stream);
// Row-per-thread kernel for the same calls (one CTA per (request, head), the row in registers).
int launch_klast_rows(const pla_b200_klast_args& a, cudaStream_t stream);

}  // namespace pla
