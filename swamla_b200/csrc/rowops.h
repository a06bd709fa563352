// Internal host-side launchers of the row kernels shared between translation units.
#pragma once
#include <cuda_runtime.h>

#include "../../include/lmoe.h"

namespace lmoe {
// x_sorted[row] = x_latent[row_src[row] / K] over the padded rows in use (zeros for pad rows).
int gather_rows(const void* x_latent, const lmoe_route* r, int K, int L, long long padded_rows, void* x_sorted,
                cudaStream_t st);
// out[t] = sum_k w[t,k] * y[pos[t*K+k]]  (w may be null: plain sum).
int combine_rows(const void* y_sorted, const int* pos, const float* w, int T, int K, int L, void* out, long long out_ld,
                 cudaStream_t st);
}  // namespace lmoe
