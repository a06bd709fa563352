// Expert-parallel regroup plan.  Rank g owns experts [g*E/G, (g+1)*E/G).  After the dispatch all-to-all its receive
// buffer holds, source rank by source rank, the rows each source routes to g's experts, sorted by (local) expert in
// the source's canonical order.  This kernel lays those rows out expert by expert (sources in rank order inside an
// expert, segments padded to 128 rows) so that the grouped GEMMs see the same padded layout as on one GPU.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"

namespace lmoe {

// One block per (source rank s, local expert j).
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int* __restrict__ counts_all, int G, int E, int rank, int* __restrict__ recv_pos,
               int* __restrict__ row_src, int* __restrict__ pad_offsets, int* __restrict__ tile_expert,
               int* __restrict__ n_tiles) {
  __shared__ int cnt[LMOE_MAX_EXPERTS];  // cnt[s' * El + j'] = rows source s' sends to local expert j'
  __shared__ int s_recv_off, s_dst_off, s_pad_off, s_tot, s_total_padded;
  const int El = E / G;
  const int e0 = rank * El;
  const int s = blockIdx.x / El, j = blockIdx.x % El;
  for (int i = threadIdx.x; i < G * El; i += blockDim.x) cnt[i] = counts_all[(i / El) * E + e0 + (i % El)];
  __syncthreads();
  if (threadIdx.x == 0) {
    int recv_off = 0;
    for (int s2 = 0; s2 < s; ++s2)
      for (int j2 = 0; j2 < El; ++j2) recv_off += cnt[s2 * El + j2];
    for (int j2 = 0; j2 < j; ++j2) recv_off += cnt[s * El + j2];
    int pad_off = 0, total_padded = 0, tot_j = 0;
    for (int j2 = 0; j2 < El; ++j2) {
      int tot = 0;
      for (int s2 = 0; s2 < G; ++s2) tot += cnt[s2 * El + j2];
      const int padded = (tot + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD * LMOE_ROW_PAD;
      if (j2 < j) pad_off += padded;
      if (j2 == j) tot_j = tot;
      total_padded += padded;
    }
    int dst_off = pad_off;
    for (int s2 = 0; s2 < s; ++s2) dst_off += cnt[s2 * El + j];
    s_recv_off = recv_off;
    s_dst_off = dst_off;
    s_pad_off = pad_off;
    s_tot = tot_j;
    s_total_padded = total_padded;
  }
  __syncthreads();
  const int n = cnt[s * El + j];
  for (int r = threadIdx.x; r < n; r += blockDim.x) {
    recv_pos[s_recv_off + r] = s_dst_off + r;
    row_src[s_dst_off + r] = s_recv_off + r;
  }
  const int padded_j = (s_tot + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD * LMOE_ROW_PAD;
  if (s == G - 1) {
    for (int r = s_pad_off + s_tot + threadIdx.x; r < s_pad_off + padded_j; r += blockDim.x) row_src[r] = -1;
  }
  if (s == 0) {
    if (threadIdx.x == 0) pad_offsets[j] = s_pad_off;
    for (int t = s_pad_off / LMOE_ROW_PAD + threadIdx.x; t < (s_pad_off + padded_j) / LMOE_ROW_PAD; t += blockDim.x)
      tile_expert[t] = j;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    pad_offsets[El] = s_total_padded;
    n_tiles[0] = s_total_padded / LMOE_ROW_PAD;
  }
}

}  // namespace lmoe

extern "C" int lmoe_ep_plan(const int32_t* counts_all, int G, int E, int rank, int32_t* recv_pos, int32_t* row_src,
                            int32_t* pad_offsets, int32_t* tile_expert, int32_t* n_tiles, void* stream) {
  if (!counts_all || !recv_pos || !row_src || !pad_offsets || !tile_expert || !n_tiles) return LMOE_ERR_ARG;
  if (G <= 0 || E <= 0 || E > LMOE_MAX_EXPERTS || (E % G) != 0 || rank < 0 || rank >= G) return LMOE_ERR_SHAPE;
  lmoe::count_launch();
  lmoe::ep_plan_kernel<<<E, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, G, E, rank, recv_pos, row_src,
                                                                        pad_offsets, tile_expert, n_tiles);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
