// Expert-parallel exchange by one-sided stores over NVLink (peer pointers of symmetric buffers).
//
// Rank g owns experts [g*E/G, (g+1)*E/G).  Every rank knows counts_all[G][E] (all-gather of the routing
// histograms), so every rank can compute where each of its rows lives in the DESTINATION's padded expert layout:
//   row of expert e = (g, j), q-th row of source r for that expert  ->  pad_off_g[j] + sum_{s<r} counts_all[s][e] + q
// The dispatch kernel reads a latent row once and stores it straight into the peer's buffer at that position; the
// return kernel does the inverse walk and stores each result row into the source's return buffer at its position
// in the source's expert-sorted order.  Nothing is sized or branched on the host: capacities are static and an
// overflow raises a status word.  Plain peer stores only (no multimem, no TMA on peer memory); the cross-rank
// ordering comes from stream-ordered collectives issued by the host code between the phases.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"

namespace lmoe {

constexpr int kStatusEpOverflow = 201;
constexpr int kEpWarps = 8;

// One block.  Tables derived from counts_all for rank `rank`:
//   src_off[s*E + e]   exclusive scan of counts_all[s][:]           (position of expert e in source s's sorted order)
//   dst_base[e]        destination padded row of this rank's first row of expert e
//   seg_cum[j*G + s]   sum_{s'<s} counts_all[s'][e0+j]              (local expert j: where source s's rows start)
//   pad_offsets[El+1], tile_expert[], n_tiles                       (this rank's padded layout)
__global__ void __launch_bounds__(256)
ep_tables_kernel(const int* __restrict__ counts_all, int G, int E, int rank, int capacity_rows, int* __restrict__ src_off,
                 int* __restrict__ dst_base, int* __restrict__ seg_cum, int* __restrict__ pad_offsets,
                 int* __restrict__ tile_expert, int* __restrict__ n_tiles, int* __restrict__ status) {
  __shared__ int tot[LMOE_MAX_EXPERTS];      // rows of expert e over all sources
  __shared__ int before[LMOE_MAX_EXPERTS];   // rows of expert e from sources < rank
  __shared__ int poff[LMOE_MAX_EXPERTS + 1]; // padded offset of expert e inside its owner's layout
  const int El = E / G;
  const int tid = threadIdx.x;
  if (tid < E) {
    int t = 0, b = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts_all[s * E + tid];
      if (s < rank) b += c;
      t += c;
    }
    tot[tid] = t;
    before[tid] = b;
  }
  // per-source exclusive scans (one thread per source; E <= 256 sequential adds)
  if (tid < G) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      src_off[tid * E + e] = run;
      run += counts_all[tid * E + e];
    }
  }
  __syncthreads();
  if (tid < G) {  // padded offsets inside owner `tid`'s layout
    int run = 0;
    for (int j = 0; j < El; ++j) {
      poff[tid * El + j] = run;
      run += (tot[tid * El + j] + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD * LMOE_ROW_PAD;
    }
    if (run > capacity_rows && status) atomicCAS(status, 0, kStatusEpOverflow);
    if (tid == rank) {
      const int used = min(run, capacity_rows) / LMOE_ROW_PAD * LMOE_ROW_PAD;
      pad_offsets[El] = used;
      n_tiles[0] = used / LMOE_ROW_PAD;
    }
  }
  __syncthreads();
  if (tid < E) dst_base[tid] = poff[tid] + before[tid];
  if (tid < El) pad_offsets[tid] = min(poff[rank * El + tid], capacity_rows);
  for (int i = tid; i < El * G; i += blockDim.x) {
    const int j = i / G, s = i % G;
    int c = 0;
    for (int s2 = 0; s2 < s; ++s2) c += counts_all[s2 * E + rank * El + j];
    seg_cum[i] = c;
  }
  // tile -> local expert
  for (int j = 0; j < El; ++j) {
    const int e = rank * El + j;
    const int t0 = poff[e] / LMOE_ROW_PAD;
    const int t1 = t0 + (tot[e] + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD;
    for (int t = t0 + tid; t < t1 && t < capacity_rows / LMOE_ROW_PAD; t += blockDim.x) tile_expert[t] = j;
  }
}

// Zero the pad rows of this rank's incoming buffer: rows [pad_off[j] + tot_j, pad_off[j+1]).  One block per local expert.
__global__ void __launch_bounds__(256)
ep_zero_pads_kernel(uint4* __restrict__ buf, int vec_per_row, const int* __restrict__ pad_offsets,
                    const int* __restrict__ seg_cum, const int* __restrict__ counts_all, int G, int E, int rank) {
  const int El = E / G;
  const int j = blockIdx.x;
  const int tot = seg_cum[j * G + (G - 1)] + counts_all[(G - 1) * E + rank * El + j];
  const long long r0 = static_cast<long long>(pad_offsets[j]) + tot, r1 = pad_offsets[j + 1];
  const long long n = (r1 - r0) * vec_per_row;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) buf[r0 * vec_per_row + i] = make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ void unpack8f(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// Dispatch: send-order row i (flat = perm[i], token = flat / K, expert e = sel[flat]) goes to the owner of e.
// MODE 0: row = src[token]                                   (forward: latent activations)
// MODE 1: row = weights[flat] * src[token], and d_weights[flat] = <src[token], y_ret[i]>   (backward: gradients)
// A warp takes 32 consecutive rows: each lane resolves the indices of one row (perm -> sel -> offsets / dst_base, a
// chain of dependent loads paid once per 32 rows), then the warp copies the rows four at a time, 16 bytes per lane.
template <int MODE>
__global__ void __launch_bounds__(kEpWarps * 32)
ep_dispatch_kernel(const uint4* __restrict__ src, const int* __restrict__ perm, const int* __restrict__ sel,
                   const int* __restrict__ offsets, const int* __restrict__ dst_base, const float* __restrict__ weights,
                   const uint4* __restrict__ y_ret, float* __restrict__ d_weights, int n_rows, int K, int El,
                   int vec_per_row, int capacity_rows, uint4* const* __restrict__ peer_bufs, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = static_cast<long long>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5);
  const long long warps_total = static_cast<long long>(gridDim.x) * kEpWarps;
  for (long long base = warp_global * 32; base < n_rows; base += warps_total * 32) {
    const long long i = base + lane;
    long long my_token = 0;
    unsigned long long my_dst = 0;  // 0: row not stored (out of range or beyond the capacity)
    float my_w = 1.0f;
    int my_flat = 0;
    if (i < n_rows) {
      my_flat = perm[i];
      const int e = sel[my_flat];
      my_token = my_flat / K;
      const int drow = dst_base[e] + static_cast<int>(i - offsets[e]);
      if (drow < capacity_rows)
        my_dst = reinterpret_cast<unsigned long long>(peer_bufs[e / El] + static_cast<long long>(drow) * vec_per_row);
      else if (status)
        atomicCAS(status, 0, kStatusEpOverflow);
      if (MODE == 1) my_w = weights[my_flat];
    }
    const int rows_here = static_cast<int>(min(32ll, static_cast<long long>(n_rows) - base));
    for (int j0 = 0; j0 < rows_here; j0 += 4) {
      long long tok[4];
      unsigned long long dst[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + u, 31);
        tok[u] = __shfl_sync(0xffffffffu, my_token, j);
        dst[u] = __shfl_sync(0xffffffffu, my_dst, j);
        w[u] = __shfl_sync(0xffffffffu, my_w, j);
        if (j0 + u >= rows_here) dst[u] = 0;
      }
      float dot[4] = {0.f, 0.f, 0.f, 0.f};
      for (int v = lane; v < vec_per_row; v += 32) {
        uint4 x[4], yv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          x[u] = src[tok[u] * vec_per_row + v];
          if (MODE == 1) yv[u] = (j0 + u < rows_here) ? y_ret[(base + j0 + u) * vec_per_row + v] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (MODE == 0) {
            if (dst[u]) reinterpret_cast<uint4*>(dst[u])[v] = x[u];
          } else {
            float g[8], yy[8], o[8];
            unpack8f(x[u], g);
            unpack8f(yv[u], yy);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              dot[u] = fmaf(g[k], yy[k], dot[u]);
              o[k] = w[u] * g[k];
            }
            if (dst[u]) reinterpret_cast<uint4*>(dst[u])[v] = pack8f(o);
          }
        }
      }
      if (MODE == 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
          const int fl = __shfl_sync(0xffffffffu, my_flat, min(j0 + u, 31));
          if (lane == 0 && j0 + u < rows_here) d_weights[fl] = dot[u];
        }
      }
    }
  }
}

// Return: padded local row p (expert j = tile_expert[p / 128]) belongs to source s (walk seg_cum) and is that
// source's row src_off[s][e] + r in its expert-sorted order; store it into s's return buffer there.  Same scheme as
// the dispatch: one lane resolves one row, the warp copies four rows at a time.
__global__ void __launch_bounds__(kEpWarps * 32)
ep_return_kernel(const uint4* __restrict__ rows, const int* __restrict__ tile_expert, const int* __restrict__ n_tiles,
                 const int* __restrict__ pad_offsets, const int* __restrict__ seg_cum, const int* __restrict__ src_off,
                 const int* __restrict__ counts_all, int G, int E, int rank, int vec_per_row, int capacity_rows,
                 uint4* const* __restrict__ peer_ret) {
  const int lane = threadIdx.x & 31;
  const int El = E / G;
  const long long used = min(static_cast<long long>(n_tiles[0]) * LMOE_ROW_PAD, static_cast<long long>(capacity_rows));
  const long long warp_global = static_cast<long long>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5);
  const long long warps_total = static_cast<long long>(gridDim.x) * kEpWarps;
  for (long long base = warp_global * 32; base < used; base += warps_total * 32) {
    const long long p = base + lane;
    unsigned long long my_dst = 0;  // 0: pad row, nothing to return
    if (p < used) {
      const int j = tile_expert[p / LMOE_ROW_PAD];
      const int e = rank * El + j;
      const int q = static_cast<int>(p - pad_offsets[j]);
      int s = -1;
      for (int s2 = G - 1; s2 >= 0; --s2) {
        if (q >= seg_cum[j * G + s2]) {
          s = s2;
          break;
        }
      }
      if (s >= 0) {
        const int r = q - seg_cum[j * G + s];
        if (r < counts_all[s * E + e])
          my_dst = reinterpret_cast<unsigned long long>(peer_ret[s] +
                                                        static_cast<long long>(src_off[s * E + e] + r) * vec_per_row);
      }
    }
    const int rows_here = static_cast<int>(min(32ll, used - base));
    for (int j0 = 0; j0 < rows_here; j0 += 4) {
      unsigned long long dst[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        dst[u] = __shfl_sync(0xffffffffu, my_dst, min(j0 + u, 31));
        if (j0 + u >= rows_here) dst[u] = 0;
      }
      for (int v = lane; v < vec_per_row; v += 32) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          x[u] = dst[u] ? rows[(base + j0 + u) * vec_per_row + v] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (dst[u]) reinterpret_cast<uint4*>(dst[u])[v] = x[u];
      }
    }
  }
}

static inline int grid_rows(long long rows) {
  long long b = (rows + kEpWarps * 32 - 1) / (kEpWarps * 32);  // a warp takes 32 rows per pass
  if (b > 148ll * 16) b = 148ll * 16;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
static inline int last_err() {
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace lmoe

using namespace lmoe;

extern "C" int lmoe_ep_tables(const int32_t* counts_all, int G, int E, int rank, int64_t capacity_rows, int32_t* src_off,
                              int32_t* dst_base, int32_t* seg_cum, int32_t* pad_offsets, int32_t* tile_expert,
                              int32_t* n_tiles, int32_t* status, void* stream) {
  if (!counts_all || !src_off || !dst_base || !seg_cum || !pad_offsets || !tile_expert || !n_tiles) return LMOE_ERR_ARG;
  if (G <= 0 || E <= 0 || E > LMOE_MAX_EXPERTS || (E % G) != 0 || rank < 0 || rank >= G || G > 256) return LMOE_ERR_SHAPE;
  if (capacity_rows <= 0 || (capacity_rows % LMOE_ROW_PAD) != 0 || capacity_rows >= (1ll << 31)) return LMOE_ERR_SHAPE;
  ep_tables_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, G, E, rank,
                                                                    static_cast<int>(capacity_rows), src_off, dst_base,
                                                                    seg_cum, pad_offsets, tile_expert, n_tiles, status);
  return last_err();
}

extern "C" int lmoe_ep_zero_pads(void* buf, int L, const int32_t* pad_offsets, const int32_t* seg_cum,
                                 const int32_t* counts_all, int G, int E, int rank, void* stream) {
  if (!buf || !pad_offsets || !seg_cum || !counts_all) return LMOE_ERR_ARG;
  if ((L & 7) != 0 || G <= 0 || (E % G) != 0) return LMOE_ERR_SHAPE;
  ep_zero_pads_kernel<<<E / G, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(buf), L / 8, pad_offsets,
                                                                           seg_cum, counts_all, G, E, rank);
  return last_err();
}

extern "C" int lmoe_ep_dispatch(const void* src_rows, const int32_t* perm, const int32_t* sel, const int32_t* offsets,
                                const int32_t* dst_base, int64_t n_rows, int K, int E, int G, int L,
                                int64_t capacity_rows, void* const* peer_bufs, int32_t* status, void* stream) {
  if (!src_rows || !perm || !sel || !offsets || !dst_base || !peer_bufs) return LMOE_ERR_ARG;
  if ((L & 7) != 0 || n_rows <= 0 || n_rows >= (1ll << 31) || G <= 0 || (E % G) != 0) return LMOE_ERR_SHAPE;
  ep_dispatch_kernel<0><<<grid_rows(n_rows), kEpWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_rows), perm, sel, offsets, dst_base, nullptr, nullptr, nullptr,
      static_cast<int>(n_rows), K, E / G, L / 8, static_cast<int>(capacity_rows),
      reinterpret_cast<uint4* const*>(peer_bufs), status);
  return last_err();
}

extern "C" int lmoe_ep_dispatch_bwd(const void* d_routed, const void* y_ret, const float* weights, const int32_t* perm,
                                    const int32_t* sel, const int32_t* offsets, const int32_t* dst_base, int64_t n_rows,
                                    int K, int E, int G, int L, int64_t capacity_rows, void* const* peer_bufs,
                                    float* d_weights, int32_t* status, void* stream) {
  if (!d_routed || !y_ret || !weights || !perm || !sel || !offsets || !dst_base || !peer_bufs || !d_weights)
    return LMOE_ERR_ARG;
  if ((L & 7) != 0 || n_rows <= 0 || n_rows >= (1ll << 31) || G <= 0 || (E % G) != 0) return LMOE_ERR_SHAPE;
  ep_dispatch_kernel<1><<<grid_rows(n_rows), kEpWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(d_routed), perm, sel, offsets, dst_base, weights, static_cast<const uint4*>(y_ret),
      d_weights, static_cast<int>(n_rows), K, E / G, L / 8, static_cast<int>(capacity_rows),
      reinterpret_cast<uint4* const*>(peer_bufs), status);
  return last_err();
}

extern "C" int lmoe_ep_return(const void* rows, const int32_t* tile_expert, const int32_t* n_tiles,
                              const int32_t* pad_offsets, const int32_t* seg_cum, const int32_t* src_off,
                              const int32_t* counts_all, int G, int E, int rank, int L, int64_t capacity_rows,
                              void* const* peer_ret, void* stream) {
  if (!rows || !tile_expert || !n_tiles || !pad_offsets || !seg_cum || !src_off || !counts_all || !peer_ret)
    return LMOE_ERR_ARG;
  if ((L & 7) != 0 || G <= 0 || (E % G) != 0 || rank < 0 || rank >= G) return LMOE_ERR_SHAPE;
  ep_return_kernel<<<grid_rows(capacity_rows), kEpWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(rows), tile_expert, n_tiles, pad_offsets, seg_cum, src_off, counts_all, G, E, rank,
      L / 8, static_cast<int>(capacity_rows), reinterpret_cast<uint4* const*>(peer_ret));
  return last_err();
}
