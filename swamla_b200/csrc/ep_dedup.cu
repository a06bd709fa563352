// Expert-parallel exchange with one row per (token, destination rank) instead of one per (token, expert).
//
// A token routed to K experts that live on fewer than K ranks would cross NVLink several times to the same rank.
// Here the source stores its latent row ONCE into a staging slot of every rank that owns at least one of the token's
// experts, together with a few words per routed row that tell the owner where the row sits in its padded expert layout:
//
//   stage[s*stride + t][L]      the latent row of token t of source s            (slot is fixed: no compaction, no scan)
//   mask[s*stride + t]          bit k set: top-k slot k of that token belongs to an expert of this rank
//   slots[(s*stride + t)*K + k] padded row of slot k in this rank's layout (-1 when the bit is clear)
//   meta[p] = {s*stride + t, w} for padded row p: its staging slot and its combine weight
//
// The owner gathers its padded layout from the staging slots (local copies), runs the grouped expert GEMMs, reduces
// the result rows of a token that belong to the same staging slot (weighted in forward, plain in backward) and stores
// ONE row per (token, owner) back into the source's return buffer ret[owner*stride + t]; the source adds the rows of
// the owners its token used.  With K experts spread uniformly over G ranks the traffic per token falls from K rows to
// G * (1 - (1 - 1/G)^K) rows each way.  The partial sums travel in bf16, so a result is rounded once per owner and once
// more at the source; the order of the additions is fixed (slot order inside an owner, owner order at the source).
//
// Plain peer stores only; cross-rank ordering comes from stream-ordered collectives between the phases.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"
#include "device_once.h"

namespace lmoe {

constexpr int kStatusEpdOverflow = 201;
constexpr int kEpdWarps = 8;
// The send kernel runs beside the shared-expert GEMM, whose SwiGLU epilogue takes 152 registers per thread: with its ten
// warps spread 3/3/2/2 over the four register files of an SM, the fullest ones keep 1,792 registers free.  A block of
// four warps (one per register file, 1,024 registers each at 32 per thread) fits there; a block of eight does not and
// would wait for the GEMM to drain (measured: no overlap at all with eight warps).
constexpr int kEpdSendWarps = 4;
constexpr int kEpdMaxVecPerLane = 4;  // rows of up to 4 * 32 * 8 = 1024 elements

__device__ __forceinline__ void epd_unpack(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 epd_pack(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// Source side.  One warp per token; lane k < K resolves top-k slot k.
// WITH_META: also writes mask / slots / meta (forward); without it only the rows travel (backward reuses the tables).
template <bool WITH_META>
__global__ void __launch_bounds__(kEpdSendWarps * 32)
epd_send_kernel(const uint4* __restrict__ src, const int* __restrict__ sel, const int* __restrict__ pos,
                const int* __restrict__ offsets, const int* __restrict__ dst_base, const float* __restrict__ weights,
                int T, int K, int El, int G, int rank, int vec_per_row, int capacity_rows, int stride,
                uint4* const* __restrict__ peer_stage, int2* const* __restrict__ peer_meta,
                unsigned* const* __restrict__ peer_mask, int* const* __restrict__ peer_slots, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kEpdSendWarps;
  for (int t = blockIdx.x * kEpdSendWarps + (threadIdx.x >> 5); t < T; t += warps_total) {
    int g = -1, drow = -1;
    float w = 0.f;
    if (lane < K) {
      const int flat = t * K + lane;
      const int e = sel[flat];
      g = e / El;
      if (WITH_META) {
        drow = dst_base[e] + (pos[flat] - offsets[e]);
        w = weights[flat];
        if (drow >= capacity_rows) {
          drow = -1;
          if (status) atomicCAS(status, 0, kStatusEpdOverflow);
        }
      }
    }
    const long long slot = static_cast<long long>(rank) * stride + t;
    for (int gi = 0; gi < G; ++gi) {
      const int d = (gi + rank + 1) % G;  // every source starts at another destination
      const bool mine = (g == d);
      const unsigned any = __ballot_sync(0xffffffffu, mine);
      if (WITH_META) {
        const unsigned m = __ballot_sync(0xffffffffu, mine && drow >= 0);
        if (lane == 0) peer_mask[d][slot] = m;
        if (any) {
          if (lane < K) peer_slots[d][slot * K + lane] = mine ? drow : -1;
          if (mine && drow >= 0) peer_meta[d][drow] = make_int2(static_cast<int>(slot), __float_as_int(w));
        }
      }
      if (any) {
        uint4* dst = peer_stage[d] + slot * vec_per_row;
        const uint4* row = src + static_cast<long long>(t) * vec_per_row;
        for (int v = lane; v < vec_per_row; v += 32) dst[v] = row[v];
      }
    }
  }
}

// Owner side, after the barrier: fill the padded layout from the staging slots.
// BWD = false: out[p] = stage[meta[p].slot]                                  (pad rows: zeros)
// BWD = true : out[p] = w_p * stage[slot],  d_w_row[p] = <stage[slot], y_sorted[p]>
// A warp takes 32 consecutive padded rows (one lane resolves one row), then copies them four at a time.
template <bool BWD>
__global__ void __launch_bounds__(kEpdWarps * 32)
epd_gather_kernel(const uint4* __restrict__ stage, const int2* __restrict__ meta, const int* __restrict__ tile_expert,
                  const int* __restrict__ n_tiles, const int* __restrict__ pad_offsets, const int* __restrict__ seg_cum,
                  const int* __restrict__ counts_all, int G, int E, int rank, int vec_per_row, int capacity_rows,
                  long long n_slots, const uint4* __restrict__ y_sorted, uint4* __restrict__ out,
                  float* __restrict__ d_w_row) {
  const int lane = threadIdx.x & 31;
  const int El = E / G;
  const long long used = min(static_cast<long long>(n_tiles[0]) * LMOE_ROW_PAD, static_cast<long long>(capacity_rows));
  const long long warp_global = static_cast<long long>(blockIdx.x) * kEpdWarps + (threadIdx.x >> 5);
  const long long warps_total = static_cast<long long>(gridDim.x) * kEpdWarps;
  for (long long base = warp_global * 32; base < used; base += warps_total * 32) {
    const long long p = base + lane;
    long long my_slot = -1;  // -1: pad row
    float my_w = 0.f;
    if (p < used) {
      const int j = tile_expert[p / LMOE_ROW_PAD];
      const int tot = seg_cum[j * G + (G - 1)] + counts_all[(G - 1) * E + rank * El + j];
      if (static_cast<int>(p - pad_offsets[j]) < tot) {
        const int2 m = meta[p];
        if (m.x >= 0 && m.x < n_slots) {  // a row whose words never arrived stays a pad row
          my_slot = m.x;
          my_w = __int_as_float(m.y);
        }
      }
    }
    const int rows_here = static_cast<int>(min(32ll, used - base));
    for (int j0 = 0; j0 < rows_here; j0 += 4) {
      long long sl[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + u, 31);
        sl[u] = __shfl_sync(0xffffffffu, my_slot, j);
        w[u] = __shfl_sync(0xffffffffu, my_w, j);
        if (j0 + u >= rows_here) sl[u] = -2;  // beyond the used rows: nothing is written
      }
      float dot[4] = {0.f, 0.f, 0.f, 0.f};
      for (int v = lane; v < vec_per_row; v += 32) {
        uint4 x[4], yv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          x[u] = sl[u] >= 0 ? stage[sl[u] * vec_per_row + v] : make_uint4(0, 0, 0, 0);
          if (BWD) yv[u] = sl[u] >= 0 ? y_sorted[(base + j0 + u) * vec_per_row + v] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (sl[u] == -2) continue;
          if (BWD) {
            float gq[8], yy[8], o[8];
            epd_unpack(x[u], gq);
            epd_unpack(yv[u], yy);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              dot[u] = fmaf(gq[k], yy[k], dot[u]);
              o[k] = w[u] * gq[k];
            }
            x[u] = epd_pack(o);
          }
          out[(base + j0 + u) * vec_per_row + v] = x[u];
        }
      }
      if (BWD) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
          if (lane == 0 && sl[u] != -2) d_w_row[base + j0 + u] = dot[u];
        }
      }
    }
  }
}

// Owner side, after the grouped GEMMs: one warp per staging slot (source s, token t).  Sums the result rows of the
// token's slots on this rank and stores one row into the source's return buffer at ret[rank*stride + t].
// WEIGHTED (forward): sum_k w_k * rows[p_k].   Otherwise (backward): sum_k rows[p_k], and the gating gradients
// d_w_row[p_k] go to the source's dw[t*K + k].
template <bool WEIGHTED>
__global__ void __launch_bounds__(kEpdWarps * 32)
epd_reduce_return_kernel(const uint4* __restrict__ rows, const int2* __restrict__ meta, const unsigned* __restrict__ mask,
                         const int* __restrict__ slots, const float* __restrict__ d_w_row,
                         const int* __restrict__ src_off, const int* __restrict__ counts_all, int G, int E, int rank,
                         int K, int vec_per_row, int stride, int capacity_rows, uint4* const* __restrict__ peer_ret,
                         float* const* __restrict__ peer_dw) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = static_cast<long long>(gridDim.x) * kEpdWarps;
  const long long n = static_cast<long long>(G) * stride;
  for (long long idx = static_cast<long long>(blockIdx.x) * kEpdWarps + (threadIdx.x >> 5); idx < n; idx += warps_total) {
    const int t = static_cast<int>(idx / G);
    const int s = static_cast<int>((idx % G + rank + 1) % G);  // neighbouring warps store to different sources
    const int tokens_s = (src_off[s * E + E - 1] + counts_all[s * E + E - 1]) / K;
    if (t >= tokens_s) continue;
    const long long slot = static_cast<long long>(s) * stride + t;
    unsigned m = mask[slot];
    if (K < 32) m &= (1u << K) - 1u;
    if (m == 0u) continue;
    int my_p = -1;
    float my_w = 1.f;
    if ((m >> lane) & 1u) my_p = slots[slot * K + lane];
    m = __ballot_sync(0xffffffffu, my_p >= 0 && my_p < capacity_rows);  // only rows inside the layout
    if (m == 0u) continue;
    if ((m >> lane) & 1u) {
      if (WEIGHTED) my_w = __int_as_float(meta[my_p].y);
      else peer_dw[s][static_cast<long long>(t) * K + lane] = d_w_row[my_p];
    }
    float acc[kEpdMaxVecPerLane][8];
#pragma unroll
    for (int i = 0; i < kEpdMaxVecPerLane; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
    unsigned rem = m;
    while (rem) {
      const int k = __ffs(rem) - 1;
      rem &= rem - 1;
      const long long p = __shfl_sync(0xffffffffu, my_p, k);
      const float w = __shfl_sync(0xffffffffu, my_w, k);
#pragma unroll
      for (int i = 0; i < kEpdMaxVecPerLane; ++i) {
        const int v = lane + 32 * i;
        if (v < vec_per_row) {
          float f[8];
          epd_unpack(rows[p * vec_per_row + v], f);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][q] = WEIGHTED ? fmaf(w, f[q], acc[i][q]) : acc[i][q] + f[q];
        }
      }
    }
    uint4* dst = peer_ret[s] + (static_cast<long long>(rank) * stride + t) * vec_per_row;
#pragma unroll
    for (int i = 0; i < kEpdMaxVecPerLane; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) dst[v] = epd_pack(acc[i]);
    }
  }
}

// Source side, after the barrier: out[t] = sum over the owners g (ascending) that hold a slot of token t of
// ret[g*stride + t].  One warp per token.
__global__ void __launch_bounds__(kEpdWarps * 32)
epd_sum_kernel(const uint4* __restrict__ ret, const int* __restrict__ sel, int T, int K, int El, int G, int vec_per_row,
               int stride, uint4* __restrict__ out, long long out_vec_stride) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * kEpdWarps;
  for (int t = blockIdx.x * kEpdWarps + (threadIdx.x >> 5); t < T; t += warps_total) {
    const int g = lane < K ? sel[t * K + lane] / El : -1;
    float acc[kEpdMaxVecPerLane][8];
#pragma unroll
    for (int i = 0; i < kEpdMaxVecPerLane; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
    for (int d = 0; d < G; ++d) {
      if (!__ballot_sync(0xffffffffu, g == d)) continue;
      const uint4* row = ret + (static_cast<long long>(d) * stride + t) * vec_per_row;
#pragma unroll
      for (int i = 0; i < kEpdMaxVecPerLane; ++i) {
        const int v = lane + 32 * i;
        if (v < vec_per_row) {
          float f[8];
          epd_unpack(row[v], f);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][q] += f[q];
        }
      }
    }
    uint4* dst = out + static_cast<long long>(t) * out_vec_stride;
#pragma unroll
    for (int i = 0; i < kEpdMaxVecPerLane; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) dst[v] = epd_pack(acc[i]);
    }
  }
}

static inline int epd_grid(long long warps) {
  long long b = (warps + kEpdWarps - 1) / kEpdWarps;
  if (b > 148ll * 16) b = 148ll * 16;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
static inline int epd_last_err() {
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
// The exchange kernels run on a side stream beside GEMMs of the main stream.  An SM runs kernels with different
// shared-memory carveouts only one after the other, so they ask for the GEMM kernel's (maximum) carveout.
static void epd_configure() {
  static PerDeviceOnce once;
  once.run([] {
  const int c = cudaSharedmemCarveoutMaxShared;
  cudaFuncSetAttribute(epd_send_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, c);
  cudaFuncSetAttribute(epd_send_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, c);
  cudaFuncSetAttribute(epd_reduce_return_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, c);
  cudaFuncSetAttribute(epd_reduce_return_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, c);
  return 0;
  });
}
static inline bool epd_dims_ok(int K, int E, int G, int rank, int L, int64_t stride) {
  return K > 0 && K <= 32 && G > 0 && G <= 256 && E > 0 && (E % G) == 0 && rank >= 0 && rank < G && L > 0 &&
         (L & 7) == 0 && L <= kEpdMaxVecPerLane * 256 && stride > 0 && stride * G < (1ll << 31);
}

}  // namespace lmoe

using namespace lmoe;

extern "C" int lmoe_epd_send(const void* src_rows, const int32_t* sel, const int32_t* pos, const int32_t* offsets,
                             const int32_t* dst_base, const float* weights, int64_t T, int K, int E, int G, int rank, int L,
                             int64_t capacity_rows, int64_t stride, void* const* peer_stage, void* const* peer_meta,
                             void* const* peer_mask, void* const* peer_slots, int32_t* status, void* stream) {
  if (!src_rows || !sel || !peer_stage) return LMOE_ERR_ARG;
  const bool with_meta = peer_meta != nullptr;
  if (with_meta && (!pos || !offsets || !dst_base || !weights || !peer_mask || !peer_slots)) return LMOE_ERR_ARG;
  if (!epd_dims_ok(K, E, G, rank, L, stride) || T <= 0 || T > stride || capacity_rows <= 0 ||
      capacity_rows >= (1ll << 31))
    return LMOE_ERR_SHAPE;
  epd_configure();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Forward (beside the SwiGLU GEMM, 152 registers per thread): one block per SM, so that whichever of the two kernels
  // reaches an SM first, the other still fits beside it.  Backward (beside a GEMM with a plain epilogue): registers are
  // no limit, eight blocks per SM leave the thread slots the GEMM CTA needs.
  long long blocks = (T + kEpdSendWarps - 1) / kEpdSendWarps;
  int sms = 0, device = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
    sms = 148;
  const long long cap = with_meta ? sms : 8ll * sms;
  if (blocks > cap) blocks = cap;
  const int grid = static_cast<int>(blocks);
  if (with_meta)
    epd_send_kernel<true><<<grid, kEpdSendWarps * 32, 0, st>>>(
        static_cast<const uint4*>(src_rows), sel, pos, offsets, dst_base, weights, static_cast<int>(T), K, E / G, G, rank,
        L / 8, static_cast<int>(capacity_rows), static_cast<int>(stride), reinterpret_cast<uint4* const*>(peer_stage),
        reinterpret_cast<int2* const*>(peer_meta), reinterpret_cast<unsigned* const*>(peer_mask),
        reinterpret_cast<int* const*>(peer_slots), status);
  else
    epd_send_kernel<false><<<grid, kEpdSendWarps * 32, 0, st>>>(
        static_cast<const uint4*>(src_rows), sel, nullptr, nullptr, nullptr, nullptr, static_cast<int>(T), K, E / G, G,
        rank, L / 8, static_cast<int>(capacity_rows), static_cast<int>(stride),
        reinterpret_cast<uint4* const*>(peer_stage), nullptr, nullptr, nullptr, status);
  return epd_last_err();
}

extern "C" int lmoe_epd_gather(const void* stage, const void* meta, const int32_t* tile_expert, const int32_t* n_tiles,
                               const int32_t* pad_offsets, const int32_t* seg_cum, const int32_t* counts_all, int G, int E,
                               int rank, int L, int64_t capacity_rows, int64_t n_slots, const void* y_sorted,
                               void* out_rows, float* d_w_row, void* stream) {
  if (!stage || !meta || !tile_expert || !n_tiles || !pad_offsets || !seg_cum || !counts_all || !out_rows)
    return LMOE_ERR_ARG;
  if ((y_sorted == nullptr) != (d_w_row == nullptr)) return LMOE_ERR_ARG;
  if (!epd_dims_ok(1, E, G, rank, L, 1) || n_slots <= 0 || capacity_rows <= 0 || (capacity_rows % LMOE_ROW_PAD) != 0 ||
      capacity_rows >= (1ll << 31))
    return LMOE_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = epd_grid((capacity_rows + 31) / 32);
  if (y_sorted)
    epd_gather_kernel<true><<<grid, kEpdWarps * 32, 0, st>>>(
        static_cast<const uint4*>(stage), static_cast<const int2*>(meta), tile_expert, n_tiles, pad_offsets, seg_cum,
        counts_all, G, E, rank, L / 8, static_cast<int>(capacity_rows), n_slots, static_cast<const uint4*>(y_sorted),
        static_cast<uint4*>(out_rows), d_w_row);
  else
    epd_gather_kernel<false><<<grid, kEpdWarps * 32, 0, st>>>(
        static_cast<const uint4*>(stage), static_cast<const int2*>(meta), tile_expert, n_tiles, pad_offsets, seg_cum,
        counts_all, G, E, rank, L / 8, static_cast<int>(capacity_rows), n_slots, nullptr, static_cast<uint4*>(out_rows),
        nullptr);
  return epd_last_err();
}

extern "C" int lmoe_epd_reduce_return(const void* rows, const void* meta, const void* mask, const int32_t* slots,
                                      const float* d_w_row, const int32_t* src_off, const int32_t* counts_all, int G, int E,
                                      int rank, int K, int L, int64_t stride, int64_t capacity_rows,
                                      void* const* peer_ret, void* const* peer_dw, void* stream) {
  if (!rows || !meta || !mask || !slots || !src_off || !counts_all || !peer_ret) return LMOE_ERR_ARG;
  if ((d_w_row == nullptr) != (peer_dw == nullptr)) return LMOE_ERR_ARG;
  if (!epd_dims_ok(K, E, G, rank, L, stride) || capacity_rows <= 0 || capacity_rows >= (1ll << 31))
    return LMOE_ERR_SHAPE;
  epd_configure();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = epd_grid(static_cast<long long>(G) * stride);
  if (d_w_row)
    epd_reduce_return_kernel<false><<<grid, kEpdWarps * 32, 0, st>>>(
        static_cast<const uint4*>(rows), static_cast<const int2*>(meta), static_cast<const unsigned*>(mask), slots,
        d_w_row, src_off, counts_all, G, E, rank, K, L / 8, static_cast<int>(stride), static_cast<int>(capacity_rows),
        reinterpret_cast<uint4* const*>(peer_ret), reinterpret_cast<float* const*>(peer_dw));
  else
    epd_reduce_return_kernel<true><<<grid, kEpdWarps * 32, 0, st>>>(
        static_cast<const uint4*>(rows), static_cast<const int2*>(meta), static_cast<const unsigned*>(mask), slots, nullptr,
        src_off, counts_all, G, E, rank, K, L / 8, static_cast<int>(stride), static_cast<int>(capacity_rows),
        reinterpret_cast<uint4* const*>(peer_ret), nullptr);
  return epd_last_err();
}

extern "C" int lmoe_epd_sum(const void* ret, const int32_t* sel, int64_t T, int K, int E, int G, int L, int64_t stride,
                            void* out, int64_t ld_out, void* stream) {
  if (!ret || !sel || !out) return LMOE_ERR_ARG;
  if (!epd_dims_ok(K, E, G, 0, L, stride) || T <= 0 || T > stride || ld_out < L || (ld_out & 7) != 0)
    return LMOE_ERR_SHAPE;
  epd_sum_kernel<<<epd_grid(T), kEpdWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(ret), sel, static_cast<int>(T), K, E / G, G, L / 8, static_cast<int>(stride),
      static_cast<uint4*>(out), ld_out / 8);
  return epd_last_err();
}

// ---------------------------------------------------------------- barrier across the ranks on flag words
// Every rank owns int32 flags[G] in symmetric memory; word s is written by rank s only.  The barrier's number comes from
// a counter in this rank's own memory that the kernel increments (every rank runs the same sequence of barriers, so
// the counters agree; a counter on the device keeps the kernel valid inside a replayed CUDA graph).  One warp: thread j
// stores the number into rank j's word for this rank (system-scope release), then waits until rank j's number has
// arrived in this rank's word j (system-scope acquire).  Stream order puts the exchange kernels queued before it in
// front of the stores, and what is queued after it behind the loads.  The wait is bounded (about two seconds): on
// expiry the kernel records status 202 and returns, so a rank that never arrives ends a step with an error instead of a
// hang.
constexpr long long kEpdBarrierBudgetCycles = 4000000000LL;
__global__ void __launch_bounds__(32) epd_flag_barrier_kernel(int* const* peer_flags, int* epoch_counter, int rank, int G,
                                                              int* status) {
  const int j = threadIdx.x;
  int epoch = 0;
  if (j == 0) {
    epoch = *epoch_counter + 1;
    *epoch_counter = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (j >= G) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flags[j] + rank), "r"(epoch) : "memory");
  const int* mine = peer_flags[rank] + j;
  const long long t0 = clock64();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - epoch >= 0) break;
    if (clock64() - t0 > kEpdBarrierBudgetCycles) {
      if (status) atomicCAS(status, 0, 202);
      break;
    }
  }
}

extern "C" int lmoe_ep_flag_barrier(void* const* peer_flags, int32_t* epoch_counter, int rank, int G, int32_t* status,
                                    void* stream) {
  if (!peer_flags || !epoch_counter || G < 1 || G > 32 || rank < 0 || rank >= G) return LMOE_ERR_ARG;
  epd_flag_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int* const*>(peer_flags),
                                                                           epoch_counter, rank, G, status);
  return epd_last_err();
}
