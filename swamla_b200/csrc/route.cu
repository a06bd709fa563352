// Router kernels: warp-level top-k with z-loss, and the deterministic histogram / scan / stable
// permutation that lays the (token, slot) pairs out expert by expert.  All HBM-bound integer work.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <mutex>

#include "../../include/lmoe.h"
#include "counters.h"
#include "device_once.h"

namespace lmoe {

constexpr int kTopkWarpsPerBlock = 8;
constexpr int kMaxPerLane = LMOE_MAX_EXPERTS / 32;  // 8 scores per lane at E = 256

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }


// One warp per token row.  Lane l holds experts l, l+32, ...
__global__ void __launch_bounds__(kTopkWarpsPerBlock * 32)
gate_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int K,
                 int* __restrict__ sel, float* __restrict__ weights, float* __restrict__ lse_out,
                 float* __restrict__ z_partial) {
  __shared__ float s_lse2[kTopkWarpsPerBlock];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kTopkWarpsPerBlock + warp;
  float lse2 = 0.f;
  if (t < T) {
    float aff[kMaxPerLane], score[kMaxPerLane];
    const float* row = logits + static_cast<long long>(t) * E;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        const float x = row[e];
        mx = fmaxf(mx, x);
        aff[j] = sigmoid_f(x);
        score[j] = aff[j] + bias[e];
      } else {
        aff[j] = 0.f;
        score[j] = -CUDART_INF_F;
      }
    }
    // logsumexp over the row
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e < E) se += expf(row[e] - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    const float lse = mx + logf(se);
    lse2 = lse * lse;
    if (lane == 0) lse_out[t] = lse;

    // Order-preserving 32-bit keys: key(a) > key(b) <=> a > b (with -0 folded onto +0), so that the
    // warp-wide maximum is one redux instruction.  Ties go to the lower expert index through a
    // second redux (minimum index among the lanes that hold the maximum).
    unsigned key[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const unsigned u = __float_as_uint(score[j] + 0.0f);
      key[j] = (lane + 32 * j < E) ? ((u & 0x80000000u) ? ~u : (u | 0x80000000u)) : 0u;
    }
    float my_aff = 0.f;  // lane k keeps the affinity of the k-th winner
    int my_idx = 0;
    float aff_sum = 0.f;
    for (int k = 0; k < K; ++k) {
      unsigned bk = 0u;
      int bj = 0;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        if (key[j] > bk) {  // strict: the lowest j (lowest expert index) wins a tie inside the lane
          bk = key[j];
          bj = j;
        }
      }
      const unsigned wmax = __reduce_max_sync(0xffffffffu, bk);
      const unsigned cand = (bk == wmax) ? static_cast<unsigned>(lane + 32 * bj) : 0xffffffffu;
      const int bi = static_cast<int>(__reduce_min_sync(0xffffffffu, cand));
      const int wl = bi & 31;
      float la = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (j == bj) la = aff[j];
      const float ba = __shfl_sync(0xffffffffu, la, wl);
      if (lane == wl) {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j)
          if (j == (bi >> 5)) key[j] = 0u;  // retire the winner (every live key has its top bit pattern > 0)
      }
      if (lane == k) {
        my_aff = ba;
        my_idx = bi;
      }
      aff_sum += ba;  // same order on every lane: slot 0, 1, ...
    }
    if (lane < K) {
      sel[static_cast<long long>(t) * K + lane] = my_idx;
      weights[static_cast<long long>(t) * K + lane] = my_aff / (aff_sum + 1e-9f);
    }
  }
  if (lane == 0) s_lse2[warp] = lse2;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < kTopkWarpsPerBlock; ++i) s += s_lse2[i];
    z_partial[blockIdx.x] = s;
  }
}

// Same result for E = 32 * PER: lane l holds the PER CONSECUTIVE experts l*PER .. l*PER+PER-1, so "lower expert index
// first" is "lower lane first, then lower slot inside the lane": the arg-max of a round is one redux (maximum key), one
// ballot (which lanes hold it) and a find-first-set, instead of two reductions.
template <int PER>
__global__ void __launch_bounds__(kTopkWarpsPerBlock * 32)
gate_topk_blocked_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int K,
                         int* __restrict__ sel, float* __restrict__ weights, float* __restrict__ lse_out,
                         float* __restrict__ z_partial) {
  constexpr int E = 32 * PER;
  __shared__ float s_lse2[kTopkWarpsPerBlock];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kTopkWarpsPerBlock + warp;
  float lse2 = 0.f;
  if (t < T) {
    float x[PER], aff[PER];
    unsigned key[PER];
    const float* row = logits + static_cast<long long>(t) * E + lane * PER;
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      x[j] = row[j];
      mx = fmaxf(mx, x[j]);
      aff[j] = sigmoid_f(x[j]);
      const unsigned u = __float_as_uint((aff[j] + bias[lane * PER + j]) + 0.0f);
      key[j] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) se += expf(x[j] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    const float lse = mx + logf(se);
    lse2 = lse * lse;
    if (lane == 0) lse_out[t] = lse;

    float my_aff = 0.f;
    int my_idx = 0;
    float aff_sum = 0.f;
    for (int k = 0; k < K; ++k) {
      unsigned bk = 0u;
      int bj = 0;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        if (key[j] > bk) {  // strict: the lowest slot wins a tie inside the lane
          bk = key[j];
          bj = j;
        }
      }
      const unsigned wmax = __reduce_max_sync(0xffffffffu, bk);
      const unsigned holders = __ballot_sync(0xffffffffu, bk == wmax);
      const int wl = __ffs(holders) - 1;  // lowest lane = lowest expert index among the maxima
      float la = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j)
        if (j == bj) la = aff[j];
      const float ba = __shfl_sync(0xffffffffu, la, wl);
      const int bi = __shfl_sync(0xffffffffu, lane * PER + bj, wl);
      if (lane == wl) {
#pragma unroll
        for (int j = 0; j < PER; ++j)
          if (j == bj) key[j] = 0u;
      }
      if (lane == k) {
        my_aff = ba;
        my_idx = bi;
      }
      aff_sum += ba;
    }
    if (lane < K) {
      sel[static_cast<long long>(t) * K + lane] = my_idx;
      weights[static_cast<long long>(t) * K + lane] = my_aff / (aff_sum + 1e-9f);
    }
  }
  if (lane == 0) s_lse2[warp] = lse2;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < kTopkWarpsPerBlock; ++i) s += s_lse2[i];
    z_partial[blockIdx.x] = s;
  }
}

// Deterministic final reduction of the z-loss partials (fixed order, one block).
__global__ void __launch_bounds__(256) zloss_finalize_kernel(const float* __restrict__ partial, int n, float scale,
                                                             float* __restrict__ z_loss) {
  __shared__ double s[256];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += 256) acc += static_cast<double>(partial[i]);
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) z_loss[0] = static_cast<float>(s[0] * static_cast<double>(scale));
}

// ----------------------------------------------------------------------------- routing tables
// The flat (token, slot) list is cut into chunks of kChunk entries, one warp per chunk.
constexpr int kChunk = 256;
constexpr int kRouteWarps = 8;

// Pass 1: per-chunk histogram -> chunk_hist[chunk][E].
__global__ void __launch_bounds__(kRouteWarps * 32)
route_hist_kernel(const int* __restrict__ sel, int n, int E, int* __restrict__ chunk_hist) {
  __shared__ int hist[kRouteWarps][LMOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * kRouteWarps + warp;
  for (int e = lane; e < E; e += 32) hist[warp][e] = 0;
  __syncwarp();
  const long long base = static_cast<long long>(chunk) * kChunk;
  if (base < n) {
    for (int s = 0; s < kChunk; s += 32) {
      const long long i = base + s + lane;
      const bool valid = i < n;
      const int e = valid ? sel[i] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (valid && (__ffs(peers) - 1) == lane) hist[warp][e] += __popc(peers);  // one writer per distinct expert
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) chunk_hist[static_cast<long long>(chunk) * E + e] = hist[warp][e];
  }
}

// Pass 2: one block per expert: exclusive scan of that expert's counts over the chunks (in place),
// total -> counts[e].
__global__ void __launch_bounds__(256) route_scan_chunks_kernel(int* __restrict__ chunk_hist, int n_chunks, int E,
                                                                int* __restrict__ counts) {
  __shared__ int warp_sums[8];
  __shared__ int carry_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < n_chunks; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const int v = (c < n_chunks) ? chunk_hist[static_cast<long long>(c) * E + e] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int warp_off = 0;
    for (int w = 0; w < warp; ++w) warp_off += warp_sums[w];
    const int carry = carry_s;
    if (c < n_chunks) chunk_hist[static_cast<long long>(c) * E + e] = carry + warp_off + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = carry + warp_off + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = carry_s;
}

// Pass 3: stable scatter.  Every block first scans the per-expert counts in shared memory (canonical
// and padded offsets); block b also publishes the tables of experts b, b + gridDim.x, ... (offsets,
// tile -> expert entries, -1 markers of the pad rows).  Then each warp walks its chunk in index order
// again: rank inside the warp step by match_any + popc, running per-expert cursors in shared memory.
__global__ void __launch_bounds__(kRouteWarps * 32)
route_scatter_kernel(const int* __restrict__ sel, int n, int E, const int* __restrict__ chunk_base,
                     const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ pad_offsets,
                     int* __restrict__ tile_expert, int* __restrict__ n_tiles, int* __restrict__ perm,
                     int* __restrict__ pos, int* __restrict__ row_src) {
  __shared__ int cursor[kRouteWarps][LMOE_MAX_EXPERTS];
  __shared__ int s_off[LMOE_MAX_EXPERTS + 1], s_poff[LMOE_MAX_EXPERTS + 1], s_cnt[LMOE_MAX_EXPERTS];
  __shared__ int s_wsum[2][kRouteWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tid = threadIdx.x;  // blockDim.x == LMOE_MAX_EXPERTS == 256
  {
    const int c = (tid < E) ? counts[tid] : 0;
    const int pc = (c + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD * LMOE_ROW_PAD;
    int ic = c, ip = pc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, ip, o);
      if (lane >= o) {
        ic += a;
        ip += b;
      }
    }
    if (lane == 31) {
      s_wsum[0][warp] = ic;
      s_wsum[1][warp] = ip;
    }
    __syncthreads();
    int wc = 0, wp = 0;
    for (int w = 0; w < warp; ++w) {
      wc += s_wsum[0][w];
      wp += s_wsum[1][w];
    }
    if (tid < E) {
      s_cnt[tid] = c;
      s_off[tid] = wc + ic - c;
      s_poff[tid] = wp + ip - pc;
      if (tid == E - 1) {
        s_off[E] = wc + ic;
        s_poff[E] = wp + ip;
      }
    }
    __syncthreads();
  }
  // publish the tables of the experts this block is responsible for
  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    if (tid == 0) {
      offsets[e] = s_off[e];
      pad_offsets[e] = s_poff[e];
    }
    for (int t = s_poff[e] / LMOE_ROW_PAD + tid; t < s_poff[e + 1] / LMOE_ROW_PAD; t += blockDim.x) tile_expert[t] = e;
    for (int r = s_poff[e] + s_cnt[e] + tid; r < s_poff[e + 1]; r += blockDim.x) row_src[r] = -1;
  }
  if (blockIdx.x == 0 && tid == 0) {
    offsets[E] = s_off[E];
    pad_offsets[E] = s_poff[E];
    n_tiles[0] = s_poff[E] / LMOE_ROW_PAD;
  }

  const int chunk = blockIdx.x * kRouteWarps + warp;
  const long long base = static_cast<long long>(chunk) * kChunk;
  if (base >= n) return;
  for (int e = lane; e < E; e += 32) cursor[warp][e] = chunk_base[static_cast<long long>(chunk) * E + e];
  __syncwarp();
  for (int s = 0; s < kChunk; s += 32) {
    const long long i = base + s + lane;
    const bool valid = i < n;
    const int e = valid ? sel[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (valid) {
      const int rank = cursor[warp][e] + __popc(peers & ((1u << lane) - 1u));
      perm[s_off[e] + rank] = static_cast<int>(i);
      const int prow = s_poff[e] + rank;
      pos[i] = prow;
      row_src[prow] = static_cast<int>(i);
    }
    __syncwarp();
    if (valid && (__ffs(peers) - 1) == lane) cursor[warp][e] += __popc(peers);
    __syncwarp();
  }
}

// Router bias update from the routing histogram.  The expected load per expert is taken from the histogram itself
// (sum of the counts / E = tokens * K / E): a histogram summed over several ranks then gives the global figure
// whatever the ranks' own token counts were.  One block; E <= LMOE_MAX_EXPERTS threads carry one expert each.
__global__ void __launch_bounds__(LMOE_MAX_EXPERTS)
bias_update_kernel(const int* __restrict__ counts, int E, float gamma, float* __restrict__ bias,
                   float* __restrict__ history) {
  __shared__ long long total_s;
  const int e = threadIdx.x;
  const int c = (e < E) ? counts[e] : 0;
  if (e == 0) total_s = 0;
  __syncthreads();
  long long part = c;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((e & 31) == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&total_s), static_cast<unsigned long long>(part));
  __syncthreads();
  if (e >= E) return;
  const float expected = static_cast<float>(static_cast<double>(total_s) / static_cast<double>(E));
  const float load = static_cast<float>(c);
  const float d = load - expected;
  const float sg = (d > 0.f) ? 1.f : ((d < 0.f) ? -1.f : 0.f);
  bias[e] -= gamma * sg;
  history[e] = 0.99f * history[e] + 0.01f * load;
}

// Kernels of this file that use static shared memory ask for the same (maximum) shared-memory carveout as the GEMM
// kernel: an SM runs kernels with different carveouts only one after the other, and these kernels are meant to run
// beside a GEMM of another stream.
template <typename F>
static inline void prefer_max_carveout(F* fn) {
  cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}
static void configure_route_kernels() {
  static PerDeviceOnce once;
  once.run([] {
  prefer_max_carveout(gate_topk_kernel);
  prefer_max_carveout(gate_topk_blocked_kernel<1>);
  prefer_max_carveout(gate_topk_blocked_kernel<2>);
  prefer_max_carveout(gate_topk_blocked_kernel<4>);
  prefer_max_carveout(gate_topk_blocked_kernel<8>);
  prefer_max_carveout(zloss_finalize_kernel);
  prefer_max_carveout(route_hist_kernel);
  prefer_max_carveout(route_scan_chunks_kernel);
  prefer_max_carveout(route_scatter_kernel);
  return 0;
  });
}

static inline int check_shape(const lmoe_shape* s) {
  if (!s) return LMOE_ERR_ARG;
  if (s->T <= 0 || s->E <= 0 || s->E > LMOE_MAX_EXPERTS || s->K <= 0 || s->K > LMOE_MAX_TOPK || s->K > s->E)
    return LMOE_ERR_SHAPE;
  if (static_cast<long long>(s->T) * s->K >= (1ll << 31)) return LMOE_ERR_SHAPE;
  return 0;
}

}  // namespace lmoe

using namespace lmoe;

extern "C" int lmoe_gate_topk_fwd(const lmoe_shape* s, const float* logits, const float* expert_bias, float z_coef,
                                  int32_t* sel, float* weights, float* lse, float* z_partial, float* z_loss,
                                  void* stream) {
  if (int rc = check_shape(s)) return rc;
  if (!logits || !expert_bias || !sel || !weights || !lse || !z_partial || !z_loss) return LMOE_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  configure_route_kernels();
  const int blocks = (s->T + kTopkWarpsPerBlock - 1) / kTopkWarpsPerBlock;
  const int thr = kTopkWarpsPerBlock * 32;
  switch (s->E) {  // blocked layout when the expert count is a multiple of the warp size
    case 32: gate_topk_blocked_kernel<1><<<blocks, thr, 0, st>>>(logits, expert_bias, s->T, s->K, sel, weights, lse, z_partial); break;
    case 64: gate_topk_blocked_kernel<2><<<blocks, thr, 0, st>>>(logits, expert_bias, s->T, s->K, sel, weights, lse, z_partial); break;
    case 128: gate_topk_blocked_kernel<4><<<blocks, thr, 0, st>>>(logits, expert_bias, s->T, s->K, sel, weights, lse, z_partial); break;
    case 256: gate_topk_blocked_kernel<8><<<blocks, thr, 0, st>>>(logits, expert_bias, s->T, s->K, sel, weights, lse, z_partial); break;
    default:
      gate_topk_kernel<<<blocks, thr, 0, st>>>(logits, expert_bias, s->T, s->E, s->K, sel, weights, lse, z_partial);
  }
  count_launch(2);
  zloss_finalize_kernel<<<1, 256, 0, st>>>(z_partial, blocks, z_coef / static_cast<float>(s->T), z_loss);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

extern "C" size_t lmoe_route_workspace_bytes(const lmoe_shape* s) {
  if (check_shape(s)) return 0;
  const long long n = static_cast<long long>(s->T) * s->K;
  const long long chunks = (n + kChunk - 1) / kChunk;
  return static_cast<size_t>(chunks) * s->E * sizeof(int);
}

extern "C" int64_t lmoe_padded_rows(const lmoe_shape* s) {
  if (check_shape(s)) return 0;
  const long long n = static_cast<long long>(s->T) * s->K;
  return (n + LMOE_ROW_PAD - 1) / LMOE_ROW_PAD * LMOE_ROW_PAD + static_cast<long long>(s->E) * LMOE_ROW_PAD;
}

extern "C" int lmoe_route_permute(const lmoe_shape* s, const int32_t* sel, const lmoe_route* r, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  if (int rc = check_shape(s)) return rc;
  if (!sel || !r || !workspace || !r->counts || !r->offsets || !r->perm || !r->pad_offsets || !r->pos || !r->row_src ||
      !r->tile_expert || !r->n_tiles)
    return LMOE_ERR_ARG;
  if (workspace_bytes < lmoe_route_workspace_bytes(s)) return LMOE_ERR_WORKSPACE;
  configure_route_kernels();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = s->T * s->K;
  const int chunks = (n + kChunk - 1) / kChunk;
  const int blocks = (chunks + kRouteWarps - 1) / kRouteWarps;
  int* chunk_hist = static_cast<int*>(workspace);
  count_launch(3);
  route_hist_kernel<<<blocks, kRouteWarps * 32, 0, st>>>(sel, n, s->E, chunk_hist);
  route_scan_chunks_kernel<<<s->E, 256, 0, st>>>(chunk_hist, chunks, s->E, r->counts);
  route_scatter_kernel<<<blocks, kRouteWarps * 32, 0, st>>>(sel, n, s->E, chunk_hist, r->counts, r->offsets,
                                                           r->pad_offsets, r->tile_expert, r->n_tiles, r->perm, r->pos,
                                                           r->row_src);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// ----------------------------------------------------------------------------- no-allocation variant
// Scratch of lmoe_route_permute_static: the per-chunk histograms live in this file-scope device array
// instead of a caller-provided workspace.  Every GPU that loads the library holds these 4 MiB until
// the process exits.  Host code must not hand `g_route_scratch` itself to a kernel (in host code the
// name is only a handle): the device address is looked up once per device with cudaGetSymbolAddress.
constexpr size_t kStaticRouteScratchInts = LMOE_STATIC_ROUTE_SCRATCH_BYTES / sizeof(int);
static __device__ __align__(256) int g_route_scratch[kStaticRouteScratchInts];

namespace {
std::mutex g_static_scratch_mutex;
int* g_static_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the CURRENT device; resolved on the first call per device.
int static_route_scratch(int** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return LMOE_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!p) return LMOE_ERR_DRIVER;
    g_static_scratch_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int lmoe_route_permute_static(const lmoe_shape* s, const int32_t* sel, const lmoe_route* r, void* stream) {
  if (int rc = check_shape(s)) return rc;
  if (!sel || !r || !r->counts || !r->offsets || !r->perm || !r->pad_offsets || !r->pos || !r->row_src ||
      !r->tile_expert || !r->n_tiles)
    return LMOE_ERR_ARG;
  if (lmoe_route_workspace_bytes(s) > LMOE_STATIC_ROUTE_SCRATCH_BYTES) return LMOE_ERR_TOO_LARGE;
  int* chunk_hist = nullptr;
  if (int rc = static_route_scratch(&chunk_hist)) return rc;
  configure_route_kernels();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = s->T * s->K;
  const int chunks = (n + kChunk - 1) / kChunk;
  const int blocks = (chunks + kRouteWarps - 1) / kRouteWarps;
  // Nothing in the scratch has to start at zero: pass 1 writes every word that passes 2 and 3 read,
  // so what an earlier call left behind is never observed.
  count_launch(3);
  route_hist_kernel<<<blocks, kRouteWarps * 32, 0, st>>>(sel, n, s->E, chunk_hist);
  route_scan_chunks_kernel<<<s->E, 256, 0, st>>>(chunk_hist, chunks, s->E, r->counts);
  route_scatter_kernel<<<blocks, kRouteWarps * 32, 0, st>>>(sel, n, s->E, chunk_hist, r->counts, r->offsets,
                                                           r->pad_offsets, r->tile_expert, r->n_tiles, r->perm, r->pos,
                                                           r->row_src);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

extern "C" int lmoe_router_bias_update(const lmoe_shape* s, const int32_t* counts, float gamma, float* expert_bias,
                                       float* load_history, void* stream) {
  if (int rc = check_shape(s)) return rc;
  if (!counts || !expert_bias || !load_history) return LMOE_ERR_ARG;
  count_launch();
  bias_update_kernel<<<1, LMOE_MAX_EXPERTS, 0, static_cast<cudaStream_t>(stream)>>>(counts, s->E, gamma, expert_bias,
                                                                                    load_history);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
