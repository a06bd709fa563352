// HBM-bound row kernels of the LatentMoE path: gather into the padded expert layout, weighted
// combine and its adjoint, SwiGLU adjoint, router adjoint, dtype casts.  One warp per row, 16-byte
// vector accesses, fp32 arithmetic.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"
#include "device_once.h"
#include "rowops.h"

namespace lmoe {

constexpr int kRowWarps = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// The three gather-type kernels below keep several independent 16-byte loads per lane in flight (rows are taken four
// or two at a time, the K rows of a token four at a time): with one row per warp at a time the bytes in flight per SM
// were too few for the HBM latency and the kernels ran at half the copy bandwidth.
constexpr int kGatherUnroll = 4;

// x_sorted[row] = x_latent[row_src[row] / K]  (zeros for pad rows); rows < 128 * n_tiles[0].
__global__ void __launch_bounds__(kRowWarps * 32)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ row_src, const int* __restrict__ n_tiles, int K,
                   int vec_per_row, uint4* __restrict__ dst, long long max_rows) {
  const int lane = threadIdx.x & 31;
  const long long rows = n_tiles ? min(static_cast<long long>(n_tiles[0]) * LMOE_ROW_PAD, max_rows) : max_rows;
  const long long warps_total = static_cast<long long>(gridDim.x) * kRowWarps;
  for (long long row0 = (static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5)) * kGatherUnroll; row0 < rows;
       row0 += warps_total * kGatherUnroll) {
    long long from[kGatherUnroll];  // source row, -1: pad row (zeros), -2: beyond the rows in use
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const long long row = row0 + u;
      from[u] = -2;
      if (row < rows) {
        const int flat = row_src[row];
        from[u] = flat >= 0 ? flat / K : -1;
      }
    }
    for (int v = lane; v < vec_per_row; v += 32) {
      uint4 x[kGatherUnroll];
#pragma unroll
      for (int u = 0; u < kGatherUnroll; ++u)
        x[u] = from[u] >= 0 ? src[from[u] * vec_per_row + v] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kGatherUnroll; ++u)
        if (from[u] != -2) dst[(row0 + u) * vec_per_row + v] = x[u];
    }
  }
}

// out[t] = (addend[t] +) sum_k w[t,k] * y[pos[t*K+k]]   (w == nullptr: plain sum).  Slot order k = 0..K-1, fp32.
__global__ void __launch_bounds__(kRowWarps * 32)
combine_kernel(const uint4* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ w, int T, int K,
               int vec_per_row, uint4* __restrict__ out, long long out_ld_vec, const uint4* __restrict__ addend,
               long long addend_ld_vec) {
  const int lane = threadIdx.x & 31;
  for (long long t = static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5); t < T;
       t += static_cast<long long>(gridDim.x) * kRowWarps) {
    for (int v = lane; v < vec_per_row; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (addend) unpack8(addend[t * addend_ld_vec + v], acc);
      for (int k0 = 0; k0 < K; k0 += kGatherUnroll) {
        uint4 rows[kGatherUnroll];
        float wk[kGatherUnroll];
#pragma unroll
        for (int u = 0; u < kGatherUnroll; ++u) {
          const long long i = t * K + min(k0 + u, K - 1);
          wk[u] = w ? w[i] : 1.0f;
          rows[u] = y[static_cast<long long>(pos[i]) * vec_per_row + v];
        }
#pragma unroll
        for (int u = 0; u < kGatherUnroll; ++u) {
          if (k0 + u < K) {  // slot order is kept: the sum has the same bits as a one-row-at-a-time loop
            float f[8];
            unpack8(rows[u], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(wk[u], f[j], acc[j]);
          }
        }
      }
      out[t * out_ld_vec + v] = pack8(acc);
    }
  }
}

// Adjoint of the weighted combine over padded rows:
//   d_y[row] = w[flat] * d_routed[t],  d_w[flat] = <d_routed[t], y[row]>,  pad rows -> 0.
__global__ void __launch_bounds__(kRowWarps * 32)
combine_bwd_kernel(const uint4* __restrict__ d_routed, const uint4* __restrict__ y, const float* __restrict__ w,
                   const int* __restrict__ row_src, const int* __restrict__ n_tiles, int K, int vec_per_row,
                   uint4* __restrict__ d_y, float* __restrict__ d_w, long long max_rows) {
  constexpr int U = 1;  // rows per warp iteration (two measured 8 us slower at 204k rows: 57 against 49 us)
  const int lane = threadIdx.x & 31;
  const long long rows = n_tiles ? min(static_cast<long long>(n_tiles[0]) * LMOE_ROW_PAD, max_rows) : max_rows;
  const long long warps_total = static_cast<long long>(gridDim.x) * kRowWarps;
  for (long long row0 = (static_cast<long long>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5)) * U; row0 < rows;
       row0 += warps_total * U) {
    int flat[U];
    float wk[U], dot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      flat[u] = (row0 + u < rows) ? row_src[row0 + u] : -2;  // -1: pad row, -2: beyond the rows in use
      wk[u] = flat[u] >= 0 ? w[flat[u]] : 0.f;
      dot[u] = 0.f;
    }
    for (int v = lane; v < vec_per_row; v += 32) {
      uint4 g4[U], y4[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        g4[u] = flat[u] >= 0 ? d_routed[static_cast<long long>(flat[u] / K) * vec_per_row + v] : make_uint4(0, 0, 0, 0);
        y4[u] = flat[u] >= 0 ? y[(row0 + u) * vec_per_row + v] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (flat[u] == -2) continue;
        float g[8], yy[8], o[8];
        unpack8(g4[u], g);
        unpack8(y4[u], yy);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot[u] = fmaf(g[j], yy[j], dot[u]);
          o[j] = wk[u] * g[j];
        }
        d_y[(row0 + u) * vec_per_row + v] = pack8(o);  // pad rows: w = 0 and g = 0 -> zeros
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
      if (lane == 0 && flat[u] >= 0) d_w[flat[u]] = dot[u];
    }
  }
}

// d_h1 = swiglu'(h1, d_hidden): gate g = h1[:, :H], up u = h1[:, H:];
//   d_u = d_h * silu(g);  d_g = d_h * u * sig(g) * (1 + g * (1 - sig(g))).
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const uint4* __restrict__ h1, const uint4* __restrict__ d_hidden, uint4* __restrict__ d_h1,
                  long long rows_host, const int* __restrict__ n_tiles, int vec_per_half, long long out_ld_vec) {
  long long rows = rows_host;
  if (n_tiles) rows = min(rows, static_cast<long long>(n_tiles[0]) * LMOE_ROW_PAD);
  const long long total = rows * vec_per_half;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_half;
    const int v = static_cast<int>(i - r * vec_per_half);
    float g[8], u[8], dh[8], dg[8], du[8];
    unpack8(h1[r * 2 * vec_per_half + v], g);
    unpack8(h1[r * 2 * vec_per_half + vec_per_half + v], u);
    unpack8(d_hidden[r * vec_per_half + v], dh);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.0f / (1.0f + __expf(-g[j]));
      du[j] = dh[j] * g[j] * sg;
      dg[j] = dh[j] * u[j] * sg * (1.0f + g[j] * (1.0f - sg));
    }
    d_h1[r * out_ld_vec + v] = pack8(dg);
    d_h1[r * out_ld_vec + vec_per_half + v] = pack8(du);
  }
}

// Router adjoint, one warp per token: dense d_logits row (bf16).
//   selected k: a = sig(logit), S = sum_j a_j + 1e-9, w = a / S,
//               d_a = (d_w_k - sum_j d_w_j w_j) / S,  d_logit = d_a * a (1 - a)
//   all e:      + d_z * z_coef * 2 * lse * softmax(logits)_e / T
__global__ void __launch_bounds__(kRowWarps * 32)
gate_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ sel, const float* __restrict__ w,
                const float* __restrict__ d_w, const float* __restrict__ lse, const float* __restrict__ d_z,
                float z_scale, int T, int E, int K, __nv_bfloat16* __restrict__ d_logits, long long out_ld) {
  __shared__ float rowbuf[kRowWarps][LMOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float dz = d_z ? d_z[0] * z_scale : 0.f;
  for (long long t = static_cast<long long>(blockIdx.x) * kRowWarps + warp; t < T;
       t += static_cast<long long>(gridDim.x) * kRowWarps) {
    const float* row = logits + t * E;
    const float l = lse[t];
    for (int e = lane; e < E; e += 32) rowbuf[warp][e] = (dz != 0.f) ? dz * 2.0f * l * expf(row[e] - l) : 0.f;
    __syncwarp();
    // per-slot quantities on lanes < K
    float a = 0.f, wk = 0.f, dwk = 0.f;
    int e_sel = 0;
    if (lane < K) {
      e_sel = sel[t * K + lane];
      a = 1.0f / (1.0f + expf(-row[e_sel]));
      wk = w[t * K + lane];
      dwk = d_w[t * K + lane];
    }
    float asum = a, dot = dwk * wk;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      asum += __shfl_xor_sync(0xffffffffu, asum, o);
      dot += __shfl_xor_sync(0xffffffffu, dot, o);
    }
    if (lane < K) {
      const float S = asum + 1e-9f;
      const float da = (dwk - dot) / S;
      rowbuf[warp][e_sel] += da * a * (1.0f - a);  // experts are distinct within a row
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) d_logits[t * out_ld + e] = __float2bfloat16_rn(rowbuf[warp][e]);
    __syncwarp();
  }
}

__global__ void cast_f32_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, long long n4,
                                     const float* __restrict__ src_tail, __nv_bfloat16* __restrict__ dst_tail, int tail) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = src[i];
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    dst[i] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail) dst_tail[threadIdx.x] = __float2bfloat16_rn(src_tail[threadIdx.x]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

static inline int grid_for(long long work_items, int per_block) {
  long long b = (work_items + per_block - 1) / per_block;
  const long long cap = 148ll * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
static inline int last_error() {
  count_launch();  // called once after every launch in this file
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int gather_rows(const void* x_latent, const lmoe_route* r, int K, int L, long long padded_rows, void* x_sorted,
                cudaStream_t st) {
  if ((L & 7) != 0) return LMOE_ERR_SHAPE;
  gather_rows_kernel<<<grid_for(padded_rows, kRowWarps), kRowWarps * 32, 0, st>>>(
      static_cast<const uint4*>(x_latent), r->row_src, r->n_tiles, K, L / 8, static_cast<uint4*>(x_sorted), padded_rows);
  return last_error();
}

int combine_rows(const void* y_sorted, const int* pos, const float* w, int T, int K, int L, void* out, long long out_ld,
                 cudaStream_t st) {
  if ((L & 7) != 0 || (out_ld & 7) != 0) return LMOE_ERR_SHAPE;
  combine_kernel<<<grid_for(T, kRowWarps), kRowWarps * 32, 0, st>>>(static_cast<const uint4*>(y_sorted), pos, w, T, K,
                                                                    L / 8, static_cast<uint4*>(out), out_ld / 8, nullptr,
                                                                    0);
  return last_error();
}

}  // namespace lmoe

using namespace lmoe;

extern "C" int lmoe_combine_bwd(const lmoe_shape* s, const void* d_routed, const void* y_sorted, const float* weights,
                                const lmoe_route* r, void* d_y_sorted, float* d_weights, void* stream) {
  if (!s || !d_routed || !y_sorted || !weights || !r || !d_y_sorted || !d_weights) return LMOE_ERR_ARG;
  if ((s->L & 7) != 0) return LMOE_ERR_SHAPE;
  const long long P = lmoe_padded_rows(s);
  combine_bwd_kernel<<<grid_for(P, kRowWarps), kRowWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(d_routed), static_cast<const uint4*>(y_sorted), weights, r->row_src, r->n_tiles, s->K,
      s->L / 8, static_cast<uint4*>(d_y_sorted), d_weights, P);
  return last_error();
}

extern "C" int lmoe_swiglu_bwd(int64_t rows, int H, const void* h1, const void* d_hidden, void* d_h1, int64_t ld_d_h1,
                               const int32_t* n_tiles_dev, void* stream) {
  if (!h1 || !d_hidden || !d_h1 || rows <= 0 || H <= 0) return LMOE_ERR_ARG;
  if ((H & 7) != 0 || (ld_d_h1 & 7) != 0 || ld_d_h1 < 2 * H) return LMOE_ERR_SHAPE;
  swiglu_bwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(h1), static_cast<const uint4*>(d_hidden), static_cast<uint4*>(d_h1), rows, n_tiles_dev,
      H / 8, ld_d_h1 / 8);
  return last_error();
}

extern "C" int lmoe_unpermute_sum_bwd(const lmoe_shape* s, const void* d_x_sorted, const lmoe_route* r, void* dgrad_cat,
                                      void* stream) {
  if (!s || !d_x_sorted || !r || !dgrad_cat) return LMOE_ERR_ARG;
  const long long ld = 2ll * s->Fs + s->L + s->E;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(dgrad_cat) + 2ll * s->Fs;
  return combine_rows(d_x_sorted, r->pos, nullptr, s->T, s->K, s->L, out, ld, static_cast<cudaStream_t>(stream));
}

extern "C" int lmoe_gate_topk_bwd(const lmoe_shape* s, const float* logits, const int32_t* sel, const float* weights,
                                  const float* d_weights, const float* lse, const float* d_z, float z_coef,
                                  void* dgrad_cat, void* stream) {
  if (!s || !logits || !sel || !weights || !d_weights || !lse || !dgrad_cat) return LMOE_ERR_ARG;
  if (s->E > LMOE_MAX_EXPERTS || s->K > 32) return LMOE_ERR_SHAPE;
  const long long ld = 2ll * s->Fs + s->L + s->E;
  __nv_bfloat16* d_logits = static_cast<__nv_bfloat16*>(dgrad_cat) + 2ll * s->Fs + s->L;
  static PerDeviceOnce once;
  once.run([] {  // same shared-memory carveout as the GEMM kernel it runs beside
    cudaFuncSetAttribute(gate_bwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return 0;
  });
  gate_bwd_kernel<<<grid_for(s->T, kRowWarps), kRowWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, sel, weights, d_weights, lse, d_z, z_coef / static_cast<float>(s->T), s->T, s->E, s->K, d_logits, ld);
  return last_error();
}

// ---- generic row primitives (used by the expert-parallel host code, which works on explicit row counts) ----
__global__ void invert_perm_kernel(const int* __restrict__ perm, int n, int* __restrict__ inv) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) inv[perm[i]] = i;
}

extern "C" int lmoe_invert_perm(const int32_t* perm, int64_t n, int32_t* inv, void* stream) {
  if (!perm || !inv || n <= 0 || n >= (1ll << 31)) return LMOE_ERR_ARG;
  invert_perm_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(perm, static_cast<int>(n), inv);
  return last_error();
}

extern "C" int lmoe_gather_rows(const void* src, const int32_t* index, int div, int64_t rows, int L,
                                const int32_t* n_tiles_dev, void* dst, void* stream) {
  if (!src || !index || !dst || rows <= 0 || div <= 0) return LMOE_ERR_ARG;
  if ((L & 7) != 0) return LMOE_ERR_SHAPE;
  gather_rows_kernel<<<grid_for(rows, kRowWarps), kRowWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), index, n_tiles_dev, div, L / 8, static_cast<uint4*>(dst), rows);
  return last_error();
}

extern "C" int lmoe_combine_rows(const void* rows_in, const int32_t* index, const float* weights, int T, int K, int L,
                                 void* out, int64_t ld_out, void* stream) {
  if (!rows_in || !index || !out || T <= 0 || K <= 0) return LMOE_ERR_ARG;
  return combine_rows(rows_in, index, weights, T, K, L, out, ld_out, static_cast<cudaStream_t>(stream));
}

extern "C" int lmoe_combine_rows_add(const void* rows_in, const int32_t* index, const float* weights, const void* addend,
                                     int64_t ld_addend, int T, int K, int L, void* out, int64_t ld_out, void* stream) {
  if (!rows_in || !index || !addend || !out || T <= 0 || K <= 0) return LMOE_ERR_ARG;
  if ((L & 7) != 0 || (ld_out & 7) != 0 || (ld_addend & 7) != 0 || ld_out < L || ld_addend < L) return LMOE_ERR_SHAPE;
  combine_kernel<<<grid_for(T, kRowWarps), kRowWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(rows_in), index, weights, T, K, L / 8, static_cast<uint4*>(out), ld_out / 8,
      static_cast<const uint4*>(addend), ld_addend / 8);
  return last_error();
}

extern "C" int lmoe_combine_bwd_rows(const void* d_routed, const void* y_rows, const float* weights,
                                     const int32_t* row_to_flat, int64_t rows, int K, int L, const int32_t* n_tiles_dev,
                                     void* d_y_rows, float* d_weights, void* stream) {
  if (!d_routed || !y_rows || !weights || !row_to_flat || !d_y_rows || !d_weights || rows <= 0 || K <= 0)
    return LMOE_ERR_ARG;
  if ((L & 7) != 0) return LMOE_ERR_SHAPE;
  combine_bwd_kernel<<<grid_for(rows, kRowWarps), kRowWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(d_routed), static_cast<const uint4*>(y_rows), weights, row_to_flat, n_tiles_dev, K,
      L / 8, static_cast<uint4*>(d_y_rows), d_weights, rows);
  return last_error();
}

extern "C" int lmoe_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream) {
  if (!src || !dst || n <= 0) return LMOE_ERR_ARG;
  const long long n4 = n / 4;
  const int tail = static_cast<int>(n - n4 * 4);
  cast_f32_bf16_kernel<<<grid_for(n4 > 0 ? n4 : 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(src), static_cast<uint2*>(dst), n4, src + n4 * 4,
      static_cast<__nv_bfloat16*>(dst) + n4 * 4, tail);
  return last_error();
}

extern "C" int lmoe_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream) {
  if (!src || !dst || n <= 0) return LMOE_ERR_ARG;
  cast_bf16_f32_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), dst, n);
  return last_error();
}
