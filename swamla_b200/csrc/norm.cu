// The two steps either side of the MoE layer inside the reference's block: x_out = x + ffn(ffn_norm(x))
// (models/mla_block.py:83-85, 159) with ffn_norm = RMSNorm (models/normalization.py:25-39).
//
//   rmsnorm_fwd   xn[t] = w * x[t] * rstd[t],  rstd[t] = rsqrt(mean(x[t]^2) + eps)      one read of x, one write of xn
//   add           out = a + b                                                            the residual add
//   rmsnorm_bwd   dx[t] = rstd * (g - x * rstd^2 * mean(g * x)) + d_res[t],  g = d_xn * w     one kernel for the adjoint of the
//                 d_w[d] = sum_t d_xn[t,d] * x[t,d] * rstd[t]                                  norm AND the residual branch
//
// bf16 rows, fp32 arithmetic, one warp per row with the row held in registers (D <= 2048).  The weight gradient is a
// two-stage sum in a fixed order (per-warp registers -> per-block shared memory in warp order -> per-block partials ->
// final kernel), so it is deterministic; no atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"

namespace lmoe {

constexpr int kNormWarps = 8;
constexpr int kNormMaxChunks = 8;  // 16-byte chunks per lane: D <= 8 * 32 * 8 = 2048
constexpr int kNormMaxBlocks = 296;

__device__ __forceinline__ void nrm_unpack(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 nrm_pack(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_fwd_kernel(const uint4* __restrict__ x, const float* __restrict__ w, float eps, long long T, int vec_per_row,
                   uint4* __restrict__ xn, float* __restrict__ rstd) {
  const int lane = threadIdx.x & 31;
  const float inv_d = 1.0f / static_cast<float>(vec_per_row * 8);
  for (long long t = static_cast<long long>(blockIdx.x) * kNormWarps + (threadIdx.x >> 5); t < T;
       t += static_cast<long long>(gridDim.x) * kNormWarps) {
    uint4 row[kNormMaxChunks];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) {
        row[i] = x[t * vec_per_row + v];
        float f[8];
        nrm_unpack(row[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss * inv_d + eps);
    if (lane == 0) rstd[t] = r;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) {
        float f[8], o[8];
        nrm_unpack(row[i], f);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = ww[j] * (f[j] * r);
        xn[t * vec_per_row + v] = nrm_pack(o);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
add_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out, long long n_vec) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float fa[8], fb[8];
    nrm_unpack(a[i], fa);
    nrm_unpack(b[i], fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) fa[j] += fb[j];
    out[i] = nrm_pack(fa);
  }
}

// partial[blockIdx.x][D]: this block's share of d_w.  Shared memory: D floats (dynamic).
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_bwd_kernel(const uint4* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd,
                   const uint4* __restrict__ d_xn, const uint4* __restrict__ d_res, long long T, int vec_per_row,
                   uint4* __restrict__ dx, float* __restrict__ partial) {
  extern __shared__ float s_dw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = vec_per_row * 8;
  const float inv_d = 1.0f / static_cast<float>(D);
  float dw[kNormMaxChunks][8];
#pragma unroll
  for (int i = 0; i < kNormMaxChunks; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;

  for (long long t = static_cast<long long>(blockIdx.x) * kNormWarps + warp; t < T;
       t += static_cast<long long>(gridDim.x) * kNormWarps) {
    const float r = rstd[t];
    uint4 xr[kNormMaxChunks], gr[kNormMaxChunks];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) {
        xr[i] = x[t * vec_per_row + v];
        gr[i] = d_xn[t * vec_per_row + v];
        float fx[8], fg[8];
        nrm_unpack(xr[i], fx);
        nrm_unpack(gr[i], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot = fmaf(fg[j] * ww[j], fx[j], dot);
          dw[i][j] = fmaf(fg[j], fx[j] * r, dw[i][j]);
        }
      }
    }
    dot = warp_sum(dot);
    const float c = r * r * r * dot * inv_d;  // rstd^3 * mean(g * x)
#pragma unroll
    for (int i = 0; i < kNormMaxChunks; ++i) {
      const int v = lane + 32 * i;
      if (v < vec_per_row) {
        float fx[8], fg[8], o[8];
        nrm_unpack(xr[i], fx);
        nrm_unpack(gr[i], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fg[j] * ww[j] * r - fx[j] * c;
        if (d_res) {
          float fr[8];
          nrm_unpack(d_res[t * vec_per_row + v], fr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += fr[j];
        }
        dx[t * vec_per_row + v] = nrm_pack(o);
      }
    }
  }
  // block sum of the weight-gradient partials, warp after warp (fixed order)
  for (int wi = 0; wi < kNormWarps; ++wi) {
    if (warp == wi) {
#pragma unroll
      for (int i = 0; i < kNormMaxChunks; ++i) {
        const int v = lane + 32 * i;
        if (v < vec_per_row) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int d = v * 8 + j;
            s_dw[d] = (wi == 0 ? 0.f : s_dw[d]) + dw[i][j];
          }
        }
      }
    }
    __syncthreads();
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) partial[static_cast<long long>(blockIdx.x) * D + d] = s_dw[d];
}

__global__ void __launch_bounds__(256)
rmsnorm_dw_finalize_kernel(const float* __restrict__ partial, int blocks, int D, float* __restrict__ d_w) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[static_cast<long long>(b) * D + d];
  d_w[d] = s;
}

static inline int norm_blocks(long long T) {
  long long b = (T + kNormWarps - 1) / kNormWarps;
  if (b > kNormMaxBlocks) b = kNormMaxBlocks;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
static inline int norm_last_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
static inline bool norm_dims_ok(long long T, int D) {
  return T > 0 && D > 0 && (D & 7) == 0 && D <= kNormMaxChunks * 256;
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace lmoe

using namespace lmoe;

extern "C" size_t lmoe_rmsnorm_workspace_bytes(int D) {
  return D > 0 ? static_cast<size_t>(kNormMaxBlocks) * D * sizeof(float) : 0;
}

extern "C" int lmoe_rmsnorm_fwd(const void* x, const float* weight, float eps, int64_t T, int D, void* xn, float* rstd,
                                void* stream) {
  if (!x || !weight || !xn || !rstd) return LMOE_ERR_ARG;
  if (!norm_dims_ok(T, D)) return LMOE_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(xn) || !aligned16(weight)) return LMOE_ERR_ALIGN;
  rmsnorm_fwd_kernel<<<norm_blocks(T), kNormWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), weight, eps, T, D / 8, static_cast<uint4*>(xn), rstd);
  count_launch();
  return norm_last_error();
}

extern "C" int lmoe_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream) {
  if (!a || !b || !out) return LMOE_ERR_ARG;
  if (n <= 0 || (n & 7) != 0) return LMOE_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return LMOE_ERR_ALIGN;
  const long long n_vec = n / 8;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 148ll * 16) blocks = 148ll * 16;
  add_bf16_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint4*>(out), n_vec);
  count_launch();
  return norm_last_error();
}

extern "C" int lmoe_rmsnorm_bwd(const void* x, const float* weight, const float* rstd, const void* d_xn,
                                const void* d_residual, int64_t T, int D, void* dx, float* d_weight, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (!x || !weight || !rstd || !d_xn || !dx || !d_weight || !workspace) return LMOE_ERR_ARG;
  if (!norm_dims_ok(T, D)) return LMOE_ERR_SHAPE;
  if (workspace_bytes < lmoe_rmsnorm_workspace_bytes(D)) return LMOE_ERR_WORKSPACE;
  if (!aligned16(x) || !aligned16(d_xn) || !aligned16(dx) || !aligned16(weight) || (d_residual && !aligned16(d_residual)))
    return LMOE_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = norm_blocks(T);
  rmsnorm_bwd_kernel<<<blocks, kNormWarps * 32, static_cast<size_t>(D) * sizeof(float), st>>>(
      static_cast<const uint4*>(x), weight, rstd, static_cast<const uint4*>(d_xn), static_cast<const uint4*>(d_residual),
      T, D / 8, static_cast<uint4*>(dx), static_cast<float*>(workspace));
  count_launch();
  if (int rc = norm_last_error()) return rc;
  rmsnorm_dw_finalize_kernel<<<(D + 255) / 256, 256, 0, st>>>(static_cast<const float*>(workspace), blocks, D, d_weight);
  count_launch();
  return norm_last_error();
}
