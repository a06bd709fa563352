// FP8 (e4m3) expert path: per-tensor dynamic scaling ("tensorwise": one amax per tensor, scale = 448 / amax,
// q = saturate(x * scale), the recipe named by optimization/fp8_native.py:103-110 of the reference), and the
// grouped expert GEMMs on tcgen05 kind::f8f6f4.  The reference applies this recipe to nn.Linear modules only;
// using it for the routed experts is this path's extension.  A tensor is quantised once and serves every GEMM
// that reads it (forward, dgrad as K-major operand, wgrad as MN-major operand) because the scale is per tensor.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lmoe.h"
#include "counters.h"
#include "gemm.cuh"
#include "gemm_host.h"

namespace lmoe {

constexpr float kE4M3Max = 448.0f;

// amax[0] = max |x| over n bf16 values (n read on the device as min(n, 128 * n_tiles[0] * row_len) when n_tiles
// is given).  Non-negative floats order like their bit patterns, so an integer atomicMax does the reduction.
__global__ void __launch_bounds__(256)
amax_kernel(const uint4* __restrict__ x, long long n_vec, const int* __restrict__ n_tiles, long long vec_per_tile,
            float* __restrict__ amax) {
  if (n_tiles) n_vec = min(n_vec, static_cast<long long>(n_tiles[0]) * vec_per_tile);
  float m = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, s[i]);
    atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
  }
}

// q = saturate_e4m3(x * 448 / amax); deq[0] = amax / 448 (1 when the tensor is all zero).
__global__ void __launch_bounds__(256)
quantize_kernel(const uint4* __restrict__ x, long long n_vec, const int* __restrict__ n_tiles, long long vec_per_tile,
                const float* __restrict__ amax, uint2* __restrict__ q, float* __restrict__ deq) {
  if (n_tiles) n_vec = min(n_vec, static_cast<long long>(n_tiles[0]) * vec_per_tile);
  const float a = amax[0];
  const float scale = (a > 0.f) ? kE4M3Max / a : 1.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) deq[0] = (a > 0.f) ? a / kE4M3Max : 1.0f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t out[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float2 f0 = __bfloat1622float2(h[2 * k]), f1 = __bfloat1622float2(h[2 * k + 1]);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f0.x * scale, f0.y * scale), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f1.x * scale, f1.y * scale), __NV_SATFINITE, __NV_E4M3);
      out[k] = lo | (hi << 16);
    }
    q[i] = make_uint2(out[0], out[1]);
  }
}

static inline int grid_vec(long long n_vec) {
  long long b = (n_vec + 255) / 256;
  if (b > 148ll * 8) b = 148ll * 8;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace lmoe

using namespace lmoe;

extern "C" int lmoe_fp8_quantize(const void* x_bf16, int64_t rows, int row_len, const int32_t* n_tiles_dev, void* q_e4m3,
                                 float* amax, float* deq, void* stream) {
  if (!x_bf16 || !q_e4m3 || !amax || !deq || rows <= 0 || row_len <= 0) return LMOE_ERR_ARG;
  if ((row_len & 7) != 0) return LMOE_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(q_e4m3) & 7) != 0)
    return LMOE_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long n_vec = rows * (row_len / 8);
  const long long vec_per_tile = static_cast<long long>(LMOE_ROW_PAD) * (row_len / 8);
  cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(float), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch(2);
  amax_kernel<<<grid_vec(n_vec), 256, 0, st>>>(static_cast<const uint4*>(x_bf16), n_vec, n_tiles_dev, vec_per_tile, amax);
  quantize_kernel<<<grid_vec(n_vec), 256, 0, st>>>(static_cast<const uint4*>(x_bf16), n_vec, n_tiles_dev, vec_per_tile,
                                                  amax, static_cast<uint2*>(q_e4m3), deq);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Generic e4m3 GEMM (test hook): C[M,N] bf16 = deq_a * deq_b * A_q[M,K] * B_q[N,K]^T.
extern "C" int lmoe_gemm_fp8(int M, int N, int K, const void* A, int64_t lda, int a_mn, const void* B, int64_t ldb,
                             int b_mn, const float* deq_a, const float* deq_b, void* C, int64_t ldc, int32_t* status,
                             void* stream) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return LMOE_ERR_ARG;
  GemmCall c;
  c.esz = 1;
  c.a_mn = a_mn ? 1 : 0;
  c.b_mn = b_mn ? 1 : 0;
  c.epi = EPI_BF16;
  c.grp = GRP_NONE;
  c.A[0] = A;
  c.lda[0] = lda;
  c.B[0] = B;
  c.ldb[0] = ldb;
  c.Kseg[0] = K;
  c.M = M;
  c.N = N;
  c.C = C;
  c.ldc = ldc;
  c.deq_a = deq_a;
  c.deq_b = deq_b;
  c.status = status;
  c.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(c);
}

// Routed gate_up in e4m3 with the SwiGLU epilogue: h1 = deq * xq * Wq[e], hidden = silu(gate) * up (both bf16).
extern "C" int lmoe_grouped_gateup_fp8(int64_t P, int E, int L, int F, const void* xq, const void* wq, const float* deq_x,
                                       const float* deq_w, const int32_t* tile_expert, const int32_t* n_tiles, void* h1,
                                       void* hidden, int32_t* status, void* stream) {
  if (!xq || !wq || !deq_x || !deq_w || !tile_expert || !n_tiles || !h1 || !hidden) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (L % 128) != 0 || (F % 128) != 0) return LMOE_ERR_SHAPE;
  GemmCall a;
  a.esz = 1;
  a.a_mn = 0;
  a.b_mn = 1;
  a.epi = EPI_SWIGLU;
  a.grp = GRP_M;
  a.A[0] = xq;
  a.lda[0] = L;
  a.B[0] = wq;
  a.ldb[0] = 2ll * F;
  a.Kseg[0] = L;
  a.M = static_cast<int>(P);
  a.N = F;
  a.C = h1;
  a.ldc = 2ll * F;
  a.C2 = hidden;
  a.ldc2 = F;
  a.padded_rows = P;
  a.groups = E;
  a.b_group_rows = L;
  a.tile_expert = tile_expert;
  a.n_m_tiles = n_tiles;
  a.deq_a = deq_x;
  a.deq_b = deq_w;
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(a);
}

// Grouped-by-rows e4m3 GEMM: out[P,N] bf16 = deq * aq[P,K] * Bq[e], Bq stacked per expert either [E*K, N]
// (b_mn = 1, the forward layout of the expert weights) or [E*N, K] (b_mn = 0, the same weights read as dgrad operand).
extern "C" int lmoe_grouped_rows_fp8(int64_t P, int E, int K, int N, const void* aq, const void* bq, int b_mn,
                                     const float* deq_a, const float* deq_b, const int32_t* tile_expert,
                                     const int32_t* n_tiles, void* out, int32_t* status, void* stream) {
  if (!aq || !bq || !deq_a || !deq_b || !tile_expert || !n_tiles || !out) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (K % 128) != 0 || (N % 16) != 0) return LMOE_ERR_SHAPE;
  GemmCall a;
  a.esz = 1;
  a.a_mn = 0;
  a.b_mn = b_mn ? 1 : 0;
  a.epi = EPI_BF16;
  a.grp = GRP_M;
  a.A[0] = aq;
  a.lda[0] = K;
  a.B[0] = bq;
  a.ldb[0] = b_mn ? N : K;
  a.Kseg[0] = K;
  a.M = static_cast<int>(P);
  a.N = N;
  a.C = out;
  a.ldc = N;
  a.padded_rows = P;
  a.groups = E;
  a.b_group_rows = b_mn ? K : N;
  a.tile_expert = tile_expert;
  a.n_m_tiles = n_tiles;
  a.deq_a = deq_a;
  a.deq_b = deq_b;
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(a);
}

// Grouped-by-contraction e4m3 GEMM (expert weight gradients): out[e][M,N] bf16 = deq * aq[rows_e, M]^T * bq[rows_e, N].
extern "C" int lmoe_grouped_wgrad_fp8(int64_t P, int E, int M, int N, const void* aq, const void* bq, const float* deq_a,
                                      const float* deq_b, const int32_t* pad_offsets, void* out, int32_t* status,
                                      void* stream) {
  if (!aq || !bq || !deq_a || !deq_b || !pad_offsets || !out) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (M % 16) != 0 || (N % 16) != 0) return LMOE_ERR_SHAPE;
  GemmCall a;
  a.esz = 1;
  a.a_mn = 1;
  a.b_mn = 1;
  a.epi = EPI_BF16;
  a.grp = GRP_K;
  a.A[0] = aq;
  a.lda[0] = M;
  a.B[0] = bq;
  a.ldb[0] = N;
  a.M = M;
  a.N = N;
  a.C = out;
  a.ldc = N;
  a.c_group_stride = static_cast<long long>(M) * N;
  a.padded_rows = P;
  a.groups = E;
  a.pad_offsets = pad_offsets;
  a.deq_a = deq_a;
  a.deq_b = deq_b;
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(a);
}
