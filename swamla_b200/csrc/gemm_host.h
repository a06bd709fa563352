// Host-side description of one launch of the tcgen05 GEMM kernel (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lmoe {

struct GemmCall {
  // operand layout
  int a_mn = 0, b_mn = 0;  // 0 = K-major, 1 = MN-major
  int epi = 0;             // EPI_*
  int grp = 0;             // GRP_*
  int bn = 0;              // 0 = choose; else 128 or 256
  int esz = 2;             // operand element size: 2 = bf16, 1 = e4m3
  const float* deq_a = nullptr;  // e4m3: device scalars, result is multiplied by deq_a[0] * deq_b[0]
  const float* deq_b = nullptr;
  // up to three K segments accumulated into the same output tile
  int nseg = 1;
  const void* A[3] = {nullptr, nullptr, nullptr};
  long long lda[3] = {0, 0, 0};  // elements
  const void* B[3] = {nullptr, nullptr, nullptr};
  long long ldb[3] = {0, 0, 0};
  int Kseg[3] = {0, 0, 0};  // contraction extent per segment (GRP_K: unused)
  // output
  int M = 0, N = 0;  // per group for GRP_K; for EPI_SWIGLU N = width of one half
  void* C = nullptr;
  long long ldc = 0;
  long long c_group_stride = 0;  // GRP_K: elements between experts' outputs; split-K: elements between planes
  void* C2 = nullptr;
  long long ldc2 = 0;
  const void* aux = nullptr;     // EPI_SWIGLU_BWD: h1 [rows, 2N] bf16; C is then d_h1 [rows, 2N]
  long long ld_aux = 0;
  // Gathered A (bf16, nseg == 1, GRP_M with K-major A or GRP_K): A[0] is the SOURCE tensor [a_src_rows, K or M]
  // and padded row i reads its row a_rows[i * a_rows_stride] / a_rows_div; a negative entry reads row a_zero_row,
  // which the caller keeps all zero.
  const int* a_rows = nullptr;
  int a_rows_stride = 1;
  int a_rows_div = 1;
  long long a_src_rows = 0;
  int a_zero_row = 0;
  int split_k = 1;               // >1 (GRP_NONE, EPI_F32): C is a [split_k, M, N] workspace of partial sums
  // grouping
  long long padded_rows = 0;         // GRP_M / GRP_K: rows of the padded routed layout (upper bound)
  int groups = 0;                    // number of experts
  int b_group_rows = 0;              // GRP_M: rows of stacked B per expert
  long long b_inner = 0;             // GRP_M: inner extent of stacked B (K for K-major, N_total for MN-major)
  const int* tile_expert = nullptr;  // GRP_M
  const int* n_m_tiles = nullptr;    // GRP_M
  const int* pad_offsets = nullptr;  // GRP_K
  int* status = nullptr;
  cudaStream_t stream = nullptr;
};

// Returns 0, a negative LMOE_ERR_* code, or a positive cudaError_t.
int launch_gemm(const GemmCall& c);

int num_sms();

// Tensor maps.  encode_2d: a row-major [outer, inner] tensor of 16-bit (esz 2) or 8-bit (esz 1) elements, box
// {128 bytes, box_outer rows}, 128-byte swizzle (operand loads, and stores from a buffer in the same layout).
// encode_out: 3-D {cols, rows, planes}, box {32 columns, 128 rows, 1}: bf16 with 64-byte swizzle or fp32 with
// 128-byte swizzle (epilogue slabs; also usable as a load of such slabs).
int encode_2d(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld_elems, int box_outer,
              int esz);
int encode_out(CUtensorMap* map, void* base, bool f32, long long cols, long long rows, long long planes,
               long long ld_elems, long long plane_elems, bool as_source = false);

// The routed expert chain (chain.cuh) in one launch.  mode 0 (forward): a = x_sorted [P, L], h1 [P, 2F] and
// mid = hidden [P, F] and out = y_sorted [P, L] are written.  mode 1 (backward): a = d_y_sorted, h1 is read,
// mid = d_h1 [P, 2F] and out = d_x_sorted [P, L] are written.
bool chain_applies(int L, int F);
// pad_offsets [E + 1] (first padded row of every expert) lets the launcher pair up tiles of the same expert on CTA
// pairs (chain_pair.cuh); NULL: one CTA per tile.
int launch_chain(int mode, long long P, int E, int L, int F, const void* a, const void* w_gate_up, const void* w_down,
                 const int* tile_expert, const int* n_tiles, const int* pad_offsets, void* h1, void* mid, void* out,
                 int* status, cudaStream_t stream);

// True when dense GEMMs of this size run on CTA pairs (256 x 256 tiles over two SMs) rather than one CTA per 128 x 256 tile.
bool pair_gemm_applies(int M, int N);

// out[rows, cols] = sum over `planes` of ws[plane][row0 + r][col0 + c]; fp32 or bf16 output.
int splitk_reduce(const float* ws, int planes, long long plane_elems, int ws_ld, int row0, int col0, int rows, int cols,
                  void* out, long long out_ld, int out_f32, cudaStream_t stream);
// The same for up to three ranges of one workspace in ONE launch (fixed summation order per element all the same).
int splitk_reduce_multi(const float* ws, int planes, long long plane_elems, int ws_ld, int n_ranges, const int* row0,
                        const int* col0, const int* rows, const int* cols, void* const* out, const long long* out_ld,
                        int out_f32, cudaStream_t stream);

}  // namespace lmoe
