// Stage-level C-ABI entry points of the LatentMoE path, assembled from the tcgen05 GEMM launcher
// and the row kernels.  Host code only: argument checks, GEMM descriptions, launches.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/lmoe.h"
#include "counters.h"
#include "chain.cuh"
#include "gemm.cuh"
#include "gemm_host.h"
#include "rowops.h"

using namespace lmoe;

namespace {

typedef __nv_bfloat16 bf16;

int check_dims(const lmoe_shape* s) {
  if (!s) return LMOE_ERR_ARG;
  if (s->T <= 0 || s->D <= 0 || s->L <= 0 || s->E <= 0 || s->K <= 0 || s->F <= 0 || s->Fs <= 0) return LMOE_ERR_SHAPE;
  if (s->E > LMOE_MAX_EXPERTS || s->K > LMOE_MAX_TOPK || s->K > s->E) return LMOE_ERR_SHAPE;
  // L and F are contraction extents of grouped GEMMs (whole 64-element k-blocks per expert); Fs is cut
  // into 32-column slabs by the SwiGLU epilogue; every extent is a multiple of 8 so rows stay 16-byte aligned.
  if ((s->L % 64) != 0 || (s->F % 64) != 0 || (s->D % 8) != 0 || (s->Fs % 32) != 0 || (s->E % 8) != 0)
    return LMOE_ERR_SHAPE;
  if (s->n_shared != 1) return LMOE_ERR_SHAPE;
  return 0;
}

GemmCall dense(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, int M, int N, int K,
               void* C, long long ldc, int epi, int* status, void* stream) {
  GemmCall c;
  c.a_mn = a_mn;
  c.b_mn = b_mn;
  c.epi = epi;
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
  c.status = status;
  c.stream = static_cast<cudaStream_t>(stream);
  return c;
}

// Number of k-slices for a weight gradient with an M x N output contracting over K rows, from a cost model in
// units of one k-block of main loop: waves x (k-blocks per slice + epilogue) + the reduce traffic of the planes.
int wgrad_split(int M, int N, int K) {
  const bool pair = pair_gemm_applies(M, N);  // 256 x 256 tiles on SM pairs: half the tiles, half the units
  const long long tiles = static_cast<long long>((M + (pair ? 255 : 127)) / (pair ? 256 : 128)) * ((N + 255) / 256);
  const int kiters = (K + 63) / 64;  // bf16 k-blocks of 64 rows
  const int sms = pair ? num_sms() / 2 : num_sms();
  const double kblock_us = 0.40;                                       // 128 x 256 x 64 on one SM
  const double plane_us = 2.0 * M * N * 4.0 / 6.5e6;                   // write + read of one fp32 plane at HBM rate
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 16 && s <= kiters; ++s) {
    const long long waves = (tiles * s + sms - 1) / sms;
    const double cost = waves * ((kiters + s - 1) / s + 8.0) * kblock_us + (s > 1 ? s * plane_us : 0.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// dW[M,N] (fp32 planes in `ws`) = Aact[K,M]^T * Bact[K,N]: both operands MN-major, contraction over rows.
int wgrad_gemm(const void* Aact, long long lda, int M, const void* Bact, long long ldb, int N, int K, float* ws,
               int split, int* status, void* stream) {
  GemmCall c = dense(Aact, lda, 1, Bact, ldb, 1, M, N, K, ws, N, EPI_F32, status, stream);
  c.split_k = split;
  c.c_group_stride = static_cast<long long>(M) * N;
  c.bn = 256;
  return launch_gemm(c);
}

}  // namespace

extern "C" int lmoe_version(void) { return LMOE_VERSION; }
extern "C" int64_t lmoe_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

extern "C" const char* lmoe_status_string(int code) {
  switch (code) {
    case LMOE_OK: return "ok";
    case LMOE_ERR_ARG: return "invalid argument (null pointer or bad enum)";
    case LMOE_ERR_SHAPE: return "unsupported shape";
    case LMOE_ERR_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case LMOE_ERR_WORKSPACE: return "workspace too small";
    case LMOE_ERR_DRIVER: return "tensor-map encoding failed or driver entry point missing";
    case LMOE_ERR_TOO_LARGE: return "problem exceeds the fixed scratch capacity of a no-allocation entry point";
    case kStatusProducerTimeout: return "device: TMA producer wait timed out";
    case kStatusMmaTimeout: return "device: MMA issuer wait timed out";
    case kStatusEpilogueTimeout: return "device: epilogue wait timed out";
    case 201: return "device: an expert-parallel shard received more rows than its buffers hold (raise ep_capacity_factor); "
                     "the excess rows were dropped and the results of that step are wrong";
    case 202: return "device: a rank of the expert-parallel group did not reach a barrier within two seconds";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

extern "C" size_t lmoe_wgrad_workspace_bytes(const lmoe_shape* s) {
  if (check_dims(s)) return 0;
  // the two dense weight-gradient GEMMs run one after the other and share the workspace
  const int Mx = 2 * s->Fs + s->L + s->E;
  const size_t a = static_cast<size_t>(wgrad_split(Mx, s->D, s->T)) * Mx * s->D;
  const int Ny = s->L + s->Fs;
  const size_t b = static_cast<size_t>(wgrad_split(s->D, Ny, s->T)) * s->D * Ny;
  return (a > b ? a : b) * sizeof(float);
}

// ------------------------------------------------------------------ forward
extern "C" int lmoe_xproj_fwd(const lmoe_shape* s, const void* x, const void* w_gate, const void* w_down, float* logits,
                              void* x_latent, int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!x || !w_gate || !w_down || !logits || !x_latent) return LMOE_ERR_ARG;
  GemmCall g = dense(x, s->D, 0, w_gate, s->D, 0, s->T, s->E, s->D, logits, s->E, EPI_F32, status, stream);
  if (int rc = launch_gemm(g)) return rc;
  GemmCall d = dense(x, s->D, 0, w_down, s->D, 0, s->T, s->L, s->D, x_latent, s->L, EPI_BF16, status, stream);
  return launch_gemm(d);
}

extern "C" int lmoe_shared_gateup_fwd(const lmoe_shape* s, const void* x, const void* w_gate_up_s, void* h1_s,
                                      void* act_cat, int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!x || !w_gate_up_s || !h1_s || !act_cat) return LMOE_ERR_ARG;
  GemmCall c = dense(x, s->D, 0, w_gate_up_s, s->D, 0, s->T, s->Fs, s->D, h1_s, 2ll * s->Fs, EPI_SWIGLU, status, stream);
  c.C2 = static_cast<bf16*>(act_cat) + s->L;  // hidden_s = act_cat[:, L:]
  c.ldc2 = s->L + s->Fs;
  return launch_gemm(c);
}

extern "C" int lmoe_gemm_swiglu_bf16(int M, int H, int K, const void* A, int64_t lda, const void* W, int64_t ldw,
                                     void* h1, int64_t ld_h1, void* hidden, int64_t ld_hidden, int32_t* status,
                                     void* stream) {
  if (!A || !W || !h1 || !hidden || M <= 0 || H <= 0 || K <= 0) return LMOE_ERR_ARG;
  if ((H % 32) != 0 || ld_h1 < 2ll * H || ld_hidden < H) return LMOE_ERR_SHAPE;
  GemmCall c = dense(A, lda, 0, W, ldw, 0, M, H, K, h1, ld_h1, EPI_SWIGLU, status, stream);
  c.C2 = hidden;
  c.ldc2 = ld_hidden;
  return launch_gemm(c);
}

// Gathered A operand of the routed GEMMs: padded row i is row row_index[i * index_stride] / index_div of src_rows.
struct GatherA {
  const int32_t* row_index = nullptr;
  int index_stride = 1;
  int index_div = 1;
  long long n_src_rows = 0;
  long long zero_row = 0;
};
static int apply_gather(GemmCall& c, const GatherA* g) {
  if (!g) return 0;
  if (!g->row_index || g->index_stride <= 0 || g->index_div <= 0 || g->n_src_rows <= 0 || g->n_src_rows >= (1ll << 31) || g->zero_row < 0 ||
      g->zero_row >= g->n_src_rows)
    return LMOE_ERR_ARG;
  c.a_rows = g->row_index;
  c.a_rows_stride = g->index_stride;
  c.a_rows_div = g->index_div;
  c.a_src_rows = g->n_src_rows;
  c.a_zero_row = static_cast<int>(g->zero_row);
  return 0;
}

static int grouped_fwd_impl(int64_t P, int E, int L, int F, const void* x_sorted, const GatherA* g, const void* w_gate_up,
                            const void* w_down, const int32_t* tile_expert, const int32_t* n_tiles,
                            const int32_t* pad_offsets, void* h1,
                            void* hidden, void* y_sorted, int32_t* status, void* stream) {
  if (!x_sorted || !w_gate_up || !w_down || !tile_expert || !n_tiles || !h1 || !hidden || !y_sorted) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (L % 64) != 0 || (F % 64) != 0) return LMOE_ERR_SHAPE;
  // one kernel for gate_up -> SwiGLU -> down per 128-row tile when the latent width fits the second accumulator
  if (!g && chain_applies(L, F))
    return launch_chain(CHAIN_FWD, P, E, L, F, x_sorted, w_gate_up, w_down, tile_expert, n_tiles, pad_offsets, h1, hidden,
                        y_sorted, status, static_cast<cudaStream_t>(stream));
  // h1 = x_sorted * Wgu[e]  (Wgu stacked [E*L, 2F], N contiguous), hidden = silu(gate) * up
  GemmCall a;
  a.a_mn = 0;
  a.b_mn = 1;
  a.epi = EPI_SWIGLU;
  a.grp = GRP_M;
  a.A[0] = x_sorted;
  a.lda[0] = L;
  a.B[0] = w_gate_up;
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
  a.pad_offsets = pad_offsets;  // lets both GEMMs run on CTA pairs that share an expert's weight loads
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  GemmCall b = a;
  if (int rc = apply_gather(a, g)) return rc;
  if (int rc = launch_gemm(a)) return rc;
  // y_sorted = hidden * Wd[e]  (Wd stacked [E*F, L], N contiguous)
  b.epi = EPI_BF16;
  b.A[0] = hidden;
  b.lda[0] = F;
  b.B[0] = w_down;
  b.ldb[0] = L;
  b.Kseg[0] = F;
  b.N = L;
  b.C = y_sorted;
  b.ldc = L;
  b.C2 = nullptr;
  b.b_group_rows = F;
  return launch_gemm(b);
}

extern "C" int lmoe_grouped_fwd(int64_t P, int E, int L, int F, const void* x_sorted, const void* w_gate_up,
                                const void* w_down, const int32_t* tile_expert, const int32_t* n_tiles,
                                const int32_t* pad_offsets, void* h1, void* hidden, void* y_sorted, int32_t* status,
                                void* stream) {
  return grouped_fwd_impl(P, E, L, F, x_sorted, nullptr, w_gate_up, w_down, tile_expert, n_tiles, pad_offsets, h1, hidden,
                          y_sorted, status, stream);
}

extern "C" int lmoe_grouped_fwd_gather(int64_t P, int E, int L, int F, const void* src_rows, int64_t n_src_rows,
                                       const int32_t* row_index, int index_stride, int index_div, int64_t zero_row,
                                       const void* w_gate_up, const void* w_down, const int32_t* tile_expert,
                                       const int32_t* n_tiles, void* h1, void* hidden, void* y_sorted, int32_t* status,
                                       void* stream) {
  GatherA g;
  g.row_index = row_index;
  g.index_stride = index_stride;
  g.index_div = index_div;
  g.n_src_rows = n_src_rows;
  g.zero_row = zero_row;
  return grouped_fwd_impl(P, E, L, F, src_rows, &g, w_gate_up, w_down, tile_expert, n_tiles, nullptr, h1, hidden, y_sorted,
                          status, stream);
}

extern "C" int lmoe_experts_fwd(const lmoe_shape* s, const void* x_latent, const void* w_gate_up, const void* w_down,
                                const lmoe_route* r, void* x_sorted, void* h1, void* hidden, void* y_sorted,
                                int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!x_latent || !w_gate_up || !w_down || !r || !x_sorted || !h1 || !hidden || !y_sorted) return LMOE_ERR_ARG;
  const long long P = lmoe_padded_rows(s);
  if (int rc = gather_rows(x_latent, r, s->K, s->L, P, x_sorted, static_cast<cudaStream_t>(stream))) return rc;
  return lmoe_grouped_fwd(P, s->E, s->L, s->F, x_sorted, w_gate_up, w_down, r->tile_expert, r->n_tiles, r->pad_offsets, h1, hidden,
                          y_sorted, status, stream);
}

extern "C" int lmoe_combine_out_fwd(const lmoe_shape* s, const void* y_sorted, const lmoe_route* r, const float* weights,
                                    void* act_cat, const void* w_down_s, const void* w_up, void* y, int32_t* status,
                                    void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!act_cat || !w_down_s || !w_up || !y) return LMOE_ERR_ARG;
  if (y_sorted && (!r || !weights)) return LMOE_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long ld = s->L + s->Fs;
  bf16* routed = static_cast<bf16*>(act_cat);
  bf16* hidden_s = routed + s->L;
  if (y_sorted)
    if (int rc = combine_rows(y_sorted, r->pos, weights, s->T, s->K, s->L, routed, ld, st)) return rc;
  // y = hidden_s * Wd_s^T + routed * Wup^T : two K segments into one accumulator
  GemmCall c = dense(hidden_s, ld, 0, w_down_s, s->Fs, 0, s->T, s->D, s->Fs, y, s->D, EPI_BF16, status, stream);
  c.nseg = 2;
  c.A[1] = routed;
  c.lda[1] = ld;
  c.B[1] = w_up;
  c.ldb[1] = s->L;
  c.Kseg[1] = s->L;
  return launch_gemm(c);
}

// ------------------------------------------------------------------ backward
extern "C" int lmoe_combine_out_bwd_dgrad(const lmoe_shape* s, const void* dy, const void* w_up, const void* w_down_s,
                                          const void* h1_s, void* d_routed, void* d_hidden_s, void* dgrad_cat,
                                          int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!dy || !w_up || !w_down_s || !h1_s || !d_routed || !dgrad_cat) return LMOE_ERR_ARG;
  // d_routed[T,L] = dy[T,D] * Wup[D,L]      (B stored [K=D, N=L]: MN-major)
  GemmCall a = dense(dy, s->D, 0, w_up, s->L, 1, s->T, s->L, s->D, d_routed, s->L, EPI_BF16, status, stream);
  if (int rc = launch_gemm(a)) return rc;
  const long long ld = 2ll * s->Fs + s->L + s->E;
  if (d_hidden_s) {
    // d_hidden_s[T,Fs] = dy * Wd_s, then the SwiGLU adjoint as a separate streaming kernel -> dgrad_cat[:, :2Fs]
    GemmCall b = dense(dy, s->D, 0, w_down_s, s->Fs, 1, s->T, s->Fs, s->D, d_hidden_s, s->Fs, EPI_BF16, status, stream);
    if (int rc = launch_gemm(b)) return rc;
    return lmoe_swiglu_bwd(s->T, s->Fs, h1_s, d_hidden_s, dgrad_cat, ld, nullptr, stream);
  }
  // fused: the SwiGLU adjoint in the epilogue of the d_hidden_s GEMM
  GemmCall b = dense(dy, s->D, 0, w_down_s, s->Fs, 1, s->T, s->Fs, s->D, dgrad_cat, ld, EPI_SWIGLU_BWD, status, stream);
  b.aux = h1_s;
  b.ld_aux = 2ll * s->Fs;
  return launch_gemm(b);
}

extern "C" int lmoe_combine_out_bwd_wgrad(const lmoe_shape* s, const void* dy, const void* act_cat, void* d_w_up,
                                          void* d_w_down_s, int grad_type, void* workspace, size_t workspace_bytes,
                                          int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!dy || !act_cat || !d_w_up || !d_w_down_s || !workspace) return LMOE_ERR_ARG;
  if (grad_type != LMOE_F32 && grad_type != LMOE_BF16) return LMOE_ERR_ARG;
  if (workspace_bytes < lmoe_wgrad_workspace_bytes(s)) return LMOE_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // [d_w_up | d_w_down_s][D, L+Fs] = dy[T,D]^T * act_cat[T, L+Fs]
  const int N = s->L + s->Fs;
  const int split = wgrad_split(s->D, N, s->T);
  float* ws = static_cast<float*>(workspace);
  if (int rc = wgrad_gemm(dy, s->D, s->D, act_cat, N, N, s->T, ws, split, status, stream)) return rc;
  const long long plane = static_cast<long long>(s->D) * N;
  const int row0[2] = {0, 0}, col0[2] = {0, s->L}, rows[2] = {s->D, s->D}, cols[2] = {s->L, s->Fs};
  void* const outs[2] = {d_w_up, d_w_down_s};
  const long long lds[2] = {s->L, s->Fs};
  return splitk_reduce_multi(ws, split, plane, N, 2, row0, col0, rows, cols, outs, lds, grad_type == LMOE_F32, st);
}

// Generic grouped-by-rows bf16 GEMM: out[P,N] = a[P,K] * B[e], B stacked [E,K,N] (b_mn = 1) or [E,N,K] (b_mn = 0).
extern "C" int lmoe_grouped_rows_bf16(int64_t P, int E, int K, int N, const void* a, const void* b, int b_mn,
                                      const int32_t* tile_expert, const int32_t* n_tiles, void* out, int32_t* status,
                                      void* stream) {
  if (!a || !b || !tile_expert || !n_tiles || !out) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (K % 64) != 0 || (N % 8) != 0) return LMOE_ERR_SHAPE;
  GemmCall c;
  c.a_mn = 0;
  c.b_mn = b_mn ? 1 : 0;
  c.epi = EPI_BF16;
  c.grp = GRP_M;
  c.A[0] = a;
  c.lda[0] = K;
  c.B[0] = b;
  c.ldb[0] = b_mn ? N : K;
  c.Kseg[0] = K;
  c.M = static_cast<int>(P);
  c.N = N;
  c.C = out;
  c.ldc = N;
  c.padded_rows = P;
  c.groups = E;
  c.b_group_rows = b_mn ? K : N;
  c.tile_expert = tile_expert;
  c.n_m_tiles = n_tiles;
  c.status = status;
  c.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(c);
}

// Generic grouped-by-contraction bf16 GEMM: out[e][M,N] = a[rows_e, M]^T * b[rows_e, N].
extern "C" int lmoe_grouped_wgrad_bf16(int64_t P, int E, int M, int N, const void* a, const void* b,
                                       const int32_t* pad_offsets, void* out, int32_t* status, void* stream) {
  if (!a || !b || !pad_offsets || !out) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (M % 8) != 0 || (N % 8) != 0) return LMOE_ERR_SHAPE;
  GemmCall c;
  c.a_mn = 1;
  c.b_mn = 1;
  c.epi = EPI_BF16;
  c.grp = GRP_K;
  c.A[0] = a;
  c.lda[0] = M;
  c.B[0] = b;
  c.ldb[0] = N;
  c.M = M;
  c.N = N;
  c.C = out;
  c.ldc = N;
  c.c_group_stride = static_cast<long long>(M) * N;
  c.padded_rows = P;
  c.groups = E;
  c.pad_offsets = pad_offsets;
  c.status = status;
  c.stream = static_cast<cudaStream_t>(stream);
  return launch_gemm(c);
}

extern "C" int lmoe_grouped_bwd_dgrad(int64_t P, int E, int L, int F, const void* d_y_sorted, const void* h1,
                                      const void* w_gate_up, const void* w_down, const int32_t* tile_expert,
                                      const int32_t* n_tiles, const int32_t* pad_offsets, void* d_hidden, void* d_h1,
                                      void* d_x_sorted,
                                      int32_t* status, void* stream) {
  if (!d_y_sorted || !h1 || !w_gate_up || !w_down || !tile_expert || !n_tiles || !d_h1 || !d_x_sorted)
    return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (L % 64) != 0 || (F % 64) != 0) return LMOE_ERR_SHAPE;
  // one kernel for d_hidden -> SwiGLU adjoint -> d_x_sorted per 128-row tile (d_hidden is not written then)
  if (chain_applies(L, F))
    return launch_chain(CHAIN_BWD, P, E, L, F, d_y_sorted, w_gate_up, w_down, tile_expert, n_tiles, pad_offsets,
                        const_cast<void*>(h1), d_h1, d_x_sorted, status, static_cast<cudaStream_t>(stream));
  // d_hidden[P,F] = d_y_sorted[P,L] * Wd[e]^T : Wd[e] is [F,L] = [N,K] row-major -> K-major B
  GemmCall a;
  a.a_mn = 0;
  a.b_mn = 0;
  a.epi = EPI_BF16;
  a.grp = GRP_M;
  a.A[0] = d_y_sorted;
  a.lda[0] = L;
  a.B[0] = w_down;
  a.ldb[0] = L;
  a.Kseg[0] = L;
  a.M = static_cast<int>(P);
  a.N = F;
  a.C = d_hidden;
  a.ldc = F;
  a.padded_rows = P;
  a.groups = E;
  a.b_group_rows = F;
  a.tile_expert = tile_expert;
  a.n_m_tiles = n_tiles;
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  if (d_hidden) {
    if (int rc = launch_gemm(a)) return rc;
    if (int rc = lmoe_swiglu_bwd(P, F, h1, d_hidden, d_h1, 2ll * F, n_tiles, stream)) return rc;
  } else {
    // fused: the SwiGLU adjoint runs in the epilogue of the d_hidden GEMM, d_hidden never reaches memory
    GemmCall f = a;
    f.epi = EPI_SWIGLU_BWD;
    f.C = d_h1;
    f.ldc = 2ll * F;
    f.aux = h1;
    f.ld_aux = 2ll * F;
    if (int rc = launch_gemm(f)) return rc;
  }
  // d_x_sorted[P,L] = d_h1[P,2F] * Wgu[e]^T : Wgu[e] is [L,2F] = [N,K] row-major -> K-major B
  GemmCall b = a;
  b.pad_offsets = pad_offsets;  // CTA pairs that share an expert's weight loads
  b.A[0] = d_h1;
  b.lda[0] = 2ll * F;
  b.B[0] = w_gate_up;
  b.ldb[0] = 2ll * F;
  b.Kseg[0] = 2 * F;
  b.N = L;
  b.C = d_x_sorted;
  b.ldc = L;
  b.b_group_rows = L;
  return launch_gemm(b);
}

extern "C" int lmoe_experts_bwd_dgrad(const lmoe_shape* s, const void* d_y_sorted, const void* h1, const void* w_gate_up,
                                      const void* w_down, const lmoe_route* r, void* d_hidden, void* d_h1,
                                      void* d_x_sorted, int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!r) return LMOE_ERR_ARG;
  return lmoe_grouped_bwd_dgrad(lmoe_padded_rows(s), s->E, s->L, s->F, d_y_sorted, h1, w_gate_up, w_down,
                                r->tile_expert, r->n_tiles, r->pad_offsets, d_hidden, d_h1, d_x_sorted, status, stream);
}

static int grouped_bwd_wgrad_impl(int64_t P, int E, int L, int F, const void* x_sorted, const GatherA* g,
                                  const void* d_h1, const void* hidden, const void* d_y_sorted,
                                  const int32_t* pad_offsets, void* d_w_gate_up, void* d_w_down, int32_t* status,
                                  void* stream) {
  if (!x_sorted || !d_h1 || !hidden || !d_y_sorted || !pad_offsets || !d_w_gate_up || !d_w_down) return LMOE_ERR_ARG;
  if (P <= 0 || (P % LMOE_ROW_PAD) != 0 || E <= 0 || (L % 64) != 0 || (F % 64) != 0) return LMOE_ERR_SHAPE;
  // d_Wgu[e][L,2F] = x_sorted[rows_e]^T * d_h1[rows_e]
  GemmCall a;
  a.a_mn = 1;
  a.b_mn = 1;
  a.epi = EPI_BF16;
  a.grp = GRP_K;
  a.A[0] = x_sorted;
  a.lda[0] = L;
  a.B[0] = d_h1;
  a.ldb[0] = 2ll * F;
  a.M = L;
  a.N = 2 * F;
  a.C = d_w_gate_up;
  a.ldc = 2ll * F;
  a.c_group_stride = static_cast<long long>(L) * 2 * F;
  a.padded_rows = P;
  a.groups = E;
  a.pad_offsets = pad_offsets;
  a.status = status;
  a.stream = static_cast<cudaStream_t>(stream);
  GemmCall b = a;
  if (int rc = apply_gather(a, g)) return rc;
  if (int rc = launch_gemm(a)) return rc;
  // d_Wd[e][F,L] = hidden[rows_e]^T * d_y_sorted[rows_e]
  b.A[0] = hidden;
  b.lda[0] = F;
  b.B[0] = d_y_sorted;
  b.ldb[0] = L;
  b.M = F;
  b.N = L;
  b.C = d_w_down;
  b.ldc = L;
  b.c_group_stride = static_cast<long long>(F) * L;
  return launch_gemm(b);
}

extern "C" int lmoe_grouped_bwd_wgrad(int64_t P, int E, int L, int F, const void* x_sorted, const void* d_h1,
                                      const void* hidden, const void* d_y_sorted, const int32_t* pad_offsets,
                                      void* d_w_gate_up, void* d_w_down, int32_t* status, void* stream) {
  return grouped_bwd_wgrad_impl(P, E, L, F, x_sorted, nullptr, d_h1, hidden, d_y_sorted, pad_offsets, d_w_gate_up,
                                d_w_down, status, stream);
}

extern "C" int lmoe_grouped_bwd_wgrad_gather(int64_t P, int E, int L, int F, const void* src_rows, int64_t n_src_rows,
                                             const int32_t* row_index, int index_stride, int index_div, int64_t zero_row,
                                             const void* d_h1, const void* hidden, const void* d_y_sorted,
                                             const int32_t* pad_offsets, void* d_w_gate_up, void* d_w_down,
                                             int32_t* status, void* stream) {
  GatherA g;
  g.row_index = row_index;
  g.index_stride = index_stride;
  g.index_div = index_div;
  g.n_src_rows = n_src_rows;
  g.zero_row = zero_row;
  return grouped_bwd_wgrad_impl(P, E, L, F, src_rows, &g, d_h1, hidden, d_y_sorted, pad_offsets, d_w_gate_up, d_w_down,
                                status, stream);
}

extern "C" int lmoe_experts_bwd_wgrad(const lmoe_shape* s, const void* x_sorted, const void* d_h1, const void* hidden,
                                      const void* d_y_sorted, const lmoe_route* r, void* d_w_gate_up, void* d_w_down,
                                      int32_t* status, void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!r) return LMOE_ERR_ARG;
  return lmoe_grouped_bwd_wgrad(lmoe_padded_rows(s), s->E, s->L, s->F, x_sorted, d_h1, hidden, d_y_sorted,
                                r->pad_offsets, d_w_gate_up, d_w_down, status, stream);
}

extern "C" int lmoe_xside_bwd(const lmoe_shape* s, const void* dgrad_cat, const void* w_gate_up_s, const void* w_down,
                              const void* w_gate, const void* x, void* dx, void* d_w_gate_up_s, void* d_w_down,
                              void* d_w_gate, int grad_type, void* workspace, size_t workspace_bytes, int32_t* status,
                              void* stream) {
  if (int rc = check_dims(s)) return rc;
  if (!dgrad_cat || !w_gate_up_s || !w_down || !w_gate || !x || !dx || !d_w_gate_up_s || !d_w_down || !d_w_gate ||
      !workspace)
    return LMOE_ERR_ARG;
  if (grad_type != LMOE_F32 && grad_type != LMOE_BF16) return LMOE_ERR_ARG;
  if (workspace_bytes < lmoe_wgrad_workspace_bytes(s)) return LMOE_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Fs2 = 2 * s->Fs;
  const long long ld = static_cast<long long>(Fs2) + s->L + s->E;
  const bf16* d_h1_s = static_cast<const bf16*>(dgrad_cat);
  const bf16* d_x_latent = d_h1_s + Fs2;
  const bf16* d_logits = d_x_latent + s->L;
  // dx = d_h1_s[T,2Fs] * Wgu_s[2Fs,D] + d_x_latent[T,L] * Wdown[L,D] + d_logits[T,E] * Wg[E,D]
  GemmCall c = dense(d_h1_s, ld, 0, w_gate_up_s, s->D, 1, s->T, s->D, Fs2, dx, s->D, EPI_BF16, status, stream);
  c.nseg = 3;
  c.A[1] = d_x_latent;
  c.lda[1] = ld;
  c.B[1] = w_down;
  c.ldb[1] = s->D;
  c.Kseg[1] = s->L;
  c.A[2] = d_logits;
  c.lda[2] = ld;
  c.B[2] = w_gate;
  c.ldb[2] = s->D;
  c.Kseg[2] = s->E;
  if (int rc = launch_gemm(c)) return rc;
  // [d_Wgu_s ; d_Wdown ; d_Wg][2Fs+L+E, D] = dgrad_cat[T, 2Fs+L+E]^T * x[T,D]
  const int M = static_cast<int>(ld);
  const int split = wgrad_split(M, s->D, s->T);
  float* ws = static_cast<float*>(workspace);
  if (int rc = wgrad_gemm(dgrad_cat, ld, M, x, s->D, s->D, s->T, ws, split, status, stream)) return rc;
  const long long plane = static_cast<long long>(M) * s->D;
  const int f32 = grad_type == LMOE_F32;
  const int row0[3] = {0, Fs2, Fs2 + s->L}, col0[3] = {0, 0, 0}, rows[3] = {Fs2, s->L, s->E}, cols[3] = {s->D, s->D, s->D};
  void* const outs[3] = {d_w_gate_up_s, d_w_down, d_w_gate};
  const long long lds[3] = {s->D, s->D, s->D};
  return splitk_reduce_multi(ws, split, plane, s->D, 3, row0, col0, rows, cols, outs, lds, f32, st);
}
