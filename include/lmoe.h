/*
 * lmoe.h -- C ABI of liblmoe.so: the LatentMoE feed-forward hot path on NVIDIA B200 (sm_100a).
 *
 * The reference (Orolol/swamla) has no native boundary for this path: its layer is Python
 * (models/moe.py: LatentMoELayer) calling two Triton entry points (models/moe_triton.py).  This
 * header is the boundary a host binds instead; each entry point names the reference lines it
 * replaces.  Conventions shared by all entry points:
 *
 *   - plain pointers and sizes only; every data pointer is a DEVICE pointer of the current
 *     device, 16-byte aligned; `stream` is a cudaStream_t passed as void*;
 *   - the caller owns every buffer (inputs, outputs, workspace); the library never allocates or
 *     frees device memory and keeps nothing between calls;
 *   - all calls are stream-ordered and never synchronise;
 *   - return value: 0 = OK; <0 = argument / shape / alignment error found on the host before any
 *     launch (see lmoe_status_string); >0 = a cudaError_t from a launch;
 *   - `status` is one device int32 the kernels write when a bounded wait inside a kernel gives up
 *     (0 = no anomaly); the host may read it lazily;
 *   - bf16 = 16-bit brain float; "rows are padded": routed rows are laid out expert by expert,
 *     each expert's segment rounded up to a multiple of LMOE_ROW_PAD rows, pad rows zero.
 *
 * Shapes (names follow the reference ctor, models/moe.py:625-700):
 *   T tokens, D = n_embd, L = latent_dim, E = routed experts as built (n_experts*latent_ratio),
 *   K = activated experts as built, F = routed expert hidden dim, Fs = shared expert hidden dim.
 */
#ifndef LMOE_H_
#define LMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LMOE_VERSION 1
#define LMOE_ROW_PAD 128
#define LMOE_MAX_EXPERTS 256
#define LMOE_MAX_TOPK 32

/* error codes (<0) */
#define LMOE_OK 0
#define LMOE_ERR_ARG (-1)        /* null pointer / bad enum */
#define LMOE_ERR_SHAPE (-2)      /* unsupported dimension */
#define LMOE_ERR_ALIGN (-3)      /* pointer or leading dimension not 16-byte aligned */
#define LMOE_ERR_WORKSPACE (-4)  /* workspace too small */
#define LMOE_ERR_DRIVER (-5)     /* tensor-map encode entry point unavailable / failed */
#define LMOE_ERR_TOO_LARGE (-6)  /* problem exceeds the fixed scratch of a no-allocation entry point */

/* element types */
#define LMOE_BF16 0
#define LMOE_F32 1
#define LMOE_E4M3 2

typedef struct lmoe_shape {
  int32_t T, D, L, E, K, F, Fs;   /* Fs: width of the shared expert; n shared experts = one of n times the width */
  int32_t n_shared;               /* informational, 1 */
} lmoe_shape;

/* Routing tables produced by lmoe_route_permute, all int32, caller-allocated.
 *   counts[E], offsets[E+1], perm[T*K]   canonical (unpadded) result, = models/moe_triton.py:36-78
 *   pad_offsets[E+1]                      start row of each expert in the padded layout
 *   pos[T*K]                              flat index t*K+k -> padded row
 *   row_src[lmoe_padded_rows]             padded row -> flat index, -1 for pad rows
 *   tile_expert[lmoe_padded_rows/128]     expert owning each 128-row tile
 *   n_tiles[1]                            number of 128-row tiles in use
 */
typedef struct lmoe_route {
  int32_t* counts;
  int32_t* offsets;
  int32_t* perm;
  int32_t* pad_offsets;
  int32_t* pos;
  int32_t* row_src;
  int32_t* tile_expert;
  int32_t* n_tiles;
} lmoe_route;

/* ---- misc ---- */
int lmoe_version(void);
const char* lmoe_status_string(int code);
/* Number of kernels this library has launched in this process so far (all entry points). */
int64_t lmoe_launch_count(void);
/* Optional timing of the tcgen05 GEMM kernel: while enabled, every GEMM launch is bracketed by CUDA events on its
 * stream; lmoe_profile_collect waits for them and returns the summed duration (ms) and the number of launches
 * since the last collect.  Host-side measurement aid of the benchmark; off by default. */
int lmoe_profile_enable(int on);
int lmoe_profile_collect(float* gemm_ms, int* gemm_launches);
/* Upper bound of padded routed rows for a shape: roundup(T*K,128) + E*128. */
int64_t lmoe_padded_rows(const lmoe_shape* s);
/* Bytes of scratch lmoe_route_permute needs (block histograms). */
size_t lmoe_route_workspace_bytes(const lmoe_shape* s);

/* Dense bf16 GEMMs with at least 256 rows and 256 columns run on CTA pairs (tcgen05 cta_group::2: two SMs share a
 * 256 x 256 tile, each loading half of B).  On unless the environment has LMOE_PAIR_GEMM=0; this call switches it for
 * the process and returns the previous setting (0 / 1).  Results are identical up to the summation order inside the
 * tensor cores.  No counterpart in the reference (a kernel-selection switch). */
int lmoe_pair_gemm_enable(int on);

/* The routed expert chain in ONE kernel per direction.  Forward: gate_up GEMM -> SwiGLU -> down GEMM per 128-row tile,
 * the hidden activation goes from the first GEMM's epilogue into the second GEMM's operand through shared memory
 * (models/moe.py:814-828 in one pass).  Backward: d_hidden GEMM -> SwiGLU adjoint -> d_x GEMM, d_hidden never reaches
 * memory.  lmoe_grouped_fwd / lmoe_grouped_bwd_dgrad (and lmoe_experts_fwd / lmoe_experts_bwd_dgrad built on them) use
 * it whenever lmoe_chain_applies(L, F) is 1: bf16, L a multiple of 64 up to 256, F a multiple of 64; otherwise they
 * launch the separate grouped GEMMs.  On unless the environment has LMOE_CHAIN=0; lmoe_chain_enable switches it for the
 * process and returns the previous setting.  Forward results are bit-identical to the separate GEMMs, backward ones
 * agree to one bf16 ulp (another summation order of d_x over the 2F columns).  No counterpart in the reference (a
 * kernel-selection switch). */
int lmoe_chain_enable(int on);
int lmoe_chain_applies(int L, int F);

/* ---- generic dense GEMM on tcgen05 (building block; also the unit-test hook) ----
 * C[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
 *   a_mn = 0: A stored [M,K] row-major (lda = row stride);  a_mn = 1: A stored [K,M] row-major.
 *   b_mn = 0: B stored [N,K] row-major (an nn.Linear weight); b_mn = 1: B stored [K,N] row-major.
 *   c_type: LMOE_BF16 or LMOE_F32.  split_k > 1 divides the contraction among split_k tiles whose fp32
 *   partial results go to `workspace` (lmoe_gemm_workspace_bytes) and are then summed in a fixed order.
 * Replaces the cuBLAS calls behind nn.Linear on this path (models/moe.py:63,69,217,722,728). */
size_t lmoe_gemm_workspace_bytes(int M, int N, int split_k);
int lmoe_gemm_bf16(int M, int N, int K, const void* A, int64_t lda, int a_mn, const void* B, int64_t ldb, int b_mn,
                   void* C, int64_t ldc, int c_type, int split_k, void* workspace, size_t workspace_bytes,
                   int32_t* status, void* stream);

/* ---- forward ----
 * Two activations are kept side by side in one buffer so that their weight gradients become one GEMM:
 *   act_cat[T, L+Fs] bf16: columns [0,L) = routed (combined expert output), [L,L+Fs) = hidden_s. */

/* Gate logits (fp32) and latent down-projection (bf16).
 * x[T,D] bf16, w_gate[E,D] bf16, w_down[L,D] bf16 -> logits[T,E] f32, x_latent[T,L] bf16.
 * Replaces models/moe.py:217 (router.gate) and models/moe.py:722 (down_proj). */
int lmoe_xproj_fwd(const lmoe_shape* s, const void* x, const void* w_gate, const void* w_down, float* logits,
                   void* x_latent, int32_t* status, void* stream);

/* Sigmoid affinity + bias, canonical top-K (higher score first, lower expert index on ties),
 * normalised gating weights, per-row logsumexp and the z-loss.
 * logits[T,E] f32, expert_bias[E] f32 -> sel[T,K] i32, weights[T,K] f32, lse[T] f32,
 * z_loss[1] f32 = z_coef * mean(lse^2).  z_partial: scratch of ceil(T/8) floats.
 * Replaces models/moe.py:220-233 (AuxLossFreeRouter.forward). */
int lmoe_gate_topk_fwd(const lmoe_shape* s, const float* logits, const float* expert_bias, float z_coef, int32_t* sel,
                       float* weights, float* lse, float* z_partial, float* z_loss, void* stream);

/* Histogram, exclusive scan and stable permutation of the flat expert ids; also the padded
 * layout tables.  Deterministic (no global atomics).  Replaces models/moe_triton.py:12-78. */
int lmoe_route_permute(const lmoe_shape* s, const int32_t* sel, const lmoe_route* r, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Same result as lmoe_route_permute, for hosts that have no device memory to give as workspace.
 * (No counterpart in the reference: this entry point exists only on this boundary.)
 * Who needs it: a caller that cannot obtain device memory at the moment of the call -- a plugin whose
 * host interface hands it input and output buffers and nothing else, a serving process whose memory
 * pool already owns the whole GPU so that a fresh cudaMalloc fails, or a code path (an error handler,
 * a callback) where allocating is forbidden.  Such a caller passes only `sel` and the output tables;
 * the chunk histograms go to a fixed array of LMOE_STATIC_ROUTE_SCRATCH_BYTES that is part of the
 * library image on every GPU that loads it (held until the process exits).
 *   - Nothing is allocated or freed, here or in any library routine this calls.
 *   - Limit: lmoe_route_workspace_bytes(s) must not exceed LMOE_STATIC_ROUTE_SCRATCH_BYTES, i.e.
 *     ceil(T*K/256) * E <= 1,048,576 (for E = 128: T*K up to 2,097,152); beyond that the call launches
 *     nothing and returns LMOE_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call before any stream capture begins.
 *   - All calls on a device share the one array.  Nothing in it needs clearing between calls (each call
 *     writes every word before reading it), but two calls that overlap on the GPU -- different streams,
 *     or different host threads without ordering between them -- race on it and corrupt each other. */
#define LMOE_STATIC_ROUTE_SCRATCH_BYTES (4u << 20)
int lmoe_route_permute_static(const lmoe_shape* s, const int32_t* sel, const lmoe_route* r, void* stream);

/* Routed experts: gather x_latent rows into the padded layout, grouped gate_up GEMM with SwiGLU
 * epilogue, grouped down GEMM.
 * x_latent[T,L] bf16, w_gate_up[E,L,2F] bf16, w_down[E,F,L] bf16 ->
 * x_sorted[P,L], h1[P,2F], hidden[P,F], y_sorted[P,L] (all bf16, P = lmoe_padded_rows).
 * Replaces models/moe.py:762-766 (expand + gather), 814 (moe_gemm #1), 822-823 (SwiGLU),
 * 828 (moe_gemm #2) and models/moe_triton.py:85-242. */
int lmoe_experts_fwd(const lmoe_shape* s, const void* x_latent, const void* w_gate_up, const void* w_down,
                     const lmoe_route* r, void* x_sorted, void* h1, void* hidden, void* y_sorted, int32_t* status,
                     void* stream);

/* Shared expert, first half: h1_s = x * w_gate_up_s^T, hidden_s = silu(gate) * up.
 * x[T,D], w_gate_up_s[2Fs,D] -> h1_s[T,2Fs] bf16, hidden_s = act_cat[:, L:].
 * Replaces models/moe.py:63-67 (SwiGLUExpert.forward). */
int lmoe_shared_gateup_fwd(const lmoe_shape* s, const void* x, const void* w_gate_up_s, void* h1_s, void* act_cat,
                           int32_t* status, void* stream);

/* Weighted combine, latent up-projection, shared down-projection and the final add:
 *   routed[t] = sum_k weights[t,k] * y_sorted[pos[t*K+k]]   -> act_cat[:, :L]
 *   y = hidden_s * w_down_s^T + routed * w_up^T             -> y[T,D] bf16
 * y_sorted == NULL: act_cat[:, :L] already holds the routed rows (r and weights are then unused).
 * Replaces models/moe.py:837, 778-782 (scatter + sum), 728 (up_proj), 69 (shared down_proj), 731. */
int lmoe_combine_out_fwd(const lmoe_shape* s, const void* y_sorted, const lmoe_route* r, const float* weights,
                         void* act_cat, const void* w_down_s, const void* w_up, void* y, int32_t* status, void* stream);

/* ---- backward (adjoints of the lines cited above; the reference defines them only through
 *      autograd, and not at all for its grouped GEMM) ----
 * The three gradients that flow back into x-side GEMMs are kept side by side:
 *   dgrad_cat[T, 2Fs+L+E] bf16: columns [0,2Fs) = d_h1_s, [2Fs,2Fs+L) = d_x_latent, then d_logits.
 * Weight gradients of the dense linears are written (not accumulated) as `grad_type` (LMOE_F32 for
 * fp32 master weights, LMOE_BF16); split-K partials go to `workspace` (lmoe_wgrad_workspace_bytes). */
size_t lmoe_wgrad_workspace_bytes(const lmoe_shape* s);

/* dgrad of the output stage: d_routed[T,L] = dy * w_up, and d_h1_s = swiglu'(h1_s, dy * w_down_s) -> dgrad_cat[:, :2Fs].
 * d_hidden_s[T,Fs]: scratch for dy * w_down_s; if NULL the SwiGLU adjoint runs in the epilogue of that GEMM instead
 * and d_hidden_s never reaches memory. */
int lmoe_combine_out_bwd_dgrad(const lmoe_shape* s, const void* dy, const void* w_up, const void* w_down_s,
                               const void* h1_s, void* d_routed, void* d_hidden_s, void* dgrad_cat, int32_t* status,
                               void* stream);
/* wgrad of the output stage, one GEMM dy^T * act_cat: d_w_up[D,L] = dy^T routed, d_w_down_s[D,Fs] = dy^T hidden_s. */
int lmoe_combine_out_bwd_wgrad(const lmoe_shape* s, const void* dy, const void* act_cat, void* d_w_up,
                               void* d_w_down_s, int grad_type, void* workspace, size_t workspace_bytes,
                               int32_t* status, void* stream);
/* Adjoint of the weighted combine, in the padded layout:
 *   d_y_sorted[row] = weights[t,k] * d_routed[t];  d_weights[t,k] = <d_routed[t], y_sorted[row]>. */
int lmoe_combine_bwd(const lmoe_shape* s, const void* d_routed, const void* y_sorted, const float* weights,
                     const lmoe_route* r, void* d_y_sorted, float* d_weights, void* stream);
/* SwiGLU adjoint: h1[R,2H] (gate | up), d_hidden[R,H] -> d_h1[R,2H] with row stride ld_d_h1 elements.
 * If n_tiles_dev is non-null the row count is read on the device as 128 * n_tiles_dev[0]. */
int lmoe_swiglu_bwd(int64_t rows, int H, const void* h1, const void* d_hidden, void* d_h1, int64_t ld_d_h1,
                    const int32_t* n_tiles_dev, void* stream);
/* Routed dgrads: d_hidden = d_y_sorted * w_down[e]^T, d_h1 = swiglu'(h1, d_hidden),
 * d_x_sorted = d_h1 * w_gate_up[e]^T.  All in the padded layout.  d_hidden may be NULL: the SwiGLU adjoint then
 * runs in the epilogue of the first GEMM and d_hidden is never written (also for lmoe_grouped_bwd_dgrad). */
int lmoe_experts_bwd_dgrad(const lmoe_shape* s, const void* d_y_sorted, const void* h1, const void* w_gate_up,
                           const void* w_down, const lmoe_route* r, void* d_hidden, void* d_h1, void* d_x_sorted,
                           int32_t* status, void* stream);
/* Routed wgrads (overwrite, bf16): d_w_gate_up[e] = x_sorted[rows_e]^T d_h1[rows_e],
 * d_w_down[e] = hidden[rows_e]^T d_y_sorted[rows_e]. */
int lmoe_experts_bwd_wgrad(const lmoe_shape* s, const void* x_sorted, const void* d_h1, const void* hidden,
                           const void* d_y_sorted, const lmoe_route* r, void* d_w_gate_up, void* d_w_down,
                           int32_t* status, void* stream);
/* Adjoint of the gather: d_x_latent[t] = sum_k d_x_sorted[pos[t*K+k]]  -> dgrad_cat[:, 2Fs:2Fs+L]. */
int lmoe_unpermute_sum_bwd(const lmoe_shape* s, const void* d_x_sorted, const lmoe_route* r, void* dgrad_cat,
                           void* stream);
/* Router adjoint: gating-weight gradient through the normalisation and the sigmoid, plus the
 * z-loss term d_z * z_coef * 2 * lse * softmax / T (d_z: device float or NULL) -> dgrad_cat[:, 2Fs+L:]. */
int lmoe_gate_topk_bwd(const lmoe_shape* s, const float* logits, const int32_t* sel, const float* weights,
                       const float* d_weights, const float* lse, const float* d_z, float z_coef, void* dgrad_cat,
                       void* stream);
/* x-side backward.  dx[T,D] = d_h1_s * w_gate_up_s + d_x_latent * w_down + d_logits * w_gate (one GEMM,
 * three K segments read from dgrad_cat); weight gradients from one GEMM dgrad_cat^T * x:
 * d_w_gate_up_s[2Fs,D], d_w_down[L,D], d_w_gate[E,D]. */
int lmoe_xside_bwd(const lmoe_shape* s, const void* dgrad_cat, const void* w_gate_up_s, const void* w_down,
                   const void* w_gate, const void* x, void* dx, void* d_w_gate_up_s, void* d_w_down, void* d_w_gate,
                   int grad_type, void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- building blocks on explicit row counts (used by the expert-parallel host code) ----
 * The routed-expert stages again, but on a caller-chosen padded row count P (multiple of 128) and expert
 * count E (the local shard), with the tile tables given directly.  lmoe_experts_* above are these plus the
 * single-GPU gather.  Same reference lines: models/moe.py:814-828 and their adjoints. */
/* pad_offsets [E + 1] (first padded row of every expert, as lmoe_route / lmoe_ep_tables write it; may be NULL): lets the
 * chain kernel put two tiles of the same expert on a CTA pair that shares the expert's weight loads. */
int lmoe_grouped_fwd(int64_t P, int E, int L, int F, const void* x_sorted, const void* w_gate_up, const void* w_down,
                     const int32_t* tile_expert, const int32_t* n_tiles, const int32_t* pad_offsets, void* h1,
                     void* hidden, void* y_sorted, int32_t* status, void* stream);
int lmoe_grouped_bwd_dgrad(int64_t P, int E, int L, int F, const void* d_y_sorted, const void* h1, const void* w_gate_up,
                           const void* w_down, const int32_t* tile_expert, const int32_t* n_tiles,
                           const int32_t* pad_offsets, void* d_hidden, void* d_h1, void* d_x_sorted, int32_t* status,
                           void* stream);
int lmoe_grouped_bwd_wgrad(int64_t P, int E, int L, int F, const void* x_sorted, const void* d_h1, const void* hidden,
                           const void* d_y_sorted, const int32_t* pad_offsets, void* d_w_gate_up, void* d_w_down,
                           int32_t* status, void* stream);

/* The same two entry points with the A operand of the gate_up GEMMs GATHERED by the TMA unit instead of read from a
 * materialised x_sorted: padded row i is row row_index[i * index_stride] / index_div of src_rows[n_src_rows, L] (bf16, row
 * stride L); a negative entry reads row `zero_row`, which the caller keeps all zero (pad rows of the routed layout).
 * With row_index = lmoe_route.row_src (flat index t*K + k) and index_div = K this removes the gather kernel of models/moe.py:749-757 (the
 * x[token_indices] copy) and the x_sorted buffer. */
int lmoe_grouped_fwd_gather(int64_t P, int E, int L, int F, const void* src_rows, int64_t n_src_rows,
                            const int32_t* row_index, int index_stride, int index_div, int64_t zero_row, const void* w_gate_up,
                            const void* w_down, const int32_t* tile_expert, const int32_t* n_tiles, void* h1, void* hidden,
                            void* y_sorted, int32_t* status, void* stream);
int lmoe_grouped_bwd_wgrad_gather(int64_t P, int E, int L, int F, const void* src_rows, int64_t n_src_rows,
                                  const int32_t* row_index, int index_stride, int index_div, int64_t zero_row, const void* d_h1,
                                  const void* hidden, const void* d_y_sorted, const int32_t* pad_offsets,
                                  void* d_w_gate_up, void* d_w_down, int32_t* status, void* stream);
/* The single GEMMs behind the three calls above, for hosts that schedule them individually:
 * out[P,N] = a[P,K] * B[e] with B stacked [E,K,N] (b_mn = 1) or [E,N,K] (b_mn = 0); out[e][M,N] = a[rows_e,M]^T b[rows_e,N]. */
int lmoe_grouped_rows_bf16(int64_t P, int E, int K, int N, const void* a, const void* b, int b_mn,
                           const int32_t* tile_expert, const int32_t* n_tiles, void* out, int32_t* status, void* stream);
int lmoe_grouped_wgrad_bf16(int64_t P, int E, int M, int N, const void* a, const void* b, const int32_t* pad_offsets,
                            void* out, int32_t* status, void* stream);
/* dst[r] = src[index[r] / div] for r < rows (zeros where index[r] < 0); rows of L bf16.  If n_tiles_dev is
 * non-null only the first 128 * n_tiles_dev[0] rows are written.  (models/moe.py:762-766 as a primitive.) */
int lmoe_gather_rows(const void* src, const int32_t* index, int div, int64_t rows, int L, const int32_t* n_tiles_dev,
                     void* dst, void* stream);
/* out[t] = sum_k weights[t,k] * rows_in[index[t*K+k]] (weights NULL: plain sum), fp32 accumulation in slot
 * order; out has row stride ld_out elements.  (models/moe.py:837,778-782 as a primitive.) */
int lmoe_combine_rows(const void* rows_in, const int32_t* index, const float* weights, int T, int K, int L, void* out,
                      int64_t ld_out, void* stream);
/* out[t] = addend[t] + sum_k weights[t*K+k] * rows_in[index[t*K+k]]  (weights == NULL: plain sum); fp32 accumulation in
 * slot order, bf16 out.  Row strides ld_addend / ld_out in elements.  The add of the routed sum onto another branch's
 * result: models/moe.py:366 (MoELayer: shared_output + routed_output) and its adjoint on the x side. */
int lmoe_combine_rows_add(const void* rows_in, const int32_t* index, const float* weights, const void* addend,
                          int64_t ld_addend, int T, int K, int L, void* out, int64_t ld_out, void* stream);

/* Dense SwiGLU up-projection: h1[M, 2H] = A[M, K] * W[2H, K]^T (gate = first H outputs), hidden[M, H] = silu(gate) * up,
 * both bf16, SwiGLU in the GEMM epilogue.  H a multiple of 32.  Replaces the first half of SwiGLUExpert.forward
 * (models/moe.py:63-67) for any width. */
int lmoe_gemm_swiglu_bf16(int M, int H, int K, const void* A, int64_t lda, const void* W, int64_t ldw, void* h1,
                          int64_t ld_h1, void* hidden, int64_t ld_hidden, int32_t* status, void* stream);

/* Adjoint of lmoe_combine_rows over `rows` rows: flat = row_to_flat[r] (t = flat / K);
 * d_y_rows[r] = weights[flat] * d_routed[t], d_weights[flat] = <d_routed[t], y_rows[r]>; zeros where flat < 0. */
int lmoe_combine_bwd_rows(const void* d_routed, const void* y_rows, const float* weights, const int32_t* row_to_flat,
                          int64_t rows, int K, int L, const int32_t* n_tiles_dev, void* d_y_rows, float* d_weights,
                          void* stream);
/* inv[perm[i]] = i. */
int lmoe_invert_perm(const int32_t* perm, int64_t n, int32_t* inv, void* stream);

/* ---- expert parallelism (no counterpart in the reference, which has data parallelism only;
 *      design note aidocs/moe.md:940-997) ----
 * Rank g of G owns experts [g*E/G, (g+1)*E/G).  counts_all[G][E] = rows every source rank routes to every
 * expert (an all-gather of the `counts` tables).  The receive buffer of the dispatch all-to-all is ordered by
 * source rank, then local expert.  Outputs, for this rank's shard:
 *   recv_pos[n_recv]  receive index -> padded local row       row_src[P_local]  padded row -> receive index | -1
 *   pad_offsets[E/G+1], tile_expert[P_local/128], n_tiles[1]   with P_local >= roundup(n_recv,128) + 128*E/G */
int lmoe_ep_plan(const int32_t* counts_all, int G, int E, int rank, int32_t* recv_pos, int32_t* row_src,
                 int32_t* pad_offsets, int32_t* tile_expert, int32_t* n_tiles, void* stream);

/* One-sided variant of the exchange: rows are stored through peer pointers (NVLink) straight into the destination
 * rank's padded expert layout, so there is no send buffer, no all-to-all and no regroup copy, and nothing is sized
 * on the host.  `capacity_rows` (multiple of 128) is the static size of every rank's incoming buffer; if a shard
 * would receive more, `status` is set to 201 and the excess rows are dropped.  The caller orders the phases across
 * ranks with stream-ordered collectives (dispatch -> barrier -> grouped GEMMs -> return -> barrier).
 *   lmoe_ep_tables   src_off[G*E], dst_base[E], seg_cum[(E/G)*G], pad_offsets[E/G+1], tile_expert[cap/128], n_tiles[1]
 *   lmoe_ep_dispatch      row i of this rank's expert-sorted order (perm, sel, offsets from lmoe_route_permute) =
 *                         src_rows[perm[i]/K]  ->  peer_bufs[owner][dst_base[e] + i - offsets[e]]
 *   lmoe_ep_dispatch_bwd  same walk with rows weights[flat] * d_routed[t]; also d_weights[flat] = <d_routed[t], y_ret[i]>
 *   lmoe_ep_zero_pads     zeroes the pad rows of this rank's incoming buffer
 *   lmoe_ep_return        padded local row p -> peer_ret[source][src_off[source][e] + r]  (inverse walk)
 * peer_bufs / peer_ret: DEVICE arrays of G device pointers (this rank's own buffer at index `rank`). */
int lmoe_ep_tables(const int32_t* counts_all, int G, int E, int rank, int64_t capacity_rows, int32_t* src_off,
                   int32_t* dst_base, int32_t* seg_cum, int32_t* pad_offsets, int32_t* tile_expert, int32_t* n_tiles,
                   int32_t* status, void* stream);
int lmoe_ep_zero_pads(void* buf, int L, const int32_t* pad_offsets, const int32_t* seg_cum, const int32_t* counts_all,
                      int G, int E, int rank, void* stream);
int lmoe_ep_dispatch(const void* src_rows, const int32_t* perm, const int32_t* sel, const int32_t* offsets,
                     const int32_t* dst_base, int64_t n_rows, int K, int E, int G, int L, int64_t capacity_rows,
                     void* const* peer_bufs, int32_t* status, void* stream);
int lmoe_ep_dispatch_bwd(const void* d_routed, const void* y_ret, const float* weights, const int32_t* perm,
                         const int32_t* sel, const int32_t* offsets, const int32_t* dst_base, int64_t n_rows, int K,
                         int E, int G, int L, int64_t capacity_rows, void* const* peer_bufs, float* d_weights,
                         int32_t* status, void* stream);
int lmoe_ep_return(const void* rows, const int32_t* tile_expert, const int32_t* n_tiles, const int32_t* pad_offsets,
                   const int32_t* seg_cum, const int32_t* src_off, const int32_t* counts_all, int G, int E, int rank,
                   int L, int64_t capacity_rows, void* const* peer_ret, void* stream);

/* De-duplicated one-sided exchange: one row per (token, destination RANK) instead of one per (token, expert).  The
 * source stores token t's latent row once into the staging slot [rank*stride + t] of every rank that owns one of its
 * experts, plus per routed row the words the owner needs (padded row, combine weight); the owner gathers its padded
 * layout locally, and after the grouped GEMMs reduces a token's result rows to ONE row per (token, owner) before it
 * stores them back (ret[owner*stride + t] at the source), where lmoe_epd_sum adds the owners' partial sums.  Partial
 * sums travel in bf16.  `stride` = slot count per source (>= every rank's token count), the same on all ranks.
 * Symmetric buffers per rank: stage [G*stride, L] bf16, meta [capacity_rows] of {int32 slot, fp32 weight},
 * mask [G*stride] uint32, slots [G*stride*K] int32, ret [G*stride, L] bf16, dw [stride*K] fp32.
 * The peer_* arguments are DEVICE arrays of G device pointers.  Tables come from lmoe_ep_tables; `pos` is the inverse
 * of the routing permutation (lmoe_invert_perm).  No counterpart in the reference (data parallelism only,
 * train.py:944-949; the sharding follows aidocs/moe.md:940-997).
 *   lmoe_epd_send           peer_meta != NULL: rows + mask/slots/meta (forward).  NULL: rows only (backward; pos,
 *                           offsets, dst_base, weights, peer_mask, peer_slots unused).  Overflow -> status 201.
 *   lmoe_epd_gather         n_slots = G*stride (a row whose slot word is outside [0, n_slots) is left a pad row).
 *                           y_sorted == NULL: out[p] = stage[slot(p)], pad rows zero.  Otherwise the adjoint of the
 *                           combine: out[p] = w_p * stage[slot(p)], d_w_row[p] = <stage[slot(p)], y_sorted[p]>.
 *   lmoe_epd_reduce_return  d_w_row == NULL: weighted sums sum_k w_k rows[p_k] (forward).  Otherwise plain sums and
 *                           d_w_row[p_k] -> peer_dw[source][t*K + k] (backward).
 *   lmoe_epd_sum            out[t] (row stride ld_out elements) = sum over the owners of token t of ret[g*stride + t] */
int lmoe_epd_send(const void* src_rows, const int32_t* sel, const int32_t* pos, const int32_t* offsets,
                  const int32_t* dst_base, const float* weights, int64_t T, int K, int E, int G, int rank, int L,
                  int64_t capacity_rows, int64_t stride, void* const* peer_stage, void* const* peer_meta,
                  void* const* peer_mask, void* const* peer_slots, int32_t* status, void* stream);
int lmoe_epd_gather(const void* stage, const void* meta, const int32_t* tile_expert, const int32_t* n_tiles,
                    const int32_t* pad_offsets, const int32_t* seg_cum, const int32_t* counts_all, int G, int E, int rank,
                    int L, int64_t capacity_rows, int64_t n_slots, const void* y_sorted, void* out_rows, float* d_w_row,
                    void* stream);
int lmoe_epd_reduce_return(const void* rows, const void* meta, const void* mask, const int32_t* slots,
                           const float* d_w_row, const int32_t* src_off, const int32_t* counts_all, int G, int E, int rank,
                           int K, int L, int64_t stride, int64_t capacity_rows, void* const* peer_ret,
                           void* const* peer_dw, void* stream);
int lmoe_epd_sum(const void* ret, const int32_t* sel, int64_t T, int K, int E, int G, int L, int64_t stride, void* out,
                 int64_t ld_out, void* stream);

/* Barrier across the G ranks of an expert-parallel group without a collective library call: peer_flags[g] points at rank
 * g's int32 flags[G] in symmetric memory, epoch_counter at an int32 in this rank's own memory (both zeroed once, before
 * the first barrier; the kernel increments the counter, so the call may sit in a replayed CUDA graph; every rank must run
 * the same sequence of barriers).  Stream-ordered like any kernel.  A rank that waits longer than about two seconds
 * records status 202 and carries on.  Replaces the one-word all-reduce the exchange used as a barrier (the reference has
 * no counterpart: its expert parallelism is pseudo-code, aidocs/moe.md:940-997). */
int lmoe_ep_flag_barrier(void* const* peer_flags, int32_t* epoch_counter, int rank, int G, int32_t* status, void* stream);

/* ---- FP8 (e4m3) expert path ----
 * Per-tensor dynamic scaling, the "tensorwise" recipe named by optimization/fp8_native.py:103-110 (torchao
 * Float8Linear; the reference applies it to nn.Linear modules only, fp8_native.py:38-66,112-116, never to the
 * routed experts -- running the expert GEMMs in e4m3 is this boundary's extension of that recipe).
 *   q = saturate_e4m3(x * 448 / amax(x)),  deq = amax(x) / 448,  result = deq_a * deq_b * (A_q * B_q^T), fp32 accumulate.
 * A tensor is quantised once and serves forward, dgrad and wgrad GEMMs alike (the scale is per tensor).
 * Contraction extents of e4m3 GEMMs must be multiples of 128. */
/* x[rows,row_len] bf16 -> q e4m3 (same shape), amax[1], deq[1].  With n_tiles_dev only the first
 * 128 * n_tiles_dev[0] rows are read and written (padded routed layout). */
int lmoe_fp8_quantize(const void* x_bf16, int64_t rows, int row_len, const int32_t* n_tiles_dev, void* q_e4m3,
                      float* amax, float* deq, void* stream);
/* C[M,N] bf16 = deq_a * deq_b * A_q[M,K] * B_q[N,K]^T; operand major-ness as in lmoe_gemm_bf16. */
int lmoe_gemm_fp8(int M, int N, int K, const void* A, int64_t lda, int a_mn, const void* B, int64_t ldb, int b_mn,
                  const float* deq_a, const float* deq_b, void* C, int64_t ldc, int32_t* status, void* stream);
/* Routed gate_up with SwiGLU epilogue (models/moe.py:814,822-823): xq[P,L], wq[E,L,2F] -> h1[P,2F], hidden[P,F] bf16. */
int lmoe_grouped_gateup_fp8(int64_t P, int E, int L, int F, const void* xq, const void* wq, const float* deq_x,
                            const float* deq_w, const int32_t* tile_expert, const int32_t* n_tiles, void* h1,
                            void* hidden, int32_t* status, void* stream);
/* out[P,N] bf16 = aq[P,K] * Bq[e]: Bq stacked [E,K,N] (b_mn = 1: forward down GEMM, models/moe.py:828) or
 * [E,N,K] (b_mn = 0: the same weights as dgrad operand). */
int lmoe_grouped_rows_fp8(int64_t P, int E, int K, int N, const void* aq, const void* bq, int b_mn, const float* deq_a,
                          const float* deq_b, const int32_t* tile_expert, const int32_t* n_tiles, void* out,
                          int32_t* status, void* stream);
/* Expert weight gradients: out[e][M,N] bf16 = aq[rows_e, M]^T * bq[rows_e, N]. */
int lmoe_grouped_wgrad_fp8(int64_t P, int E, int M, int N, const void* aq, const void* bq, const float* deq_a,
                           const float* deq_b, const int32_t* pad_offsets, void* out, int32_t* status, void* stream);

/* The steps either side of the layer in the reference's block, x_out = x + ffn(ffn_norm(x)) (models/mla_block.py:83-85,
 * 159), as fused row kernels: RMSNorm (models/normalization.py:25-39; fp32 arithmetic on bf16 rows, one read and one
 * write instead of the five element-wise passes of the eager module), the residual add, and ONE backward kernel for the
 * adjoint of the norm plus the residual branch:
 *   lmoe_rmsnorm_fwd   xn[T,D] = weight * x * rstd,  rstd[t] = rsqrt(mean(x[t]^2) + eps)  (x, xn bf16; weight, rstd fp32)
 *   lmoe_add_bf16      out = a + b over n bf16 elements (n % 8 == 0)
 *   lmoe_rmsnorm_bwd   dx = rstd * (g - x * rstd^2 * mean(g * x)) + d_residual (nullable), g = d_xn * weight;
 *                      d_weight[D] fp32 = sum_t d_xn * x * rstd, summed in a fixed order (deterministic)
 * D a multiple of 8, D <= 2048.  workspace: lmoe_rmsnorm_workspace_bytes(D). */
size_t lmoe_rmsnorm_workspace_bytes(int D);
int lmoe_rmsnorm_fwd(const void* x, const float* weight, float eps, int64_t T, int D, void* xn, float* rstd, void* stream);
int lmoe_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream);
int lmoe_rmsnorm_bwd(const void* x, const float* weight, const float* rstd, const void* d_xn, const void* d_residual,
                     int64_t T, int D, void* dx, float* d_weight, void* workspace, size_t workspace_bytes, void* stream);

/* ---- router bias update (after backward) ----
 * load = histogram(sel) (= counts); bias -= gamma * sign(load - T*K/E); history = .99 history + .01 load.
 * T*K is read from the histogram (sum of counts), so `counts` may be the sum of several ranks' histograms
 * (expert parallelism) whatever their token counts; s->T is not used.  Replaces models/moe.py:254-275. */
int lmoe_router_bias_update(const lmoe_shape* s, const int32_t* counts, float gamma, float* expert_bias,
                            float* load_history, void* stream);

/* ---- small utilities ---- */
int lmoe_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream);
int lmoe_cast_bf16_to_f32(const void* src, float* dst, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LMOE_H_ */
