// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] = A[M,K] * B[N,K]^T      bf16 (kind::f16) or e4m3 (kind::f8f6f4) operands, fp32 accumulation in
//                                   tensor memory; e4m3 results are multiplied by two per-tensor de-scale factors
//
// One CTA per SM walks a static tile schedule.  Roles:
//   warp 0      TMA producer: fills a ring of shared-memory stages (A tile 128 x 64, B tile BN x 64)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) and commits to mbarriers;
//               also owns the tensor-memory allocation (two accumulators of BN columns)
//   warps 2..9  epilogue, two groups of four warps: tcgen05.ld the finished accumulator (a warp owns the 32
//               lanes = rows of its quadrant), convert, write 32-column slabs into a swizzled shared-memory
//               staging buffer and hand it to a TMA store.  Group 0 takes the even slabs, group 1 the odd
//               ones, each with its own buffer, named barrier and issuing thread, so one group's store
//               drains while the other computes and every scheduler has two warps to hide latency with.
//               The accumulator is released as soon as its last slab is in registers, so the next tile's
//               main loop overlaps the stores
//
// Operand major-ness (template): K-major = the contraction index is contiguous in memory
// (activations [rows,K], nn.Linear weights [N,K]); MN-major = the row/column index is contiguous
// (routed expert weights [K,N], both operands of every weight gradient).
//
// Grouping (template):
//   GRP_M  rows are the padded routed layout; a 128-row tile belongs to one expert (tile_expert) and
//          B is that expert's slice of a stacked weight tensor
//   GRP_K  one output matrix per expert; the contraction runs over that expert's padded row range
//
// K segments: up to three (A_i, B_i) pairs are accumulated into one tile, which fuses sums of
// products such as hidden_s*Wd_s^T + routed*Wup^T without a concatenated copy.
// Split-K (dense only): the k-blocks are divided among `split_k` tiles; slice s writes its partial
// result to plane s of a [split_k, M, N] fp32 workspace (third coordinate of the output map) and a
// separate deterministic kernel reduces the planes.
#pragma once
#include "common/ptx.cuh"

namespace lmoe {

// EPI_SWIGLU_BWD: the accumulator is d_hidden; the epilogue reads the saved gate/up of the same rows and
// columns (aux = h1) and writes d_h1 = [d_gate | d_up] -- the SwiGLU adjoint without a d_hidden round trip.
enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_SWIGLU_BWD = 3 };
enum : int { GRP_NONE = 0, GRP_M = 1, GRP_K = 2 };

constexpr int kBM = 128;
constexpr int kBKBytes = 128;  // bytes per k-block row (one 128-byte swizzle row): 64 bf16 or 128 e4m3 elements
constexpr int kGemmThreads = 320;
constexpr int kEpiGroupThreads = 128;
constexpr int kSlabCols = 32;  // output columns per epilogue slab

// status codes written by a wait that gave up
constexpr int kStatusProducerTimeout = 101;
constexpr int kStatusMmaTimeout = 102;
constexpr int kStatusEpilogueTimeout = 103;

struct alignas(64) GemmParams {
  CUtensorMap tmA[3];
  CUtensorMap tmB[3];
  CUtensorMap tmC;   // 3-D {N, M, planes}: main output (h1 for SwiGLU)
  CUtensorMap tmC2;  // SwiGLU: hidden output
  int seg_kiters[3];
  int nseg;
  int M, N;              // output extent (per group for GRP_K); SwiGLU: N = width of one half
  int m_tiles, n_tiles;  // tile counts (per group for GRP_K; upper bound for GRP_M)
  int groups;            // GRP_K: number of experts
  int split_k;           // GRP_NONE: number of k-slices (each writes its own output plane)
  int half;              // SwiGLU: width of the gate half (F or Fs)
  const int* tile_expert;  // GRP_M
  const int* n_m_tiles;    // GRP_M: device scalar, number of 128-row tiles in use
  int b_group_rows;        // GRP_M: rows of the stacked B tensor per expert
  const int* pad_offsets;  // GRP_K
  const float* deq_a;      // e4m3: per-tensor de-scale factors (amax / 448) of A and B, device scalars
  const float* deq_b;
  const void* aux;         // EPI_SWIGLU_BWD: h1 [rows, 2*N] bf16 (gate | up), row stride ld_aux elements
  long long ld_aux;
  CUtensorMap tmAux;       // EPI_SWIGLU_BWD: the same tensor as 128-row boxes of 64 columns (128-byte swizzle), staged by TMA
  // Gathered A operand (bf16, one K segment): row i of the padded routed layout is row
  // a_rows[i * a_rows_stride] / a_rows_div of the tensor behind tmA[0] (negative entry: a_zero_row, a row of zeros).  GRP_M with K-major A gathers the tile's M rows,
  // GRP_K (MN-major A) gathers the contraction rows.  NULL: A is read in place.
  const int* a_rows;
  int a_rows_stride;
  int a_rows_div;
  int a_zero_row;
  int* status;
};

template <int BN, int EPI, int GRP = 0>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBKBytes;
  static constexpr int kBBytes = BN * kBKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // one slab = 128 rows x 32 columns: 8 KB in bf16 (64-byte rows), 16 KB in fp32 (128-byte rows)
  static constexpr int kSlabBytes = (EPI == EPI_F32) ? 16384 : 8192;
  // SwiGLU with 256-wide tiles: the hidden slab is staged in the gate slab's buffer once the gate store has read it, so
  // that two slabs per group are enough and the operand ring gets a fourth 48 KB stage (bytes in flight are what
  // these kernels are short of; measured 5 us per GEMM and stage)
  static constexpr bool kHiddenReusesGate = (EPI == EPI_SWIGLU && BN == 256);
  static constexpr int kStreams = (EPI == EPI_SWIGLU) ? (kHiddenReusesGate ? 2 : 3) : (EPI == EPI_SWIGLU_BWD ? 2 : 1);
  // staging buffers per epilogue group: two for the plain bf16 epilogue (its slabs are cheap to produce, so the
  // read latency of the previous TMA store would otherwise be exposed on every slab) and for the adjoint epilogue of
  // the grouped GEMM (four k-blocks per tile: three stages are enough, the second buffer gains 3 %); one for the
  // others, whose long contractions need the shared memory for a fourth stage
  static constexpr int kBufsPerGroup =
      (EPI == EPI_BF16 || (EPI == EPI_SWIGLU_BWD && GRP == 1) || (EPI == EPI_SWIGLU && BN == 128)) ? 2 : 1;
  static constexpr int kStagingBytes = 2 * kBufsPerGroup * kStreams * kSlabBytes;
  // EPI_SWIGLU_BWD: per epilogue group the saved gate / up of its 64 columns of the next tile (two 16 KB boxes)
  // (2 groups x 2 buffers x (gate 8 KB + up 8 KB))
  static constexpr int kAuxBytes = (EPI == EPI_SWIGLU_BWD) ? 65536 : 0;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kBudget = 232448 - 1024 - kBarrierBytes - kStagingBytes - kAuxBytes;
  static constexpr int kStagesMax = kBudget / kStageBytes;
  static constexpr int kStages = kStagesMax > 6 ? 6 : kStagesMax;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kAuxBytes + kBarrierBytes + 1024;  // +1024: alignment
  static_assert(kStages >= 3, "pipeline too shallow");
};

// sigmoid(g) = 0.5 + 0.5 * tanh(g / 2) on the hardware tanh unit: ONE special-function instruction per value
// (exp2 + reciprocal take two, and a full-precision division many more; the SwiGLU epilogues are bound by instruction
// issue, not by memory).  tanh.approx.f32 has a relative error of 2^-11, an eighth of a bf16 ulp.
__device__ __forceinline__ float sigmoid_fast(float g) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
  return fmaf(0.5f, t, 0.5f);
}
// silu(g) = g * sigmoid(g)
__device__ __forceinline__ float silu_f(float g) { return g * sigmoid_fast(g); }

// Named barrier over the 128 threads of one epilogue group (barrier id 1 or 2).
__device__ __forceinline__ void epi_bar_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
// AND-reduction of a predicate over the 128 threads of one epilogue group.
__device__ __forceinline__ bool epi_bar_all(int id, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %2, 0;\n"
      "bar.red.and.pred q, %1, 128, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(out)
      : "r"(id), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

// 3-D tiled store; c0 = innermost (column) coordinate.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// One 128 x 32 bf16 slab row (64 bytes) into a 64-byte-swizzled staging buffer: the 16-byte chunk j of
// row r lands at chunk j ^ ((r >> 1) & 3), which is what a SWIZZLE_64B tensor map expects.
__device__ __forceinline__ void stage_row_bf16(uint8_t* buf, int r, const uint32_t (&p)[16]) {
  const int sw = (r >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    *reinterpret_cast<uint4*>(buf + r * 64 + ((j ^ sw) << 4)) = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
  }
}
// One 128 x 32 fp32 slab row (128 bytes), 128-byte swizzle: chunk j of row r lands at chunk j ^ (r & 7).
__device__ __forceinline__ void stage_row_f32(uint8_t* buf, int r, const float (&v)[32]) {
  const int sw = r & 7;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    *reinterpret_cast<float4*>(buf + r * 128 + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
}

// ESZ = operand element size in bytes: 2 (bf16) or 1 (e4m3).
template <bool A_MN, bool B_MN, int BN, int EPI, int GRP, int ESZ = 2>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  using S = GemmSmem<BN, EPI, GRP>;
  constexpr int STAGES = S::kStages;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  static_assert(BN == 128 || BN == 256, "BN");
  static_assert(ESZ == 1 || ESZ == 2, "ESZ");
  constexpr bool kSwiglu = (EPI == EPI_SWIGLU);
  constexpr int BK_E = kBKBytes / ESZ;   // elements per k-block
  constexpr int CH = 128 / ESZ;          // width (elements) of one MN-major chunk: 128 bytes of row/column index
  constexpr int CH_BYTES = BK_E * 128;   // one MN-major chunk: BK_E k-rows of 128 bytes
  constexpr int UK = 32 / ESZ;           // elements per tcgen05.mma along K
  static_assert(!(kSwiglu && B_MN && (BN / 2) < CH), "gate and up halves must each be whole MN-major chunks");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * S::kStageBytes;  // 1024-aligned: stage sizes are multiples of 1024
  uint8_t* aux_stage = staging + S::kStagingBytes;       // EPI_SWIGLU_BWD only (kAuxBytes == 0 otherwise)
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(aux_stage + S::kAuxBytes);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_tfull = bar_empty + STAGES;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint64_t* bar_aux = bar_tempty + 2;                    // [4]: one per epilogue group in use
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_aux + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_tfull[i], 1);
      mbar_init(&bar_tempty[i], 8);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&bar_aux[i], 1);
    if (EPI == EPI_SWIGLU_BWD) tma_prefetch_desc(&p.tmAux);
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < p.nseg; ++i) {
      tma_prefetch_desc(&p.tmA[i]);
      tma_prefetch_desc(&p.tmB[i]);
    }
    tma_prefetch_desc(&p.tmC);
    if (kSwiglu) tma_prefetch_desc(&p.tmC2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- tile schedule (identical arithmetic in every role) ----
  int m_tiles = p.m_tiles;
  if (GRP == GRP_M) m_tiles = min(*p.n_m_tiles, p.m_tiles);
  const int tiles_mn = m_tiles * p.n_tiles;
  int total_tiles = tiles_mn;
  if (GRP == GRP_NONE) total_tiles = tiles_mn * p.split_k;
  if (GRP == GRP_K) total_tiles = tiles_mn * p.groups;

  struct Tile {
    int m0, nt, plane, grp, kb, ke, krow0;
  };
  auto decode = [&](int id) {
    Tile t;
    const int outer = id / tiles_mn;
    const int rem = id - outer * tiles_mn;
    t.m0 = (rem / p.n_tiles) * kBM;
    t.nt = rem % p.n_tiles;
    t.plane = 0;
    t.grp = 0;
    t.kb = 0;
    t.ke = p.seg_kiters[0];
    t.krow0 = 0;
    if (GRP == GRP_NONE) {
      if (p.split_k > 1) {
        const int per = (p.seg_kiters[0] + p.split_k - 1) / p.split_k;
        t.kb = min(outer * per, p.seg_kiters[0]);
        t.ke = min(t.kb + per, p.seg_kiters[0]);
        t.plane = outer;
      }
    } else if (GRP == GRP_M) {
      t.grp = p.tile_expert[t.m0 / kBM];
    } else {
      t.grp = outer;
      t.plane = outer;
      const int r0 = p.pad_offsets[outer], r1 = p.pad_offsets[outer + 1];
      t.krow0 = r0;
      t.ke = (r1 - r0) / BK_E;
    }
    return t;
  };
  auto tile_kiters = [&](const Tile& t) {
    int n = t.ke - t.kb;
    for (int s = 1; s < p.nseg; ++s) n += p.seg_kiters[s];
    return n;
  };

  // B tile of one pipeline stage (issued by one thread)
  auto load_b = [&](uint8_t* sb, uint64_t* bar, const Tile& t, int s, int kcoord) {
    const int grp_rows = (GRP == GRP_M) ? t.grp * p.b_group_rows : 0;
    if (!B_MN) {
      if (kSwiglu) {
        const int nh = t.nt * (BN / 2);
        tma_load_2d(sb, &p.tmB[s], bar, kcoord, grp_rows + nh);
        tma_load_2d(sb + (BN / 2) * 128, &p.tmB[s], bar, kcoord, grp_rows + p.half + nh);
      } else {
        tma_load_2d(sb, &p.tmB[s], bar, kcoord, grp_rows + t.nt * BN);
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN / CH; ++j) {
        constexpr int kHalfChunks = BN / (2 * CH);
        int ncol;
        if (kSwiglu) {
          const int nh = t.nt * (BN / 2);
          ncol = (j < kHalfChunks) ? (nh + j * CH) : (p.half + nh + (j - kHalfChunks) * CH);
        } else {
          ncol = t.nt * BN + j * CH;
        }
        tma_load_2d(sb + j * CH_BYTES, &p.tmB[s], bar, ncol, grp_rows + kcoord);
      }
    }
  };

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (ESZ == 2 && GRP != GRP_NONE && p.a_rows != nullptr) {
      // Gathered A: the whole warp runs the loop; lane l issues the gather of four rows (l-th group of four) of
      // every stage, lane 0 also arms the barrier and loads B.  A stage holds 128 rows of 128 bytes either way
      // (K-major: 128 tile rows; MN-major: two chunks of 64 contraction rows), i.e. 32 gathers of 512 bytes.
      static_assert(kBM * kBKBytes == 32 * 4 * 128, "one gather of four rows per lane");
      auto load_idx = [&](long long first_row) {
        int4 v;
        const int* q = p.a_rows + first_row * p.a_rows_stride;
        v.x = q[0];
        v.y = q[p.a_rows_stride];
        v.z = q[2 * p.a_rows_stride];
        v.w = q[3 * p.a_rows_stride];
        v.x = v.x < 0 ? p.a_zero_row : v.x / p.a_rows_div;
        v.y = v.y < 0 ? p.a_zero_row : v.y / p.a_rows_div;
        v.z = v.z < 0 ? p.a_zero_row : v.z / p.a_rows_div;
        v.w = v.w < 0 ? p.a_zero_row : v.w / p.a_rows_div;
        return v;
      };
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        const Tile t = decode(id);
        int4 idx = make_int4(0, 0, 0, 0);
        if (!A_MN) idx = load_idx(static_cast<long long>(t.m0) + 4 * lane);
        for (int kit = t.kb; kit < t.ke; ++kit) {
          if (A_MN) idx = load_idx(static_cast<long long>(t.krow0) + kit * BK_E + 4 * (lane & 15));
          if (!mbar_wait(&bar_empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          if (lane == 0) mbar_expect_tx(&bar_full[stage], S::kStageBytes);
          __syncwarp();
          const int kcoord = t.krow0 + kit * BK_E;
          if (!A_MN) {
            tma_gather4_2d(sa + lane * 512, &p.tmA[0], &bar_full[stage], kit * BK_E, idx.x, idx.y, idx.z, idx.w);
          } else {
            const int j = lane >> 4;  // which 64-column chunk of the tile's M extent
            tma_gather4_2d(sa + j * CH_BYTES + (lane & 15) * 512, &p.tmA[0], &bar_full[stage], t.m0 + j * CH, idx.x,
                           idx.y, idx.z, idx.w);
          }
          if (lane == 0) load_b(sb, &bar_full[stage], t, 0, kcoord);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    } else if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        const Tile t = decode(id);
        for (int s = 0; s < p.nseg && ok; ++s) {
          const int kb = (s == 0) ? t.kb : 0;
          const int ke = (s == 0) ? t.ke : p.seg_kiters[s];
          for (int kit = kb; kit < ke; ++kit) {
            if (!mbar_wait(&bar_empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * S::kStageBytes;
            uint8_t* sb = sa + S::kABytes;
            mbar_expect_tx(&bar_full[stage], S::kStageBytes);
            const int kcoord = t.krow0 + kit * BK_E;  // element (K-major) or row (MN-major) coordinate along K
            if (!A_MN) {
              tma_load_2d(sa, &p.tmA[s], &bar_full[stage], kcoord, t.m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / CH; ++j)
                tma_load_2d(sa + j * CH_BYTES, &p.tmA[s], &bar_full[stage], t.m0 + j * CH, kcoord);
            }
            load_b(sb, &bar_full[stage], t, s, kcoord);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0) {
      constexpr uint32_t fmt = (ESZ == 2) ? 1u : 0u;  // kind::f16: 1 = bf16;  kind::f8f6f4: 0 = e4m3
      constexpr uint32_t idesc = make_idesc(fmt, fmt, A_MN, B_MN, kBM, BN);
      constexpr uint32_t a_lbo = A_MN ? static_cast<uint32_t>(CH_BYTES) : 0u;
      constexpr uint32_t b_lbo = B_MN ? static_cast<uint32_t>(CH_BYTES) : 0u;
      constexpr uint32_t a_kstep = A_MN ? static_cast<uint32_t>(UK * 128) : 32u;  // bytes per tcgen05.mma along K
      constexpr uint32_t b_kstep = B_MN ? static_cast<uint32_t>(UK * 128) : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        const Tile t = decode(id);
        const int nk = tile_kiters(t);
        if (nk == 0) continue;
        if (!mbar_wait(&bar_tempty[acc], acc_phase ^ 1, abort_flag, p.status, kStatusMmaTimeout)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < nk; ++it) {
          if (!mbar_wait(&bar_full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < BK_E / UK; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            if (ESZ == 2)
              umma_f16(d_tmem, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
            else
              umma_f8(d_tmem, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bar_empty[stage]);  // stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&bar_tfull[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ============================= epilogue =============================
    const int q = warp & 3;             // TMEM lane quadrant this warp may access
    const int group = (warp - 2) >> 2;  // 0: even slabs, 1: odd slabs
    const int bar_id = 1 + group;
    const int r = q * 32 + lane;        // row of the tile owned by this thread
    const bool issuer = (((warp - 2) & 3) == 0) && lane == 0;
    uint8_t* const sbuf0 = staging + group * (S::kBufsPerGroup * S::kStreams * S::kSlabBytes);
    int buf = 0;  // which of the group's staging buffers the next slab uses
    float deq = 1.0f;
    if (ESZ == 1) deq = (p.deq_a ? p.deq_a[0] : 1.0f) * (p.deq_b ? p.deq_b[0] : 1.0f);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // EPI_SWIGLU_BWD (BN = 128): group g owns the tile's columns [64 g, 64 g + 64), i.e. slabs 2g and 2g + 1, and the
    // saved gate / up of those columns arrive as TWO 128-row boxes of 64 columns (128-byte rows, 128-byte swizzle: a
    // TMA load costs the SM one request slot per box row whatever the row's width, so 64-column boxes halve what the
    // 32-column slabs cost).  One 32 KB buffer per group: every thread takes its two rows (gate, up: 128 bytes each)
    // into registers at the start of the tile, which frees the buffer for the group's NEXT tile a whole tile's
    // epilogue ahead of its use.
    constexpr bool kAdj = (EPI == EPI_SWIGLU_BWD);
    const int n_per_tile_e = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
    auto slabs_of = [&](const Tile& tt) {
      const int n0_ = tt.nt * n_per_tile_e;
      int sl = (p.N - n0_ + kSlabCols - 1) / kSlabCols;
      return sl > n_per_tile_e / kSlabCols ? n_per_tile_e / kSlabCols : sl;
    };
    int aux_seq = 0;             // tiles whose rows this group has taken from its buffer
    int pre_id = blockIdx.x;     // next tile to stage (issuer only)
    auto stage_next = [&]() {    // issues the loads of the group's next tile that has columns for it, if there is one
      while (pre_id < total_tiles) {
        const Tile tt = decode(pre_id);
        pre_id += gridDim.x;
        if (2 * group < slabs_of(tt)) {
          uint8_t* dst = aux_stage + group * 32768;
          const int col = tt.nt * BN + group * 64;
          mbar_expect_tx(&bar_aux[group], 32768);
          tma_load_2d(dst, &p.tmAux, &bar_aux[group], col, tt.m0);                 // gate; rows / columns beyond the
          tma_load_2d(dst + 16384, &p.tmAux, &bar_aux[group], p.N + col, tt.m0);   // up      tensor arrive as zeros
          return;
        }
      }
    };
    if (kAdj && issuer) stage_next();
    for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
      const Tile t = decode(id);
      const int nk = tile_kiters(t);
      if (nk > 0) {
        if (!mbar_wait(&bar_tfull[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
        tc_fence_after();
      }
      // All threads of the group must agree before entering the (unbounded) named barriers below:
      // a barrier-wide AND, which every thread reaches on every tile whatever its wait returned.
      ok = epi_bar_all(bar_id, ok);
      if (!ok) break;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int n_per_tile = kSwiglu ? BN / 2 : BN;
      const int n0 = t.nt * n_per_tile;
      const int n_lim = kSwiglu ? p.half : p.N;
      int slabs = (n_lim - n0 + kSlabCols - 1) / kSlabCols;
      if (slabs > n_per_tile / kSlabCols) slabs = n_per_tile / kSlabCols;
      // this group's slabs: group, group + 2, ... (adjoint epilogue: 2 group, 2 group + 1); the accumulator is released
      // after the last one is loaded
      const int c_begin = kAdj ? 2 * group : group;
      const int c_step = kAdj ? 1 : 2;
      const int c_end = kAdj ? min(slabs, 2 * group + 2) : slabs;
      const int last = (c_end > c_begin) ? c_begin + ((c_end - 1 - c_begin) / c_step) * c_step : -1;
      if (nk > 0 && last < 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_tempty[acc]);
      }

      uint4 hg8[kAdj ? 8 : 1], hu8[kAdj ? 8 : 1];  // adjoint epilogue: saved gate / up of this row, 64 columns each
      if (kAdj && c_end > c_begin) {
        if (!mbar_wait(&bar_aux[group], aux_seq & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
        const uint8_t* src = aux_stage + group * 32768 + r * 128;
        const int sw = r & 7;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          hg8[j] = *reinterpret_cast<const uint4*>(src + ((j ^ sw) << 4));
          hu8[j] = *reinterpret_cast<const uint4*>(src + 16384 + ((j ^ sw) << 4));
        }
        ++aux_seq;
        ok = epi_bar_all(bar_id, ok);  // every thread of the group holds its rows: the buffer is free
        if (!ok) break;
        if (issuer) stage_next();
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += c_step) {
        float v[32], u[32];
        uint4 hg[4], hu[4];  // adjoint epilogue: the 32 columns of this slab
        if (kAdj) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            hg[j] = (c == c_begin) ? hg8[j] : hg8[(kAdj ? 4 : 0) + j];   // (index 0 when the arrays are dummies)
            hu[j] = (c == c_begin) ? hu8[j] : hu8[(kAdj ? 4 : 0) + j];
          }
        }
        if (nk > 0) {
          tmem_ld32(taddr + c * 32, v);
          if (kSwiglu) tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (c == last) {
            // last slab of this warp is in registers: hand the accumulator back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tempty[acc]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = u[j] = 0.f;
        }
        if (ESZ == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] *= deq;
            if (kSwiglu) u[j] *= deq;
          }
        }
        uint32_t pk[16], pu[16], ph[16];
        if (EPI == EPI_BF16) {
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
        } else if (EPI == EPI_SWIGLU_BWD) {
          const uint32_t* wg = reinterpret_cast<const uint32_t*>(hg);
          const uint32_t* wu = reinterpret_cast<const uint32_t*>(hu);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // d_hidden is rounded to bf16 first (what a stored d_hidden would hold), then
            //   d_up = dh * g * sig(g),  d_gate = dh * u * sig(g) * (1 + g * (1 - sig(g)))
            const uint32_t dh2 = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            float dh[2] = {__uint_as_float(dh2 << 16), __uint_as_float(dh2 & 0xffff0000u)};
            float g[2] = {__uint_as_float(wg[j] << 16), __uint_as_float(wg[j] & 0xffff0000u)};
            float uu[2] = {__uint_as_float(wu[j] << 16), __uint_as_float(wu[j] & 0xffff0000u)};
            float dg[2], du[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const float sg = sigmoid_fast(g[k]);
              du[k] = dh[k] * g[k] * sg;
              dg[k] = dh[k] * uu[k] * sg * (1.0f + g[k] * (1.0f - sg));
            }
            pk[j] = pack_bf16x2(dg[0], dg[1]);
            pu[j] = pack_bf16x2(du[0], du[1]);
          }
        } else if (EPI == EPI_SWIGLU) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // gate/up are saved as bf16; hidden is formed from the rounded values (one packed convert
            // per pair, unpacked again with shifts)
            pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            pu[j] = pack_bf16x2(u[2 * j], u[2 * j + 1]);
            const float g0 = __uint_as_float(pk[j] << 16), g1 = __uint_as_float(pk[j] & 0xffff0000u);
            const float u0 = __uint_as_float(pu[j] << 16), u1 = __uint_as_float(pu[j] & 0xffff0000u);
            ph[j] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
          }
        }
        // the staging buffer about to be written was last read by the store issued kBufsPerGroup slabs ago
        uint8_t* sbuf = sbuf0 + buf * (S::kStreams * S::kSlabBytes);
        if (issuer) {
          if (S::kBufsPerGroup == 2)
            tma_store_wait_read_1();
          else
            tma_store_wait_read_all();
        }
        epi_bar_sync(bar_id);
        if (EPI == EPI_F32) {
          stage_row_f32(sbuf, r, v);
        } else if (EPI == EPI_BF16) {
          stage_row_bf16(sbuf, r, pk);
        } else if (EPI == EPI_SWIGLU_BWD) {
          stage_row_bf16(sbuf, r, pk);
          stage_row_bf16(sbuf + S::kSlabBytes, r, pu);
        } else {
          stage_row_bf16(sbuf, r, pk);
          stage_row_bf16(sbuf + S::kSlabBytes, r, pu);
          if (!S::kHiddenReusesGate) stage_row_bf16(sbuf + 2 * S::kSlabBytes, r, ph);
        }
        fence_proxy_async_smem();
        epi_bar_sync(bar_id);
        if (kSwiglu && S::kHiddenReusesGate) {
          const int col = n0 + c * kSlabCols;
          if (issuer) {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, 0);
            tma_store_commit();
            tma_store_3d(&p.tmC, sbuf + S::kSlabBytes, p.half + col, t.m0, 0);
            tma_store_commit();
            tma_store_wait_read_1();   // the gate store (all but the latest group) has read its slab
          }
          epi_bar_sync(bar_id);
          stage_row_bf16(sbuf, r, ph);
          fence_proxy_async_smem();
          epi_bar_sync(bar_id);
          if (issuer) {
            tma_store_3d(&p.tmC2, sbuf, col, t.m0, 0);
            tma_store_commit();
          }
        } else if (issuer) {
          const int col = n0 + c * kSlabCols;
          if (kSwiglu) {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, 0);
            tma_store_3d(&p.tmC, sbuf + S::kSlabBytes, p.half + col, t.m0, 0);
            tma_store_3d(&p.tmC2, sbuf + 2 * S::kSlabBytes, col, t.m0, 0);
          } else if (EPI == EPI_SWIGLU_BWD) {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, 0);                        // d_gate
            tma_store_3d(&p.tmC, sbuf + S::kSlabBytes, p.N + col, t.m0, 0);  // d_up
          } else {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, t.plane);
          }
          tma_store_commit();
        }
        if (S::kBufsPerGroup == 2) buf ^= 1;
      }
      if (nk > 0) {
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    if (issuer) tma_store_wait0();  // staging memory must outlive the last reads
  }

  // ---- teardown: every role falls through to here, also after an abort ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace lmoe
