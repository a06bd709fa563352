// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T      bf16 (or e4m3) operands, fp32 accumulation in tensor memory
//
// One CTA per SM walks a static tile schedule.  Roles:
//   warp 0      TMA producer: fills a ring of shared-memory stages (A tile 128 x 64, B tile BN x 64)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) and commits to mbarriers;
//               also owns the tensor-memory allocation (two accumulators of BN columns)
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp owns 32 lanes = 32 rows),
//               apply the epilogue and store; overlaps the next tile's main loop
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
#pragma once
#include "common/ptx.cuh"

namespace lmoe {

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ATOMIC = 2, EPI_SWIGLU = 3, EPI_SWIGLU_BWD = 4 };
enum : int { GRP_NONE = 0, GRP_M = 1, GRP_K = 2 };

constexpr int kBM = 128;
constexpr int kBK = 64;  // 16-bit elements per k-block (one 128-byte swizzle row)
constexpr int kGemmThreads = 192;

// status codes written by a wait that gave up
constexpr int kStatusProducerTimeout = 101;
constexpr int kStatusMmaTimeout = 102;
constexpr int kStatusEpilogueTimeout = 103;

struct alignas(64) GemmParams {
  CUtensorMap tmA[3];
  CUtensorMap tmB[3];
  int seg_kiters[3];
  int nseg;
  int M, N;              // output extent (per group for GRP_K)
  int m_tiles, n_tiles;  // tile counts (per group for GRP_K; upper bound for GRP_M)
  int groups;            // GRP_K: number of experts
  int split_k;           // GRP_NONE: k-blocks are divided among split_k tiles which ADD into C
  void* C;
  long long ldc;
  long long c_group_stride;  // GRP_K: elements between consecutive experts' outputs
  void* C2;                  // EPI_SWIGLU: hidden output;  EPI_SWIGLU_BWD: h1 input
  long long ldc2;
  int half;                  // EPI_SWIGLU*: width of the gate half (F or Fs)
  const int* tile_expert;    // GRP_M
  const int* n_m_tiles;      // GRP_M: device scalar, number of 128-row tiles in use
  int b_group_rows;          // GRP_M: rows of the stacked B tensor per expert
  const int* pad_offsets;    // GRP_K
  int* status;
};

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024: manual alignment
};

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <bool A_MN, bool B_MN, int BN, int EPI, int GRP>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::kStages;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  static_assert(BN == 128 || BN == 256, "BN");
  constexpr bool kSwiglu = (EPI == EPI_SWIGLU);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_tfull = bar_empty + STAGES;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
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
      mbar_init(&bar_tempty[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    for (int i = 0; i < p.nseg; ++i) {
      tma_prefetch_desc(&p.tmA[i]);
      tma_prefetch_desc(&p.tmB[i]);
    }
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
    int m0, nt, grp, kb, ke, krow0;
  };
  auto decode = [&](int id) {
    Tile t;
    const int outer = id / tiles_mn;
    const int rem = id - outer * tiles_mn;
    t.m0 = (rem / p.n_tiles) * kBM;
    t.nt = rem % p.n_tiles;
    t.grp = 0;
    t.kb = 0;
    t.ke = p.seg_kiters[0];
    t.krow0 = 0;
    if (GRP == GRP_NONE) {
      if (p.split_k > 1) {
        const int per = (p.seg_kiters[0] + p.split_k - 1) / p.split_k;
        t.kb = min(outer * per, p.seg_kiters[0]);
        t.ke = min(t.kb + per, p.seg_kiters[0]);
      }
    } else if (GRP == GRP_M) {
      t.grp = p.tile_expert[t.m0 / kBM];
    } else {
      t.grp = outer;
      const int r0 = p.pad_offsets[outer], r1 = p.pad_offsets[outer + 1];
      t.krow0 = r0;
      t.ke = (r1 - r0) / kBK;
    }
    return t;
  };
  auto tile_kiters = [&](const Tile& t) {
    int n = t.ke - t.kb;
    for (int s = 1; s < p.nseg; ++s) n += p.seg_kiters[s];
    return n;
  };

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
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
            const int kcoord = t.krow0 + kit * kBK;  // element (K-major) or row (MN-major) coordinate along K
            // ---- A ----
            if (!A_MN) {
              tma_load_2d(sa, &p.tmA[s], &bar_full[stage], kcoord, t.m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                tma_load_2d(sa + j * 8192, &p.tmA[s], &bar_full[stage], t.m0 + j * 64, kcoord);
            }
            // ---- B ----
            const int grp_rows = (GRP == GRP_M) ? t.grp * p.b_group_rows : 0;
            if (!B_MN) {
              if (kSwiglu) {
                const int nh = t.nt * (BN / 2);
                tma_load_2d(sb, &p.tmB[s], &bar_full[stage], kcoord, grp_rows + nh);
                tma_load_2d(sb + (BN / 2) * 128, &p.tmB[s], &bar_full[stage], kcoord, grp_rows + p.half + nh);
              } else {
                tma_load_2d(sb, &p.tmB[s], &bar_full[stage], kcoord, grp_rows + t.nt * BN);
              }
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) {
                int ncol;
                if (kSwiglu) {
                  const int nh = t.nt * (BN / 2);
                  ncol = (j < BN / 128) ? (nh + j * 64) : (p.half + nh + (j - BN / 128) * 64);
                } else {
                  ncol = t.nt * BN + j * 64;
                }
                tma_load_2d(sb + j * 8192, &p.tmB[s], &bar_full[stage], ncol, grp_rows + kcoord);
              }
            }
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
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, kBM, BN);
      constexpr uint32_t a_lbo = A_MN ? 8192u : 0u;
      constexpr uint32_t b_lbo = B_MN ? 8192u : 0u;
      constexpr uint32_t a_kstep = A_MN ? 2048u : 32u;  // bytes per 16-element k-step
      constexpr uint32_t b_kstep = B_MN ? 2048u : 32u;
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
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_f16(d_tmem, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
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
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int id = blockIdx.x; id < total_tiles; id += gridDim.x) {
      const Tile t = decode(id);
      const int nk = tile_kiters(t);
      if (nk == 0 && EPI == EPI_F32_ATOMIC) continue;  // nothing to add
      if (nk > 0) {
        if (!mbar_wait(&bar_tfull[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout)) break;
        tc_fence_after();
      }
      const long long grow = t.m0 + row_in_tile;
      const bool row_ok = (GRP == GRP_M) ? true : (grow < p.M);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;

      if (EPI == EPI_SWIGLU) {
        // accumulator columns [0,BN/2) = gate, [BN/2,BN) = up, for output columns nh..nh+BN/2
        const int nh = t.nt * (BN / 2);
        __nv_bfloat16* h1 = reinterpret_cast<__nv_bfloat16*>(p.C) + grow * p.ldc;
        __nv_bfloat16* hid = reinterpret_cast<__nv_bfloat16*>(p.C2) + grow * p.ldc2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          float g[32], u[32];
          if (nk > 0) {
            tmem_ld32(taddr + c * 32, g);
            tmem_ld32(taddr + BN / 2 + c * 32, u);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = u[j] = 0.f;
          }
          const int col = nh + c * 32;
          if (row_ok && col < p.half) {
            uint32_t pg[16], pu[16], ph[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // the saved gate/up are bf16; hidden is formed from the rounded values
              const float g0 = bf16_round(g[2 * j]), g1 = bf16_round(g[2 * j + 1]);
              const float u0 = bf16_round(u[2 * j]), u1 = bf16_round(u[2 * j + 1]);
              pg[j] = pack_bf16x2(g0, g1);
              pu[j] = pack_bf16x2(u0, u1);
              ph[j] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
            }
            uint4* dg = reinterpret_cast<uint4*>(h1 + col);
            uint4* du = reinterpret_cast<uint4*>(h1 + p.half + col);
            uint4* dh = reinterpret_cast<uint4*>(hid + col);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col + j * 8 < p.half) {
                dg[j] = make_uint4(pg[4 * j], pg[4 * j + 1], pg[4 * j + 2], pg[4 * j + 3]);
                du[j] = make_uint4(pu[4 * j], pu[4 * j + 1], pu[4 * j + 2], pu[4 * j + 3]);
                dh[j] = make_uint4(ph[4 * j], ph[4 * j + 1], ph[4 * j + 2], ph[4 * j + 3]);
              }
            }
          }
        }
      } else {
        const int n0 = t.nt * BN;
        const long long cbase = (GRP == GRP_K ? static_cast<long long>(t.grp) * p.c_group_stride : 0) + grow * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          if (nk > 0) {
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          const int col = n0 + c * 32;
          if (row_ok && col < p.N) {
            if (EPI == EPI_BF16) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + cbase + col;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col + j * 8 < p.N) {
                  reinterpret_cast<uint4*>(dst)[j] =
                      make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                                 pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
                }
              }
            } else if (EPI == EPI_F32) {
              float* dst = reinterpret_cast<float*>(p.C) + cbase + col;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (col + j * 4 < p.N)
                  reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            } else if (EPI == EPI_F32_ATOMIC) {
              float* dst = reinterpret_cast<float*>(p.C) + cbase + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < p.N) atomicAdd(dst + j, v[j]);
              }
            }
          }
        }
      }
      if (nk > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_tempty[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
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
