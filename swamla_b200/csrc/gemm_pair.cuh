// Dense bf16 GEMM on CTA PAIRS (tcgen05 cta_group::2): two CTAs of a cluster share one 256 x 256 output tile.
//
// Why: with one CTA per 128 x 256 tile every k-block needs 16 KB of A and 32 KB of B per SM; the tensor pipe then
// outruns what one SM can pull in.  A pair splits B: each CTA loads its own 128 rows of A and HALF of the B tile
// (16 KB + 16 KB per k-block), the MMA with M = 256 reads both halves, and each CTA ends up with the accumulators of
// its own 128 rows in its own tensor memory.  A third less fill traffic per FLOP and a six-deep ring instead of four.
//
// Roles per CTA as in gemm.cuh (warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warps 2-9 two epilogue
// groups); differences:
//   * rank 0's "full" barrier of a stage collects the bytes of BOTH CTAs' loads (the loads name rank 0's barrier through
//     its shared::cluster address; no multicast anywhere);
//   * only rank 0 issues MMAs; its tcgen05.commit arrives at the "empty" / "accumulator full" barriers of both CTAs;
//   * the epilogue warps of both CTAs release an accumulator on rank 0's "accumulator empty" barrier (16 arrivals);
//   * the CTAs meet at a cluster barrier after set-up and before tear-down.
// Dense GEMMs only (no expert grouping), bf16 operands, BN = 256, epilogues bf16 / fp32 (split-K planes) / SwiGLU.
// Every wait is bounded as in gemm.cuh; a CTA whose wait expires stops issuing work, its partner's waits expire in turn.
#pragma once
#include "gemm.cuh"

namespace lmoe {

template <int EPI>
struct PairSmem {
  static constexpr int kABytes = kBM * kBKBytes;       // 128 rows of A
  static constexpr int kBBytes = 128 * kBKBytes;       // this CTA's half of the 256-wide B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSlabBytes = (EPI == EPI_F32) ? 16384 : 8192;
  static constexpr int kStreams = (EPI == EPI_SWIGLU) ? 3 : 1;
  static constexpr int kBufsPerGroup = (EPI == EPI_BF16) ? 2 : 1;
  static constexpr int kStagingBytes = 2 * kBufsPerGroup * kStreams * kSlabBytes;
  static constexpr int kBarrierBytes = 1536;  // barriers + the per-expert table of the grouped form (<= 257 ints)
  static constexpr int kBudget = 232448 - 1024 - kBarrierBytes - kStagingBytes;
  static constexpr int kStagesMax = kBudget / kStageBytes;
  static constexpr int kStages = kStagesMax > 6 ? 6 : kStagesMax;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
  static_assert(kStages >= 4, "pipeline too shallow");
};

// GRP == GRP_M (grouped over rows, K-major A): the rows are the padded routed layout; the two CTAs of a pair take two
// consecutive 128-row tiles of the SAME expert (tiles 2j, 2j+1 of its run, from pad_offsets) and share that expert's
// slice of the stacked B tensor.  An expert with an odd number of tiles ends with a pair whose second CTA recomputes
// the first tile and stores nothing.
template <bool A_MN, bool B_MN, int EPI, int GRP = GRP_NONE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  static_assert(GRP == GRP_NONE || (GRP == GRP_M && !A_MN), "grouped form: rows of a K-major A");
  using S = PairSmem<EPI>;
  constexpr int BN = 256;
  constexpr int STAGES = S::kStages;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr bool kSwiglu = (EPI == EPI_SWIGLU);
  constexpr int BK_E = kBKBytes / 2;   // 64 bf16 per k-block
  constexpr int CH = 64;               // MN-major chunk width (elements)
  constexpr int CH_BYTES = BK_E * 128;
  constexpr int UK = 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * S::kStageBytes;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(staging + S::kStagingBytes);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_tfull = bar_empty + STAGES;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* etab = reinterpret_cast<int*>(tmem_slot + 2);  // GRP_M: first tile of expert e | experts before e with an odd tile count << 23

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: issues the MMAs and owns the pair's "full" / "accumulator empty" barriers
  if (GRP == GRP_M) {
    const int E = p.groups;
    const int cap_rows = p.m_tiles * kBM;   // m_tiles: capacity of the padded layout in 128-row tiles
    if (static_cast<int>(threadIdx.x) <= E) etab[threadIdx.x] = min(p.pad_offsets[threadIdx.x], cap_rows) / kBM;
    __syncthreads();
    if (warp == 0) {  // lane l scans experts 8l .. 8l+7, a shuffle scan joins the lanes
      int odd[8], sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;
        odd[i] = (e < E) ? ((etab[e + 1] - etab[e]) & 1) : 0;
        sum += odd[i];
      }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      __syncwarp();
      int run = incl - sum;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;
        if (e < E) etab[e] |= run << 23;
        run += odd[i];
        if (e + 1 == E) etab[E] |= run << 23;
      }
    }
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&bar_full[i], 1);    // rank 0's: one arrive.expect_tx by its producer, bytes of both CTAs
      mbar_init(&bar_empty[i], 1);   // one tcgen05.commit arrival per CTA
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_tfull[i], 1);
      mbar_init(&bar_tempty[i], 16);  // rank 0's: 8 epilogue warps of each CTA
    }
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
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival or load completion
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- tile schedule over pairs (identical arithmetic in every role of both CTAs) ----
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  auto first_tile = [&](int e) { return etab[e] & 0x7fffff; };
  auto pairs_before = [&](int e) { return ((etab[e] & 0x7fffff) - (etab[0] & 0x7fffff) + (etab[e] >> 23)) >> 1; };
  // m_tiles counts 256-row tiles (dense) or is the layout's capacity in 128-row tiles (grouped: pairs come from etab)
  const int tiles_mn = (GRP == GRP_M ? pairs_before(p.groups) : p.m_tiles) * p.n_tiles;
  const int total_tiles = tiles_mn * p.split_k;

  struct Tile {
    int m0, nt, plane, kb, ke;
    int grp;   // GRP_M: expert of the pair
    int live;  // GRP_M: 0 for the tile-less second CTA of an odd run (loads the first tile, stores nothing)
  };
  auto decode = [&](int id) {
    Tile t;
    t.grp = 0;
    t.live = 1;
    if (GRP == GRP_M) {
      const int pid = id / p.n_tiles;
      t.nt = id - pid * p.n_tiles;
      int lo = 0, hi = p.groups - 1;  // largest e with pairs_before(e) <= pid
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (pairs_before(mid) <= pid) lo = mid;
        else hi = mid - 1;
      }
      const int first = first_tile(lo) + 2 * (pid - pairs_before(lo));
      const int own = first + static_cast<int>(rank);
      t.grp = lo;
      t.live = own < first_tile(lo + 1) ? 1 : 0;
      t.m0 = (t.live ? own : first) * kBM;
      t.plane = 0;
      t.kb = 0;
      t.ke = p.seg_kiters[0];
      return t;
    }
    const int outer = id / tiles_mn;
    const int rem = id - outer * tiles_mn;
    t.m0 = (rem / p.n_tiles) * 256 + static_cast<int>(rank) * kBM;  // this CTA's 128 rows
    t.nt = rem % p.n_tiles;
    t.plane = 0;
    t.kb = 0;
    t.ke = p.seg_kiters[0];
    if (p.split_k > 1) {
      const int per = (p.seg_kiters[0] + p.split_k - 1) / p.split_k;
      t.kb = min(outer * per, p.seg_kiters[0]);
      t.ke = min(t.kb + per, p.seg_kiters[0]);
      t.plane = outer;
    }
    return t;
  };
  auto tile_kiters = [&](const Tile& t) {
    int n = t.ke - t.kb;
    for (int s = 1; s < p.nseg; ++s) n += p.seg_kiters[s];
    return n;
  };

  if (warp == 0) {
    // =========================== TMA producer (both CTAs) ===========================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int id = pair_id; id < total_tiles && ok; id += n_pairs) {
        const Tile t = decode(id);
        // first row / column of this CTA's half of B
        int b0;
        if (kSwiglu)
          b0 = (rank == 0 ? 0 : p.half) + t.nt * (BN / 2);  // rank 0: gate rows, rank 1: up rows
        else
          b0 = t.nt * BN + static_cast<int>(rank) * 128;
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
            if (rank == 0) mbar_expect_tx(&bar_full[stage], 2 * S::kStageBytes);
            const uint32_t full0 = mapa_shared(smem_u32(&bar_full[stage]), 0);
            const int kcoord = kit * BK_E;
            if (!A_MN) {
              tma_load_2d_pair(sa, &p.tmA[s], full0, kcoord, t.m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / CH; ++j) tma_load_2d_pair(sa + j * CH_BYTES, &p.tmA[s], full0, t.m0 + j * CH, kcoord);
            }
            const int grp_rows = (GRP == GRP_M) ? t.grp * p.b_group_rows : 0;  // this expert's slice of the stacked B
            if (!B_MN) {
              tma_load_2d_pair(sb, &p.tmB[s], full0, kcoord, grp_rows + b0);
            } else {
#pragma unroll
              for (int j = 0; j < 128 / CH; ++j)
                tma_load_2d_pair(sb + j * CH_BYTES, &p.tmB[s], full0, b0 + j * CH, grp_rows + kcoord);
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
    // ============================ MMA issuer (rank 0 only) ============================
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(1u, 1u, A_MN, B_MN, 256, BN);
      constexpr uint32_t a_lbo = A_MN ? static_cast<uint32_t>(CH_BYTES) : 0u;
      constexpr uint32_t b_lbo = B_MN ? static_cast<uint32_t>(CH_BYTES) : 0u;
      constexpr uint32_t a_kstep = A_MN ? static_cast<uint32_t>(UK * 128) : 32u;
      constexpr uint32_t b_kstep = B_MN ? static_cast<uint32_t>(UK * 128) : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int id = pair_id; id < total_tiles && ok; id += n_pairs) {
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
            umma_f16_pair(d_tmem, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&bar_empty[stage], 0x3);  // both CTAs may refill the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&bar_tfull[acc], 0x3);  // accumulators complete in both CTAs
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ============================= epilogue (both CTAs, own 128 rows) =============================
    const int q = warp & 3;
    const int group = (warp - 2) >> 2;
    const int bar_id = 1 + group;
    const int r = q * 32 + lane;
    const bool issuer = (((warp - 2) & 3) == 0) && lane == 0;
    uint8_t* const sbuf0 = staging + group * (S::kBufsPerGroup * S::kStreams * S::kSlabBytes);
    int buf = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int id = pair_id; id < total_tiles && ok; id += n_pairs) {
      const Tile t = decode(id);
      const int nk = tile_kiters(t);
      if (nk > 0) {
        if (!mbar_wait(&bar_tfull[acc], acc_phase, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
        tc_fence_after();
      }
      ok = epi_bar_all(bar_id, ok);
      if (!ok) break;
      const uint32_t tempty0 = mapa_shared(smem_u32(&bar_tempty[acc]), 0);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int n_per_tile = kSwiglu ? BN / 2 : BN;
      const int n0 = t.nt * n_per_tile;
      const int n_lim = kSwiglu ? p.half : p.N;
      int slabs = (n_lim - n0 + kSlabCols - 1) / kSlabCols;
      if (slabs > n_per_tile / kSlabCols) slabs = n_per_tile / kSlabCols;
      const int last = ((slabs - 1 - group) >= 0) ? group + ((slabs - 1 - group) & ~1) : -1;
      if (nk > 0 && last < 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty0);
      }

#pragma unroll 1
      for (int c = group; c < slabs; c += 2) {
        float v[32], u[32];
        if (nk > 0) {
          tmem_ld32(taddr + c * 32, v);
          if (kSwiglu) tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (c == last) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = u[j] = 0.f;
        }
        uint32_t pk[16], pu[16], ph[16];
        if (EPI == EPI_BF16) {
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
        } else if (EPI == EPI_SWIGLU) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            pu[j] = pack_bf16x2(u[2 * j], u[2 * j + 1]);
            const float g0 = __uint_as_float(pk[j] << 16), g1 = __uint_as_float(pk[j] & 0xffff0000u);
            const float u0 = __uint_as_float(pu[j] << 16), u1 = __uint_as_float(pu[j] & 0xffff0000u);
            ph[j] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
          }
        }
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
        } else {
          stage_row_bf16(sbuf, r, pk);
          stage_row_bf16(sbuf + S::kSlabBytes, r, pu);
          stage_row_bf16(sbuf + 2 * S::kSlabBytes, r, ph);
        }
        fence_proxy_async_smem();
        epi_bar_sync(bar_id);
        if (issuer && t.live && (GRP == GRP_M || t.m0 < p.M)) {  // dense: the second half of a ragged last tile may lie outside
          const int col = n0 + c * kSlabCols;
          if (kSwiglu) {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, 0);
            tma_store_3d(&p.tmC, sbuf + S::kSlabBytes, p.half + col, t.m0, 0);
            tma_store_3d(&p.tmC2, sbuf + 2 * S::kSlabBytes, col, t.m0, 0);
          } else {
            tma_store_3d(&p.tmC, sbuf, col, t.m0, t.plane);
          }
        }
        if (issuer) tma_store_commit();
        if (S::kBufsPerGroup == 2) buf ^= 1;
      }
      if (nk > 0) {
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    if (issuer) tma_store_wait0();
  }

  // ---- teardown: every role of both CTAs falls through to here, also after an abort ----
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while its partner may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace lmoe
