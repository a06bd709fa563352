// The routed expert chain (chain.cuh) on CTA PAIRS (tcgen05 cta_group::2): two CTAs of a cluster work on two 128-row
// tiles of the SAME expert and share every weight slice.
//
// Why: the chain is bound by what an SM can pull out of L2 (about 65 GB/s per SM with all SMs loading), and per
// 128-row tile that is mostly the expert's weights (384 KB of weights against 64 KB of activations at L = F = 256).
// In a pair each CTA loads HALF of every weight slice (its half of the N extent), the MMA with M = 256 reads both
// halves, and each CTA keeps the accumulators of its own 128 rows in its own tensor memory: half the weight traffic
// per tile.
//
// Pairs are formed inside an expert's run of tiles (tiles 2j and 2j+1 of expert e); an expert with an odd number of
// tiles ends with a pair whose second CTA recomputes the first tile and stores nothing.  pad_offsets[E+1] (rows, multiples
// of 128, fewer than 2^23 tiles) gives the runs; the pair index -> (expert, tile) map comes from a small per-expert table
// in shared memory.
//
// Roles per CTA (384 threads): warp 0 producer of the A operand and the first GEMM's weights, warp 10 producer of the
// second GEMM's weights, warp 1 / warp 11 MMA issuers of the first / second GEMM (separate threads and separate rings, so
// the first GEMM runs ahead by its two accumulators and never queues behind the second GEMM's wait for the epilogue),
// warps 2-9 epilogue as in chain.cuh.  As in gemm_pair.cuh:
//   * rank 0's "full" barriers collect the bytes of BOTH CTAs' loads (the loads name rank 0's barrier through its
//     shared::cluster address; no multicast load anywhere);
//   * only rank 0 issues MMAs; its tcgen05.commit arrives at the barriers of both CTAs (ring / A / A2 "empty",
//     accumulator "full");
//   * the epilogue warps of both CTAs release accumulators on rank 0's barriers (16 arrivals), and both CTAs' chunk
//     issuers report their A2 buffer on rank 0's barrier (2 arrivals);
//   * cluster barriers after set-up and before tear-down.
// L must be a multiple of 128 (each CTA's half of the second GEMM's N extent is whole 64-wide chunks).
#pragma once
#include "chain.cuh"

namespace lmoe {

struct alignas(64) ChainPairParams {
  CUtensorMap tmA;    // [P, L] box {64, 128}
  CUtensorMap tmB1;   // FWD: Wgu [E*L, 2F] box {64, 64};   BWD: Wd [E*F, L] box {64 k, 32 rows}
  CUtensorMap tmB2;   // FWD: Wd [E*F, L] box {64, 64};     BWD: Wgu [E*L, 2F] box {64 k, L/2 rows}
  CUtensorMap tmAux;  // h1 [P, 2F] box {32, 128} (64-byte swizzle): FWD store, BWD load
  CUtensorMap tmMid;  // box {64, 128} (128-byte swizzle): FWD hidden [P, F]; BWD d_h1 [P, 2F]
  CUtensorMap tmOut;  // [P, L] box {32, 128} (64-byte swizzle)
  int L, F, E;
  int max_tiles;
  int prefetch_a;
  const int* pad_offsets;   // [E + 1] first padded row of every expert (multiples of 128)
  int* status;
};

constexpr int kChainPairThreads = 384;  // 12 warps: two producers, two MMA issuers, eight epilogue warps

// Shared memory of one CTA of a pair.  Two weight rings, one per GEMM, each fed by its own producer thread and drained
// by its own MMA-issuing thread: the first GEMM runs ahead of the epilogue warps by as many chunks as its two
// accumulators allow and never waits behind the second GEMM's dependence on them.
template <int MODE>
struct ChainPairSmem {
  static constexpr bool kFwd = (MODE == CHAIN_FWD);
  // FWD: two hidden chunks (one per epilogue group); BWD: d_gate + d_up chunk (also the staging slabs of the tile
  // epilogue, which runs when both are free)
  static constexpr int kA2Bytes = 32768;
  // FWD: per epilogue group a gate slab and an up slab on their way to h1 (the tile epilogue's slab reuses the first);
  // BWD: saved gate/up, two chunks
  static constexpr int kAuxBytes = kFwd ? 32768 : 65536;
  static constexpr int kOutBytes = 0;
  static constexpr int kR1Stages = kFwd ? 4 : 2, kR1Bytes = 16384;         // first GEMM: two chunks ahead
  static constexpr int kR2Stages = kFwd ? 2 : 4, kR2Bytes = kFwd ? 16384 : 8192;  // second GEMM: two chunks | one chunk
  static constexpr int kBarrierBytes = 2048;
  static constexpr int kFixed = kChainA1Bytes + kA2Bytes + kAuxBytes + kOutBytes;
  static constexpr int kTotal = 1024 + kFixed + kR1Stages * kR1Bytes + kR2Stages * kR2Bytes + kBarrierBytes;
  static_assert(kTotal <= 232448, "shared memory");
};

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kChainPairThreads, 1)
chain_pair_kernel(const __grid_constant__ ChainPairParams p) {
  using S = ChainPairSmem<MODE>;
  constexpr int R1 = S::kR1Stages, R2 = S::kR2Stages;
  constexpr bool FWD = (MODE == CHAIN_FWD);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ACC2_COL = 256;

  CHAIN_TRACE_DECL
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* const a1 = smem;
  uint8_t* const a2 = a1 + kChainA1Bytes;
  uint8_t* const aux = a2 + S::kA2Bytes;
  uint8_t* const outb = a2;  // backward: tile-epilogue slabs
  uint8_t* const ring1 = aux + S::kAuxBytes + S::kOutBytes;
  uint8_t* const ring2 = ring1 + R1 * S::kR1Bytes;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(ring2 + R2 * S::kR2Bytes);
  uint64_t* const r1_full = bars;                        // rank 0's: bytes of both CTAs
  uint64_t* const r1_empty = r1_full + R1;               // local: one commit arrival
  uint64_t* const r2_full = r1_empty + R1;               // rank 0's
  uint64_t* const r2_empty = r2_full + R2;               // local
  uint64_t* const a1_full = r2_empty + R2;               // [4] rank 0's
  uint64_t* const a1_empty = a1_full + 4;                // [4] local
  uint64_t* const acc1_full = a1_empty + 4;              // [2] local
  uint64_t* const acc1_empty = acc1_full + 2;            // [2] rank 0's: 16 arrivals
  uint64_t* const a2_full = acc1_empty + 2;              // [2] rank 0's: 2 arrivals (forward: one per epilogue group)
  uint64_t* const a2_empty = a2_full + 2;                // [2] local
  uint64_t* const acc2_full = a2_empty + 2;              // [1] local
  uint64_t* const acc2_empty = acc2_full + 1;            // [1] rank 0's: 16 arrivals
  uint64_t* const gu_full = acc2_empty + 1;              // [2] local (BWD)
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(gu_full + 2);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* const etab = reinterpret_cast<int*>(tmem_slot + 2);  // [E + 1] per-expert table (<= 257 ints), see below

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();

  if (threadIdx.x == 0) {
    for (int i = 0; i < R1; ++i) {
      mbar_init(&r1_full[i], 1);
      mbar_init(&r1_empty[i], 1);
    }
    for (int i = 0; i < R2; ++i) {
      mbar_init(&r2_full[i], 1);
      mbar_init(&r2_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&a1_full[i], 1);
      mbar_init(&a1_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc1_full[i], 1);
      mbar_init(&acc1_empty[i], FWD ? 8 : 16);  // forward: one epilogue group (four warps) per CTA reads a buffer
      mbar_init(&gu_full[i], 1);
      mbar_init(&a2_full[i], 2);
      mbar_init(&a2_empty[i], 1);
    }
    mbar_init(acc2_full, 1);
    mbar_init(acc2_empty, 16);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB1);
    tma_prefetch_desc(&p.tmB2);
    tma_prefetch_desc(&p.tmAux);
    tma_prefetch_desc(&p.tmMid);
    tma_prefetch_desc(&p.tmOut);
  }
  // Per-expert table in shared memory: etab[e] = first tile of expert e (low 23 bits) | number of experts before e with
  // an odd tile count (high 9 bits).  Pairs before expert e = (first_tile(e) - first_tile(0) + odd_before(e)) / 2.
  const int E = p.E;
  {
    const int cap_rows = p.max_tiles * kBM;
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
      __syncwarp();  // every lane has read its nine entries before any is rewritten
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
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrival or load completion
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- schedule: identical arithmetic in every role of both CTAs ----
  const int L = p.L, F = p.F;
  const int KB1 = L / 64;   // k-blocks of the first GEMM
  const int NC = F / 64;    // chunks per tile
  auto first_tile = [&](int e) { return etab[e] & 0x7fffff; };
  auto pairs_before = [&](int e) { return ((etab[e] & 0x7fffff) - (etab[0] & 0x7fffff) + (etab[e] >> 23)) >> 1; };
  const int n_pairs = pairs_before(E);
  const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
  const int n_clusters = static_cast<int>(gridDim.x) >> 1;
  struct Cur {
    int pid, c;   // pair index, chunk
    int e;        // expert of the pair
    int tile;     // the 128-row tile this CTA loads (its own, or the pair's first one when it has none)
    int live;     // 1: this CTA's tile exists and its results are stored
  };
  auto locate = [&](int pid, int c) {
    Cur k;
    k.pid = pid;
    k.c = c;
    k.e = 0;
    k.tile = 0;
    k.live = 0;
    if (pid >= n_pairs) return k;
    int lo = 0, hi = E - 1;  // largest e with pairs_before(e) <= pid
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (pairs_before(mid) <= pid) lo = mid;
      else hi = mid - 1;
    }
    k.e = lo;
    const int t1 = first_tile(lo + 1);
    const int first = first_tile(lo) + 2 * (pid - pairs_before(lo));
    const int own = first + static_cast<int>(rank);
    k.live = own < t1 ? 1 : 0;
    k.tile = k.live ? own : first;
    return k;
  };
  auto valid = [&](const Cur& k) { return k.pid < n_pairs; };
  auto next = [&](const Cur& k) {
    if (k.c + 1 < NC) {
      Cur n = k;
      n.c = k.c + 1;
      return n;
    }
    return locate(k.pid + n_clusters, 0);
  };

  // A ring as seen by one thread: producers wait on "empty" and arm rank 0's "full"; MMA issuers wait on "full" and
  // release with a commit to both CTAs.
  struct Ring {
    uint8_t* base;
    uint64_t *full, *empty;
    int stages, stage_bytes;
    int stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
  };

  if (warp == 0) {
    // =========== producer 1 (both CTAs): the first GEMM's weight slices ===========
    // (the tile's A operand comes from producer 2: this thread never blocks on the A buffer, so the weight ring stays
    //  two chunks ahead across tile boundaries)
    if (lane == 0) {
      Ring rg{ring1, r1_full, r1_empty, R1, S::kR1Bytes};
      bool ok = true;
      for (Cur k = locate(cluster_id, 0); ok && valid(k); k = next(k)) {
        // FWD: this CTA's half of the chunk's B: rank 0 the 64 gate columns, rank 1 the 64 up columns of Wgu[e], two
        //      k-blocks (8 KB each) per stage.
        // BWD: rows [c*64 + rank*32, +32) of Wd[e] (its half of the chunk's d_hidden columns), 4 KB per k-block, all
        //      k-blocks of the chunk in one stage.
        const int n_stage = FWD ? (KB1 + 1) / 2 : 1;
        CHAIN_TRACE(4, 30);
        for (int s = 0; s < n_stage && ok; ++s) {
          if (!mbar_wait(&rg.empty[rg.stage], rg.phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* st = rg.base + rg.stage * rg.stage_bytes;
          const uint32_t full0 = mapa_shared(smem_u32(&rg.full[rg.stage]), 0);
          if (FWD) {
            const int nkb = min(2, KB1 - 2 * s);
            if (rank == 0) mbar_expect_tx(&rg.full[rg.stage], 2 * nkb * 8192);
            for (int h = 0; h < nkb; ++h)
              tma_load_2d_pair(st + h * 8192, &p.tmB1, full0, static_cast<int>(rank) * F + k.c * 64, k.e * L + (2 * s + h) * 64);
          } else {
            if (rank == 0) mbar_expect_tx(&rg.full[rg.stage], 2 * KB1 * 4096);
            for (int kb = 0; kb < KB1; ++kb)
              tma_load_2d_pair(st + kb * 4096, &p.tmB1, full0, kb * 64, k.e * F + k.c * 64 + static_cast<int>(rank) * 32);
          }
          rg.advance();
        }
      }
    }
  } else if (warp == 10) {
    // =========== producer 2 (both CTAs): the second GEMM's weight slices ===========
    if (lane == 0) {
      Ring rg{ring2, r2_full, r2_empty, R2, S::kR2Bytes};
      bool ok = true;
      const int half = L / 2;  // this CTA's share of the second GEMM's N extent
      int tiles_loaded = 0;
      // this CTA's A operand of tile `t`, k-block by k-block as the previous tile's last chunk releases the buffers
      auto load_a = [&](const Cur& t) {
        for (int kb = 0; kb < KB1; ++kb) {
          if (!mbar_wait(&a1_empty[kb], (tiles_loaded & 1) ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            return;
          }
          if (rank == 0) mbar_expect_tx(&a1_full[kb], 2 * 16384);
          tma_load_2d_pair(a1 + kb * 16384, &p.tmA, mapa_shared(smem_u32(&a1_full[kb]), 0), kb * 64, t.tile * kBM);
        }
        ++tiles_loaded;
      };
      // The next tile's A operand is requested in front of the weights of chunk NC - 2: the buffers come free when the
      // first GEMM of the tile's LAST chunk completes, which is about when the epilogue warps start on chunk NC - 3, well
      // before the second GEMM of chunk NC - 2 needs its weights.
      const int a_slot = NC >= 2 ? NC - 2 : 0;
      {
        const Cur k0 = locate(cluster_id, 0);
        if (valid(k0)) load_a(k0);
      }
      for (Cur k = locate(cluster_id, 0); ok && valid(k); k = next(k)) {
        if (k.c == a_slot) {
          const Cur nx = locate(k.pid + n_clusters, 0);
          if (valid(nx)) {
            load_a(nx);
            if (!ok) break;
            if (p.prefetch_a) {  // and the one after it into L2
              const Cur nx2 = locate(nx.pid + n_clusters, 0);
              if (valid(nx2))
                for (int kb = 0; kb < KB1; ++kb) tma_prefetch_2d(&p.tmA, kb * 64, nx2.tile * kBM);
            }
          }
        }
        // FWD: rows [c*64, +64) of Wd[e], columns [rank*L/2, +L/2): L/128 MN-major chunks of 8 KB, one stage.
        // BWD: per part (gate columns, up columns of Wgu[e]) and per 128-column slice s of d_x: rows
        //      [s*128 + rank*64, +64) x k columns [part*F + c*64, +64), one 8 KB stage each.
        const int n_stage = FWD ? 1 : 2 * (L / 128);
        for (int s = 0; s < n_stage && ok; ++s) {
          if (!mbar_wait(&rg.empty[rg.stage], rg.phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          uint8_t* st = rg.base + rg.stage * rg.stage_bytes;
          const uint32_t full0 = mapa_shared(smem_u32(&rg.full[rg.stage]), 0);
          if (FWD) {
            if (rank == 0) mbar_expect_tx(&rg.full[rg.stage], 2 * half * 128);
            for (int j = 0; j < half / 64; ++j)
              tma_load_2d_pair(st + j * 8192, &p.tmB2, full0, static_cast<int>(rank) * half + j * 64, k.e * F + k.c * 64);
          } else {
            const int part = s / (L / 128), sl = s % (L / 128);
            if (rank == 0) mbar_expect_tx(&rg.full[rg.stage], 2 * 8192);
            tma_load_2d_pair(st, &p.tmB2, full0, part * F + k.c * 64, k.e * L + sl * 128 + static_cast<int>(rank) * 64);
          }
          rg.advance();
        }
      }
    }
  } else if (warp == 1) {
    // =========== MMA issuer 1 (rank 0 only): the first GEMM of every chunk ===========
    if (lane == 0 && rank == 0) {
      Ring rg{ring1, r1_full, r1_empty, R1, S::kR1Bytes};
      bool ok = true;
      const uint32_t a1_addr = smem_u32(a1);
      int tiles_g1 = 0, gi = 0;
      for (Cur k = locate(cluster_id, 0); ok && valid(k); k = next(k), ++gi) {
        const int b = gi & 1;
        if (!mbar_wait(&acc1_empty[b], ((gi >> 1) & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * 128;
        const uint32_t a_par = tiles_g1 & 1;
        CHAIN_TRACE(1, 1);
        const int n_stage = FWD ? (KB1 + 1) / 2 : 1;
        for (int s = 0; s < n_stage && ok; ++s) {
          if (!mbar_wait(&rg.full[rg.stage], rg.phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sb = smem_u32(rg.base + rg.stage * rg.stage_bytes);
          const int kb0 = FWD ? 2 * s : 0;
          const int nkb = FWD ? min(2, KB1 - 2 * s) : KB1;
          for (int h = 0; h < nkb && ok; ++h) {
            const int kb = kb0 + h;
            if (k.c == 0) {
              if (!mbar_wait(&a1_full[kb], a_par, abort_flag, p.status, kStatusMmaTimeout)) {
                ok = false;
                break;
              }
              tc_fence_after();
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a1_addr + kb * 16384 + kk * 32, 0, 1024);
              if (FWD) {
                constexpr uint32_t idesc = make_idesc(1u, 1u, false, true, 256, 128);
                const uint64_t db = make_smem_desc_sw128(sb + h * 8192 + kk * 2048, 8192, 1024);
                umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
              } else {
                constexpr uint32_t idesc = make_idesc(1u, 1u, false, false, 256, 64);
                const uint64_t db = make_smem_desc_sw128(sb + kb * 4096 + kk * 32, 0, 1024);
                umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
              }
            }
            if (k.c == NC - 1) umma_commit_pair(&a1_empty[kb], 0x3);  // last reader of this k-block of the A operand
          }
          if (!ok) break;
          umma_commit_pair(&rg.empty[rg.stage], 0x3);
          rg.advance();
        }
        if (!ok) break;
        if (k.c == 0) ++tiles_g1;
        umma_commit_pair(&acc1_full[b], 0x3);
        CHAIN_TRACE(1, 2);
      }
    }
  } else if (warp == 11) {
    // =========== MMA issuer 2 (rank 0 only): the second GEMM of every chunk ===========
    if (lane == 0 && rank == 0) {
      Ring rg{ring2, r2_full, r2_empty, R2, S::kR2Bytes};
      bool ok = true;
      const uint32_t a2_addr = smem_u32(a2);
      int tiles_g2 = 0, gi = 0;
      for (Cur k = locate(cluster_id, 0); ok && valid(k); k = next(k), ++gi) {
        if (k.c == 0) {
          if (!mbar_wait(acc2_empty, (tiles_g2 & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) break;
          ++tiles_g2;
        }
        // both CTAs' epilogue warps have written their A2 buffers and handed them to the async proxy
        CHAIN_TRACE(0, 3);
        const int b2 = FWD ? (gi & 1) : 0;                          // forward: the A2 buffer of the chunk's epilogue group
        const uint32_t par2 = FWD ? ((gi >> 1) & 1) : (gi & 1);
        if (!mbar_wait(&a2_full[b2], par2, abort_flag, p.status, kStatusMmaTimeout)) break;
        tc_fence_after();
        CHAIN_TRACE(0, 4);
        const int n_stage = FWD ? 1 : 2 * (L / 128);
        for (int s = 0; s < n_stage && ok; ++s) {
          if (!mbar_wait(&rg.full[rg.stage], rg.phase, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sb = smem_u32(rg.base + rg.stage * rg.stage_bytes);
          if (FWD) {
            const uint32_t idesc = make_idesc(1u, 1u, false, true, 256, static_cast<uint32_t>(L));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a2_addr + b2 * 16384 + kk * 32, 0, 1024);
              const uint64_t db = make_smem_desc_sw128(sb + kk * 2048, 8192, 1024);
              umma_f16_pair(tmem_base + ACC2_COL, da, db, idesc, (k.c > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
            constexpr uint32_t idesc = make_idesc(1u, 1u, false, false, 256, 128);
            const int part = s / (L / 128), sl = s % (L / 128);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a2_addr + part * 16384 + kk * 32, 0, 1024);
              const uint64_t db = make_smem_desc_sw128(sb + kk * 32, 0, 1024);
              umma_f16_pair(tmem_base + ACC2_COL + sl * 128, da, db, idesc, (k.c > 0 || part > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit_pair(&rg.empty[rg.stage], 0x3);
          rg.advance();
        }
        if (!ok) break;
        CHAIN_TRACE(0, 5);
        umma_commit_pair(&a2_empty[b2], 0x3);                  // the A2 buffers may be rewritten once these MMAs have read them
        if (k.c == NC - 1) umma_commit_pair(acc2_full, 0x3);   // the tile's result is complete in both CTAs
      }
    }
  } else if constexpr (FWD) {
    // ================= epilogue, forward (both CTAs, own 128 rows): two groups on ALTERNATING chunks =================
    // Group s (four warps, one per tensor-memory lane quadrant) owns the chunks whose running index has parity s, the
    // first GEMM's accumulator s and the hidden buffer s: while one group turns its chunk into the second GEMM's
    // operand, the other is one chunk ahead or behind, the second GEMM of either never waits for a CTA-wide barrier, and
    // a buffer is rewritten two chunks after the MMAs that read it were issued.  A chunk is done in two 32-column
    // halves through one pair of 8 KB slabs (gate, up on their way to h1).  The tile's result (eight 32-column slabs at
    // L = 256) is drained half by each group: the group of the last chunk right after it, the other after its first
    // chunk of the NEXT tile, so that neither idles while the last chunk's second GEMM completes.
    const int q = warp & 3;
    const int gs = (warp - 2) >> 2;
    const int bar_id = 1 + gs;
    const int r = q * 32 + lane;
    const bool issuer = (((warp - 2) & 3) == 0) && lane == 0;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint8_t* const slabs = aux + gs * 16384;
    uint8_t* const a2g = a2 + gs * 16384;
    const uint32_t acc1_empty0 = mapa_shared(smem_u32(&acc1_empty[gs]), 0);
    const uint32_t acc2_empty0 = mapa_shared(smem_u32(acc2_empty), 0);
    const uint32_t a2_full0 = mapa_shared(smem_u32(&a2_full[gs]), 0);
    const int nsl = L / kSlabCols;
    int tiles_done = 0;
    bool ok = true;
    // the second GEMM's accumulator of tile `t` -> bf16 -> y_sorted: slabs gs, gs + 2, ...
    auto tile_epilogue = [&](const Cur& t) {
      if (issuer) CHAIN_TRACE(2 + gs, 20);
      if (!mbar_wait(acc2_full, tiles_done & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (issuer) CHAIN_TRACE(2 + gs, 21);
      tc_fence_after();
      ok = epi_bar_all(bar_id, ok);
      if (!ok) return;
      const int m0 = t.tile * kBM;
#pragma unroll 1
      for (int c = gs; c < nsl; c += 2) {
        float v[32];
        tmem_ld32(lane_addr + ACC2_COL + c * 32, v);
        tmem_ld_wait();
        if (c + 2 >= nsl) {  // this warp's last slab is in registers: hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc2_empty0);
        }
        if (!t.live) continue;  // uniform over the CTA: a tile-less second CTA only drains its accumulator
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
        if (issuer) tma_store_wait_read_all();
        epi_bar_sync(bar_id);
        stage_row_bf16(slabs, r, pk);
        fence_proxy_async_smem();
        epi_bar_sync(bar_id);
        if (issuer) {
          tma_store_3d(&p.tmOut, slabs, c * kSlabCols, m0, 0);
          tma_store_commit();
        }
      }
      ++tiles_done;
      if (issuer) CHAIN_TRACE(2 + gs, 22);
    };
    Cur cur = locate(cluster_id, 0);
    if (gs == 1 && valid(cur)) cur = next(cur);
    Cur pend = cur;
    bool pending = false;  // group 0: a tile whose result slabs are still to be drained
    for (int n = 0; valid(cur); ++n) {
      const int m0 = cur.tile * kBM;
      if (issuer) CHAIN_TRACE(2 + gs, 10);
      if (!mbar_wait(&acc1_full[gs], n & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (issuer) CHAIN_TRACE(2 + gs, 11);
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t pa[16], pb[16], pc[16];
        if (ok) {
          float v[32], u[32];
          tmem_ld32(lane_addr + gs * 128 + h * 32, v);        // gate
          tmem_ld32(lane_addr + gs * 128 + 64 + h * 32, u);   // up
          tmem_ld_wait();
          if (issuer) CHAIN_TRACE(2 + gs, 18);
          if (h == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc1_empty0);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // gate/up are saved as bf16; hidden is formed from the rounded values
            pa[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            pb[j] = pack_bf16x2(u[2 * j], u[2 * j + 1]);
            const float g0 = __uint_as_float(pa[j] << 16), g1 = __uint_as_float(pa[j] & 0xffff0000u);
            const float u0 = __uint_as_float(pb[j] << 16), u1 = __uint_as_float(pb[j] & 0xffff0000u);
            pc[j] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
          }
        }
        // the hidden buffer: the second GEMM of this group's previous chunk has read it; the slabs (and, first half, the
        // hidden buffer): the stores issued from them have read their source
        if (issuer) CHAIN_TRACE(2 + gs, 12);
        if (h == 0 && ok && !mbar_wait(&a2_empty[gs], (n & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
        if (issuer) CHAIN_TRACE(2 + gs, 13);
        if (issuer) tma_store_wait_read_all();
        if (issuer) CHAIN_TRACE(2 + gs, 14);
        ok = epi_bar_all(bar_id, ok);
        if (!ok) break;
        stage_row_bf16(slabs, r, pa);
        stage_row_bf16(slabs + 8192, r, pb);
        a2_write_half(a2g, r, h, pc);
        fence_proxy_async_smem();
        if (issuer) CHAIN_TRACE(2 + gs, 15);
        epi_bar_sync(bar_id);
        if (issuer) {
          if (h == 1) {
            CHAIN_TRACE(2 + gs, 16);
            mbar_arrive_cluster(a2_full0);  // the MMAs issued by rank 0 read this CTA's buffer
          }
          if (cur.live) {
            tma_store_3d(&p.tmAux, slabs, cur.c * 64 + h * 32, m0, 0);             // gate -> h1
            tma_store_3d(&p.tmAux, slabs + 8192, F + cur.c * 64 + h * 32, m0, 0);  // up   -> h1
            if (h == 1) tma_store_2d(&p.tmMid, a2g, cur.c * 64, m0);               // hidden
          }
          tma_store_commit();
        }
      }
      if (!ok) break;
      if (cur.c == 0 && pending) {
        tile_epilogue(pend);
        pending = false;
        if (!ok) break;
      }
      if (cur.c == NC - 1) {
        tile_epilogue(cur);
        if (!ok) break;
      } else if (cur.c == NC - 2) {
        pend = cur;
        pending = true;
      }
      cur = next(cur);
      if (valid(cur)) cur = next(cur);
    }
    if (ok && pending) tile_epilogue(pend);
    if (issuer) tma_store_wait0();
  } else {
    // ============================= epilogue, backward (both CTAs, own 128 rows) =============================
    const int q = warp & 3;
    const int group = (warp - 2) >> 2;
    const int bar_id = 1 + group;
    const int r = q * 32 + lane;
    const bool chunk_issuer = (warp == 2 && lane == 0);
    const bool group_issuer = (((warp - 2) & 3) == 0) && lane == 0;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint8_t* const out_slab = outb + group * 8192;
    // rank 0's barriers that this CTA's epilogue arrives on
    const uint32_t acc1_empty0[2] = {mapa_shared(smem_u32(&acc1_empty[0]), 0), mapa_shared(smem_u32(&acc1_empty[1]), 0)};
    const uint32_t acc2_empty0 = mapa_shared(smem_u32(acc2_empty), 0);
    const uint32_t a2_full0 = mapa_shared(smem_u32(a2_full), 0);
    int tiles_done = 0;
    bool ok = true;
    Cur cur = locate(cluster_id, 0);
    // Backward: saved gate / up of a chunk staged by TMA two chunks ahead (see chain.cuh); local to each CTA.
    auto load_gu = [&](const Cur& k, int b) {
      mbar_expect_tx(&gu_full[b], 32768);
      uint8_t* dst = aux + b * 32768;
      const int row0 = k.tile * kBM;
      for (int gr = 0; gr < 2; ++gr) {
        tma_load_3d(dst + gr * 16384, &p.tmAux, &gu_full[b], k.c * 64 + gr * 32, row0, 0);
        tma_load_3d(dst + gr * 16384 + 8192, &p.tmAux, &gu_full[b], F + k.c * 64 + gr * 32, row0, 0);
      }
    };
    if (!FWD && chunk_issuer && valid(cur)) {
      load_gu(cur, 0);
      const Cur c1 = next(cur);
      if (valid(c1)) load_gu(c1, 1);
    }
    for (int gi = 0; valid(cur); ++gi, cur = next(cur)) {
      const int b = gi & 1;
      const int m0 = cur.tile * kBM;
      // ---------------- chunk epilogue ----------------
      if (chunk_issuer) CHAIN_TRACE(2, 10);
      if (!mbar_wait(&acc1_full[b], (gi >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (chunk_issuer) CHAIN_TRACE(2, 11);
      if (!FWD && ok && !mbar_wait(&gu_full[b], (gi >> 1) & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      tc_fence_after();
      uint32_t pa[16], pb[16], pc[16];
      if (ok) {
        if (FWD) {
          float v[32], u[32];
          tmem_ld32(lane_addr + b * 128 + group * 32, v);        // gate
          tmem_ld32(lane_addr + b * 128 + 64 + group * 32, u);   // up
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc1_empty0[b]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pa[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            pb[j] = pack_bf16x2(u[2 * j], u[2 * j + 1]);
            const float g0 = __uint_as_float(pa[j] << 16), g1 = __uint_as_float(pa[j] & 0xffff0000u);
            const float u0 = __uint_as_float(pb[j] << 16), u1 = __uint_as_float(pb[j] & 0xffff0000u);
            pc[j] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
          }
        } else {
          float v[32];
          tmem_ld32(lane_addr + b * 128 + group * 32, v);        // d_hidden
          tmem_ld_wait();
          tc_fence_before();
          uint32_t sg[16], su[16];
          const uint8_t* gu = aux + b * 32768 + group * 16384;
          slab_read_row(gu, r, sg);
          slab_read_row(gu + 8192, r, su);
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc1_empty0[b]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t dh2 = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            const float dh[2] = {__uint_as_float(dh2 << 16), __uint_as_float(dh2 & 0xffff0000u)};
            const float g[2] = {__uint_as_float(sg[j] << 16), __uint_as_float(sg[j] & 0xffff0000u)};
            const float uu[2] = {__uint_as_float(su[j] << 16), __uint_as_float(su[j] & 0xffff0000u)};
            float dg[2], du[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const float s = sigmoid_fast(g[t]);
              du[t] = dh[t] * g[t] * s;
              dg[t] = dh[t] * uu[t] * s * (1.0f + g[t] * (1.0f - s));
            }
            pa[j] = pack_bf16x2(dg[0], dg[1]);
            pb[j] = pack_bf16x2(du[0], du[1]);
          }
        }
      }
      if (chunk_issuer) CHAIN_TRACE(2, 12);
      if (ok && !mbar_wait(a2_empty, (gi & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (chunk_issuer) CHAIN_TRACE(2, 13);
      // stores issued from the buffers about to be rewritten have read their source (backward: the tile epilogue's slabs
      // share the A2 buffer, and each group's issuer committed its own)
      if (FWD ? chunk_issuer : group_issuer) tma_store_wait_read_all();
      if (chunk_issuer) CHAIN_TRACE(2, 14);
      ok = epi_all_and(ok);
      if (!ok) break;
      if (!FWD && chunk_issuer) {  // every thread holds its gate / up rows in registers: refill the buffer (chunk gi + 2)
        const Cur c2 = next(next(cur));
        if (valid(c2)) load_gu(c2, b);
      }
      if (FWD) {
        uint8_t* slabs = aux + group * 16384;
        stage_row_bf16(slabs, r, pa);
        stage_row_bf16(slabs + 8192, r, pb);
        a2_write_half(a2, r, group, pc);
      } else {
        a2_write_half(a2, r, group, pa);
        a2_write_half(a2 + 16384, r, group, pb);
      }
      if (chunk_issuer) CHAIN_TRACE(2, 15);
      fence_proxy_async_smem();
      if (chunk_issuer) CHAIN_TRACE(2, 17);
      epi_all_sync();
      if (chunk_issuer) {
        CHAIN_TRACE(2, 16);
        mbar_arrive_cluster(a2_full0);  // the MMAs issued by rank 0 read this CTA's A2 buffer
        if (cur.live) {
          if (FWD) {
            for (int gr = 0; gr < 2; ++gr) {
              tma_store_3d(&p.tmAux, aux + gr * 16384, cur.c * 64 + gr * 32, m0, 0);
              tma_store_3d(&p.tmAux, aux + gr * 16384 + 8192, F + cur.c * 64 + gr * 32, m0, 0);
            }
            tma_store_2d(&p.tmMid, a2, cur.c * 64, m0);
          } else {
            tma_store_2d(&p.tmMid, a2, cur.c * 64, m0);
            tma_store_2d(&p.tmMid, a2 + 16384, F + cur.c * 64, m0);
          }
        }
        tma_store_commit();
      }
      if (cur.c != NC - 1) continue;
      // ---------------- tile epilogue ----------------
      if (chunk_issuer) CHAIN_TRACE(2, 20);
      if (!mbar_wait(acc2_full, tiles_done & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (chunk_issuer) CHAIN_TRACE(2, 21);
      tc_fence_after();
      if (!FWD && chunk_issuer) tma_store_wait_read_all();  // the last chunk's stores have read the A2 buffer (slabs go there)
      ok = epi_all_and(ok);
      if (!ok) break;
      const int slabs = L / kSlabCols;
      const int last = ((slabs - 1 - group) >= 0) ? group + ((slabs - 1 - group) & ~1) : -1;
      if (last < 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc2_empty0);
      }
#pragma unroll 1
      for (int c = group; c < slabs; c += 2) {
        float v[32];
        tmem_ld32(lane_addr + ACC2_COL + c * 32, v);
        tmem_ld_wait();
        if (c == last) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc2_empty0);
        }
        if (!cur.live) continue;  // uniform over the CTA: a tile-less second CTA only drains its accumulator
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
        if (group_issuer) tma_store_wait_read_all();
        epi_bar_sync(bar_id);
        stage_row_bf16(out_slab, r, pk);
        fence_proxy_async_smem();
        epi_bar_sync(bar_id);
        if (group_issuer) {
          tma_store_3d(&p.tmOut, out_slab, c * kSlabCols, m0, 0);
          tma_store_commit();
        }
      }
      ++tiles_done;
      if (chunk_issuer) CHAIN_TRACE(2, 22);
    }
    if (group_issuer) tma_store_wait0();
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
