// Two chained tcgen05 GEMMs per 128-row tile of the padded routed layout, in ONE persistent kernel: the
// intermediate of the routed SwiGLU expert never makes an HBM round trip between them.
//
//   CHAIN_FWD   h1 = x_sorted * Wgu[e]          (64 gate + 64 up columns per chunk, fp32 in tensor memory)
//               hidden = silu(gate) * up        (epilogue warps; written as the bf16 A operand of the second GEMM
//                                                into shared memory and, from the same buffer, to HBM for backward)
//               y_sorted = hidden * Wd[e]       (accumulated chunk by chunk into a second tensor-memory region)
//   CHAIN_BWD   d_hidden = d_y_sorted * Wd[e]^T (64 columns per chunk)
//               d_h1 = swiglu'(h1, d_hidden)    (epilogue warps; the saved gate/up of the chunk is staged by TMA;
//                                                d_gate / d_up become the A operand of the second GEMM and go to HBM
//                                                from the same buffer for the weight gradients)
//               d_x_sorted = d_h1 * Wgu[e]^T    (accumulated chunk by chunk)
//
// Replaces, per direction, two grouped GEMM launches plus (backward) the streaming SwiGLU-adjoint kernel:
// `hidden` is read back from HBM by nobody in forward, and d_hidden never exists in memory.
//
// One CTA per SM walks a CONTIGUOUS range of tiles (ceil(n_tiles / grid) each); a tile belongs to one expert
// (tile_expert).  Contiguous ranges keep a CTA on the same expert for several tiles in a row, so after the first tile
// its weight slices come from L2 at L2 latency; with a round-robin assignment all CTAs that share an expert would ask
// for the same weight lines at the same moment and every load would see the latency of the one HBM fetch behind it.  Roles (320 threads):
//   warp 0      TMA producer.  The tile's A operand (128 x L, K-major) is resident for the whole tile; the weight
//               slices stream through a ring of 16 KB stages in exactly the order the MMA warp consumes them
//   warp 1      MMA issuer (one thread) and owner of the 512 tensor-memory columns:
//               [0,256) two accumulators of the first GEMM (chunk g uses buffer g & 1), [256,512) the second GEMM's
//   warps 2..9  epilogue: the chunk epilogue (all eight warps together, one 32-column half of the chunk per group of
//               four) and the tile epilogue (32-column slabs alternating between the two groups, as in gemm.cuh)
// The MMA warp issues the first GEMM of chunk g+1 BEFORE the second GEMM of chunk g, so the tensor pipe works on
// chunk g+1 while the epilogue warps turn chunk g's accumulator into the second GEMM's operand.
//
// Every wait is bounded (common/ptx.cuh): on expiry the waiter records a status code, raises the CTA's abort flag,
// all roles fall through to the tensor-memory release.
#pragma once
#include "gemm.cuh"

namespace lmoe {

enum : int { CHAIN_FWD = 0, CHAIN_BWD = 1 };

constexpr int kChainMaxL = 256;                // width of the second GEMM's output (tensor-memory columns 256..511)
constexpr int kChainStageBytes = 16384;
constexpr int kChainA1Bytes = (kChainMaxL / 64) * 16384;  // resident A tile: up to four k-blocks of 128 x 64

struct alignas(64) ChainParams {
  CUtensorMap tmA;    // A of the first GEMM  [P, L]  box {64, 128}            (x_sorted | d_y_sorted)
  CUtensorMap tmB1;   // FWD: Wgu [E*L, 2F] box {64, 64};   BWD: Wd [E*F, L] box {64, 64}
  CUtensorMap tmB2;   // FWD: Wd [E*F, L] box {64, 64};     BWD: Wgu [E*L, 2F] box {64, min(L, 128)}
  CUtensorMap tmAux;  // FWD: store h1 [P, 2F] box {32, 128} (64-byte swizzle);  BWD: load of the same tensor
  CUtensorMap tmMid;  // store from the A2 buffer, box {64, 128} (128-byte swizzle): FWD hidden [P, F]; BWD d_h1 [P, 2F]
  CUtensorMap tmOut;  // store of the second GEMM's result [P, L] box {32, 128} (64-byte swizzle)
  int L, F;
  int max_tiles;            // capacity of the padded layout in tiles
  int prefetch_a;           // 1: prefetch the next tile's A operand into L2
  int contiguous;           // 1: contiguous tile range per CTA; 0: round-robin
  const int* tile_expert;
  const int* n_tiles;       // device scalar: tiles in use
  int* status;
};

// Development aid (compiled only with -DLMOE_CHAIN_TRACE): CTA 0 records (tag, globaltimer) pairs per role.
#ifdef LMOE_CHAIN_TRACE
constexpr int kTraceSlots = 4096;
constexpr int kTraceRoles = 5;
__device__ long long g_chain_trace[kTraceRoles][kTraceSlots][2];
__device__ int g_chain_trace_n[kTraceRoles];
// The slot counter lives in a register of the (single) thread that records for a role: no load on the recording path.
__device__ __forceinline__ void chain_trace(int role, int tag, int& i) {
  if (blockIdx.x != 0 || i >= kTraceSlots) return;
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  g_chain_trace[role][i][0] = tag;
  g_chain_trace[role][i][1] = t;
  g_chain_trace_n[role] = ++i;
}
#define CHAIN_TRACE(role, tag) chain_trace(role, tag, trace_i)
#define CHAIN_TRACE_DECL int trace_i = 0;
#else
#define CHAIN_TRACE(role, tag)
#define CHAIN_TRACE_DECL
#endif

template <int MODE>
struct ChainSmem {
  static constexpr int kA2Bytes = (MODE == CHAIN_FWD) ? 16384 : 32768;  // hidden chunk | d_gate + d_up chunk
  // FWD: gate/up slabs on their way to h1 (2 groups x 2 x 8 KB); BWD: saved gate/up staged by TMA, two chunks deep
  static constexpr int kAuxBytes = (MODE == CHAIN_FWD) ? 32768 : 65536;
  static constexpr int kOutBytes = 16384;  // one 128 x 32 bf16 slab per epilogue group
  static constexpr int kBarrierBytes = 2048;  // barriers, and the pair kernel's per-expert prefix table
  static constexpr int kFixed = kChainA1Bytes + kA2Bytes + kAuxBytes + kOutBytes;
  static constexpr int kStages = (232448 - 1024 - kBarrierBytes - kFixed) / kChainStageBytes;
  static constexpr int kTotal = 1024 + kFixed + kStages * kChainStageBytes + kBarrierBytes;
  static_assert(kStages >= 3, "ring too shallow");
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1)
               : "memory");
}
// AND-reduction of a predicate over the 256 epilogue threads (named barrier 3).
__device__ __forceinline__ bool epi_all_and(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %1, 0;\n"
      "bar.red.and.pred q, 3, 256, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void epi_all_sync() { asm volatile("bar.sync 3, 256;" ::: "memory"); }

// Row r's 32-column half `half32` (0 | 1) of a 128 x 64 bf16 K-major tile in the 128-byte-swizzled layout that both a
// TMA store with SWIZZLE_128B and a tcgen05 K-major descriptor read: 16-byte chunk j of row r sits at chunk j ^ (r & 7).
__device__ __forceinline__ void a2_write_half(uint8_t* tile, int r, int half32, const uint32_t (&p)[16]) {
  const int sw = r & 7;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int chunk = (half32 * 4 + j) ^ sw;
    *reinterpret_cast<uint4*>(tile + r * 128 + (chunk << 4)) = make_uint4(p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
  }
}
// Row r of a 128 x 32 bf16 slab in the 64-byte-swizzled layout (what stage_row_bf16 writes and a SWIZZLE_64B load leaves).
__device__ __forceinline__ void slab_read_row(const uint8_t* buf, int r, uint32_t (&p)[16]) {
  const int sw = (r >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = *reinterpret_cast<const uint4*>(buf + r * 64 + ((j ^ sw) << 4));
    p[4 * j] = v.x;
    p[4 * j + 1] = v.y;
    p[4 * j + 2] = v.z;
    p[4 * j + 3] = v.w;
  }
}

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) chain_kernel(const __grid_constant__ ChainParams p) {
  using S = ChainSmem<MODE>;
  constexpr int STAGES = S::kStages;
  constexpr bool FWD = (MODE == CHAIN_FWD);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ACC2_COL = 256;

  CHAIN_TRACE_DECL
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* const a1 = smem;                              // [KB1][128 x 64] K-major, 128-byte swizzle
  uint8_t* const a2 = a1 + kChainA1Bytes;                // FWD: hidden chunk; BWD: d_gate chunk, d_up chunk
  uint8_t* const aux = a2 + S::kA2Bytes;
  uint8_t* const outb = aux + S::kAuxBytes;
  uint8_t* const ring = outb + S::kOutBytes;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(ring + STAGES * kChainStageBytes);
  uint64_t* const ring_full = bars;
  uint64_t* const ring_empty = ring_full + STAGES;
  uint64_t* const a1_full = ring_empty + STAGES;         // [4]
  uint64_t* const a1_empty = a1_full + 4;                // [4]
  uint64_t* const acc1_full = a1_empty + 4;              // [2]
  uint64_t* const acc1_empty = acc1_full + 2;            // [2]
  uint64_t* const a2_full = acc1_empty + 2;              // [1]
  uint64_t* const a2_empty = a2_full + 1;                // [1]
  uint64_t* const acc2_full = a2_empty + 1;              // [1]
  uint64_t* const acc2_empty = acc2_full + 1;            // [1]
  uint64_t* const gu_full = acc2_empty + 1;              // [2] (BWD)
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(gu_full + 2);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&a1_full[i], 1);
      mbar_init(&a1_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc1_full[i], 1);
      mbar_init(&acc1_empty[i], 8);
      mbar_init(&gu_full[i], 1);
    }
    mbar_init(a2_full, 1);
    mbar_init(a2_empty, 1);
    mbar_init(acc2_full, 1);
    mbar_init(acc2_empty, 8);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB1);
    tma_prefetch_desc(&p.tmB2);
    tma_prefetch_desc(&p.tmAux);
    tma_prefetch_desc(&p.tmMid);
    tma_prefetch_desc(&p.tmOut);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- schedule: identical arithmetic in every role ----
  const int L = p.L, F = p.F;
  const int KB1 = L / 64;             // k-blocks of the first GEMM
  const int NC = F / 64;              // chunks per tile
  const int NH = (L + 127) / 128;     // 128-column halves of the second GEMM's output
  const int n_tiles = min(*p.n_tiles, p.max_tiles);
  struct Cur {
    int tile, c;
  };
  // p.contiguous: CTA b takes tiles [b * per, (b + 1) * per); otherwise tiles b, b + grid, b + 2 * grid, ...
  const int tiles_per_cta = (n_tiles + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int tile_step = p.contiguous ? 1 : static_cast<int>(gridDim.x);
  const int tile_begin = p.contiguous ? static_cast<int>(blockIdx.x) * tiles_per_cta : static_cast<int>(blockIdx.x);
  const int tile_end = p.contiguous ? min(tile_begin + tiles_per_cta, n_tiles) : n_tiles;
  auto valid = [&](const Cur& k) { return k.tile < tile_end; };
  auto next = [&](Cur k) {
    if (++k.c == NC) {
      k.c = 0;
      k.tile += tile_step;
    }
    return k;
  };

  if (warp == 0) {
    // ======================================= TMA producer =======================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto acquire = [&](uint32_t bytes) -> uint8_t* {  // next ring stage, armed for `bytes`
        CHAIN_TRACE(0, 31);
        if (!mbar_wait(&ring_empty[stage], phase ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
          ok = false;
          return nullptr;
        }
        CHAIN_TRACE(0, 32);
        mbar_expect_tx(&ring_full[stage], bytes);
        return ring + stage * kChainStageBytes;
      };
      auto advance = [&]() {
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      };
      int tiles_loaded = 0;  // tiles whose A operand has been requested
      auto emit_g1 = [&](const Cur& k, int gi) {
        CHAIN_TRACE(0, 30);
        const int e = p.tile_expert[k.tile];
        const int m0 = k.tile * kBM;
        if (k.c == 0) {  // the tile's A operand, k-block by k-block as the previous tile's last chunk releases them
          for (int kb = 0; kb < KB1 && ok; ++kb) {
            if (!mbar_wait(&a1_empty[kb], (tiles_loaded & 1) ^ 1, abort_flag, p.status, kStatusProducerTimeout)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&a1_full[kb], 16384);
            tma_load_2d(a1 + kb * 16384, &p.tmA, &a1_full[kb], kb * 64, m0);
          }
          ++tiles_loaded;
          // the A operand of the tile after this one: bring it into L2 a whole tile period ahead, so that its load
          // (which can only start when this tile's last chunk releases the buffer) does not wait for HBM
          const int nt_tile = k.tile + tile_step;
          if (p.prefetch_a && nt_tile < tile_end)
            for (int kb = 0; kb < KB1; ++kb) tma_prefetch_2d(&p.tmA, kb * 64, nt_tile * kBM);
        }
        if (!ok) return;
        if (FWD) {
          // one stage per k-block: gate columns [c*64, +64) and up columns [F + c*64, +64) of Wgu[e] rows [kb*64, +64)
          for (int kb = 0; kb < KB1; ++kb) {
            uint8_t* st = acquire(16384);
            if (!st) return;
            tma_load_2d(st, &p.tmB1, &ring_full[stage], k.c * 64, e * L + kb * 64);
            tma_load_2d(st + 8192, &p.tmB1, &ring_full[stage], F + k.c * 64, e * L + kb * 64);
            advance();
          }
        } else {
          // one stage per pair of k-blocks: rows [c*64, +64) of Wd[e] (the chunk's d_hidden columns), 64 k each
          for (int kb = 0; kb < KB1; kb += 2) {
            const int nkb = min(2, KB1 - kb);
            uint8_t* st = acquire(nkb * 8192);
            if (!st) return;
            for (int h = 0; h < nkb; ++h)
              tma_load_2d(st + h * 8192, &p.tmB1, &ring_full[stage], (kb + h) * 64, e * F + k.c * 64);
            advance();
          }
        }
      };
      auto emit_g2 = [&](const Cur& k) {
        CHAIN_TRACE(0, 35);
        const int e = p.tile_expert[k.tile];
        if (FWD) {
          // rows [c*64, +64) of Wd[e], 128 output columns per stage (two 64-wide MN-major chunks)
          for (int s = 0; s < NH; ++s) {
            const int n_this = min(128, L - s * 128);
            uint8_t* st = acquire(n_this * 128);
            if (!st) return;
            for (int j = 0; j < n_this / 64; ++j)
              tma_load_2d(st + j * 8192, &p.tmB2, &ring_full[stage], s * 128 + j * 64, e * F + k.c * 64);
            advance();
          }
        } else {
          // Wgu[e] rows (output columns of d_x) [s*128, +n), k columns [c*64, +64) (gate part) then [F + c*64, +64)
          // (the box always holds min(L, 128) rows; a last half with fewer rows of this expert also brings rows of
          //  the next one, or zeros past the end of the tensor, which the MMA's N extent leaves out)
          const int box_n = min(L, 128);
          for (int part = 0; part < 2; ++part)
            for (int s = 0; s < NH; ++s) {
              uint8_t* st = acquire(box_n * 128);
              if (!st) return;
              tma_load_2d(st, &p.tmB2, &ring_full[stage], part * F + k.c * 64, e * L + s * 128);
              advance();
            }
        }
      };
      Cur cur{tile_begin, 0};
      int gi = 0;
      if (valid(cur)) emit_g1(cur, 0);
      while (ok && valid(cur)) {
        const Cur nx = next(cur);
        if (valid(nx)) emit_g1(nx, gi + 1);
        if (!ok) break;
        emit_g2(cur);
        cur = nx;
        ++gi;
      }
    }
  } else if (warp == 1) {
    // ======================================== MMA issuer ========================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto wait_stage = [&]() -> uint32_t {
        if (!mbar_wait(&ring_full[stage], phase, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          return 0u;
        }
        tc_fence_after();
        return smem_u32(ring + stage * kChainStageBytes);
      };
      auto release_stage = [&]() {
        umma_commit(&ring_empty[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      };
      const uint32_t a1_addr = smem_u32(a1), a2_addr = smem_u32(a2);
      int tiles_g1 = 0;  // tiles whose first GEMM has started (parity of the a1_full barriers)
      int tiles_g2 = 0;  // tiles whose second GEMM has started (parity of acc2_empty)
      auto issue_g1 = [&](const Cur& k, int gi) {
        const int b = gi & 1;
        if (!mbar_wait(&acc1_empty[b], ((gi >> 1) & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          return;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * 128;
        const uint32_t a_par = tiles_g1 & 1;
        CHAIN_TRACE(1, 1);
        if (FWD) {
          constexpr uint32_t idesc = make_idesc(1u, 1u, false, true, kBM, 128);
          for (int kb = 0; kb < KB1; ++kb) {
            const uint32_t sb = wait_stage();
            if (!ok) return;
            if (k.c == 0) {
              if (!mbar_wait(&a1_full[kb], a_par, abort_flag, p.status, kStatusMmaTimeout)) {
                ok = false;
                return;
              }
              tc_fence_after();
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a1_addr + kb * 16384 + kk * 32, 0, 1024);
              const uint64_t db = make_smem_desc_sw128(sb + kk * 2048, 8192, 1024);
              umma_f16(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            release_stage();
            if (k.c == NC - 1) umma_commit(&a1_empty[kb]);  // last reader of this k-block of the tile's A operand
          }
        } else {
          constexpr uint32_t idesc = make_idesc(1u, 1u, false, false, kBM, 64);
          for (int kb = 0; kb < KB1; kb += 2) {
            const uint32_t sb = wait_stage();
            if (!ok) return;
            const int nkb = min(2, KB1 - kb);
            for (int h = 0; h < nkb; ++h) {
              if (k.c == 0) {
                if (!mbar_wait(&a1_full[kb + h], a_par, abort_flag, p.status, kStatusMmaTimeout)) {
                  ok = false;
                  return;
                }
                tc_fence_after();
              }
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const uint64_t da = make_smem_desc_sw128(a1_addr + (kb + h) * 16384 + kk * 32, 0, 1024);
                const uint64_t db = make_smem_desc_sw128(sb + h * 8192 + kk * 32, 0, 1024);
                umma_f16(d_tmem, da, db, idesc, (kb + h > 0 || kk > 0) ? 1u : 0u);
              }
              if (k.c == NC - 1) umma_commit(&a1_empty[kb + h]);
            }
            release_stage();
          }
        }
        if (k.c == 0) ++tiles_g1;
        umma_commit(&acc1_full[b]);
        CHAIN_TRACE(1, 2);
      };
      auto issue_g2 = [&](const Cur& k, int gi) {
        if (k.c == 0) {
          if (!mbar_wait(acc2_empty, (tiles_g2 & 1) ^ 1, abort_flag, p.status, kStatusMmaTimeout)) {
            ok = false;
            return;
          }
          ++tiles_g2;
        }
        CHAIN_TRACE(1, 3);
        if (!mbar_wait(a2_full, gi & 1, abort_flag, p.status, kStatusMmaTimeout)) {
          ok = false;
          return;
        }
        tc_fence_after();
        CHAIN_TRACE(1, 4);
        if (FWD) {
          for (int s = 0; s < NH; ++s) {
            const int n_this = min(128, L - s * 128);
            const uint32_t idesc = make_idesc(1u, 1u, false, true, kBM, static_cast<uint32_t>(n_this));
            const uint32_t sb = wait_stage();
            if (!ok) return;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = make_smem_desc_sw128(a2_addr + kk * 32, 0, 1024);
              const uint64_t db = make_smem_desc_sw128(sb + kk * 2048, 8192, 1024);
              umma_f16(tmem_base + ACC2_COL + s * 128, da, db, idesc, (k.c > 0 || kk > 0) ? 1u : 0u);
            }
            release_stage();
          }
        } else {
          for (int part = 0; part < 2; ++part)
            for (int s = 0; s < NH; ++s) {
              const int n_this = min(128, L - s * 128);
              const uint32_t idesc = make_idesc(1u, 1u, false, false, kBM, static_cast<uint32_t>(n_this));
              const uint32_t sb = wait_stage();
              if (!ok) return;
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const uint64_t da = make_smem_desc_sw128(a2_addr + part * 16384 + kk * 32, 0, 1024);
                const uint64_t db = make_smem_desc_sw128(sb + kk * 32, 0, 1024);
                umma_f16(tmem_base + ACC2_COL + s * 128, da, db, idesc, (k.c > 0 || part > 0 || kk > 0) ? 1u : 0u);
              }
              release_stage();
            }
        }
        umma_commit(a2_empty);                       // the A2 buffer may be rewritten once these MMAs have read it
        CHAIN_TRACE(1, 5);
        if (k.c == NC - 1) umma_commit(acc2_full);   // the tile's result is complete
      };
      Cur cur{tile_begin, 0};
      int gi = 0;
      if (valid(cur)) issue_g1(cur, 0);
      while (ok && valid(cur)) {
        const Cur nx = next(cur);
        if (valid(nx)) issue_g1(nx, gi + 1);
        if (!ok) break;
        issue_g2(cur, gi);
        cur = nx;
        ++gi;
      }
    }
  } else {
    // ========================================= epilogue =========================================
    const int q = warp & 3;             // tensor-memory lane quadrant of this warp
    const int group = (warp - 2) >> 2;  // 0 | 1: which 32-column half of a chunk, which slabs of the tile epilogue
    const int bar_id = 1 + group;
    const int r = q * 32 + lane;        // row of the tile owned by this thread
    const bool chunk_issuer = (warp == 2 && lane == 0);
    const bool group_issuer = (((warp - 2) & 3) == 0) && lane == 0;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint8_t* const out_slab = outb + group * 8192;
    int tiles_done = 0;
    bool ok = true;
    Cur cur{tile_begin, 0};
    // Backward: the saved gate / up of chunk `k` (four 128 x 32 slabs: group 0 gate, up; group 1 gate, up) staged by TMA
    // into buffer `b`.  Issued by one epilogue thread two chunks ahead of their use: the buffer of chunk g is free as
    // soon as every epilogue thread has passed chunk g's first barrier (its rows are in registers by then), so no
    // "empty" barrier is needed, and the lead of two chunk periods covers the HBM latency.
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
          if (lane == 0) mbar_arrive(&acc1_empty[b]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // gate/up are saved as bf16; hidden is formed from the rounded values
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
          if (lane == 0) mbar_arrive(&acc1_empty[b]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // d_hidden is rounded to bf16 first (what a stored d_hidden would hold), then
            //   d_up = dh * g * sig(g),  d_gate = dh * u * sig(g) * (1 + g * (1 - sig(g)))
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
      // The A2 buffer (and, forward, the gate/up slabs) may be rewritten once the second GEMM of the previous chunk
      // has read it and the stores issued from it have read their source.
      if (chunk_issuer) CHAIN_TRACE(2, 12);
      if (ok && !mbar_wait(a2_empty, (gi & 1) ^ 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (chunk_issuer) CHAIN_TRACE(2, 13);
      if (chunk_issuer) tma_store_wait_read_all();
      if (chunk_issuer) CHAIN_TRACE(2, 14);
      ok = epi_all_and(ok);  // every epilogue thread reaches this barrier on every chunk, whatever its waits returned
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
      fence_proxy_async_smem();
      if (chunk_issuer) CHAIN_TRACE(2, 15);
      epi_all_sync();
      if (chunk_issuer) {
        CHAIN_TRACE(2, 16);
        mbar_arrive(a2_full);  // the MMA warp may issue the second GEMM of this chunk
        if (FWD) {
          for (int gr = 0; gr < 2; ++gr) {
            tma_store_3d(&p.tmAux, aux + gr * 16384, cur.c * 64 + gr * 32, m0, 0);             // gate -> h1
            tma_store_3d(&p.tmAux, aux + gr * 16384 + 8192, F + cur.c * 64 + gr * 32, m0, 0);  // up   -> h1
          }
          tma_store_2d(&p.tmMid, a2, cur.c * 64, m0);                                          // hidden
        } else {
          tma_store_2d(&p.tmMid, a2, cur.c * 64, m0);                                          // d_gate -> d_h1
          tma_store_2d(&p.tmMid, a2 + 16384, F + cur.c * 64, m0);                              // d_up   -> d_h1
        }
        tma_store_commit();
      }
      if (cur.c != NC - 1) continue;
      // ---------------- tile epilogue: the second GEMM's accumulator -> bf16 -> [P, L] ----------------
      if (chunk_issuer) CHAIN_TRACE(2, 20);
      if (!mbar_wait(acc2_full, tiles_done & 1, abort_flag, p.status, kStatusEpilogueTimeout)) ok = false;
      if (chunk_issuer) CHAIN_TRACE(2, 21);
      tc_fence_after();
      ok = epi_all_and(ok);
      if (!ok) break;
      const int slabs = L / kSlabCols;
      const int last = ((slabs - 1 - group) >= 0) ? group + ((slabs - 1 - group) & ~1) : -1;
      if (last < 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc2_empty);
      }
#pragma unroll 1
      for (int c = group; c < slabs; c += 2) {
        float v[32];
        tmem_ld32(lane_addr + ACC2_COL + c * 32, v);
        tmem_ld_wait();
        if (c == last) {  // this warp's last slab is in registers: hand the accumulator back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc2_empty);
        }
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
    if (group_issuer) tma_store_wait0();  // shared memory must outlive the last reads
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
