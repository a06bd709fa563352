// Host launcher of the routed expert chain kernel (chain.cuh): tensor maps, grid sizing, the on/off switch.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "../../include/lmoe.h"
#include "chain_pair.cuh"
#include "counters.h"
#include "device_once.h"
#include "gemm_host.h"

namespace lmoe {

static int g_chain = -1;  // -1: not yet read from the environment (LMOE_CHAIN=1 switches the kernel on)
static bool chain_enabled() {
  if (g_chain < 0) {
    const char* e = getenv("LMOE_CHAIN");
    g_chain = (e && e[0] == '1') ? 1 : 0;
  }
  return g_chain == 1;
}

bool chain_applies(int L, int F) {
  return chain_enabled() && L >= 64 && L <= kChainMaxL && (L % 64) == 0 && F >= 64 && (F % 64) == 0;
}

// Tiles of the same expert on CTA pairs (chain_pair.cuh); LMOE_CHAIN_PAIR=0 keeps one CTA per tile.
static bool chain_pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LMOE_CHAIN_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int MODE>
static int launch_chain_pair_inst(const ChainPairParams& p, int total_tiles, cudaStream_t stream) {
  auto kfn = chain_pair_kernel<MODE>;
  constexpr int smem = ChainPairSmem<MODE>::kTotal;
  static PerDeviceOnce once;
  static int max_pairs_dev[kMaxDevices] = {};
  const int dev = current_device();
  if (int rc = once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        cudaFuncSetAttribute(kfn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (num_sms() / 2), 1, 1);
        cfg.blockDim = dim3(kChainPairThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kfn, &cfg) != cudaSuccess || n <= 0) {
          cudaGetLastError();
          n = num_sms() / 2;
        }
        max_pairs_dev[dev] = n;
        return 0;
      }))
    return rc;
  // at most one pair slot per two tiles plus one per expert (odd runs); never more clusters than the device holds
  long long want = (static_cast<long long>(total_tiles) + 1) / 2 + p.E;
  if (want > max_pairs_dev[dev]) want = max_pairs_dev[dev];
  if (want < 1) want = 1;
  kfn<<<2 * static_cast<int>(want), kChainPairThreads, smem, stream>>>(p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

template <int MODE>
static int launch_chain_inst(const ChainParams& p, int grid, cudaStream_t stream) {
  auto kfn = chain_kernel<MODE>;
  constexpr int smem = ChainSmem<MODE>::kTotal;
  static PerDeviceOnce once;
  if (int rc = once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        cudaFuncSetAttribute(kfn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        return 0;
      }))
    return rc;
  kfn<<<grid, kGemmThreads, smem, stream>>>(p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

static int launch_chain_pair(int mode, long long P, int E, int L, int F, const void* a, const void* w_gate_up,
                             const void* w_down, const int* pad_offsets, void* h1, void* mid, void* out, int* status,
                             cudaStream_t stream) {
  ChainPairParams p;
  memset(&p, 0, sizeof(p));
  int rc = encode_2d(&p.tmA, a, L, P, L, kBM, 2);
  if (rc) return rc;
  const long long wgu_rows = static_cast<long long>(E) * L, wd_rows = static_cast<long long>(E) * F;
  if (mode == CHAIN_FWD) {
    if ((rc = encode_2d(&p.tmB1, w_gate_up, 2ll * F, wgu_rows, 2ll * F, 64, 2))) return rc;
    if ((rc = encode_2d(&p.tmB2, w_down, L, wd_rows, L, 64, 2))) return rc;
    if ((rc = encode_2d(&p.tmMid, mid, F, P, F, kBM, 2))) return rc;
  } else {
    if ((rc = encode_2d(&p.tmB1, w_down, L, wd_rows, L, 32, 2))) return rc;               // 32 of the chunk's 64 rows
    if ((rc = encode_2d(&p.tmB2, w_gate_up, 2ll * F, wgu_rows, 2ll * F, 64, 2))) return rc;     // 64 of d_x's columns
    if ((rc = encode_2d(&p.tmMid, mid, 2ll * F, P, 2ll * F, kBM, 2))) return rc;
  }
  if ((rc = encode_out(&p.tmAux, h1, false, 2ll * F, P, 1, 2ll * F, 0, mode == CHAIN_BWD))) return rc;
  if ((rc = encode_out(&p.tmOut, out, false, L, P, 1, L, 0))) return rc;
  p.L = L;
  p.F = F;
  p.E = E;
  p.max_tiles = static_cast<int>(P / kBM);
  {
    const char* e = getenv("LMOE_CHAIN_PREFETCH");
    p.prefetch_a = (e && e[0] == '0') ? 0 : 1;
  }
  p.pad_offsets = pad_offsets;
  p.status = status;
  return mode == CHAIN_FWD ? launch_chain_pair_inst<CHAIN_FWD>(p, p.max_tiles, stream)
                           : launch_chain_pair_inst<CHAIN_BWD>(p, p.max_tiles, stream);
}

int launch_chain(int mode, long long P, int E, int L, int F, const void* a, const void* w_gate_up, const void* w_down,
                 const int* tile_expert, const int* n_tiles, const int* pad_offsets, void* h1, void* mid, void* out,
                 int* status, cudaStream_t stream) {
  if (!a || !w_gate_up || !w_down || !tile_expert || !n_tiles || !h1 || !mid || !out) return LMOE_ERR_ARG;
  if (P <= 0 || (P % kBM) != 0 || E <= 0 || !chain_applies(L, F)) return LMOE_ERR_SHAPE;
  if (pad_offsets && chain_pair_enabled() && (L % 128) == 0 && (F % 128) == 0 && E <= LMOE_MAX_EXPERTS && P / kBM < (1 << 23))
    return launch_chain_pair(mode, P, E, L, F, a, w_gate_up, w_down, pad_offsets, h1, mid, out, status, stream);
  ChainParams p;
  memset(&p, 0, sizeof(p));
  int rc = encode_2d(&p.tmA, a, L, P, L, kBM, 2);
  if (rc) return rc;
  const long long wgu_rows = static_cast<long long>(E) * L, wd_rows = static_cast<long long>(E) * F;
  if (mode == CHAIN_FWD) {
    if ((rc = encode_2d(&p.tmB1, w_gate_up, 2ll * F, wgu_rows, 2ll * F, 64, 2))) return rc;
    if ((rc = encode_2d(&p.tmB2, w_down, L, wd_rows, L, 64, 2))) return rc;
    if ((rc = encode_2d(&p.tmMid, mid, F, P, F, kBM, 2))) return rc;            // hidden [P, F]
  } else {
    if ((rc = encode_2d(&p.tmB1, w_down, L, wd_rows, L, 64, 2))) return rc;
    if ((rc = encode_2d(&p.tmB2, w_gate_up, 2ll * F, wgu_rows, 2ll * F, L < 128 ? L : 128, 2))) return rc;
    if ((rc = encode_2d(&p.tmMid, mid, 2ll * F, P, 2ll * F, kBM, 2))) return rc;  // d_h1 [P, 2F]
  }
  if ((rc = encode_out(&p.tmAux, h1, false, 2ll * F, P, 1, 2ll * F, 0, mode == CHAIN_BWD))) return rc;
  if ((rc = encode_out(&p.tmOut, out, false, L, P, 1, L, 0))) return rc;
  p.L = L;
  p.F = F;
  p.max_tiles = static_cast<int>(P / kBM);
  {
    const char* e = getenv("LMOE_CHAIN_PREFETCH");
    p.prefetch_a = (e && e[0] == '0') ? 0 : 1;
    const char* c = getenv("LMOE_CHAIN_CONTIG");
    p.contiguous = (c && c[0] == '1') ? 1 : 0;
  }
  p.tile_expert = tile_expert;
  p.n_tiles = n_tiles;
  p.status = status;
  const int sms = num_sms();
  const int grid = p.max_tiles < sms ? p.max_tiles : sms;
  return mode == CHAIN_FWD ? launch_chain_inst<CHAIN_FWD>(p, grid, stream) : launch_chain_inst<CHAIN_BWD>(p, grid, stream);
}

}  // namespace lmoe

extern "C" int lmoe_chain_enable(int on) {
  const int before = lmoe::chain_enabled() ? 1 : 0;
  lmoe::g_chain = on ? 1 : 0;
  return before;
}

extern "C" int lmoe_chain_applies(int L, int F) { return lmoe::chain_applies(L, F) ? 1 : 0; }

#ifdef LMOE_CHAIN_TRACE
// Development aid: copies CTA 0's event trace of the last chain launch to the host and clears it.
extern "C" int lmoe_chain_trace_read(long long* host, int* counts) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host, lmoe::g_chain_trace, sizeof(long long) * lmoe::kTraceRoles * lmoe::kTraceSlots * 2);
  cudaMemcpyFromSymbol(counts, lmoe::g_chain_trace_n, sizeof(int) * lmoe::kTraceRoles);
  int zero[lmoe::kTraceRoles] = {};
  cudaMemcpyToSymbol(lmoe::g_chain_trace_n, zero, sizeof(zero));
  return 0;
}
#endif
