// Host launcher of the tcgen05 GEMM: tensor-map encoding, template dispatch, grid sizing.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/lmoe.h"
#include "counters.h"
#include "device_once.h"
#include "gemm.cuh"
#include "gemm_pair.cuh"
#include "gemm_host.h"

namespace lmoe {

std::atomic<long long> g_launch_count{0};

// ---------------------------------------------------------------- driver entry point
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int num_sms() {
  static PerDeviceOnce once;
  static int n[kMaxDevices] = {};
  const int dev = current_device();
  once.run([&] {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
    return 0;
  });
  return n[dev];
}

// Operand map: 2-D over a row-major [outer, inner] tensor of 16-bit (esz 2) or 8-bit (esz 1) elements,
// 128-byte swizzle; the inner box extent is always 128 bytes.
int encode_2d(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld_elems,
                     int box_outer, int esz) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return LMOE_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld_elems * esz) & 15) != 0) return LMOE_ERR_ALIGN;
  if (inner <= 0 || outer <= 0 || box_outer > 256) return LMOE_ERR_SHAPE;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * esz};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esz), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : LMOE_ERR_DRIVER;
}

// Output map: 3-D {cols, rows, planes}; one 128 x 32 slab per store.  bf16: 64-byte rows in shared
// memory (SWIZZLE_64B); fp32: 128-byte rows (SWIZZLE_128B).
int encode_out(CUtensorMap* map, void* base, bool f32, long long cols, long long rows, long long planes,
               long long ld_elems, long long plane_elems, bool as_source) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return LMOE_ERR_DRIVER;
  const int es = f32 ? 4 : 2;
  if (planes <= 1) {
    planes = 1;
    plane_elems = rows * ld_elems;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld_elems * es) & 15) != 0 || ((plane_elems * es) & 15) != 0)
    return LMOE_ERR_ALIGN;
  if (cols <= 0 || rows <= 0) return LMOE_ERR_SHAPE;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld_elems) * es, static_cast<cuuint64_t>(plane_elems) * es};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kSlabCols), static_cast<cuuint32_t>(kBM), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  // a slab row is 64 bytes: as a load source, let L2 fetch whole 256-byte pieces from HBM once, so that the
                  // neighbouring slabs (read by the other epilogue group a moment later) hit L2
                  as_source ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : LMOE_ERR_DRIVER;
}

// ---------------------------------------------------------------- optional per-launch timing of the GEMM kernel
// When enabled, every GEMM launch is bracketed by CUDA events on its own stream; lmoe_profile_collect synchronises
// and returns the summed duration.  Used by the benchmark to report the tensor-core kernel's own throughput.
static std::mutex g_prof_mutex;
static bool g_prof_enabled = false;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_prof_events;

// ---------------------------------------------------------------- dispatch
template <bool A_MN, bool B_MN, int BN, int EPI, int GRP, int ESZ>
static int launch_inst(const GemmParams& p, int grid, cudaStream_t stream) {
  auto kfn = gemm_kernel<A_MN, B_MN, BN, EPI, GRP, ESZ>;
  constexpr int smem = GemmSmem<BN, EPI, GRP>::kTotal;
  static PerDeviceOnce once;  // one per template instantiation
  if (int rc = once.run([&] {
        cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        // ask for the largest shared-memory carveout so that what the GEMM leaves unused stays available to small
        // kernels of other streams running beside it
        cudaFuncSetAttribute(kfn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        return 0;
      }))
    return rc;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  if (g_prof_enabled) {
    cudaEventCreate(&ev0);
    cudaEventCreate(&ev1);
    cudaEventRecord(ev0, stream);
  }
  kfn<<<grid, kGemmThreads, smem, stream>>>(p);
  if (ev0) {
    cudaEventRecord(ev1, stream);
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_events.emplace_back(ev0, ev1);
  }
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

#define LMOE_KEY(am, bm, bn256, epi, grp, esz) \
  ((am) | ((bm) << 1) | ((bn256) << 2) | ((epi) << 3) | ((grp) << 6) | (((esz) == 1 ? 1 : 0) << 9))
#define LMOE_CASE(am, bm, bn, epi, grp, esz)          \
  case LMOE_KEY(am, bm, (bn == 256), epi, grp, esz):  \
    return launch_inst<(am != 0), (bm != 0), bn, epi, grp, esz>(p, grid, stream);
#define LMOE_CASE_BN(am, bm, epi, grp, esz) LMOE_CASE(am, bm, 128, epi, grp, esz) LMOE_CASE(am, bm, 256, epi, grp, esz)
#define LMOE_CASE_MAJORS(epi, grp, esz)                                                                      \
  LMOE_CASE_BN(0, 0, epi, grp, esz) LMOE_CASE_BN(0, 1, epi, grp, esz) LMOE_CASE_BN(1, 0, epi, grp, esz) \
      LMOE_CASE_BN(1, 1, epi, grp, esz)

static int dispatch(const GemmCall& c, int bn, const GemmParams& p, int grid, cudaStream_t stream) {
  switch (LMOE_KEY(c.a_mn, c.b_mn, (bn == 256), c.epi, c.grp, c.esz)) {
    // ---- bf16 ----
    // dense
    LMOE_CASE_MAJORS(EPI_BF16, GRP_NONE, 2)
    LMOE_CASE_MAJORS(EPI_F32, GRP_NONE, 2)
    LMOE_CASE_BN(0, 0, EPI_SWIGLU, GRP_NONE, 2)
    // grouped over rows (routed forward and dgrads)
    LMOE_CASE_BN(0, 1, EPI_SWIGLU, GRP_M, 2)
    LMOE_CASE_BN(0, 1, EPI_BF16, GRP_M, 2)
    LMOE_CASE_BN(0, 0, EPI_BF16, GRP_M, 2)
    // grouped over the contraction (routed wgrads)
    LMOE_CASE_BN(1, 1, EPI_BF16, GRP_K, 2)
    // dgrad with the SwiGLU adjoint in the epilogue (routed and shared)
    LMOE_CASE(0, 0, 128, EPI_SWIGLU_BWD, GRP_M, 2)
    LMOE_CASE(0, 1, 128, EPI_SWIGLU_BWD, GRP_NONE, 2)
    // ---- e4m3 ----
    LMOE_CASE_MAJORS(EPI_BF16, GRP_NONE, 1)
    LMOE_CASE(0, 1, 256, EPI_SWIGLU, GRP_M, 1)
    LMOE_CASE_BN(0, 1, EPI_BF16, GRP_M, 1)
    LMOE_CASE_BN(0, 0, EPI_BF16, GRP_M, 1)
    LMOE_CASE_BN(1, 1, EPI_BF16, GRP_K, 1)
    default:
      return LMOE_ERR_ARG;
  }
}

// ---------------------------------------------------------------- CTA-pair kernel (dense GEMMs)
// Dense bf16 GEMMs with at least 256 rows and 256 columns run on CTA pairs (gemm_pair.cuh) unless LMOE_PAIR_GEMM=0.
static int g_pair_gemm = -1;  // -1: not yet read from the environment
static bool pair_gemm_enabled() {
  if (g_pair_gemm < 0) {
    const char* e = getenv("LMOE_PAIR_GEMM");
    g_pair_gemm = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pair_gemm == 1;
}

bool pair_gemm_applies(int M, int N) { return pair_gemm_enabled() && M >= 256 && N >= 256; }

template <bool A_MN, bool B_MN, int EPI, int GRP = GRP_NONE>
static int launch_pair_inst(const GemmParams& p, long long total_tiles, cudaStream_t stream) {
  auto kfn = gemm_pair_kernel<A_MN, B_MN, EPI, GRP>;
  constexpr int smem = PairSmem<EPI>::kTotal;
  static PerDeviceOnce once;  // one per template instantiation
  static int max_pairs_dev[kMaxDevices] = {};
  const int dev = current_device();
  if (int rc = once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaFuncSetAttribute(kfn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    // how many pairs the device holds at once (SM pairs must share a cluster-capable group)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (num_sms() / 2), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
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
  const int max_pairs = max_pairs_dev[dev];
  const int pairs = static_cast<int>(total_tiles < max_pairs ? total_tiles : max_pairs);
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  if (g_prof_enabled) {
    cudaEventCreate(&ev0);
    cudaEventCreate(&ev1);
    cudaEventRecord(ev0, stream);
  }
  kfn<<<2 * pairs, kGemmThreads, smem, stream>>>(p);
  if (ev0) {
    cudaEventRecord(ev1, stream);
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_events.emplace_back(ev0, ev1);
  }
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Same contract as launch_gemm for a dense bf16 GEMM (GRP_NONE; EPI_BF16, EPI_F32 with optional split-K, EPI_SWIGLU).
static int launch_gemm_pair(const GemmCall& c) {
  const bool swiglu = (c.epi == EPI_SWIGLU);
  const int bk = kBKBytes / 2;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int m_tiles = (c.M + 255) / 256;
  const int split = c.split_k > 1 ? c.split_k : 1;
  const int n_per_tile = swiglu ? 128 : 256;
  const int n_tiles = (c.N + n_per_tile - 1) / n_per_tile;
  for (int s = 0; s < c.nseg; ++s) {
    if (!c.A[s] || !c.B[s]) return LMOE_ERR_ARG;
    const int K = c.Kseg[s];
    if (K <= 0) return LMOE_ERR_SHAPE;
    p.seg_kiters[s] = (K + bk - 1) / bk;
    int rc = !c.a_mn ? encode_2d(&p.tmA[s], c.A[s], K, c.M, c.lda[s], kBM, 2)
                     : encode_2d(&p.tmA[s], c.A[s], c.M, K, c.lda[s], bk, 2);
    if (rc) return rc;
    const int n_b_total = swiglu ? 2 * c.N : c.N;
    rc = !c.b_mn ? encode_2d(&p.tmB[s], c.B[s], K, n_b_total, c.ldb[s], 128, 2)   // this CTA's half: 128 rows of B
                 : encode_2d(&p.tmB[s], c.B[s], n_b_total, K, c.ldb[s], bk, 2);
    if (rc) return rc;
  }
  {
    const bool f32 = (c.epi == EPI_F32);
    const long long cols = swiglu ? 2ll * c.N : c.N;
    long long planes = 1, plane_elems = 0;
    if (split > 1) {
      planes = split;
      plane_elems = c.c_group_stride;
      if (plane_elems < static_cast<long long>(c.M) * c.ldc) return LMOE_ERR_ARG;
    }
    int rc = encode_out(&p.tmC, c.C, f32, cols, c.M, planes, c.ldc, plane_elems);
    if (rc) return rc;
    if (swiglu) {
      rc = encode_out(&p.tmC2, c.C2, false, c.N, c.M, 1, c.ldc2, 0);
      if (rc) return rc;
    }
  }
  p.nseg = c.nseg;
  p.M = c.M;
  p.N = c.N;
  p.m_tiles = m_tiles;
  p.n_tiles = n_tiles;
  p.split_k = split;
  p.half = c.N;
  p.status = c.status;
  const long long total = static_cast<long long>(m_tiles) * n_tiles * split;
  const int key = c.a_mn | (c.b_mn << 1) | (c.epi << 2);
  switch (key) {
    case 0 | (EPI_BF16 << 2): return launch_pair_inst<false, false, EPI_BF16>(p, total, c.stream);
    case 1 | (EPI_BF16 << 2): return launch_pair_inst<true, false, EPI_BF16>(p, total, c.stream);
    case 2 | (EPI_BF16 << 2): return launch_pair_inst<false, true, EPI_BF16>(p, total, c.stream);
    case 3 | (EPI_BF16 << 2): return launch_pair_inst<true, true, EPI_BF16>(p, total, c.stream);
    case 0 | (EPI_F32 << 2): return launch_pair_inst<false, false, EPI_F32>(p, total, c.stream);
    case 1 | (EPI_F32 << 2): return launch_pair_inst<true, false, EPI_F32>(p, total, c.stream);
    case 2 | (EPI_F32 << 2): return launch_pair_inst<false, true, EPI_F32>(p, total, c.stream);
    case 3 | (EPI_F32 << 2): return launch_pair_inst<true, true, EPI_F32>(p, total, c.stream);
    case 0 | (EPI_SWIGLU << 2): return launch_pair_inst<false, false, EPI_SWIGLU>(p, total, c.stream);
    default: return LMOE_ERR_ARG;
  }
}

// Grouped-over-rows GEMM on CTA pairs: two tiles of the same expert share the expert's B loads (gemm_pair.cuh, GRP_M).
// Needs the per-expert padded offsets; K-major A, one K segment, plain bf16 or SwiGLU epilogue.
// Off unless the environment has LMOE_PAIR_GROUPED=1 (2: only the SwiGLU GEMM, 3: only the plain ones): with the
// 256-element contractions of the routed experts a tile's main loop is four k-blocks long, an expert with an odd tile
// count wastes half a pair and the last round of pairs is mostly empty (measured at E = 128, L = F = 256, 1,594 tiles:
// gate_up + down 140 us on pairs against 134 us with one CTA per tile).
static int pair_grouped_mode() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LMOE_PAIR_GROUPED");
    v = (e && e[0] >= '1' && e[0] <= '3') ? e[0] - '0' : 0;
  }
  return v;
}
static bool pair_grouped_applies(const GemmCall& c) {
  const bool swiglu = (c.epi == EPI_SWIGLU);
  const int mode = pair_grouped_mode();
  if (mode == 0 || (mode == 2 && !swiglu) || (mode == 3 && swiglu)) return false;
  return c.grp == GRP_M && c.pad_offsets && pair_gemm_enabled() && c.esz == 2 && !c.a_rows && !c.a_mn && c.nseg == 1 &&
         c.bn == 0 && (c.epi == EPI_BF16 || (swiglu && c.b_mn)) && c.groups > 0 && c.groups <= LMOE_MAX_EXPERTS &&
         c.padded_rows / kBM < (1 << 23) && (c.N % (swiglu ? 128 : 32)) == 0 && (c.Kseg[0] % 64) == 0;
}

static int launch_gemm_pair_grouped(const GemmCall& c) {
  const bool swiglu = (c.epi == EPI_SWIGLU);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int K = c.Kseg[0];
  const int n_per_tile = swiglu ? 128 : 256;
  const int n_tiles = (c.N + n_per_tile - 1) / n_per_tile;
  const int n_b_total = swiglu ? 2 * c.N : c.N;
  const long long b_outer = static_cast<long long>(c.groups) * c.b_group_rows;
  p.seg_kiters[0] = K / 64;
  int rc = encode_2d(&p.tmA[0], c.A[0], K, c.padded_rows, c.lda[0], kBM, 2);
  if (rc) return rc;
  rc = !c.b_mn ? encode_2d(&p.tmB[0], c.B[0], K, b_outer, c.ldb[0], 128, 2)       // this CTA's 128 rows of B[e]
               : encode_2d(&p.tmB[0], c.B[0], n_b_total, b_outer, c.ldb[0], 64, 2);
  if (rc) return rc;
  rc = encode_out(&p.tmC, c.C, false, swiglu ? 2ll * c.N : c.N, c.padded_rows, 1, c.ldc, 0);
  if (rc) return rc;
  if (swiglu) {
    rc = encode_out(&p.tmC2, c.C2, false, c.N, c.padded_rows, 1, c.ldc2, 0);
    if (rc) return rc;
  }
  p.nseg = 1;
  p.M = static_cast<int>(c.padded_rows);
  p.N = c.N;
  p.m_tiles = static_cast<int>(c.padded_rows / kBM);
  p.n_tiles = n_tiles;
  p.groups = c.groups;
  p.split_k = 1;
  p.half = c.N;
  p.b_group_rows = c.b_group_rows;
  p.pad_offsets = c.pad_offsets;
  p.status = c.status;
  // pairs are counted on the device; at most one per two tiles plus one per expert
  const long long total = (static_cast<long long>(p.m_tiles + 1) / 2 + c.groups) * n_tiles;
  if (swiglu) return launch_pair_inst<false, true, EPI_SWIGLU, GRP_M>(p, total, c.stream);
  if (c.b_mn) return launch_pair_inst<false, true, EPI_BF16, GRP_M>(p, total, c.stream);
  return launch_pair_inst<false, false, EPI_BF16, GRP_M>(p, total, c.stream);
}

int launch_gemm(const GemmCall& c) {
  if (c.nseg < 1 || c.nseg > 3 || !c.C || c.M <= 0 || c.N <= 0) return LMOE_ERR_ARG;
  if (c.split_k > 1 && (c.epi != EPI_F32 || c.nseg != 1 || c.grp != GRP_NONE)) return LMOE_ERR_ARG;
  const bool swiglu = (c.epi == EPI_SWIGLU);
  if (c.esz != 1 && c.esz != 2) return LMOE_ERR_ARG;
  const int esz = c.esz;
  const int bk = kBKBytes / esz;  // elements per k-block
  const int ch = 128 / esz;       // MN-major chunk width in elements
  if ((c.N & 7) != 0) return LMOE_ERR_SHAPE;
  if (swiglu && ((c.N % kSlabCols) != 0 || !c.C2)) return LMOE_ERR_SHAPE;
  const bool swiglu_bwd = (c.epi == EPI_SWIGLU_BWD);
  if (swiglu_bwd && ((c.N % kSlabCols) != 0 || !c.aux || (reinterpret_cast<uintptr_t>(c.aux) & 15) != 0 ||
                     ((c.ld_aux * 2) & 15) != 0))
    return LMOE_ERR_SHAPE;

  const bool gather = c.a_rows != nullptr;
  if (pair_grouped_applies(c)) return launch_gemm_pair_grouped(c);
  if (c.grp == GRP_NONE && esz == 2 && !gather && c.bn != 128 && pair_gemm_applies(c.M, swiglu ? 2 * c.N : c.N) &&
      (c.epi == EPI_BF16 || c.epi == EPI_F32 || (swiglu && !c.a_mn && !c.b_mn)))
    return launch_gemm_pair(c);
  if (gather) {
    const bool shape_ok = (c.grp == GRP_M && !c.a_mn) || (c.grp == GRP_K && c.a_mn);
    if (!shape_ok || esz != 2 || c.nseg != 1 || c.a_src_rows <= 0 || c.a_rows_stride <= 0 || c.a_rows_div <= 0 || c.a_zero_row < 0 ||
        c.a_zero_row >= c.a_src_rows)
      return LMOE_ERR_ARG;
  }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  // ---- tile geometry ----
  const int sms = num_sms();
  const long long rows_total = (c.grp == GRP_M) ? c.padded_rows : c.M;
  const int m_tiles = static_cast<int>((rows_total + kBM - 1) / kBM);
  const int split = c.split_k > 1 ? c.split_k : 1;
  int bn = c.bn;
  if (bn == 0) {
    // N per tile: BN for plain epilogues, BN/2 output columns for SwiGLU (gate + up accumulators)
    const int n_eff = swiglu ? 2 * c.N : c.N;
    const long long tiles256 =
        static_cast<long long>(m_tiles) * ((n_eff + 255) / 256) * (c.grp == GRP_K ? c.groups : 1) * split;
    bn = (n_eff >= 256 && tiles256 >= sms) ? 256 : 128;
    if (esz == 1 && swiglu && c.b_mn) bn = 256;  // gate and up halves must each be a whole 128-wide chunk
    // per-expert weight gradients contract over thousands of rows: wide tiles even when they do not fill a wave
    // (128-wide tiles measured 2.5x slower for 32 experts per GPU)
    if (c.grp == GRP_K && n_eff >= 256) bn = 256;
    if (swiglu_bwd) bn = 128;  // the staged gate / up slabs take 64 KB of shared memory: 32 KB stages
  }
  if (bn != 128 && bn != 256) return LMOE_ERR_ARG;
  const int n_per_tile = swiglu ? bn / 2 : bn;
  const int n_tiles = (c.N + n_per_tile - 1) / n_per_tile;

  // ---- operand maps ----
  for (int s = 0; s < c.nseg; ++s) {
    if (!c.A[s] || !c.B[s]) return LMOE_ERR_ARG;
    int rc;
    if (c.grp == GRP_K) {
      // both operands are [padded rows, extent] row-major and contract over rows
      if (!c.a_mn || !c.b_mn) return LMOE_ERR_ARG;
      if (gather)  // box of one row: the kernel gathers the contraction rows four at a time
        rc = encode_2d(&p.tmA[s], c.A[s], c.M, c.a_src_rows, c.lda[s], 1, esz);
      else
        rc = encode_2d(&p.tmA[s], c.A[s], c.M, c.padded_rows, c.lda[s], bk, esz);
      if (rc) return rc;
      rc = encode_2d(&p.tmB[s], c.B[s], c.N, c.padded_rows, c.ldb[s], bk, esz);
      if (rc) return rc;
      p.seg_kiters[s] = 0;
      continue;
    }
    const int K = c.Kseg[s];
    if (K <= 0) return LMOE_ERR_SHAPE;
    p.seg_kiters[s] = (K + bk - 1) / bk;
    // A
    if (gather)
      rc = encode_2d(&p.tmA[s], c.A[s], K, c.a_src_rows, c.lda[s], 1, esz);
    else if (!c.a_mn)
      rc = encode_2d(&p.tmA[s], c.A[s], K, rows_total, c.lda[s], kBM, esz);
    else
      rc = encode_2d(&p.tmA[s], c.A[s], c.M, K, c.lda[s], bk, esz);
    if (rc) return rc;
    // B
    const int n_b_total = swiglu ? 2 * c.N : c.N;  // columns (or rows) of B addressed by this GEMM
    if (c.grp == GRP_M) {
      if ((K % bk) != 0 || c.groups <= 0 || c.b_group_rows <= 0) return LMOE_ERR_SHAPE;
      const long long outer = static_cast<long long>(c.groups) * c.b_group_rows;
      if (!c.b_mn)
        rc = encode_2d(&p.tmB[s], c.B[s], K, outer, c.ldb[s], swiglu ? bn / 2 : bn, esz);
      else
        rc = encode_2d(&p.tmB[s], c.B[s], n_b_total, outer, c.ldb[s], bk, esz);
    } else {
      if (!c.b_mn)
        rc = encode_2d(&p.tmB[s], c.B[s], K, n_b_total, c.ldb[s], swiglu ? bn / 2 : bn, esz);
      else
        rc = encode_2d(&p.tmB[s], c.B[s], n_b_total, K, c.ldb[s], bk, esz);
    }
    if (rc) return rc;
  }

  // ---- output maps ----
  {
    const bool f32 = (c.epi == EPI_F32);
    const long long cols = (swiglu || swiglu_bwd) ? 2ll * c.N : c.N;
    long long planes = 1, plane_elems = 0;
    if (c.grp == GRP_K) {
      planes = c.groups;
      plane_elems = c.c_group_stride;
    } else if (split > 1) {
      planes = split;
      plane_elems = c.c_group_stride;
      if (plane_elems < static_cast<long long>(c.M) * c.ldc) return LMOE_ERR_ARG;
    }
    int rc = encode_out(&p.tmC, c.C, f32, cols, rows_total, planes, c.ldc, plane_elems);
    if (rc) return rc;
    if (swiglu) {
      rc = encode_out(&p.tmC2, c.C2, false, c.N, rows_total, 1, c.ldc2, 0);
      if (rc) return rc;
    }
    if (swiglu_bwd) {  // the saved gate / up as a source of 128-row x 64-column boxes; rows past the end read as zeros
      rc = encode_2d(&p.tmAux, c.aux, 2ll * c.N, rows_total, c.ld_aux, kBM, 2);
      if (rc) return rc;
    }
  }

  p.nseg = c.nseg;
  p.M = c.M;
  p.N = c.N;
  p.m_tiles = m_tiles;
  p.n_tiles = n_tiles;
  p.groups = c.groups;
  p.split_k = split;
  p.half = c.N;
  p.tile_expert = c.tile_expert;
  p.n_m_tiles = c.n_m_tiles;
  p.b_group_rows = c.b_group_rows;
  p.pad_offsets = c.pad_offsets;
  p.deq_a = c.deq_a;
  p.deq_b = c.deq_b;
  p.aux = c.aux;
  p.ld_aux = c.ld_aux;
  p.a_rows = c.a_rows;
  p.a_rows_stride = c.a_rows_stride;
  p.a_rows_div = c.a_rows_div;
  p.a_zero_row = c.a_zero_row;
  p.status = c.status;
  (void)ch;
  if (c.grp == GRP_M && (!c.tile_expert || !c.n_m_tiles)) return LMOE_ERR_ARG;
  if (c.grp == GRP_K && (!c.pad_offsets || c.groups <= 0)) return LMOE_ERR_ARG;

  long long total = static_cast<long long>(m_tiles) * n_tiles;
  if (c.grp == GRP_NONE) total *= split;
  if (c.grp == GRP_K) total *= c.groups;
  const int grid = static_cast<int>(total < sms ? total : sms);
  return dispatch(c, bn, p, grid, c.stream);
}

// ---------------------------------------------------------------- split-K reduction
// out[r, c] = sum_s ws[s, r, c] for a row range of the workspace, written as fp32 or bf16 with its own
// leading dimension.  Fixed summation order: deterministic.
// Up to three row/column ranges of the workspace per launch, each with its own output: the ranges of one weight-gradient
// GEMM are reduced by one kernel.
struct SplitKRange {
  int row0, col0, rows, cols;
  void* out;
  long long out_ld;
  long long vec_begin;  // first float4 of this range in the launch's linear index space
};
struct SplitKRanges {
  SplitKRange r[3];
  int n;
  long long total;
};

__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int planes, long long plane_elems, int ws_ld, const SplitKRanges rg,
                     int out_f32) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < rg.total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    int k = 0;
    if (rg.n > 1 && i >= rg.r[1].vec_begin) k = 1;
    if (rg.n > 2 && i >= rg.r[2].vec_begin) k = 2;
    const SplitKRange& q = rg.r[k];
    const long long li = i - q.vec_begin;
    const int vec_per_row = q.cols / 4;
    const int r = static_cast<int>(li / vec_per_row);
    const int c = static_cast<int>(li - static_cast<long long>(r) * vec_per_row) * 4;
    const float* src = ws + static_cast<long long>(q.row0 + r) * ws_ld + q.col0 + c;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < planes; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * plane_elems);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    if (out_f32) {
      *reinterpret_cast<float4*>(static_cast<float*>(q.out) + r * q.out_ld + c) = acc;
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(q.out) + r * q.out_ld + c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    }
  }
}

int splitk_reduce_multi(const float* ws, int planes, long long plane_elems, int ws_ld, int n_ranges, const int* row0,
                        const int* col0, const int* rows, const int* cols, void* const* out, const long long* out_ld,
                        int out_f32, cudaStream_t stream) {
  if (n_ranges < 1 || n_ranges > 3 || (ws_ld & 3) != 0) return LMOE_ERR_SHAPE;
  SplitKRanges rg;
  memset(&rg, 0, sizeof(rg));
  rg.n = n_ranges;
  long long total = 0;
  for (int k = 0; k < n_ranges; ++k) {
    if ((cols[k] & 3) != 0 || (col0[k] & 3) != 0 || (out_ld[k] & 3) != 0 || rows[k] <= 0 || cols[k] <= 0) return LMOE_ERR_SHAPE;
    rg.r[k].row0 = row0[k];
    rg.r[k].col0 = col0[k];
    rg.r[k].rows = rows[k];
    rg.r[k].cols = cols[k];
    rg.r[k].out = out[k];
    rg.r[k].out_ld = out_ld[k];
    rg.r[k].vec_begin = total;
    total += static_cast<long long>(rows[k]) * (cols[k] / 4);
  }
  rg.total = total;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(ws, planes, plane_elems, ws_ld, rg, out_f32);
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int splitk_reduce(const float* ws, int planes, long long plane_elems, int ws_ld, int row0, int col0, int rows, int cols,
                  void* out, long long out_ld, int out_f32, cudaStream_t stream) {
  return splitk_reduce_multi(ws, planes, plane_elems, ws_ld, 1, &row0, &col0, &rows, &cols, &out, &out_ld, out_f32, stream);
}

}  // namespace lmoe

// ---------------------------------------------------------------- C ABI
extern "C" int lmoe_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(lmoe::g_prof_mutex);
  lmoe::g_prof_enabled = (on != 0);
  return 0;
}

extern "C" int lmoe_profile_collect(float* gemm_ms, int* gemm_launches) {
  if (!gemm_ms || !gemm_launches) return LMOE_ERR_ARG;
  std::lock_guard<std::mutex> lock(lmoe::g_prof_mutex);
  float total = 0.f;
  for (auto& pr : lmoe::g_prof_events) {
    cudaEventSynchronize(pr.second);
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess) total += ms;
    cudaEventDestroy(pr.first);
    cudaEventDestroy(pr.second);
  }
  *gemm_ms = total;
  *gemm_launches = static_cast<int>(lmoe::g_prof_events.size());
  lmoe::g_prof_events.clear();
  return 0;
}

extern "C" size_t lmoe_gemm_workspace_bytes(int M, int N, int split_k) {
  if (split_k <= 1 || M <= 0 || N <= 0) return 0;
  return static_cast<size_t>(split_k) * M * N * sizeof(float);
}

extern "C" int lmoe_pair_gemm_enable(int on) {
  const int before = lmoe::pair_gemm_enabled() ? 1 : 0;
  lmoe::g_pair_gemm = on ? 1 : 0;
  return before;
}

extern "C" int lmoe_gemm_bf16(int M, int N, int K, const void* A, int64_t lda, int a_mn, const void* B, int64_t ldb,
                              int b_mn, void* C, int64_t ldc, int c_type, int split_k, void* workspace,
                              size_t workspace_bytes, int32_t* status, void* stream) {
  using namespace lmoe;
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return LMOE_ERR_ARG;
  if (c_type != LMOE_BF16 && c_type != LMOE_F32) return LMOE_ERR_ARG;
  GemmCall c;
  c.a_mn = a_mn ? 1 : 0;
  c.b_mn = b_mn ? 1 : 0;
  c.grp = GRP_NONE;
  c.A[0] = A;
  c.lda[0] = lda;
  c.B[0] = B;
  c.ldb[0] = ldb;
  c.Kseg[0] = K;
  c.M = M;
  c.N = N;
  c.status = status;
  c.stream = static_cast<cudaStream_t>(stream);
  if (split_k > 1) {
    if (!workspace || workspace_bytes < lmoe_gemm_workspace_bytes(M, N, split_k)) return LMOE_ERR_WORKSPACE;
    if ((N & 3) != 0) return LMOE_ERR_SHAPE;
    c.epi = EPI_F32;
    c.C = workspace;
    c.ldc = N;
    c.c_group_stride = static_cast<long long>(M) * N;
    c.split_k = split_k;
    if (int rc = launch_gemm(c)) return rc;
    return splitk_reduce(static_cast<const float*>(workspace), split_k, c.c_group_stride, N, 0, 0, M, N, C, ldc,
                         c_type == LMOE_F32, c.stream);
  }
  c.epi = (c_type == LMOE_F32) ? EPI_F32 : EPI_BF16;
  c.C = C;
  c.ldc = ldc;
  return launch_gemm(c);
}
