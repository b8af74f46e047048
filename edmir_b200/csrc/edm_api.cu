// C ABI over the fused tensor-parallel GEMM kernel: argument checks, tensor-map encoding,
// symmetric-memory contexts and launches.  No torch types, no allocation on the launch path.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/edm_b200.h"
#include "tp_gemm.cuh"

using namespace edm;

namespace {

thread_local int g_last_cuda_error = 0;
uint64_t g_timeout_ns = 2000ull * 1000ull * 1000ull;
int g_profile = 0;

// Tuning knobs for experiments, read from the environment once: EDM_STAGE_LIMIT (ring stages),
// EDM_BAND (row blocks per band of the tile walk), EDM_PUSH_STRIDE (every n-th CTA pushes all-gather
// shards with the sm transport), EDM_SIDE_STREAMS (copy-engine transport), EDM_CTA_GROUP (1 or 2),
// EDM_BLOCK_N (32 or 256: tile width of the single-CTA plain GEMM), EDM_TAIL_SPLIT (most pieces a
// tile of an incomplete last wave is cut into along K; 0 or 1: none).
struct Tuning {
  int stage_limit = 0, band = 0, push_stride = 1, side_streams = 2, cta_group = 0, block_n = 0, tail_split = kTailMaxParts;
  Tuning() {
    auto get = [](const char* name, int dflt) {
      const char* e = std::getenv(name);
      return e ? std::atoi(e) : dflt;
    };
    stage_limit = get("EDM_STAGE_LIMIT", 0);
    band = get("EDM_BAND", 0);
    push_stride = get("EDM_PUSH_STRIDE", 1);
    if (push_stride < 1) push_stride = 1;
    side_streams = get("EDM_SIDE_STREAMS", 2);
    cta_group = get("EDM_CTA_GROUP", 0);
    block_n = get("EDM_BLOCK_N", 0);
    tail_split = get("EDM_TAIL_SPLIT", kTailMaxParts);
  }
};
const Tuning& tuning() {
  static const Tuning t;
  return t;
}
bool capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  return cudaStreamIsCapturing(s, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone;
}
// Most pieces a tile may be cut into along K by a launch on `s`.  The pieces' flags carry a launch
// counter kept on the host; a replay of a captured launch would repeat its value and find the
// flags of the previous replay already raised, so captured launches do not split.
int max_tail_parts(cudaStream_t s) { return capturing(s) ? 0 : tuning().tail_split; }
void apply_tuning(LaunchParams& lp, cudaStream_t s) {
  lp.stage_limit = tuning().stage_limit;
  lp.band = tuning().band;
  lp.push_stride = tuning().push_stride;
  lp.tail_split = max_tail_parts(s);
  // flags of the split last wave carry a value no earlier launch of this process used
  static std::atomic<uint32_t> tail_epoch{0};
  lp.tail_epoch = tail_epoch.fetch_add(1u) + 1u;
}

#define EDM_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e__ = (expr);                            \
    if (e__ != cudaSuccess) {                            \
      g_last_cuda_error = static_cast<int>(e__);         \
      return EDM_ERR_CUDA;                               \
    }                                                    \
  } while (0)

// ---- driver entry point for tensor-map encoding (no link against libcuda) -------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

using WriteValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
WriteValue32Fn write_value_fn() {
  static WriteValue32Fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<WriteValue32Fn>(p);
  });
  return fn;
}

// K-major matrix [rows, k] with leading dimension ld (elements); box = 128 bytes of K x box_rows.
// Encoding is a pure function of its arguments, so the last few results are kept: a decode-sized
// launch is short enough for two driver calls per operand to show.
struct TmapKey {
  const void* base; int64_t rows, k, ld; int elem_bytes, box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && k == o.k && ld == o.ld && elem_bytes == o.elem_bytes &&
           box_rows == o.box_rows;
  }
};
int make_tmap(CUtensorMap* m, const void* base, int64_t rows, int64_t k, int64_t ld, int elem_bytes,
              int box_rows) {
  constexpr int kCache = 16;
  thread_local TmapKey keys[kCache] = {};
  thread_local CUtensorMap maps[kCache];
  thread_local int next = 0;
  const TmapKey key{base, rows, k, ld, elem_bytes, box_rows};
  for (int i = 0; i < kCache; ++i)
    if (keys[i].base != nullptr && keys[i] == key) { *m = maps[i]; return EDM_OK; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return EDM_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((ld * elem_bytes) & 15)) return EDM_ERR_BAD_ARG;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstr[1] = {static_cast<cuuint64_t>(ld * elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes / elem_bytes),
                       static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = 100000 + static_cast<int>(r);
    return EDM_ERR_CUDA;
  }
  keys[next] = key;
  maps[next] = *m;
  next = (next + 1) % kCache;
  return EDM_OK;
}

int num_sms() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

// One launch path for every variant: plain, cooperative (emulated ranks must be co-resident),
// and/or as clusters of 2 (CTA pairs).
template <int kCG, int kBN, bool kTf32, typename OutT>
struct Variant {
  static void* fn() { return reinterpret_cast<void*>(&tp_gemm_kernel<kCG, kBN, kTf32, OutT>); }
  static int configure() {
    static bool done = false;
    if (!done) {
      EDM_CUDA(cudaFuncSetAttribute(fn(), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      done = true;
    }
    return EDM_OK;
  }
  // Number of CTAs that can be resident at once (whole pairs for kCG == 2).
  static int max_resident(int sms, int* out) {
    static int cached = 0;
    if (!cached) {
      int rc = configure();
      if (rc) return rc;
      if (kCG == 1) {
        cached = sms;
      } else {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms - sms % 2); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int clusters = 0;
        EDM_CUDA(cudaOccupancyMaxActiveClusters(&clusters, fn(), &cfg));
        cached = 2 * clusters;
        if (cached > sms - sms % 2) cached = sms - sms % 2;
        if (cached <= 0) return EDM_ERR_CUDA;
      }
    }
    *out = cached;
    return EDM_OK;
  }
  static int launch(const LaunchParams& lp, int grid, bool cooperative, cudaStream_t stream) {
    int rc = configure();
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    int n = 0;
    if (kCG == 2) {
      at[n].id = cudaLaunchAttributeClusterDimension;
      at[n].val.clusterDim.x = 2; at[n].val.clusterDim.y = 1; at[n].val.clusterDim.z = 1;
      ++n;
    }
    if (cooperative) {
      at[n].id = cudaLaunchAttributeCooperative;
      at[n].val.cooperative = 1;
      ++n;
    }
    cfg.attrs = at; cfg.numAttrs = n;
    void* args[1] = {const_cast<LaunchParams*>(&lp)};
    EDM_CUDA(cudaLaunchKernelExC(&cfg, fn(), args));
    return EDM_OK;
  }
};

int launch_variant(int dtype, int cg, int bn, const LaunchParams& lp, int grid, bool coop, cudaStream_t stream) {
  if (dtype == EDM_DTYPE_BF16) {
    if (cg == 2) return Variant<2, 256, false, __nv_bfloat16>::launch(lp, grid, coop, stream);
    if (bn == 32) return Variant<1, 32, false, __nv_bfloat16>::launch(lp, grid, coop, stream);
    return Variant<1, 256, false, __nv_bfloat16>::launch(lp, grid, coop, stream);
  }
  return Variant<1, 256, true, float>::launch(lp, grid, coop, stream);
}

// Tile width of the plain bf16 GEMM.  With a single row block (M <= 128: decode) the job is to
// stream the weights once through as many SMs as possible.  Two ways to get there: 128x32 tiles
// (8x more tiles, each CTA re-reads its 128 rows of A over the whole K), or 128x256 tiles cut along
// K over the idle CTAs (TailSplit; the pieces then exchange partial sums).  Measured per CTA:
// 0.30 us per K block with narrow tiles, 0.54 us per K block plus 7.4 us for the exchange with
// wide pieces; the choice compares the two.
int pick_block_n(int dtype, int cg, int64_t M, int64_t N, int64_t K, int sms, int max_parts) {
  if (dtype != EDM_DTYPE_BF16 || cg != 1) return kBlockN;
  if (tuning().block_n == 32 || tuning().block_n == 256) return tuning().block_n;
  const int64_t wide_tiles = ((M + kBlockM - 1) / kBlockM) * ((N + kBlockN - 1) / kBlockN);
  if (M > kBlockM || wide_tiles * 2 > sms) return kBlockN;
  const int64_t kb = (K * 2 + kBlockKBytes - 1) / kBlockKBytes;
  const TailSplit split(static_cast<int>(wide_tiles), sms, static_cast<int>(kb), max_parts);
  const int64_t narrow_ns = 300 * kb;
  const int64_t wide_ns = 540 * ((kb + split.parts - 1) / split.parts) + (split.parts > 1 ? 7400 : 0);
  return wide_ns < narrow_ns ? kBlockN : 32;
}

int max_resident_ctas(int dtype, int cg, int sms, int* out) {
  if (dtype == EDM_DTYPE_BF16 && cg == 2) return Variant<2, 256, false, __nv_bfloat16>::max_resident(sms, out);
  *out = sms;
  return EDM_OK;
}

// CTA pairs pay off once there are whole 256-row tiles; EDM_CTA_GROUP=1|2 forces a variant.
int pick_cta_group(int dtype, int op, int64_t M, int world) {
  if (dtype != EDM_DTYPE_BF16) return 1;
  int want = M >= 256 ? 2 : 1;
  if (tuning().cta_group == 1 || tuning().cta_group == 2) want = tuning().cta_group;
  if (want == 2 && op == EDM_OP_GEMM_RS && world > 1 && (M / world) % (2 * kBlockM) != 0) want = 1;
  return want;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Split-fp32 scratch: tf32 high/low copies of A and B, then one fp32 running-sum tile per CTA.
constexpr int kSegKBlocks = 8;      // 256 K elements per TMEM accumulation segment
constexpr int kMaxGridCtas = 256;   // upper bound on CTAs of one launch
constexpr size_t kRunningSumBytes = static_cast<size_t>(kMaxGridCtas) * kBlockM * kBlockN * 4;

size_t split_ws_bytes(int64_t M, int64_t N, int64_t K) {
  return 2 * (align_up(static_cast<size_t>(M) * K * 4, 256) + align_up(static_cast<size_t>(N) * K * 4, 256)) +
         kRunningSumBytes;
}

// Fills tmap_a/tmap_b (and runs the tf32 split for fp32) for a GEMM A[M,K] x B[N,K].
// `cg` = CTAs sharing a tile of width `bn`: each loads bn / cg rows of the B tile per stage.
int prepare_operands(RankParams& P, int dtype, int cg, int bn, const void* a, int64_t lda, int64_t a_rows,
                     const void* b, int64_t ldb, int64_t N, int64_t K, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  if (dtype == EDM_DTYPE_BF16) {
    if (K % 8 || N % 8) return EDM_ERR_BAD_ARG;
    int rc = make_tmap(&P.tmap_a[0], a, a_rows, K, lda, 2, kBlockM);
    if (rc) return rc;
    P.tmap_a[1] = P.tmap_a[0];
    rc = make_tmap(&P.tmap_b[0], b, N, K, ldb, 2, bn / cg);
    if (rc) return rc;
    P.tmap_b[1] = P.tmap_b[0];
    P.passes = 1;
    return EDM_OK;
  }
  if (dtype != EDM_DTYPE_FP32) return EDM_ERR_BAD_ARG;
  if (K % 4 || N % 4) return EDM_ERR_BAD_ARG;
  if (!ws || ws_bytes < split_ws_bytes(a_rows, N, K)) return EDM_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(ws) & 255u) return EDM_ERR_BAD_ARG;
  char* w = static_cast<char*>(ws);
  const size_t a_sz = align_up(static_cast<size_t>(a_rows) * K * 4, 256);
  const size_t b_sz = align_up(static_cast<size_t>(N) * K * 4, 256);
  float* a_hi = reinterpret_cast<float*>(w);
  float* a_lo = reinterpret_cast<float*>(w + a_sz);
  float* b_hi = reinterpret_cast<float*>(w + 2 * a_sz);
  float* b_lo = reinterpret_cast<float*>(w + 2 * a_sz + b_sz);
  split_tf32_kernel<<<296, 256, 0, stream>>>(static_cast<const float*>(a), a_hi, a_lo, a_rows, K, lda);
  split_tf32_kernel<<<296, 256, 0, stream>>>(static_cast<const float*>(b), b_hi, b_lo, N, K, ldb);
  EDM_CUDA(cudaGetLastError());
  int rc;
  if ((rc = make_tmap(&P.tmap_a[0], a_hi, a_rows, K, K, 4, kBlockM))) return rc;
  if ((rc = make_tmap(&P.tmap_a[1], a_lo, a_rows, K, K, 4, kBlockM))) return rc;
  if ((rc = make_tmap(&P.tmap_b[0], b_hi, N, K, K, 4, bn / cg))) return rc;
  if ((rc = make_tmap(&P.tmap_b[1], b_lo, N, K, K, 4, bn / cg))) return rc;
  P.passes = 3;
  P.seg_kblocks = kSegKBlocks;
  P.scratch = reinterpret_cast<float*>(w + 2 * a_sz + 2 * b_sz);
  return EDM_OK;
}

int check_dims(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return EDM_ERR_BAD_ARG;
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return EDM_ERR_BAD_ARG;
  return EDM_OK;
}

// CTAs of a launch over `tiles` tiles: one unit (CTA or pair) per tile up to what fits on the GPU,
// or, with fewer tiles than units and a launch that may cut tiles along K, one unit per piece.
int grid_for_tiles(int tiles, int cg, int resident, bool may_split, int64_t K, int max_parts) {
  const int units = resident / cg;
  if (tiles >= units) return units * cg;
  int work = tiles;
  if (may_split) {
    const TailSplit split(tiles, units, static_cast<int>((K * 2 + kBlockKBytes - 1) / kBlockKBytes), max_parts);
    if (split.parts > 1) work = split.tiles * split.parts;
  }
  return (work < units ? work : units) * cg;
}

// Launches that may cut tiles along K share one scratch array, claim counter and flag set per
// device.  Two of them on the same stream are ordered anyway; across streams this event keeps them
// apart (a launch waits for the previous one that was issued on another stream).  Launches under
// stream capture are left alone: whoever builds the graph orders them.
struct ScratchGuard {
  std::mutex mu;
  cudaEvent_t ev = nullptr;
  cudaStream_t last = nullptr;
  bool recorded = false;
};
ScratchGuard* scratch_guard() {
  static ScratchGuard guards[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return &guards[dev];
}
int scratch_guard_before(cudaStream_t s) {
  ScratchGuard* g = scratch_guard();
  if (!g || capturing(s)) return EDM_OK;
  std::lock_guard<std::mutex> lock(g->mu);
  if (g->recorded && g->last != s) EDM_CUDA(cudaStreamWaitEvent(s, g->ev, 0));
  return EDM_OK;
}
int scratch_guard_after(cudaStream_t s) {
  ScratchGuard* g = scratch_guard();
  if (!g || capturing(s)) return EDM_OK;
  std::lock_guard<std::mutex> lock(g->mu);
  if (!g->ev) EDM_CUDA(cudaEventCreateWithFlags(&g->ev, cudaEventDisableTiming));
  EDM_CUDA(cudaEventRecord(g->ev, s));
  g->last = s;
  g->recorded = true;
  return EDM_OK;
}

int plain_gemm(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
               int64_t M, int64_t N, int64_t K, void* ws, size_t ws_bytes, void* stream) {
  if (!a || !b || !d) return EDM_ERR_BAD_ARG;
  int rc = check_dims(M, N, K);
  if (rc) return rc;
  const int out_bytes = dtype == EDM_DTYPE_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(d) & 15u) || ((ldd * out_bytes) & 15) || ldd < N) return EDM_ERR_BAD_ARG;
  if (lda < K || ldb < K) return EDM_ERR_BAD_ARG;
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  RankParams& P = lp.r[0];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cg = pick_cta_group(dtype, EDM_OP_GEMM, M, 1);
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  const int bn = pick_block_n(dtype, cg, M, N, K, sms, max_tail_parts(s));
  rc = prepare_operands(P, dtype, cg, bn, a, lda, M, b, ldb, N, K, ws, ws_bytes, s);
  if (rc) return rc;
  P.M = static_cast<int32_t>(M); P.N = static_cast<int32_t>(N); P.K = static_cast<int32_t>(K);
  P.rank = 0; P.world = 1; P.mode = kPlain; P.epoch = 1;
  P.out = d; P.ld_out = ldd;
  int resident = 0;
  if ((rc = max_resident_ctas(dtype, cg, sms, &resident))) return rc;
  const int tiles = static_cast<int>(((M + kBlockM * cg - 1) / (kBlockM * cg)) * ((N + bn - 1) / bn));
  apply_tuning(lp, s);
  const int grid = grid_for_tiles(tiles, cg, resident, bn == kBlockN && dtype == EDM_DTYPE_BF16, K, lp.tail_split);
  lp.num_vranks = 1;
  lp.ctas_per_vrank = grid;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  if ((rc = scratch_guard_before(s))) return rc;
  if ((rc = launch_variant(dtype, cg, bn, lp, grid, false, s))) return rc;
  return scratch_guard_after(s);
}

}  // namespace

// ======================================================================== allocation-free fp32 GEMM
// Scratch for edm_gemm_fp32_static: the tf32 high/low copies of A and B (first
// kStaticSplitBytes) followed by one fp32 running-sum tile for each of kStaticCtas CTAs.  The
// array is part of the library image: every GPU that loads the library keeps these 12 MiB until
// the process exits.  In host code the name below is only a handle for the runtime, never a
// device address; the address a kernel may use comes from cudaGetSymbolAddress.
namespace {
constexpr size_t kStaticSplitBytes = 8u << 20;
constexpr int kStaticCtas = 32;
constexpr size_t kStaticScratchBytes = kStaticSplitBytes + static_cast<size_t>(kStaticCtas) * kBlockM * kBlockN * 4;
constexpr int kMaxDevices = 64;
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

extern "C" int edm_gemm_fp32_static(const void* a, int64_t lda, const void* b, int64_t ldb, void* d,
                                    int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream) {
  if (!a || !b || !d) return EDM_ERR_BAD_ARG;
  int rc = check_dims(M, N, K);
  if (rc) return rc;
  if (K % 4 || N % 4 || lda < K || ldb < K || ldd < N) return EDM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(d) & 15u) || ((ldd * 4) & 15)) return EDM_ERR_BAD_ARG;
  const size_t a_sz = align_up(static_cast<size_t>(M) * K * 4, 256);
  const size_t b_sz = align_up(static_cast<size_t>(N) * K * 4, 256);
  if (2 * (a_sz + b_sz) > kStaticSplitBytes) return EDM_ERR_CAPACITY;  // operands too large for the fixed scratch

  // Set-up, once per device, with that device current: resolve the device address of the array.
  static char* scratch_of_device[kMaxDevices] = {};
  int dev = 0;
  EDM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return EDM_ERR_UNSUPPORTED;
  if (scratch_of_device[dev] == nullptr) {
    void* p = nullptr;
    EDM_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return EDM_ERR_CUDA;
    scratch_of_device[dev] = static_cast<char*>(p);
  }
  char* w = scratch_of_device[dev];

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* a_hi = reinterpret_cast<float*>(w);
  float* a_lo = reinterpret_cast<float*>(w + a_sz);
  float* b_hi = reinterpret_cast<float*>(w + 2 * a_sz);
  float* b_lo = reinterpret_cast<float*>(w + 2 * a_sz + b_sz);
  // both splits and the running sums are fully rewritten by every call: nothing has to start at zero
  split_tf32_kernel<<<296, 256, 0, s>>>(static_cast<const float*>(a), a_hi, a_lo, M, K, lda);
  split_tf32_kernel<<<296, 256, 0, s>>>(static_cast<const float*>(b), b_hi, b_lo, N, K, ldb);
  EDM_CUDA(cudaGetLastError());

  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  RankParams& P = lp.r[0];
  if ((rc = make_tmap(&P.tmap_a[0], a_hi, M, K, K, 4, kBlockM))) return rc;
  if ((rc = make_tmap(&P.tmap_a[1], a_lo, M, K, K, 4, kBlockM))) return rc;
  if ((rc = make_tmap(&P.tmap_b[0], b_hi, N, K, K, 4, kBlockN))) return rc;
  if ((rc = make_tmap(&P.tmap_b[1], b_lo, N, K, K, 4, kBlockN))) return rc;
  P.passes = 3;
  P.seg_kblocks = kSegKBlocks;
  P.scratch = reinterpret_cast<float*>(w + kStaticSplitBytes);  // indexed by CTA: the grid stays <= kStaticCtas
  P.M = static_cast<int32_t>(M); P.N = static_cast<int32_t>(N); P.K = static_cast<int32_t>(K);
  P.rank = 0; P.world = 1; P.mode = kPlain; P.epoch = 1;
  P.out = d; P.ld_out = ldd;
  const int64_t tiles = ((M + kBlockM - 1) / kBlockM) * ((N + kBlockN - 1) / kBlockN);
  const int grid = static_cast<int>(tiles < kStaticCtas ? tiles : kStaticCtas);
  lp.num_vranks = 1;
  lp.ctas_per_vrank = grid;
  lp.timeout_ns = g_timeout_ns;
  return launch_variant(EDM_DTYPE_FP32, 1, kBlockN, lp, grid, false, s);
}

// ======================================================================== contexts
struct edm_comm {
  int rank = 0, world = 1;
  int device = 0;
  char* base[EDM_MAX_RANKS] = {};  // every rank's allocation as mapped in this process
  bool imported[EDM_MAX_RANKS] = {};
  size_t flag_bytes = 0;     // both parities
  size_t counter_bytes = 0;
  size_t window_bytes = 0;   // both parities
  size_t heap_bytes = 0;
  size_t heap_used = 0;
  size_t total_bytes = 0;
  uint32_t epoch = 0;
  // copy-engine transport of the all-gather: a side stream and the events that tie it to the caller's
  // (several streams so that copies to different peers run on different copy engines at once)
  static constexpr int kSideStreams = 4;
  cudaStream_t side[kSideStreams] = {};
  cudaEvent_t ev_in = nullptr, ev_out[kSideStreams] = {};

  size_t off_flags() const { return 0; }
  size_t off_counters() const { return flag_bytes; }
  size_t off_window() const { return flag_bytes + counter_bytes; }
  size_t off_heap() const { return flag_bytes + counter_bytes + window_bytes; }
};

namespace {
constexpr size_t kFlagBytesPerParity = 2u << 20;  // 512 Ki flag words per parity
constexpr size_t kCounterBytes = 64u << 10;

struct Layout {
  int64_t m_blocks, n_blocks, total;
  int32_t max_owned = 0;
  uint32_t partial_off = 0, result_off = 0, gather_off = 0, flag_words = 0;
  size_t window_need = 0;
};

int plan_layout(const edm_comm* c, const edm_tp_call_t& call, int out_bytes, int elem_bytes, int cg, Layout& L) {
  const int W = c->world;
  const int tile_m = kBlockM * cg;  // a CTA pair schedules 256-row tiles; slots and flags stay per 128 rows
  L.m_blocks = (call.M + tile_m - 1) / tile_m;
  L.n_blocks = (call.N + kBlockN - 1) / kBlockN;
  L.total = L.m_blocks * L.n_blocks;
  if (L.total > (1 << 24)) return EDM_ERR_BAD_ARG;
  const size_t tile_bytes = static_cast<size_t>(kBlockM) * kBlockN * out_bytes;
  if (call.op == EDM_OP_GEMM_RS) {
    if (call.M % W) return EDM_ERR_BAD_ARG;
    const int64_t rows = call.M / W;
    if (rows % tile_m) return EDM_ERR_UNSUPPORTED;  // tiles must not straddle owners
    L.max_owned = static_cast<int32_t>(rows / tile_m * L.n_blocks) * cg;
    L.window_need = tile_bytes * L.max_owned * W;
    L.flag_words = static_cast<uint32_t>(W) * L.max_owned * 4;
  } else if (call.op == EDM_OP_GEMM_AR) {
    L.max_owned = static_cast<int32_t>((L.total + W - 1) / W) * cg;
    L.window_need = tile_bytes * L.max_owned * W;
    L.partial_off = 0;
    L.result_off = static_cast<uint32_t>(W) * L.max_owned * 4;
    L.flag_words = L.result_off + static_cast<uint32_t>(L.total) * cg * 4;
  } else if (call.op == EDM_OP_AG_GEMM) {
    if (call.M % W || call.chunks < 1 || call.chunks > 4096 || call.chunks > call.M / W)
      return EDM_ERR_BAD_ARG;
    L.window_need = static_cast<size_t>(call.M) * call.K * elem_bytes;
    L.gather_off = 0;
    L.flag_words = static_cast<uint32_t>(W) * call.chunks;
    if (static_cast<size_t>(W) * call.chunks * 4 > c->counter_bytes) return EDM_ERR_CAPACITY;
  } else {
    return EDM_ERR_BAD_ARG;
  }
  if (L.window_need > c->window_bytes / 2) return EDM_ERR_CAPACITY;
  if (static_cast<size_t>(L.flag_words) * 4 > c->flag_bytes / 2) return EDM_ERR_CAPACITY;
  return EDM_OK;
}

// Builds one rank's kernel parameters; bumps the context epoch.
int build_rank_params(edm_comm* c, const edm_tp_call_t& call, int cg, RankParams& P, cudaStream_t stream) {
  if (!c || !call.a || !call.b || !call.d) return EDM_ERR_BAD_ARG;
  int rc = check_dims(call.M, call.N, call.K);
  if (rc) return rc;
  const int W = c->world;
  for (int p = 0; p < W; ++p)
    if (!c->base[p]) return EDM_ERR_BAD_ARG;  // peers not linked yet
  const int elem_bytes = call.dtype == EDM_DTYPE_BF16 ? 2 : 4;
  const int out_bytes = elem_bytes;
  if (call.dtype != EDM_DTYPE_BF16 && call.dtype != EDM_DTYPE_FP32) return EDM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(call.d) & 15u) || ((call.ldd * out_bytes) & 15) || call.ldd < call.N)
    return EDM_ERR_BAD_ARG;
  if (call.lda < call.K || call.ldb < call.K) return EDM_ERR_BAD_ARG;

  std::memset(&P, 0, sizeof(P));
  P.M = static_cast<int32_t>(call.M); P.N = static_cast<int32_t>(call.N); P.K = static_cast<int32_t>(call.K);
  P.rank = c->rank; P.world = W;
  P.out = call.d; P.ld_out = call.ldd;

  if (W == 1 || call.op == EDM_OP_GEMM) {
    // a one-rank group needs no exchange
    if (call.op == EDM_OP_GEMM_AR || call.op == EDM_OP_GEMM_RS || call.op == EDM_OP_GEMM ||
        call.op == EDM_OP_AG_GEMM) {
      P.mode = kPlain; P.epoch = 1;
      return prepare_operands(P, call.dtype, cg, kBlockN, call.a, call.lda, call.M, call.b, call.ldb, call.N,
                              call.K, call.workspace, call.workspace_bytes, stream);
    }
    return EDM_ERR_BAD_ARG;
  }

  Layout L;
  rc = plan_layout(c, call, out_bytes, elem_bytes, cg, L);
  if (rc) return rc;

  const uint32_t epoch = c->epoch + 1;
  const size_t par = epoch & 1u;
  for (int p = 0; p < W; ++p) {
    P.flags[p] = reinterpret_cast<uint32_t*>(c->base[p] + c->off_flags() + par * (c->flag_bytes / 2));
    P.win[p] = c->base[p] + c->off_window() + par * (c->window_bytes / 2);
    P.gather[p] = P.win[p];
  }
  P.counters = reinterpret_cast<uint32_t*>(c->base[c->rank] + c->off_counters());
  P.epoch = epoch;
  P.max_owned = L.max_owned;
  P.partial_flag_off = L.partial_off;
  P.result_flag_off = L.result_off;
  P.gather_flag_off = L.gather_off;

  if (call.op == EDM_OP_AG_GEMM) {
    if (call.dtype != EDM_DTYPE_BF16) return EDM_ERR_UNSUPPORTED;
    if (call.K % 8 || call.N % 8) return EDM_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(call.a) & 15u || (call.lda * 2) & 15) return EDM_ERR_BAD_ARG;
    const int64_t rows = call.M / W;
    P.mode = kAG;
    P.ag_chunks = call.chunks;
    P.ag_local_direct = (rows % kBlockM == 0) ? 1 : 0;
    P.x_local = call.a; P.ld_x = call.lda;
    P.ag_external = call.transport == EDM_TRANSPORT_COPY_ENGINE ? 1 : 0;
    P.passes = 1;
    // A comes from the local gather buffer [M,K]; the own shard is read in place when it
    // covers whole row blocks
    if ((rc = make_tmap(&P.tmap_a[0], P.gather[c->rank], call.M, call.K, call.K, 2, kBlockM))) return rc;
    if ((rc = make_tmap(&P.tmap_a[1], call.a, rows, call.K, call.lda, 2, kBlockM))) return rc;
    if ((rc = make_tmap(&P.tmap_b[0], call.b, call.N, call.K, call.ldb, 2, kBlockN / cg))) return rc;
    P.tmap_b[1] = P.tmap_b[0];
  } else {
    P.mode = call.op == EDM_OP_GEMM_RS ? kRS : kAR;
    if (call.op == EDM_OP_GEMM_AR) {
      // peers store reduced tiles straight into this tensor: it must sit in the symmetric heap
      const char* d = static_cast<const char*>(call.d);
      const char* heap0 = c->base[c->rank] + c->off_heap();
      const size_t span = (static_cast<size_t>(call.M - 1) * call.ldd + call.N) * out_bytes;
      if (d < heap0 || d + span > heap0 + c->heap_bytes) return EDM_ERR_NOT_SYMMETRIC;
      const size_t off = static_cast<size_t>(d - c->base[c->rank]);
      for (int p = 0; p < W; ++p) P.peer_out[p] = c->base[p] + off;
    }
    rc = prepare_operands(P, call.dtype, cg, kBlockN, call.a, call.lda, call.M, call.b, call.ldb, call.N, call.K,
                          call.workspace, call.workspace_bytes, stream);
    if (rc) return rc;
  }
  c->epoch = epoch;
  return EDM_OK;
}

// Copy-engine transport of one all-gather: after the caller's stream has produced the shard, the
// side stream copies it into every peer's gather buffer chunk by chunk (peer order rank-1,
// rank-2, ...: every GPU sends to and receives from one peer at a time) and raises each chunk's
// flag with a stream-ordered 32-bit write, which cannot overtake the copy before it.  No SM takes
// part, so the GEMM's operand traffic is not disturbed.  `after_launch` closes the bracket: later
// work on the caller's stream waits until the outgoing copies have read the shard.
int ag_copy_engine_issue(edm_comm* c, const RankParams& P, cudaStream_t stream) {
  WriteValue32Fn wv = write_value_fn();
  if (!wv) return EDM_ERR_UNSUPPORTED;
  const int W = P.world;
  const int64_t rows = P.M / W;
  const int elem = 2;
  const size_t row_bytes = static_cast<size_t>(P.K) * elem;
  const int64_t chunk_rows = (rows + P.ag_chunks - 1) / P.ag_chunks;
  int nstreams = tuning().side_streams;
  if (nstreams < 1) nstreams = 1;
  if (nstreams > edm_comm::kSideStreams) nstreams = edm_comm::kSideStreams;
  EDM_CUDA(cudaEventRecord(c->ev_in, stream));
  for (int i = 0; i < edm_comm::kSideStreams; ++i) EDM_CUDA(cudaStreamWaitEvent(c->side[i], c->ev_in, 0));
  // when the shard does not cover whole row blocks the kernel also reads the own rows from the
  // gather buffer: deliver them (d = 0) like a peer's
  for (int d = P.ag_local_direct ? 1 : 0; d < W; ++d) {
    const int peer = (P.rank - d + W) % W;
    cudaStream_t side = c->side[d % nstreams];
    char* dst0 = static_cast<char*>(P.gather[peer]) + static_cast<size_t>(P.rank) * rows * row_bytes;
    const char* src0 = static_cast<const char*>(P.x_local);
    for (int ch = 0; ch < P.ag_chunks; ++ch) {
      const int64_t r_lo = ch * chunk_rows;
      const int64_t r_hi = r_lo + chunk_rows < rows ? r_lo + chunk_rows : rows;
      if (r_hi > r_lo) {
        if (P.ld_x == P.K)  // contiguous shard: a plain copy is the fastest thing a copy engine does
          EDM_CUDA(cudaMemcpyAsync(dst0 + r_lo * row_bytes, src0 + r_lo * row_bytes,
                                   static_cast<size_t>(r_hi - r_lo) * row_bytes, cudaMemcpyDeviceToDevice, side));
        else
          EDM_CUDA(cudaMemcpy2DAsync(dst0 + r_lo * row_bytes, row_bytes, src0 + r_lo * P.ld_x * elem,
                                     static_cast<size_t>(P.ld_x) * elem, row_bytes, static_cast<size_t>(r_hi - r_lo),
                                     cudaMemcpyDeviceToDevice, side));
      }
      uint32_t* flag = P.flags[peer] + P.gather_flag_off + P.rank * P.ag_chunks + ch;
      CUresult r = wv(reinterpret_cast<CUstream>(side), reinterpret_cast<CUdeviceptr>(flag), P.epoch, 0);
      if (r != CUDA_SUCCESS) { g_last_cuda_error = 100000 + static_cast<int>(r); return EDM_ERR_CUDA; }
    }
  }
  return EDM_OK;
}
int ag_copy_engine_after_launch(edm_comm* c, cudaStream_t stream) {
  for (int i = 0; i < edm_comm::kSideStreams; ++i) {
    EDM_CUDA(cudaEventRecord(c->ev_out[i], c->side[i]));
    EDM_CUDA(cudaStreamWaitEvent(stream, c->ev_out[i], 0));
  }
  return EDM_OK;
}

int grid_for(const RankParams& P, int cg, int resident) {
  if (P.mode == kAG) return resident;  // push warps of every CTA help move the shard
  const int tiles = ((P.M + kBlockM * cg - 1) / (kBlockM * cg)) * ((P.N + kBlockN - 1) / kBlockN);
  return tiles * cg < resident ? tiles * cg : resident;
}
}  // namespace

extern "C" {

int edm_version(void) { return 1; }
int edm_last_cuda_error(void) { return g_last_cuda_error; }

int edm_status_read(uint32_t out[16]) {
  if (!out) return EDM_ERR_BAD_ARG;
  EDM_CUDA(cudaDeviceSynchronize());
  EDM_CUDA(cudaMemcpyFromSymbol(out, g_status, sizeof(uint32_t) * 16));
  return EDM_OK;
}
int edm_status_clear(void) {
  uint32_t z[16] = {};
  EDM_CUDA(cudaDeviceSynchronize());
  EDM_CUDA(cudaMemcpyToSymbol(g_status, z, sizeof(z)));
  // a launch that gave up may have left the claim counters of the split last wave part-way
  EDM_CUDA(cudaMemcpyToSymbol(g_tail_next, z, sizeof(uint32_t) * kMaxVirtualRanks));
  return EDM_OK;
}
int edm_profile_enable(int on) {
  g_profile = on ? 1 : 0;
  return EDM_OK;
}
int edm_profile_read(uint64_t out[24], int reset) {
  if (!out) return EDM_ERR_BAD_ARG;
  EDM_CUDA(cudaDeviceSynchronize());
  EDM_CUDA(cudaMemcpyFromSymbol(out, g_prof, sizeof(uint64_t) * 24));
  if (reset) {
    uint64_t z[24] = {};
    EDM_CUDA(cudaMemcpyToSymbol(g_prof, z, sizeof(z)));
  }
  return EDM_OK;
}
int edm_set_timeout_ms(uint32_t ms) {
  if (ms == 0) return EDM_ERR_BAD_ARG;
  g_timeout_ns = static_cast<uint64_t>(ms) * 1000000ull;
  return EDM_OK;
}

int edm_gemm_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
                  int64_t M, int64_t N, int64_t K, void* stream) {
  return plain_gemm(EDM_DTYPE_BF16, a, lda, b, ldb, d, ldd, M, N, K, nullptr, 0, stream);
}

size_t edm_gemm_fp32_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return split_ws_bytes(M, N, K);
}
int edm_gemm_fp32(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
                  int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                  void* stream) {
  return plain_gemm(EDM_DTYPE_FP32, a, lda, b, ldb, d, ldd, M, N, K, workspace, workspace_bytes, stream);
}

int edm_comm_create(int rank, int world, size_t window_bytes, size_t heap_bytes, edm_comm_t** out) {
  if (!out || world < 1 || world > EDM_MAX_RANKS || rank < 0 || rank >= world) return EDM_ERR_BAD_ARG;
  edm_comm* c = new (std::nothrow) edm_comm();
  if (!c) return EDM_ERR_CAPACITY;
  c->rank = rank; c->world = world;
  EDM_CUDA(cudaGetDevice(&c->device));
  c->flag_bytes = 2 * kFlagBytesPerParity;
  c->counter_bytes = kCounterBytes;
  c->window_bytes = align_up(window_bytes / 2 + (window_bytes & 1), 1024) * 2;
  c->heap_bytes = align_up(heap_bytes, 1024);
  c->total_bytes = c->flag_bytes + c->counter_bytes + c->window_bytes + c->heap_bytes;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, c->total_bytes);
  if (e != cudaSuccess) { g_last_cuda_error = e; delete c; return EDM_ERR_CUDA; }
  e = cudaMemset(p, 0, c->flag_bytes + c->counter_bytes);
  if (e != cudaSuccess) { g_last_cuda_error = e; cudaFree(p); delete c; return EDM_ERR_CUDA; }
  c->base[rank] = static_cast<char*>(p);
  bool ok = cudaEventCreateWithFlags(&c->ev_in, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < edm_comm::kSideStreams; ++i)
    ok = cudaStreamCreateWithFlags(&c->side[i], cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    g_last_cuda_error = static_cast<int>(cudaGetLastError());
    edm_comm_destroy(c);
    return EDM_ERR_CUDA;
  }
  *out = c;
  return EDM_OK;
}

int edm_comm_destroy(edm_comm_t* c) {
  if (!c) return EDM_ERR_BAD_ARG;
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (c->imported[p] && c->base[p]) cudaIpcCloseMemHandle(c->base[p]);
  if (c->base[c->rank]) cudaFree(c->base[c->rank]);
  if (c->ev_in) cudaEventDestroy(c->ev_in);
  for (int i = 0; i < edm_comm::kSideStreams; ++i) {
    if (c->ev_out[i]) cudaEventDestroy(c->ev_out[i]);
    if (c->side[i]) cudaStreamDestroy(c->side[i]);
  }
  delete c;
  return EDM_OK;
}

int edm_comm_export(edm_comm_t* c, void* handle64) {
  if (!c || !handle64) return EDM_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == EDM_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  EDM_CUDA(cudaIpcGetMemHandle(&h, c->base[c->rank]));
  std::memcpy(handle64, &h, sizeof(h));
  return EDM_OK;
}

int edm_comm_import(edm_comm_t* c, int peer, const void* handle64) {
  if (!c || !handle64 || peer < 0 || peer >= c->world || peer == c->rank) return EDM_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  EDM_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  c->base[peer] = static_cast<char*>(p);
  c->imported[peer] = true;
  return EDM_OK;
}

int edm_comm_link_local(edm_comm_t* c, int peer, edm_comm_t* other) {
  if (!c || !other || peer < 0 || peer >= c->world || peer == c->rank) return EDM_ERR_BAD_ARG;
  if (other->rank != peer || other->world != c->world || other->total_bytes != c->total_bytes)
    return EDM_ERR_BAD_ARG;
  c->base[peer] = other->base[other->rank];
  c->imported[peer] = false;
  return EDM_OK;
}

int edm_comm_heap_alloc(edm_comm_t* c, size_t bytes, void** out) {
  if (!c || !out || bytes == 0) return EDM_ERR_BAD_ARG;
  const size_t start = align_up(c->heap_used, 256);
  if (start + bytes > c->heap_bytes) return EDM_ERR_CAPACITY;
  *out = c->base[c->rank] + c->off_heap() + start;
  c->heap_used = start + bytes;
  return EDM_OK;
}
int edm_comm_heap_reset(edm_comm_t* c) {
  if (!c) return EDM_ERR_BAD_ARG;
  c->heap_used = 0;
  return EDM_OK;
}
int edm_comm_rank(const edm_comm_t* c) { return c ? c->rank : -1; }
int edm_comm_world(const edm_comm_t* c) { return c ? c->world : -1; }

int edm_tile_walk(int op, int rank, int world, int64_t M, int64_t N, int tile_m, int tile_n, int band_rows,
                  int units, int32_t* out, int64_t capacity, int64_t* positions) {
  if (op < EDM_OP_GEMM || op > EDM_OP_AG_GEMM || world < 1 || world > 8 || rank < 0 || rank >= world || M <= 0 ||
      N <= 0 || M > INT32_MAX || N > INT32_MAX || tile_m <= 0 || tile_n <= 0 || units < 1 || !positions)
    return EDM_ERR_BAD_ARG;
  const int mode = op == EDM_OP_GEMM ? kPlain : op == EDM_OP_GEMM_RS ? kRS : op == EDM_OP_GEMM_AR ? kAR : kAG;
  const TileWalk walk(mode, rank, world, static_cast<int>(M), static_cast<int>(N), tile_m, tile_n, band_rows, units);
  if (mode == kRS && world > 1 && walk.mb_per_rank == 0) return EDM_ERR_UNSUPPORTED;
  *positions = walk.positions;
  if (!out) return EDM_OK;
  if (capacity < walk.positions) return EDM_ERR_CAPACITY;
  for (int i = 0; i < walk.positions; ++i) {
    const Tile t = walk.at(i);
    out[4 * i + 0] = t.valid ? t.m_blk : -1;
    out[4 * i + 1] = t.valid ? t.n_blk : -1;
    out[4 * i + 2] = t.owner;
    out[4 * i + 3] = t.owned_idx;
  }
  return EDM_OK;
}

int edm_gemm_plan(int64_t M, int64_t N, int64_t K, int sms, int32_t out[4]) {
  if (!out || sms < 2 || sms > 4096) return EDM_ERR_BAD_ARG;
  int rc = check_dims(M, N, K);
  if (rc) return rc;
  const int max_parts = tuning().tail_split;
  const int cg = pick_cta_group(EDM_DTYPE_BF16, EDM_OP_GEMM, M, 1);
  const int bn = pick_block_n(EDM_DTYPE_BF16, cg, M, N, K, sms, max_parts);
  const int resident = cg == 2 ? sms - sms % 2 : sms;
  const int tiles = static_cast<int>(((M + kBlockM * cg - 1) / (kBlockM * cg)) * ((N + bn - 1) / bn));
  const int grid = grid_for_tiles(tiles, cg, resident, bn == kBlockN, K, max_parts);
  const TailSplit split(tiles, grid / cg, static_cast<int>((K * 2 + kBlockKBytes - 1) / kBlockKBytes),
                        bn == kBlockN ? max_parts : 0);
  out[0] = cg; out[1] = bn; out[2] = grid; out[3] = split.parts;
  return EDM_OK;
}

int edm_tail_split(int64_t tiles, int units, int64_t k_blocks, int32_t out[3]) {
  if (tiles < 0 || tiles > INT32_MAX || units < 1 || k_blocks < 1 || k_blocks > INT32_MAX || !out) return EDM_ERR_BAD_ARG;
  const TailSplit t(static_cast<int>(tiles), units, static_cast<int>(k_blocks), tuning().tail_split);
  out[0] = t.first; out[1] = t.tiles; out[2] = t.parts;
  return EDM_OK;
}

int edm_comm_p2p_probe(edm_comm_t* c, int peer, size_t bytes, int mode, void* stream) {
  if (!c || peer < 0 || peer >= c->world || !c->base[peer] || (mode != 0 && mode != 1)) return EDM_ERR_BAD_ARG;
  if (bytes == 0 || bytes % 8192 || bytes > c->window_bytes / 2) return EDM_ERR_CAPACITY;
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  static bool configured = false;
  const int smem = 8 * 2 * 8192 + 128;
  if (!configured) {
    EDM_CUDA(cudaFuncSetAttribute(p2p_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  // source: first half of the local window; destination: second half of the peer's
  const char* src = c->base[c->rank] + c->off_window();
  char* dst = c->base[peer] + c->off_window() + c->window_bytes / 2;
  p2p_probe_kernel<<<sms, 256, smem, static_cast<cudaStream_t>(stream)>>>(src, dst, bytes, mode);
  EDM_CUDA(cudaGetLastError());
  return EDM_OK;
}

int edm_tp_launch(edm_comm_t* comm, const edm_tp_call_t* call, void* stream) {
  if (!comm || !call) return EDM_ERR_BAD_ARG;
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the exchange flags carry the context's call counter, which a replay of a captured launch
  // would repeat: fused launches cannot be captured
  if (comm->world > 1 && capturing(s)) return EDM_ERR_UNSUPPORTED;
  const int cg = pick_cta_group(call->dtype, call->op, call->M, comm->world);
  int rc = build_rank_params(comm, *call, cg, lp.r[0], s);
  if (rc) return rc;
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  int resident = 0;
  if ((rc = max_resident_ctas(call->dtype, cg, sms, &resident))) return rc;
  const int grid = grid_for(lp.r[0], cg, resident);
  lp.num_vranks = 1;
  lp.ctas_per_vrank = grid;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  apply_tuning(lp, s);
  const bool ce = lp.r[0].mode == kAG && lp.r[0].ag_external;
  if (ce && (rc = ag_copy_engine_issue(comm, lp.r[0], s))) return rc;
  const bool may_split = lp.r[0].mode == kAG;  // the only fused mode that writes its tiles in place
  if (may_split && (rc = scratch_guard_before(s))) return rc;
  rc = launch_variant(call->dtype, cg, kBlockN, lp, grid, false, s);
  if (rc) return rc;
  if (may_split && (rc = scratch_guard_after(s))) return rc;
  if (ce) return ag_copy_engine_after_launch(comm, s);
  return EDM_OK;
}

int edm_tp_launch_emulated(edm_comm_t* const* comms, const edm_tp_call_t* calls, int n, void* stream) {
  if (!comms || !calls || n < 1 || n > kMaxVirtualRanks) return EDM_ERR_BAD_ARG;
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (capturing(s)) return EDM_ERR_UNSUPPORTED;  // see edm_tp_launch
  const int cg = pick_cta_group(calls[0].dtype, calls[0].op, calls[0].M, comms[0] ? comms[0]->world : 1);
  for (int i = 0; i < n; ++i) {
    if (!comms[i] || calls[i].dtype != calls[0].dtype || calls[i].op != calls[0].op ||
        calls[i].M != calls[0].M)
      return EDM_ERR_BAD_ARG;
    int rc = build_rank_params(comms[i], calls[i], cg, lp.r[i], s);
    if (rc) return rc;
  }
  const int sms = num_sms();
  if (sms < n) return EDM_ERR_CUDA;
  int resident = 0;
  int rc = max_resident_ctas(calls[0].dtype, cg, sms, &resident);
  if (rc) return rc;
  lp.num_vranks = n;
  // all CTAs co-resident (the emulated ranks wait on one another); whole pairs per rank
  lp.ctas_per_vrank = resident / n / cg * cg;
  if (lp.ctas_per_vrank < cg) return EDM_ERR_CUDA;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  apply_tuning(lp, s);
  for (int i = 0; i < n; ++i)
    if (lp.r[i].mode == kAG && lp.r[i].ag_external && (rc = ag_copy_engine_issue(comms[i], lp.r[i], s))) return rc;
  if ((rc = scratch_guard_before(s))) return rc;
  rc = launch_variant(calls[0].dtype, cg, kBlockN, lp, lp.ctas_per_vrank * n, true, s);
  if (rc) return rc;
  if ((rc = scratch_guard_after(s))) return rc;
  for (int i = 0; i < n; ++i)
    if (lp.r[i].mode == kAG && lp.r[i].ag_external && (rc = ag_copy_engine_after_launch(comms[i], s))) return rc;
  return EDM_OK;
}

static int tp_bf16(edm_comm_t* comm, int op, const void* a, int64_t lda, const void* b, int64_t ldb,
                   void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, int32_t chunks, void* stream) {
  edm_tp_call_t c;
  std::memset(&c, 0, sizeof(c));
  c.op = op; c.dtype = EDM_DTYPE_BF16;
  c.a = a; c.lda = lda; c.b = b; c.ldb = ldb; c.d = d; c.ldd = ldd;
  c.M = M; c.N = N; c.K = K; c.chunks = chunks; c.transport = EDM_TRANSPORT_SM;
  return edm_tp_launch(comm, &c, stream);
}
int edm_gemm_rs_bf16(edm_comm_t* comm, const void* a, int64_t lda, const void* b, int64_t ldb,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream) {
  return tp_bf16(comm, EDM_OP_GEMM_RS, a, lda, b, ldb, d, ldd, M, N, K, 1, stream);
}
int edm_gemm_ar_bf16(edm_comm_t* comm, const void* a, int64_t lda, const void* b, int64_t ldb,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream) {
  return tp_bf16(comm, EDM_OP_GEMM_AR, a, lda, b, ldb, d, ldd, M, N, K, 1, stream);
}
int edm_ag_gemm_bf16(edm_comm_t* comm, const void* x, int64_t ldx, const void* w, int64_t ldw,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, int32_t chunks,
                     void* stream) {
  return tp_bf16(comm, EDM_OP_AG_GEMM, x, ldx, w, ldw, d, ldd, M, N, K, chunks, stream);
}

}  // extern "C"
