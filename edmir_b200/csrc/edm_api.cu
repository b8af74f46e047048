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
#include "moe.cuh"
#include "ar_oneshot.cuh"
#include "decode_gemm.cuh"

using namespace edm;

namespace {

thread_local int g_last_cuda_error = 0;
// process-wide settings: written by their setters, read by every launch (relaxed atomics)
std::atomic<uint64_t> g_timeout_ns{2000ull * 1000ull * 1000ull};
std::atomic<int> g_profile{0};
constexpr int kMaxDevices = 64;

// Index of the current device into the per-device tables below, or -1.
int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// Tuning knobs for experiments, read from the environment once (the operators pass their schedule
// through edm_tp_call_t, not through these): EDM_STAGE_LIMIT (ring stages),
// EDM_BAND / EDM_BAND_COLS (row blocks per band of the tile walk / column blocks per super-tile), EDM_PUSH_STRIDE (every n-th CTA pushes all-gather
// shards with the sm transport), EDM_SIDE_STREAMS (copy-engine transport), EDM_CTA_GROUP (1 or 2),
// EDM_BLOCK_N (32 or 256: tile width of the single-CTA plain GEMM), EDM_TAIL_SPLIT (most pieces a
// tile of an incomplete last wave is cut into along K; 0 or 1: none), EDM_DECODE (most rows a GEMM
// may have to run the decode kernel instead of the general one; 0: never).
constexpr int kDecodeMaxRows = 64;  // beyond that the general kernel is as fast (measured at 96 and 128 rows)
struct Tuning {
  int stage_limit = 0, band = 0, band_cols = 0, push_stride = 1, side_streams = 2, cta_group = 0, block_n = 0,
      tail_split = kTailMaxParts, decode = kDecodeMaxRows;
  Tuning() {
    auto get = [](const char* name, int dflt) {
      const char* e = std::getenv(name);
      return e ? std::atoi(e) : dflt;
    };
    stage_limit = get("EDM_STAGE_LIMIT", 0);
    band = get("EDM_BAND", 0);
    band_cols = get("EDM_BAND_COLS", 0);
    push_stride = get("EDM_PUSH_STRIDE", 1);
    if (push_stride < 1) push_stride = 1;
    side_streams = get("EDM_SIDE_STREAMS", 2);
    cta_group = get("EDM_CTA_GROUP", 0);
    block_n = get("EDM_BLOCK_N", 0);
    tail_split = get("EDM_TAIL_SPLIT", kTailMaxParts);
    decode = get("EDM_DECODE", kDecodeMaxRows);
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
  lp.band_cols = tuning().band_cols > 0 ? tuning().band_cols : 0;
  lp.push_stride = tuning().push_stride;
  lp.tail_split = max_tail_parts(s);
  // flags of the split last wave carry a value no earlier launch of this process used
  static std::atomic<uint32_t> tail_epoch{0};
  lp.tail_epoch = tail_epoch.fetch_add(1u) + 1u;
}

// Checking build (-DEDM_DEBUG_BOUNDS): the entry points collect every range a launch may touch
// and publish the table to the device before the kernel is enqueued; see tp_gemm.cuh.
#ifdef EDM_DEBUG_BOUNDS
struct DbgRanges {
  unsigned long long lo[kDbgMaxRanges], hi[kDbgMaxRanges];
  int n = 0;
  void add(const void* p, size_t bytes) {
    if (!p || !bytes || n >= kDbgMaxRanges) return;
    lo[n] = reinterpret_cast<unsigned long long>(p);
    hi[n] = lo[n] + bytes;
    ++n;
  }
};
thread_local DbgRanges g_dbg;
void dbg_reset() { g_dbg.n = 0; }
void dbg_add(const void* p, size_t bytes) { g_dbg.add(p, bytes); }
void dbg_add_matrix(const void* p, int64_t rows, int64_t cols, int64_t ld, int elem) {
  if (rows > 0) g_dbg.add(p, (static_cast<size_t>(rows - 1) * ld + cols) * elem);
}
int dbg_publish(cudaStream_t s) {
  // the table is uploaded and awaited per launch: not possible while the stream is being captured
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone) return EDM_ERR_UNSUPPORTED;
  void* p = nullptr;
  // the library's own device arrays
  if (cudaGetSymbolAddress(&p, g_tail_scratch) == cudaSuccess) g_dbg.add(p, sizeof(g_tail_scratch));
  if (cudaGetSymbolAddress(&p, g_tail_flags) == cudaSuccess) g_dbg.add(p, sizeof(g_tail_flags));
  if (cudaGetSymbolAddress(&p, g_tail_claim) == cudaSuccess) g_dbg.add(p, sizeof(g_tail_claim));
  if (cudaMemcpyToSymbolAsync(g_dbg_lo, g_dbg.lo, sizeof(unsigned long long) * g_dbg.n, 0, cudaMemcpyHostToDevice, s) != cudaSuccess ||
      cudaMemcpyToSymbolAsync(g_dbg_hi, g_dbg.hi, sizeof(unsigned long long) * g_dbg.n, 0, cudaMemcpyHostToDevice, s) != cudaSuccess ||
      cudaMemcpyToSymbolAsync(g_dbg_n, &g_dbg.n, sizeof(int), 0, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return EDM_ERR_CUDA;
  return cudaStreamSynchronize(s) == cudaSuccess ? EDM_OK : EDM_ERR_CUDA;  // the table is per launch: no overlap in this build
}
#else
inline void dbg_reset() {}
inline void dbg_add(const void*, size_t) {}
inline void dbg_add_matrix(const void*, int64_t, int64_t, int64_t, int) {}
inline int dbg_publish(cudaStream_t) { return EDM_OK; }
#endif

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
  // Function attributes and occupancy belong to a device: one slot per device, filled under a lock
  // on the first launch there (the attribute call is idempotent, so a race would be harmless, but
  // the lock also keeps the tables coherent for several host threads).
  static std::mutex& lock() { static std::mutex m; return m; }
  static int configure() {
    static bool done[kMaxDevices] = {};
    const int dev = current_device();
    if (dev < 0) return EDM_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> g(lock());
    if (!done[dev]) {
      EDM_CUDA(cudaFuncSetAttribute(fn(), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      done[dev] = true;
    }
    return EDM_OK;
  }
  // Number of CTAs that can be resident at once (whole pairs for kCG == 2).
  static int max_resident(int sms, int* out) {
    static int per_device[kMaxDevices] = {};
    const int dev = current_device();
    if (dev < 0) return EDM_ERR_UNSUPPORTED;
    int rc = configure();
    if (rc) return rc;
    std::lock_guard<std::mutex> g(lock());
    int& cached = per_device[dev];
    if (!cached) {
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
  if (int rc = dbg_publish(stream)) return rc;
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

// Operand bytes the split needs (tf32 high and low copies of A and B), or 0 when the sum does not
// fit in `limit` -- evaluated term by term so that extents near 2^30 cannot wrap around.
size_t split_operand_bytes(int64_t M, int64_t N, int64_t K, size_t limit) {
  const size_t cap = limit / 8;  // elements of A and B together: 2 copies x 4 bytes each
  const size_t k = static_cast<size_t>(K);
  if (k == 0 || static_cast<size_t>(M) > cap / k || static_cast<size_t>(N) > cap / k) return 0;
  const size_t a_sz = align_up(static_cast<size_t>(M) * k * 4, 256), b_sz = align_up(static_cast<size_t>(N) * k * 4, 256);
  if (a_sz > limit / 2 || b_sz > limit / 2 - a_sz) return 0;
  return 2 * (a_sz + b_sz);
}
size_t split_ws_bytes(int64_t M, int64_t N, int64_t K) {
  const size_t ops = split_operand_bytes(M, N, K, static_cast<size_t>(1) << 46);  // 64 TiB: beyond any device
  return ops ? ops + kRunningSumBytes : 0;
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
  const size_t ws_need = split_ws_bytes(a_rows, N, K);
  if (!ws || ws_need == 0 || ws_bytes < ws_need) return EDM_ERR_CAPACITY;
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
// Launches that do not cut any tile (most of them) skip all of this.
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
// Would the kernel cut tiles of this launch along K?  Mirrors the condition in tp_gemm_kernel.
bool launch_splits(const LaunchParams& lp, const RankParams& P, int dtype, int cg, int bn, int grid) {
  if (dtype != EDM_DTYPE_BF16 || bn != kBlockN || P.passes != 1 || grid > kTailMaxCtas) return false;
  if ((P.mode != kPlain && P.mode != kAG) || P.group_table != nullptr) return false;
  const int pushers = (P.mode == kAG && P.world > 1 && !P.ag_external) ? lp.pusher_ctas : 0;
  const int units = (lp.ctas_per_vrank - pushers) / cg;
  const int64_t tiles = ((static_cast<int64_t>(P.M) + kBlockM * cg - 1) / (kBlockM * cg)) *
                        ((static_cast<int64_t>(P.N) + bn - 1) / bn);
  if (tiles > INT32_MAX) return false;
  const TailSplit split(static_cast<int>(tiles), units, (P.K * 2 + kBlockKBytes - 1) / kBlockKBytes, lp.tail_split);
  return split.parts > 1;
}
// Runs `launch` (which enqueues one kernel on `s`).  When that kernel uses the shared scratch, the
// lock is held from the wait on the previous user's event until this launch's event is recorded,
// so two host threads cannot both pass the check and overlap on the GPU.
template <typename F>
int launch_with_scratch(bool uses_scratch, cudaStream_t s, F&& launch) {
  ScratchGuard* g = uses_scratch && !capturing(s) ? scratch_guard() : nullptr;
  if (!g) return launch();
  std::lock_guard<std::mutex> lock(g->mu);
  if (g->recorded && g->last != s) EDM_CUDA(cudaStreamWaitEvent(s, g->ev, 0));
  const int rc = launch();
  if (rc) return rc;
  if (!g->ev) EDM_CUDA(cudaEventCreateWithFlags(&g->ev, cudaEventDisableTiming));
  EDM_CUDA(cudaEventRecord(g->ev, s));
  g->last = s;
  g->recorded = true;
  return EDM_OK;
}

// Decode kernel (decode_gemm.cuh): bf16, at most 64 rows, and no more 128-column tiles than SMs
// (every piece of every tile is resident at once; wider outputs take the general kernel).
// `split`: pieces a tile's K range is cut into -- as many as fill the GPU, each at least 4 K blocks.
int decode_tok(int64_t M) { return M <= 32 ? 32 : 64; }
bool decode_plan(int dtype, int64_t M, int64_t N, int64_t K, int sms, int* tiles_out, int* split_out) {
  if (dtype != EDM_DTYPE_BF16 || M > kDecodeMaxRows || M > tuning().decode || K % 8 || N % 8) return false;
  const int64_t tiles = (N + kBlockM - 1) / kBlockM;
  if (tiles > sms) return false;
  const int64_t kb = (K * 2 + kBlockKBytes - 1) / kBlockKBytes;
  const int tok = decode_tok(M);
  const int max_split = tok == 32 ? DecodeShape<32>::kMaxSplit : DecodeShape<64>::kMaxSplit;
  int split = 1;
  while (split * 2 <= max_split && tiles * split * 2 <= sms && kb / (split * 2) >= 4) split *= 2;
  *tiles_out = static_cast<int>(tiles);
  *split_out = split;
  return true;
}

int decode_gemm(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd, int64_t M, int64_t N,
                int64_t K, int tiles, int split, cudaStream_t s) {
  DecodeParams p;
  std::memset(&p, 0, sizeof(p));
  int rc;
  if ((rc = make_tmap(&p.tmap_w, b, N, K, ldb, 2, kBlockM))) return rc;
  const int tok = decode_tok(M);
  if ((rc = make_tmap(&p.tmap_x, a, M, K, lda, 2, tok))) return rc;
  p.out = d; p.ld_out = ldd;
  p.M = static_cast<int32_t>(M); p.N = static_cast<int32_t>(N); p.K = static_cast<int32_t>(K);
  p.split = split;
  p.timeout_ns = g_timeout_ns;
  p.profile = g_profile;
  void* fn = tok == 32 ? reinterpret_cast<void*>(decode_gemm_kernel<32>) : reinterpret_cast<void*>(decode_gemm_kernel<64>);
  static std::atomic<bool> configured[kMaxDevices][2] = {};
  const int dev = current_device();
  if (dev < 0) return EDM_ERR_UNSUPPORTED;
  std::atomic<bool>& done = configured[dev][tok == 32 ? 0 : 1];
  if (!done.load(std::memory_order_acquire)) {
    EDM_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes));
    done.store(true, std::memory_order_release);
  }
  dbg_reset();
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kDecThreads); cfg.dynamicSmemBytes = kDecSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  // Every cluster must be resident at once or the launch runs in waves (a cluster needs `split`
  // free SMs inside one GPC; with one CTA per SM not every split that fits by SM count fits by
  // cluster count).  Clusters that can be active per (variant, split), asked once per device.
  static std::atomic<int> active[kMaxDevices][2][4] = {};
  for (; split > 1; split /= 2) {
    const int si = split == 2 ? 1 : (split == 4 ? 2 : 3);
    std::atomic<int>& slot = active[dev][tok == 32 ? 0 : 1][si];
    int n = slot.load(std::memory_order_acquire);
    if (n == 0) {
      cfg.gridDim = dim3(tiles * split);
      at[0].val.clusterDim.x = split;
      if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = -1; }
      slot.store(n, std::memory_order_release);
    }
    if (n < 0 || tiles <= n) break;  // (unknown: keep the planned split)
  }
  p.split = split;
  cfg.gridDim = dim3(tiles * split);
  at[0].val.clusterDim.x = split;
  void* args[1] = {&p};
  EDM_CUDA(cudaLaunchKernelExC(&cfg, fn, args));
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
  if (dtype == EDM_DTYPE_FP32) {  // before any CUDA call: a bad size must never reach a launch
    const size_t need = split_ws_bytes(M, N, K);
    if (!ws || need == 0 || ws_bytes < need) return EDM_ERR_CAPACITY;
  }
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  RankParams& P = lp.r[0];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cg = pick_cta_group(dtype, EDM_OP_GEMM, M, 1);
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  int dec_tiles = 0, dec_split = 0;
  if (decode_plan(dtype, M, N, K, sms, &dec_tiles, &dec_split))
    return decode_gemm(a, lda, b, ldb, d, ldd, M, N, K, dec_tiles, dec_split, s);
  const int bn = pick_block_n(dtype, cg, M, N, K, sms, max_tail_parts(s));
  rc = prepare_operands(P, dtype, cg, bn, a, lda, M, b, ldb, N, K, ws, ws_bytes, s);
  if (rc) return rc;
  P.M = static_cast<int32_t>(M); P.N = static_cast<int32_t>(N); P.K = static_cast<int32_t>(K);
  P.rank = 0; P.world = 1; P.mode = kPlain; P.epoch = 1;
  P.out = d; P.ld_out = ldd;
  dbg_reset();
  dbg_add_matrix(d, M, N, ldd, out_bytes);
  dbg_add(ws, ws_bytes);
  int resident = 0;
  if ((rc = max_resident_ctas(dtype, cg, sms, &resident))) return rc;
  const int tiles = static_cast<int>(((M + kBlockM * cg - 1) / (kBlockM * cg)) * ((N + bn - 1) / bn));
  apply_tuning(lp, s);
  const int grid = grid_for_tiles(tiles, cg, resident, bn == kBlockN && dtype == EDM_DTYPE_BF16, K, lp.tail_split);
  lp.num_vranks = 1;
  lp.ctas_per_vrank = grid;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  return launch_with_scratch(launch_splits(lp, P, dtype, cg, bn, grid), s,
                             [&] { return launch_variant(dtype, cg, bn, lp, grid, false, s); });
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
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

extern "C" int edm_gemm_fp32_static(const void* a, int64_t lda, const void* b, int64_t ldb, void* d,
                                    int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream) {
  if (!a || !b || !d) return EDM_ERR_BAD_ARG;
  int rc = check_dims(M, N, K);
  if (rc) return rc;
  if (K % 4 || N % 4 || lda < K || ldb < K || ldd < N) return EDM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(d) & 15u) || ((ldd * 4) & 15)) return EDM_ERR_BAD_ARG;
  // operands too large for the fixed scratch (checked term by term: huge extents must not wrap)
  if (split_operand_bytes(M, N, K, kStaticSplitBytes) == 0) return EDM_ERR_CAPACITY;
  const size_t a_sz = align_up(static_cast<size_t>(M) * K * 4, 256);
  const size_t b_sz = align_up(static_cast<size_t>(N) * K * 4, 256);

  // Set-up, once per device, with that device current: resolve the device address of the array.
  static std::atomic<char*> scratch_of_device[kMaxDevices] = {};
  int dev = 0;
  EDM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return EDM_ERR_UNSUPPORTED;
  char* w = scratch_of_device[dev].load(std::memory_order_acquire);
  if (w == nullptr) {
    void* p = nullptr;
    EDM_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return EDM_ERR_CUDA;
    w = static_cast<char*>(p);
    scratch_of_device[dev].store(w, std::memory_order_release);  // two threads may both resolve it: same value
  }

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
  dbg_reset();
  dbg_add_matrix(d, M, N, ldd, 4);
  dbg_add(w, kStaticScratchBytes);
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
  int streams_in_use = 0;    // side streams the launch being issued has put copies on

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
    if (static_cast<size_t>(W) * call.chunks * 4 > c->counter_bytes / 2) return EDM_ERR_CAPACITY;
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
    dbg_add_matrix(call.d, call.M, call.N, call.ldd, out_bytes);
    dbg_add(call.workspace, call.workspace_bytes);
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
  // two banks of arrival counters, by epoch parity: a call uses one and clears the other
  P.counters = reinterpret_cast<uint32_t*>(c->base[c->rank] + c->off_counters() + par * (c->counter_bytes / 2));
  P.counters_next = reinterpret_cast<uint32_t*>(c->base[c->rank] + c->off_counters() + (par ^ 1u) * (c->counter_bytes / 2));
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
    // which peers (rank-d, d = 1 .. W-1; d = 0 is the own shard when it is not read in place) get
    // the shard from copy engines: all, none, or the ce_peers farthest ones
    const int first_d = P.ag_local_direct ? 1 : 0;
    if (call.transport == EDM_TRANSPORT_COPY_ENGINE || call.transport == EDM_TRANSPORT_COPY_ENGINE_STRIPED) {
      P.ag_ce_lo = first_d;
    } else if (call.transport == EDM_TRANSPORT_HYBRID) {
      if (call.ce_peers < 0 || call.ce_peers > W - 1) return EDM_ERR_BAD_ARG;
      P.ag_ce_lo = W - call.ce_peers;
    } else if (call.transport == EDM_TRANSPORT_SM) {
      P.ag_ce_lo = W;
    } else {
      return EDM_ERR_BAD_ARG;
    }
    P.ag_external = P.ag_ce_lo <= first_d ? 1 : 0;
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
  const int64_t a_rows = call.op == EDM_OP_AG_GEMM ? call.M / W : call.M;
  dbg_add_matrix(call.a, a_rows, call.K, call.lda, elem_bytes);
  dbg_add_matrix(call.d, call.op == EDM_OP_GEMM_RS ? call.M / W : call.M, call.N, call.ldd, out_bytes);
  dbg_add(call.workspace, call.workspace_bytes);
  for (int p = 0; p < W; ++p) dbg_add(c->base[p], c->total_bytes);
  return EDM_OK;
}

// Copy-engine transport of one all-gather: after the caller's stream has produced the shard, the
// side stream copies it into every peer's gather buffer chunk by chunk (peer order rank-1,
// rank-2, ...: every GPU sends to and receives from one peer at a time) and raises each chunk's
// flag with a stream-ordered 32-bit write, which cannot overtake the copy before it.  No SM takes
// part, so the GEMM's operand traffic is not disturbed.  `after_launch` closes the bracket: later
// work on the caller's stream waits until the outgoing copies have read the shard.
// The caller's stream must have recorded c->ev_in at the point the shard is ready
// (ag_copy_engine_mark); the copies wait for that event only, so they may be enqueued after the
// GEMM kernel that consumes them.
int ag_copy_engine_mark(edm_comm* c, cudaStream_t stream) {
  EDM_CUDA(cudaEventRecord(c->ev_in, stream));
  return EDM_OK;
}
int ag_copy_engine_issue(edm_comm* c, const RankParams& P, int side_streams, bool striped, cudaStream_t stream) {
  (void)stream;
  WriteValue32Fn wv = write_value_fn();
  if (!wv) return EDM_ERR_UNSUPPORTED;
  const int W = P.world;
  const int64_t rows = P.M / W;
  const int elem = 2;
  const size_t row_bytes = static_cast<size_t>(P.K) * elem;
  const int64_t chunk_rows = (rows + P.ag_chunks - 1) / P.ag_chunks;
  int nstreams = side_streams > 0 ? side_streams : tuning().side_streams;
  if (nstreams < 1) nstreams = 1;
  if (nstreams > edm_comm::kSideStreams) nstreams = edm_comm::kSideStreams;
  const int d_lo = P.ag_ce_lo > (P.ag_local_direct ? 1 : 0) ? P.ag_ce_lo : (P.ag_local_direct ? 1 : 0);
  // streams are dealt by peer, or -- striped -- by chunk: then all of them serve one peer at a time
  const int lanes = striped ? P.ag_chunks : W - d_lo;
  if (lanes < nstreams) nstreams = lanes > 0 ? lanes : 1;
  c->streams_in_use = nstreams;
  for (int i = 0; i < nstreams; ++i) EDM_CUDA(cudaStreamWaitEvent(c->side[i], c->ev_in, 0));
  // when the shard does not cover whole row blocks the kernel also reads the own rows from the
  // gather buffer: deliver them (d = 0) like a peer's
  // every copy must stay inside the half of the peer's window this call uses
  if (static_cast<size_t>(P.M) * row_bytes > c->window_bytes / 2) return EDM_ERR_CAPACITY;
  for (int d = d_lo; d < W; ++d) {
    const int peer = (P.rank - d + W) % W;
    char* dst0 = static_cast<char*>(P.gather[peer]) + static_cast<size_t>(P.rank) * rows * row_bytes;
    const char* src0 = static_cast<const char*>(P.x_local);
    for (int ch = 0; ch < P.ag_chunks; ++ch) {
      const int64_t r_lo = ch * chunk_rows;
      const int64_t r_hi = r_lo + chunk_rows < rows ? r_lo + chunk_rows : rows;
      cudaStream_t side = c->side[(striped ? ch : d) % nstreams];
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
  for (int i = 0; i < c->streams_in_use; ++i) {
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
int edm_status_check(void) {
  uint32_t st[16];
  const int rc = edm_status_read(st);
  if (rc) return rc;
  return st[0] == 0 ? EDM_OK : EDM_ERR_DEVICE_TIMEOUT;
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
int edm_comm_poison(edm_comm_t* c, int byte_value, void* stream) {
  if (!c || !c->base[c->rank]) return EDM_ERR_BAD_ARG;
  EDM_CUDA(cudaMemsetAsync(c->base[c->rank] + c->off_window(), byte_value & 0xFF, c->window_bytes,
                           static_cast<cudaStream_t>(stream)));
  return EDM_OK;
}
int edm_comm_rank(const edm_comm_t* c) { return c ? c->rank : -1; }
int edm_comm_world(const edm_comm_t* c) { return c ? c->world : -1; }

int edm_tile_walk(int op, int rank, int world, int64_t M, int64_t N, int tile_m, int tile_n, int band_rows,
                  int band_cols, int units, int32_t* out, int64_t capacity, int64_t* positions) {
  if (op < EDM_OP_GEMM || op > EDM_OP_AG_GEMM || world < 1 || world > 8 || rank < 0 || rank >= world || M <= 0 ||
      N <= 0 || M > INT32_MAX || N > INT32_MAX || tile_m <= 0 || tile_n <= 0 || units < 1 || band_cols < 0 || !positions)
    return EDM_ERR_BAD_ARG;
  const int mode = op == EDM_OP_GEMM ? kPlain : op == EDM_OP_GEMM_RS ? kRS : op == EDM_OP_GEMM_AR ? kAR : kAG;
  const TileWalk walk(mode, rank, world, static_cast<int>(M), static_cast<int>(N), tile_m, tile_n, band_rows, units,
                      band_cols);
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
  int dec_tiles = 0, dec_split = 0;
  if (decode_plan(EDM_DTYPE_BF16, M, N, K, sms, &dec_tiles, &dec_split)) {
    // decode kernel: tiles of all rows x 128 columns, each cut into `split` pieces along K
    out[0] = 1; out[1] = kBlockM; out[2] = dec_tiles * dec_split; out[3] = dec_split;
    return EDM_OK;
  }
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
  if (!c || peer < 0 || peer >= c->world || !c->base[peer] || mode < 0 || mode > 3) return EDM_ERR_BAD_ARG;
  if (bytes == 0 || bytes % 32768 || bytes > c->window_bytes / 2) return EDM_ERR_CAPACITY;
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  static std::atomic<bool> configured[kMaxDevices] = {};
  const int smem = 6 * 2 * 16384 + 128;  // the largest of the modes' staging
  const int dev = current_device();
  if (dev < 0) return EDM_ERR_UNSUPPORTED;
  if (!configured[dev].load(std::memory_order_acquire)) {
    EDM_CUDA(cudaFuncSetAttribute(p2p_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev].store(true, std::memory_order_release);
  }
  // source: first half of the local window; destination: second half of the peer's
  const char* src = c->base[c->rank] + c->off_window();
  char* dst = c->base[peer] + c->off_window() + c->window_bytes / 2;
  p2p_probe_kernel<<<sms, 256, smem, static_cast<cudaStream_t>(stream)>>>(src, dst, bytes, mode);
  EDM_CUDA(cudaGetLastError());
  return EDM_OK;
}

// Row blocks per band of the tile walk of an all-gather launch, when the caller leaves it open.
// The walk of a band finishes all its row blocks column by column, so a band reaches as far ahead
// as it is tall: with weights small enough to stay in L2 whatever the band height (B re-read per
// band costs nothing then) the band is one chunk of a shard, and tiles start as soon as the first
// chunk of a shard has landed instead of when its last one has.  0: the kernel's default.
static int ag_band_for(const edm_tp_call_t& call, const RankParams& P, int cg) {
  if (P.mode != kAG || P.world <= 1 || call.band_rows > 0 || tuning().band > 0) return 0;
  if (static_cast<int64_t>(P.N) * P.K * 2 > (32ll << 20)) return 0;
  const int64_t chunk_rows = (P.M / P.world + P.ag_chunks - 1) / P.ag_chunks;
  const int64_t blocks = chunk_rows / (kBlockM * cg);
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 16 ? 16 : blocks));
}

// Dedicated pusher CTAs of an all-gather launch with `per_rank` CTAs per rank: whole pairs, and at
// least one unit is left for the tiles.  0 when the kernel pushes nothing.
static int pusher_ctas_for(const edm_tp_call_t& call, const RankParams& P, int cg, int per_rank, int* out) {
  *out = 0;
  if (P.mode != kAG || P.world <= 1 || P.ag_external) return EDM_OK;
  if (call.pusher_ctas < 0) return EDM_ERR_BAD_ARG;
  const int n = call.pusher_ctas / cg * cg;
  if (n > per_rank - cg) return EDM_ERR_BAD_ARG;
  *out = n;
  return EDM_OK;
}

// One-shot all-reduce: fills one rank's parameters (bumping the context's call counter) and runs
// that rank's plain GEMM into its window bank.
static int one_shot_rank(edm_comm* c, const edm_tp_call_t& call, OneShotRank& R, cudaStream_t s) {
  if (!c || !call.a || !call.b || !call.d) return EDM_ERR_BAD_ARG;
  if (call.op != EDM_OP_GEMM_AR || c->world < 2 || c->world > kOneShotMaxRanks) return EDM_ERR_BAD_ARG;
  if (call.dtype != EDM_DTYPE_BF16 && call.dtype != EDM_DTYPE_FP32) return EDM_ERR_BAD_ARG;
  int rc = check_dims(call.M, call.N, call.K);
  if (rc) return rc;
  const int ob = call.dtype == EDM_DTYPE_BF16 ? 2 : 4;
  if ((call.N * ob) & 15 || (call.ldd * ob) & 15 || call.ldd < call.N || (reinterpret_cast<uintptr_t>(call.d) & 15u))
    return EDM_ERR_BAD_ARG;
  const size_t need = static_cast<size_t>(call.M) * static_cast<size_t>(call.N) * ob;
  if (need > c->window_bytes / 2) return EDM_ERR_CAPACITY;
  for (int p = 0; p < c->world; ++p)
    if (!c->base[p]) return EDM_ERR_BAD_ARG;  // peers not linked yet
  const uint32_t epoch = c->epoch + 1;
  const size_t par = epoch & 1u;
  std::memset(&R, 0, sizeof(R));
  for (int p = 0; p < c->world; ++p) {
    R.part[p] = c->base[p] + c->off_window() + par * (c->window_bytes / 2);
    R.flags[p] = reinterpret_cast<uint32_t*>(c->base[p] + c->off_flags() + par * (c->flag_bytes / 2));
  }
  R.out = call.d; R.ld_out = call.ldd;
  R.M = static_cast<int32_t>(call.M); R.N = static_cast<int32_t>(call.N);
  R.rank = c->rank; R.world = c->world; R.epoch = epoch; R.out_bytes = ob;
  rc = plain_gemm(call.dtype, call.a, call.lda, call.b, call.ldb, const_cast<char*>(R.part[c->rank]), call.N,
                  call.M, call.N, call.K, call.workspace, call.workspace_bytes, s);
  if (rc) return rc;
  c->epoch = epoch;
  return EDM_OK;
}

// CTAs per rank of the one-shot reduction: about one 16-byte vector per thread (the kernel is a
// single round trip of loads then), within what is co-resident.
static int one_shot_ctas(const OneShotRank& R, int limit) {
  const int64_t vecs = static_cast<int64_t>(R.M) * R.N * R.out_bytes / 16;
  int64_t n = (vecs + kOneShotThreads - 1) / kOneShotThreads;
  if (n > limit) n = limit;
  return static_cast<int>(n < 1 ? 1 : n);
}

static int one_shot_launch(OneShotParams& lp, int n, bool coop, cudaStream_t s) {
  lp.num_vranks = n;
  lp.timeout_ns = g_timeout_ns;
  dbg_reset();
  for (int i = 0; i < n; ++i) {
    const OneShotRank& R = lp.r[i];
    dbg_add_matrix(R.out, R.M, R.N, R.ld_out, R.out_bytes);
    for (int p = 0; p < R.world; ++p) {
      dbg_add(const_cast<char*>(R.part[p]), static_cast<size_t>(R.M) * R.N * R.out_bytes);
      dbg_add(R.flags[p], static_cast<size_t>(R.world) * 4);
    }
  }
  if (int rc = dbg_publish(s)) return rc;
  const int grid = lp.ctas_per_vrank * n;
  if (coop) {
    void* args[] = {&lp};
    EDM_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ar_one_shot_kernel), dim3(grid), dim3(kOneShotThreads),
                                         args, 0, s));
  } else {
    ar_one_shot_kernel<<<grid, kOneShotThreads, 0, s>>>(lp);
    EDM_CUDA(cudaGetLastError());
  }
  return EDM_OK;
}

int edm_tp_launch(edm_comm_t* comm, const edm_tp_call_t* call, void* stream) {
  if (!comm || !call) return EDM_ERR_BAD_ARG;
  if (call->one_shot != 0 && call->one_shot != 1) return EDM_ERR_BAD_ARG;
  if (call->one_shot && comm->world > 1) {
    cudaStream_t s1 = static_cast<cudaStream_t>(stream);
    if (capturing(s1)) return EDM_ERR_UNSUPPORTED;  // the flags carry the call counter (see below)
    OneShotParams op;
    std::memset(&op, 0, sizeof(op));
    if (int rc = one_shot_rank(comm, *call, op.r[0], s1)) return rc;
    const int sms = num_sms();
    if (sms <= 0) return EDM_ERR_CUDA;
    op.ctas_per_vrank = one_shot_ctas(op.r[0], sms);
    return one_shot_launch(op, 1, false, s1);
  }
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the exchange flags carry the context's call counter, which a replay of a captured launch
  // would repeat: fused launches cannot be captured
  if (comm->world > 1 && capturing(s)) return EDM_ERR_UNSUPPORTED;
  const int cg = pick_cta_group(call->dtype, call->op, call->M, comm->world);
  dbg_reset();
  int rc = build_rank_params(comm, *call, cg, lp.r[0], s);
  if (rc) return rc;
  const RankParams& P = lp.r[0];
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  int resident = 0;
  if ((rc = max_resident_ctas(call->dtype, cg, sms, &resident))) return rc;
  const int grid = grid_for(P, cg, resident);
  lp.num_vranks = 1;
  lp.ctas_per_vrank = grid;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  apply_tuning(lp, s);
  if (call->band_rows > 0) lp.band = call->band_rows;
  else if (const int b = ag_band_for(*call, P, cg)) lp.band = b;
  if (call->band_cols > 0) lp.band_cols = call->band_cols;
  if ((rc = pusher_ctas_for(*call, P, cg, grid, &lp.pusher_ctas))) return rc;
  const bool ce = P.mode == kAG && P.world > 1 && P.ag_ce_lo < P.world;
  // the kernel goes first (it starts on this rank's own shard); the copies only wait for the
  // point on the caller's stream where the shard was ready
  if (ce && (rc = ag_copy_engine_mark(comm, s))) return rc;
  rc = launch_with_scratch(launch_splits(lp, P, call->dtype, cg, kBlockN, grid), s,
                           [&] { return launch_variant(call->dtype, cg, kBlockN, lp, grid, false, s); });
  if (rc) return rc;
  if (ce) {
    if ((rc = ag_copy_engine_issue(comm, P, call->side_streams, call->transport == EDM_TRANSPORT_COPY_ENGINE_STRIPED, s)))
      return rc;
    return ag_copy_engine_after_launch(comm, s);
  }
  return EDM_OK;
}

int edm_tp_launch_emulated(edm_comm_t* const* comms, const edm_tp_call_t* calls, int n, void* stream) {
  if (!comms || !calls || n < 1 || n > kMaxVirtualRanks) return EDM_ERR_BAD_ARG;
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (capturing(s)) return EDM_ERR_UNSUPPORTED;  // see edm_tp_launch
  if (calls[0].one_shot != 0 && calls[0].one_shot != 1) return EDM_ERR_BAD_ARG;
  if (calls[0].one_shot && comms[0] && comms[0]->world > 1) {
    // every rank's GEMM first, then one cooperative launch in which the ranks' CTAs exchange flags
    OneShotParams op;
    std::memset(&op, 0, sizeof(op));
    for (int i = 0; i < n; ++i) {
      if (!comms[i] || calls[i].one_shot != 1 || calls[i].dtype != calls[0].dtype || calls[i].M != calls[0].M ||
          calls[i].N != calls[0].N)
        return EDM_ERR_BAD_ARG;
      if (int rc = one_shot_rank(comms[i], calls[i], op.r[i], s)) return rc;
    }
    const int sms = num_sms();
    if (sms < n) return EDM_ERR_CUDA;
    op.ctas_per_vrank = one_shot_ctas(op.r[0], sms / n);
    return one_shot_launch(op, n, true, s);
  }
  const int cg = pick_cta_group(calls[0].dtype, calls[0].op, calls[0].M, comms[0] ? comms[0]->world : 1);
  dbg_reset();
  for (int i = 0; i < n; ++i) {
    if (!comms[i] || calls[i].dtype != calls[0].dtype || calls[i].op != calls[0].op ||
        calls[i].M != calls[0].M || calls[i].pusher_ctas != calls[0].pusher_ctas ||
        calls[i].band_rows != calls[0].band_rows || calls[i].band_cols != calls[0].band_cols)
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
  if (calls[0].band_rows > 0) lp.band = calls[0].band_rows;
  else if (const int b = ag_band_for(calls[0], lp.r[0], cg)) lp.band = b;
  if (calls[0].band_cols > 0) lp.band_cols = calls[0].band_cols;
  if ((rc = pusher_ctas_for(calls[0], lp.r[0], cg, lp.ctas_per_vrank, &lp.pusher_ctas))) return rc;
  // Copies between buffers of ONE device may be carried out by kernels, which cannot start while
  // the cooperative launch holds every SM (a chunked copy would then starve behind it until the
  // kernel's waits run out).  The emulation therefore lets the copies finish first: the kernel
  // still finds its rows through the chunk flags and the gather buffer, only the overlap -- which
  // a single device cannot show anyway -- is given up.
  bool splits = false;
  for (int i = 0; i < n; ++i) {
    const RankParams& P = lp.r[i];
    splits = splits || launch_splits(lp, P, calls[0].dtype, cg, kBlockN, lp.ctas_per_vrank * n);
    if (P.mode == kAG && P.world > 1 && P.ag_ce_lo < P.world) {
      if ((rc = ag_copy_engine_mark(comms[i], s))) return rc;
      if ((rc = ag_copy_engine_issue(comms[i], P, calls[i].side_streams,
                                     calls[i].transport == EDM_TRANSPORT_COPY_ENGINE_STRIPED, s)))
        return rc;
      if ((rc = ag_copy_engine_after_launch(comms[i], s))) return rc;
    }
  }
  return launch_with_scratch(splits, s, [&] {
    return launch_variant(calls[0].dtype, cg, kBlockN, lp, lp.ctas_per_vrank * n, true, s);
  });
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

// ======================================================================== mixture of experts
namespace {

struct MoeLayout {
  int W, E_local, C, max_blocks;
  // window (inside the parity half)
  size_t w_counts, w_xbuf, w_meta, w_cbuf, window_need;
  // workspace
  size_t s_idx, s_w, s_slot, s_tgu, s_tdn, s_nblk, s_ctr, s_y, s_act, s_z, workspace_need;
};

int moe_layout(int64_t T, int64_t H, int64_t F, int64_t E, int W, MoeLayout& L) {
  if (T < 1 || H < 8 || F < 8 || E < 2 || W < 1 || W > EDM_MAX_RANKS) return EDM_ERR_BAD_ARG;
  if (E > kMoeMaxExperts || E % W || H % 8 || F % 8) return EDM_ERR_BAD_ARG;
  if (T > (1 << 22) || H > (1 << 20) || F > (1 << 20)) return EDM_ERR_BAD_ARG;
  L.W = W;
  L.E_local = static_cast<int>(E / W);
  L.C = static_cast<int>(align_up(static_cast<size_t>(T) * W, 256));  // a token sends at most one row to an expert
  L.max_blocks = L.E_local * (L.C / 256);
  const size_t rows = static_cast<size_t>(L.E_local) * L.C;
  size_t o = 0;
  auto take = [&](size_t bytes) { const size_t at = o; o = align_up(o + bytes, 256); return at; };
  L.w_counts = take(static_cast<size_t>(W) * E * 4);
  L.w_xbuf = take(rows * H * 2);
  L.w_meta = take(rows * 4);
  L.w_cbuf = take(static_cast<size_t>(T) * 2 * H * 2);
  L.window_need = o;
  o = 0;
  L.s_idx = take(static_cast<size_t>(T) * 2 * 4);
  L.s_w = take(static_cast<size_t>(T) * 2 * 4);
  L.s_slot = take(static_cast<size_t>(T) * 2 * 4);
  L.s_tgu = take(static_cast<size_t>(L.max_blocks) * 16);
  L.s_tdn = take(static_cast<size_t>(L.max_blocks) * 16);
  L.s_nblk = take(4);
  L.s_ctr = take(8);
  L.s_y = take(rows * 2 * F * 2);
  L.s_act = take(rows * F * 2);
  L.s_z = take(rows * H * 2);
  L.workspace_need = o;
  return EDM_OK;
}

// One launch of the GEMM kernel over the row blocks an earlier kernel listed in `table`.
int grouped_gemm(const void* a, int64_t lda, int64_t a_rows, const void* b, int64_t ldb, int64_t b_rows, void* d,
                 int64_t ldd, int64_t N, int64_t K, const int32_t* table, const int32_t* count, int max_blocks,
                 cudaStream_t s) {
  LaunchParams lp;
  std::memset(&lp, 0, sizeof(lp));
  RankParams& P = lp.r[0];
  const int cg = 2;
  int rc;
  if ((rc = make_tmap(&P.tmap_a[0], a, a_rows, K, lda, 2, kBlockM))) return rc;
  if ((rc = make_tmap(&P.tmap_b[0], b, b_rows, K, ldb, 2, kBlockN / cg))) return rc;
  P.tmap_a[1] = P.tmap_a[0];
  P.tmap_b[1] = P.tmap_b[0];
  P.passes = 1;
  P.M = max_blocks * kBlockM * cg;
  P.N = static_cast<int32_t>(N); P.K = static_cast<int32_t>(K);
  P.rank = 0; P.world = 1; P.mode = kPlain; P.epoch = 1;
  P.out = d; P.ld_out = ldd;
  P.group_table = table; P.group_count = count;
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  int resident = 0;
  if ((rc = max_resident_ctas(EDM_DTYPE_BF16, cg, sms, &resident))) return rc;
  apply_tuning(lp, s);
  lp.tail_split = 0;  // row blocks come from a device-side table: no split of a last wave
  lp.num_vranks = 1;
  lp.ctas_per_vrank = resident;
  lp.timeout_ns = g_timeout_ns;
  lp.profile = g_profile;
  return launch_variant(EDM_DTYPE_BF16, cg, kBlockN, lp, resident, false, s);
}

int moe_forward_impl(edm_comm_t* const* comms, const edm_moe_call_t* calls, int n, cudaStream_t s) {
  MoeParams mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.num_vranks = n;
  mp.timeout_ns = g_timeout_ns;
  MoeLayout L[kMaxVirtualRanks];
  dbg_reset();
  for (int i = 0; i < n; ++i) {
    edm_comm* c = comms[i];
    const edm_moe_call_t& call = calls[i];
    if (!c || !call.x || !call.logits || !call.w1 || !call.w2 || !call.out || !call.workspace) return EDM_ERR_BAD_ARG;
    const int W = c->world;
    for (int p = 0; p < W; ++p)
      if (!c->base[p]) return EDM_ERR_BAD_ARG;
    int rc = moe_layout(call.tokens, call.hidden, call.ffn, call.experts, W, L[i]);
    if (rc) return rc;
    if (call.tokens != calls[0].tokens || call.hidden != calls[0].hidden || call.ffn != calls[0].ffn ||
        call.experts != calls[0].experts)
      return EDM_ERR_BAD_ARG;
    if (L[i].window_need > c->window_bytes / 2 || static_cast<size_t>(3 * W) * 4 > c->flag_bytes / 2)
      return EDM_ERR_CAPACITY;
    if (call.workspace_bytes < L[i].workspace_need) return EDM_ERR_CAPACITY;
    if ((reinterpret_cast<uintptr_t>(call.workspace) & 255u) || (reinterpret_cast<uintptr_t>(call.x) & 15u) ||
        (reinterpret_cast<uintptr_t>(call.out) & 15u) || ((call.ldx * 2) & 15) || ((call.ldo * 2) & 15) ||
        call.ldx < call.hidden || call.ldo < call.hidden || call.ld_logits < call.experts ||
        call.ldw1 < call.hidden || call.ldw2 < call.ffn)
      return EDM_ERR_BAD_ARG;
    MoeRank& R = mp.r[i];
    R.T = call.tokens; R.H = call.hidden; R.F = call.ffn; R.E = call.experts;
    R.E_local = L[i].E_local; R.W = W; R.rank = c->rank; R.C = L[i].C; R.max_blocks = L[i].max_blocks;
    const uint32_t epoch = c->epoch + 1;
    R.epoch = epoch;
    const size_t par = epoch & 1u;
    R.x = static_cast<const __nv_bfloat16*>(call.x); R.ld_x = call.ldx;
    R.logits = call.logits; R.ld_logits = call.ld_logits;
    R.out = static_cast<__nv_bfloat16*>(call.out); R.ld_out = call.ldo;
    char* ws = static_cast<char*>(call.workspace);
    R.topk_idx = reinterpret_cast<int32_t*>(ws + L[i].s_idx);
    R.topk_w = reinterpret_cast<float*>(ws + L[i].s_w);
    R.slot = reinterpret_cast<int32_t*>(ws + L[i].s_slot);
    R.table_gu = reinterpret_cast<int32_t*>(ws + L[i].s_tgu);
    R.table_dn = reinterpret_cast<int32_t*>(ws + L[i].s_tdn);
    R.n_blocks = reinterpret_cast<int32_t*>(ws + L[i].s_nblk);
    R.done_ctr = reinterpret_cast<uint32_t*>(ws + L[i].s_ctr);
    R.Y = reinterpret_cast<const __nv_bfloat16*>(ws + L[i].s_y);
    R.act = reinterpret_cast<__nv_bfloat16*>(ws + L[i].s_act);
    R.Z = reinterpret_cast<const __nv_bfloat16*>(ws + L[i].s_z);
    for (int p = 0; p < W; ++p) {
      char* win = c->base[p] + c->off_window() + par * (c->window_bytes / 2);
      R.counts[p] = reinterpret_cast<uint32_t*>(win + L[i].w_counts);
      R.xbuf[p] = reinterpret_cast<__nv_bfloat16*>(win + L[i].w_xbuf);
      R.meta[p] = reinterpret_cast<int32_t*>(win + L[i].w_meta);
      R.cbuf[p] = reinterpret_cast<__nv_bfloat16*>(win + L[i].w_cbuf);
      R.flags[p] = reinterpret_cast<uint32_t*>(c->base[p] + c->off_flags() + par * (c->flag_bytes / 2));
      dbg_add(c->base[p], c->total_bytes);
    }
    dbg_add(call.workspace, call.workspace_bytes);
    dbg_add_matrix(call.out, call.tokens, call.hidden, call.ldo, 2);
    EDM_CUDA(cudaMemsetAsync(R.done_ctr, 0, 8, s));
  }
  if (int rc = dbg_publish(s)) return rc;
  const int sms = num_sms();
  if (sms <= 0) return EDM_ERR_CUDA;
  const dim3 wide(static_cast<unsigned>(sms / n > 0 ? sms / n : 1), static_cast<unsigned>(n));
  const dim3 one(1, static_cast<unsigned>(n));
  // the row-copy and elementwise stages are latency-bound per warp: two to four CTAs per SM
  const dim3 wide2(wide.x * 2, wide.y), wide4(wide.x * 4, wide.y);
  moe_route_kernel<<<one, kMoeRouteThreads, 0, s>>>(mp);
  moe_dispatch_kernel<<<wide2, 256, 0, s>>>(mp);
  moe_plan_kernel<<<one, 64, 0, s>>>(mp);
  EDM_CUDA(cudaGetLastError());
  for (int i = 0; i < n; ++i) {
    const MoeRank& R = mp.r[i];
    const int64_t rows = static_cast<int64_t>(R.E_local) * R.C;
    int rc = grouped_gemm(R.xbuf[R.rank], R.H, rows, calls[i].w1, calls[i].ldw1, static_cast<int64_t>(R.E_local) * 2 * R.F,
                          const_cast<__nv_bfloat16*>(R.Y), 2 * R.F, 2 * R.F, R.H, R.table_gu, R.n_blocks, R.max_blocks, s);
    if (rc) return rc;
  }
  moe_silu_mul_kernel<<<wide4, 256, 0, s>>>(mp);
  EDM_CUDA(cudaGetLastError());
  for (int i = 0; i < n; ++i) {
    const MoeRank& R = mp.r[i];
    const int64_t rows = static_cast<int64_t>(R.E_local) * R.C;
    int rc = grouped_gemm(R.act, R.F, rows, calls[i].w2, calls[i].ldw2, static_cast<int64_t>(R.E_local) * R.H,
                          const_cast<__nv_bfloat16*>(R.Z), R.H, R.H, R.F, R.table_dn, R.n_blocks, R.max_blocks, s);
    if (rc) return rc;
  }
  moe_combine_kernel<<<wide2, 256, 0, s>>>(mp);
  moe_finish_kernel<<<wide4, 256, 0, s>>>(mp);
  EDM_CUDA(cudaGetLastError());
  for (int i = 0; i < n; ++i) comms[i]->epoch += 1;
  return EDM_OK;
}

}  // namespace

extern "C" {

size_t edm_moe_window_bytes(int64_t tokens, int64_t hidden, int64_t experts, int world) {
  MoeLayout L;
  if (moe_layout(tokens, hidden, 8, experts, world, L)) return 0;
  return 2 * align_up(L.window_need, 1024);
}
size_t edm_moe_workspace_bytes(int64_t tokens, int64_t hidden, int64_t ffn, int64_t experts, int world) {
  MoeLayout L;
  if (moe_layout(tokens, hidden, ffn, experts, world, L)) return 0;
  return L.workspace_need;
}
int edm_moe_routing_offsets(int64_t tokens, int64_t hidden, int64_t ffn, int64_t experts, int world, size_t out[3]) {
  MoeLayout L;
  if (!out) return EDM_ERR_BAD_ARG;
  int rc = moe_layout(tokens, hidden, ffn, experts, world, L);
  if (rc) return rc;
  out[0] = L.s_idx; out[1] = L.s_w; out[2] = L.s_slot;
  return EDM_OK;
}
int edm_moe_forward(edm_comm_t* comm, const edm_moe_call_t* call, void* stream) {
  if (!comm || !call) return EDM_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (capturing(s)) return EDM_ERR_UNSUPPORTED;  // flags carry the context's call counter
  edm_comm_t* comms[1] = {comm};
  return moe_forward_impl(comms, call, 1, s);
}
int edm_moe_forward_emulated(edm_comm_t* const* comms, const edm_moe_call_t* calls, int n, void* stream) {
  if (!comms || !calls || n < 1 || n > kMaxVirtualRanks) return EDM_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (capturing(s)) return EDM_ERR_UNSUPPORTED;
  return moe_forward_impl(comms, calls, n, s);
}

}  // extern "C"
