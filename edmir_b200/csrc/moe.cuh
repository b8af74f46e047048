// Expert-parallel mixture-of-experts layer: routing, dispatch, activation, combine.
//
// One layer call on rank r is a sequence of launches on one stream; the two grouped GEMMs between
// them are launches of tp_gemm_kernel with a row-block table (RankParams::group_table):
//
//   route     top-2 experts and their softmax weights per token; for every (token, choice) pair
//             its slot among this rank's pairs for the same expert; the per-expert counts are
//             stored into every peer's counts table and a flag is raised there
//   dispatch  waits for every rank's counts, derives where this rank's pairs start in each
//             expert's buffer, stores the token rows (and a word naming their origin) into the
//             buffer of the rank that owns the expert; the last CTA raises a flag at every peer
//   plan      waits for every rank's rows, builds the row-block tables of the two grouped GEMMs
//   [GEMM]    Y = X_e W1_e^T for the experts of this rank              (gate and up projections)
//   silu_mul  act = silu(Y[:, :F]) * Y[:, F:]
//   [GEMM]    Z = act W2_e^T                                            (down projection)
//   combine   stores every row of Z into the combine buffer of the rank its token came from,
//             at (token, choice); the last CTA raises a flag at every peer
//   finish    waits for every rank's rows, out[t] = w0 * C[t,0] + w1 * C[t,1]
//
// The all-to-all exchanges are stores into symmetric peer windows plus release/acquire flag
// words, like the tile pushes of the fused linears.  A stage only ever waits for what the peers'
// PREVIOUS stage produced, so no launch depends on a launch behind it on any rank, and when
// several ranks are emulated on one device (every stage is then one launch over all ranks,
// blockIdx.y = rank) every wait is already satisfied when its kernel starts.  All waits are
// bounded (wait_flag); a wait that gives up makes its kernel return without touching anything.
//
// Integer conventions (they make routing results comparable bit for bit with a host restatement):
// equal logits go to the lower expert index; pairs are ordered by (source rank, token, choice);
// expert e lives on rank e / (E / W).
#pragma once
#include "tp_gemm.cuh"

namespace edm {

constexpr int kMoeMaxExperts = 64;
constexpr int kMoeRouteThreads = 1024;

struct MoeRank {
  int32_t T, H, F, E, E_local, W, rank;
  int32_t C;            // rows reserved per local expert (a multiple of 256: row blocks never straddle experts)
  uint32_t epoch;
  int32_t max_blocks;   // capacity of the row-block tables
  const __nv_bfloat16* x; int64_t ld_x;       // [T, H]
  const float* logits; int64_t ld_logits;     // [T, E]
  __nv_bfloat16* out; int64_t ld_out;         // [T, H]
  // local scratch
  int32_t* topk_idx;    // [T * 2]
  float* topk_w;        // [T * 2]
  int32_t* slot;        // [T * 2] position of the pair among this rank's pairs for its expert
  int32_t* table_gu;    // [max_blocks][4] row blocks of the gate_up GEMM
  int32_t* table_dn;    // [max_blocks][4] row blocks of the down GEMM
  int32_t* n_blocks;    // [1]
  uint32_t* done_ctr;   // [2] CTAs that have finished their stores (dispatch, combine); zero between calls
  const __nv_bfloat16* Y;    // [E_local * C, 2F]
  __nv_bfloat16* act;        // [E_local * C, F]
  const __nv_bfloat16* Z;    // [E_local * C, H]
  // symmetric: the same objects on every rank, as mapped here
  uint32_t* counts[kMaxRanks];      // [W][E] pairs rank w sends to expert e
  __nv_bfloat16* xbuf[kMaxRanks];   // [E_local * C, H] rows received per expert
  int32_t* meta[kMaxRanks];         // [E_local * C] origin of each row: rank << 24 | token * 2 + choice
  __nv_bfloat16* cbuf[kMaxRanks];   // [T * 2, H] expert outputs returned per (token, choice)
  uint32_t* flags[kMaxRanks];       // [3 * W] counts / rows / results of rank w have landed
};
struct MoeParams {
  int32_t num_vranks;
  uint64_t timeout_ns;
  MoeRank r[kMaxVirtualRanks];
};

// Exclusive prefix sum of `v` over the block (blockDim.x a multiple of 32, at most 1024); *total
// receives the block-wide sum.  `tmp` holds 33 words.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* tmp, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += up;
  }
  if (lane == 31) tmp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    uint32_t w = lane < nw ? tmp[lane] : 0u, winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += up;
    }
    tmp[lane] = winc - w;                 // offset of each warp
    if (lane == 31) tmp[32] = winc;       // block total
  }
  __syncthreads();
  const uint32_t base = tmp[warp];
  *total = tmp[32];
  __syncthreads();  // tmp may be reused right away
  return base + inc - v;
}

// ------------------------------------------------------------------ route
__global__ void __launch_bounds__(kMoeRouteThreads, 1) moe_route_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  __shared__ uint32_t tmp[33];
  __shared__ uint32_t totals[kMoeMaxExperts];
  const int tid = threadIdx.x;
  // top-2 and weights
  for (int t = tid; t < R.T; t += blockDim.x) {
    const float* row = R.logits + static_cast<int64_t>(t) * R.ld_logits;
    int i0 = 0;
    float l0 = row[0];
    for (int e = 1; e < R.E; ++e) {
      const float v = row[e];
      if (v > l0) { l0 = v; i0 = e; }   // strict: equal logits stay with the lower index
    }
    int i1 = i0 == 0 ? 1 : 0;
    float l1 = row[i1];
    for (int e = i1 + 1; e < R.E; ++e) {
      if (e == i0) continue;
      const float v = row[e];
      if (v > l1) { l1 = v; i1 = e; }
    }
    const float e1 = __expf(l1 - l0);   // l0 >= l1
    R.topk_idx[2 * t] = i0; R.topk_idx[2 * t + 1] = i1;
    R.topk_w[2 * t] = 1.f / (1.f + e1); R.topk_w[2 * t + 1] = e1 / (1.f + e1);
  }
  __syncthreads();
  // slots: thread i owns a run of consecutive pairs, so (token, choice) order is thread order
  const int pairs = 2 * R.T;
  const int per = (pairs + blockDim.x - 1) / blockDim.x;
  const int lo = min(tid * per, pairs), hi = min(lo + per, pairs);
  for (int e = 0; e < R.E; ++e) {
    uint32_t mine = 0;
    for (int i = lo; i < hi; ++i) mine += R.topk_idx[i] == e ? 1u : 0u;
    uint32_t total;
    uint32_t at = block_exclusive_scan(mine, tmp, &total);
    for (int i = lo; i < hi; ++i)
      if (R.topk_idx[i] == e) R.slot[i] = static_cast<int32_t>(at++);
    if (tid == 0) totals[e] = total;
  }
  __syncthreads();
  // every rank learns how many pairs this rank sends to each expert
  for (int i = tid; i < R.W * R.E; i += blockDim.x) {
    const int peer = i / R.E, e = i - peer * R.E;
    uint32_t* dst = R.counts[peer] + R.rank * R.E + e;
    if (EDM_ADDR_OK(dst, 4, 30u)) *reinterpret_cast<volatile uint32_t*>(dst) = totals[e];
  }
  __syncthreads();
  if (tid == 0) {
    fence_acq_rel_sys();
    for (int peer = 0; peer < R.W; ++peer)
      if (EDM_ADDR_OK(R.flags[peer] + R.rank, 4, 31u)) st_relaxed_sys(R.flags[peer] + R.rank, R.epoch);
  }
}

// All threads of the block return true when the W flags at R.flags[rank][base .. base+W) have
// reached the epoch.
__device__ __forceinline__ bool moe_wait_all(const MoeRank& R, int base, uint64_t timeout_ns, uint32_t code) {
  bool ok = true;
  if (static_cast<int>(threadIdx.x) < R.W)
    ok = wait_flag(R.flags[R.rank] + base + threadIdx.x, R.epoch, timeout_ns, code, base + threadIdx.x);
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Called by every thread after the block's stores: the last block of the grid row to arrive
// raises the flag `slot` of this rank at every peer and re-arms the counter.
__device__ __forceinline__ void moe_publish_when_last(const MoeRank& R, uint32_t* ctr, int slot) {
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
      *reinterpret_cast<volatile uint32_t*>(ctr) = 0u;
      fence_acq_rel_sys();
      for (int peer = 0; peer < R.W; ++peer)
        if (EDM_ADDR_OK(R.flags[peer] + slot * R.W + R.rank, 4, 32u))
          st_relaxed_sys(R.flags[peer] + slot * R.W + R.rank, R.epoch);
    }
  }
}

// One warp copies `bytes` (a multiple of 16) from src to dst with 16-byte accesses.
__device__ __forceinline__ void warp_copy_row(char* dst, const char* src, int bytes, int lane, uint32_t site) {
  if (!EDM_ADDR_OK(dst, bytes, site)) return;
  for (int v = lane * 16; v < bytes; v += 32 * 16 * 4) {
    uint4 b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v + u * 512 < bytes) b[u] = ld_cg_v4(src + v + u * 512);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v + u * 512 < bytes) st_global_v4(dst + v + u * 512, b[u]);
  }
}

// ------------------------------------------------------------------ dispatch
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  __shared__ uint32_t base[kMoeMaxExperts];
  if (!moe_wait_all(R, 0, p.timeout_ns, kTimeoutGatherFlag)) return;
  if (static_cast<int>(threadIdx.x) < R.E) {
    uint32_t b = 0;
    for (int w = 0; w < R.rank; ++w) b += ld_relaxed_sys(R.counts[R.rank] + w * R.E + threadIdx.x);
    base[threadIdx.x] = b;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int row_bytes = R.H * 2;
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < 2 * R.T; i += warps) {
    const int e = R.topk_idx[i];
    const int dst_rank = e / R.E_local;
    const int64_t row = static_cast<int64_t>(e - dst_rank * R.E_local) * R.C + base[e] + R.slot[i];
    warp_copy_row(reinterpret_cast<char*>(R.xbuf[dst_rank]) + row * row_bytes,
                  reinterpret_cast<const char*>(R.x) + static_cast<int64_t>(i >> 1) * R.ld_x * 2, row_bytes, lane, 33u);
    if (lane == 0 && EDM_ADDR_OK(R.meta[dst_rank] + row, 4, 34u)) R.meta[dst_rank][row] = (R.rank << 24) | i;
  }
  moe_publish_when_last(R, R.done_ctr, 1);
}

// ------------------------------------------------------------------ plan
__global__ void __launch_bounds__(64) moe_plan_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  const bool ok = moe_wait_all(R, R.W, p.timeout_ns, kTimeoutGatherFlag);
  if (threadIdx.x != 0) return;
  int j = 0;
  if (ok) {
    for (int el = 0; el < R.E_local; ++el) {
      const int e = R.rank * R.E_local + el;
      int rows = 0;
      for (int w = 0; w < R.W; ++w) rows += static_cast<int>(ld_relaxed_sys(R.counts[R.rank] + w * R.E + e));
      for (int r0 = 0; r0 < rows && j < R.max_blocks; r0 += 256, ++j) {
        const int n = min(256, rows - r0);
        reinterpret_cast<int4*>(R.table_gu)[j] = make_int4(el * R.C + r0, el * 2 * R.F, n, e);
        reinterpret_cast<int4*>(R.table_dn)[j] = make_int4(el * R.C + r0, el * R.H, n, e);
      }
    }
  }
  *R.n_blocks = j;  // zero when the wait gave up: the GEMMs then do nothing
}

// Rows of the expert buffers that hold a token, in table order: q = block * 256 + row.
__device__ __forceinline__ bool moe_row_of(const MoeRank& R, int q, int64_t& row) {
  const int4 e = reinterpret_cast<const int4*>(R.table_dn)[q >> 8];
  if ((q & 255) >= e.z) return false;
  row = static_cast<int64_t>(e.x) + (q & 255);
  return true;
}

// ------------------------------------------------------------------ silu(gate) * up
__global__ void __launch_bounds__(256) moe_silu_mul_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int total = *R.n_blocks * 256;
  for (int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); q < total; q += warps) {
    int64_t row;
    if (!moe_row_of(R, q, row)) continue;
    const int row_bytes = R.F * 2;
    const char* y = reinterpret_cast<const char*>(R.Y) + row * (2 * R.F) * 2;
    char* a = reinterpret_cast<char*>(R.act) + row * R.F * 2;
    // a pure HBM pass (3 F elements per row): eight 16-byte loads per lane are in flight before
    // any is used -- with two the kernel ran at a quarter of the copy bandwidth
    constexpr int kU = 4;
    for (int v0 = lane * 16; v0 < row_bytes; v0 += 32 * 16 * kU) {
      uint4 g[kU], u[kU];
#pragma unroll
      for (int j = 0; j < kU; ++j) {
        const int v = v0 + j * 32 * 16;
        if (v < row_bytes) {
          g[j] = ld_cg_v4(y + v);
          u[j] = ld_cg_v4(y + row_bytes + v);
        }
      }
#pragma unroll
      for (int j = 0; j < kU; ++j) {
        const int v = v0 + j * 32 * 16;
        if (v < row_bytes) {
          const uint32_t gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w}, uw[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
          uint32_t ow[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xFFFF0000u);
            const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xFFFF0000u);
            const __nv_bfloat162 o = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
            ow[k] = *reinterpret_cast<const uint32_t*>(&o);
          }
          st_global_v4(a + v, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
      }
    }
  }
}

// ------------------------------------------------------------------ combine
__global__ void __launch_bounds__(256) moe_combine_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int total = *R.n_blocks * 256;
  const int row_bytes = R.H * 2;
  for (int q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); q < total; q += warps) {
    int64_t row;
    if (!moe_row_of(R, q, row)) continue;
    const int m = R.meta[R.rank][row];
    const int src = m >> 24, pair = m & 0xFFFFFF;
    if (src < 0 || src >= R.W || pair >= 2 * R.T) continue;  // a row nobody wrote (only after a failed wait)
    warp_copy_row(reinterpret_cast<char*>(R.cbuf[src]) + static_cast<int64_t>(pair) * row_bytes,
                  reinterpret_cast<const char*>(R.Z) + row * row_bytes, row_bytes, lane, 35u);
  }
  moe_publish_when_last(R, R.done_ctr + 1, 2);
}

// ------------------------------------------------------------------ finish
__global__ void __launch_bounds__(256) moe_finish_kernel(const __grid_constant__ MoeParams p) {
  const MoeRank& R = p.r[blockIdx.y];
  if (!moe_wait_all(R, 2 * R.W, p.timeout_ns, kTimeoutResultFlag)) return;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const char* c = reinterpret_cast<const char*>(R.cbuf[R.rank]);
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < R.T; t += warps) {
    const float w0 = R.topk_w[2 * t], w1 = R.topk_w[2 * t + 1];
    const char* r0 = c + static_cast<int64_t>(2 * t) * R.H * 2;
    const char* r1 = r0 + R.H * 2;
    char* o = reinterpret_cast<char*>(R.out) + static_cast<int64_t>(t) * R.ld_out * 2;
    for (int v = lane * 16; v < R.H * 2; v += 32 * 16) {
      const uint4 a = ld_cg_v4(r0 + v), b = ld_cg_v4(r1 + v);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = w0 * __uint_as_float(aw[k] << 16) + w1 * __uint_as_float(bw[k] << 16);
        const float hi = w0 * __uint_as_float(aw[k] & 0xFFFF0000u) + w1 * __uint_as_float(bw[k] & 0xFFFF0000u);
        const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
        ow[k] = *reinterpret_cast<const uint32_t*>(&r);
      }
      st_global_v4(o + v, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
  }
}

}  // namespace edm
