// Decode-sized GEMM: D[M, N] = X[M, K] * W[N, K]^T with M <= 64 tokens.
//
// With a handful of tokens the job is to stream the weights through the SMs once, at the rate of
// the HBM.  The general kernel puts the tokens on the 128 TMEM lanes (the MMA's M side) and 32 or
// 256 weight rows on its N side; an MMA then costs the same however few of its 128 rows are real,
// and a CTA cannot issue them fast enough to keep up with its share of the weights.  Here the
// operands are swapped: 128 weight rows are the MMA's M side, the tokens (padded to kTok = 32 or
// 64) its N side, so every MMA consumes 4 KiB of weights.  (kTok = 128 also works but is no faster
// than the general kernel: every CTA then re-reads as many token bytes as it streams weights.)  A tile is 128 output columns for all tokens.
// With N = 4096 that makes 32 tiles, so each tile's K range is cut into `split` pieces that run
// as the CTAs of one thread-block cluster; the pieces' fp32 partial sums meet in the leader CTA's
// shared memory (distributed shared memory stores, two cluster barriers) and the leader writes the
// transposed result.  No global scratch, no flags: the launch can be captured.
//
// Per CTA: warp 0 loads (TMA: 128x64 weights + kTok x 64 tokens per stage), warp 1 issues the MMAs,
// warps 2-5 read the accumulator (lanes = weight rows, columns = tokens).
#pragma once
#include "tp_gemm.cuh"

namespace edm {

constexpr int kDecThreads = 192;
constexpr int kDecStageW = kBlockM * kBlockKBytes;            // 16 KiB of weights per stage
constexpr int kDecRingBytes = 192 * 1024;
constexpr int kDecSmemBytes = kDecRingBytes + 1024 /*align*/;
constexpr int kDecMaxStages = 9;
// kTok = tokens per tile = N of the MMA
template <int kTok> struct DecodeShape {
  static constexpr int kStageX = kTok * kBlockKBytes;          // 4 or 8 KiB of tokens per stage
  static constexpr int kStageBytes = kDecStageW + kStageX;
  static constexpr int kStages = kDecRingBytes / kStageBytes;  // 9 or 8
  // the pieces' partial sums (fp32, [piece-1][token][weight row]) are parked in the leader's ring
  static constexpr int kMaxSplit = kDecRingBytes / (kTok * kBlockM * 4) + 1 >= 8 ? 8 : (kDecRingBytes / (kTok * kBlockM * 4) + 1 >= 4 ? 4 : 2);
  static_assert(kStages <= kDecMaxStages && (kMaxSplit - 1) * kTok * kBlockM * 4 <= kDecRingBytes, "ring too small");
};

struct DecodeParams {
  CUtensorMap tmap_w;  // W [N, K]: box 128 rows x 64 elements
  CUtensorMap tmap_x;  // X [M, K]: box kTok rows x 64 elements (rows beyond M read as zero)
  void* out;           // [M, N] bf16
  int64_t ld_out;      // elements
  int32_t M, N, K;
  int32_t split;       // pieces of K = CTAs per cluster (1, 2, 4 or 8; at most DecodeShape::kMaxSplit)
  uint64_t timeout_ns;
  int32_t profile;     // accumulate per-CTA times into the profile slots (kernel, accumulator wait, epilogue)
};

__device__ __forceinline__ void st_shared_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

template <int kTok>
__global__ void __launch_bounds__(kDecThreads, 1)
decode_gemm_kernel(const __grid_constant__ DecodeParams p) {
  constexpr int kDecStages = DecodeShape<kTok>::kStages;
  constexpr int kDecStageBytes = DecodeShape<kTok>::kStageBytes;
  constexpr int kDecTok = kTok;
  extern __shared__ uint8_t dec_smem_raw[];
  __shared__ uint64_t bars[2 * kDecMaxStages + 1];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool prof = p.profile != 0;
  ProfTimer prof_kernel(prof && threadIdx.x == 0);
  ProfTimer prof_acc(prof && threadIdx.x == 64);   // first epilogue warp: launch to accumulator complete
  const int split = p.split;
  const int tile = blockIdx.x / split;
  const int piece = split > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int n0 = tile * kBlockM;
  const int kb_total = (p.K * 2 + kBlockKBytes - 1) / kBlockKBytes;
  const int per = (kb_total + split - 1) / split;
  const int k_lo = min(piece * per, kb_total), k_hi = min(k_lo + per, kb_total);
  const int nkb = k_hi - k_lo;  // K blocks of this piece (0: the piece contributes nothing)

  const uint32_t ring = (smem_u32(dec_smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kDecStages]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * kDecStages]);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc<1>(smem_u32(&tmem_base_slot), kDecTok);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);

  bool acc_ready = false;  // epilogue warps: the accumulator holds this piece's sum (the leader always has K blocks)
  if (warp == 0) {
    // ============================ TMA producer ============================
    if (lane == 0 && nkb > 0) {
      tma_prefetch_desc(&p.tmap_w);
      tma_prefetch_desc(&p.tmap_x);
      uint32_t s = 0, ph = 0;
      for (int j = k_lo; j < k_hi; ++j, s = (s + 1 == kDecStages ? 0 : s + 1), ph ^= (s == 0)) {
        if (!wait_mbar(bar_empty + 8 * s, ph ^ 1u, p.timeout_ns, kTimeoutEmptyBar, j)) break;
        const uint32_t sa = ring + s * kDecStageBytes;
        mbar_arrive_expect_tx(bar_full + 8 * s, kDecStageBytes);
        tma_load_2d(sa, &p.tmap_w, j * (kBlockKBytes / 2), n0, bar_full + 8 * s);
        tma_load_2d(sa + kDecStageW, &p.tmap_x, j * (kBlockKBytes / 2), 0, bar_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0 && nkb > 0) {
      constexpr uint32_t idesc = make_idesc<1, kDecTok, false>();
      const uint64_t adesc0 = make_smem_desc(ring);
      uint32_t s = 0, ph = 0;
      bool alive = true;
      for (int kb = 0; kb < nkb; ++kb, s = (s + 1 == kDecStages ? 0 : s + 1), ph ^= (s == 0)) {
        if (!wait_mbar(bar_full + 8 * s, ph, p.timeout_ns, kTimeoutFullBar, kb)) { alive = false; break; }
        tc_fence_after();
        const uint64_t adesc = adesc0 + s * (kDecStageBytes >> 4);
        const uint64_t bdesc = adesc + (kDecStageW >> 4);
#pragma unroll
        for (int k = 0; k < kBlockKBytes / 32; ++k)
          umma_ss<1, false>(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(bar_empty + 8 * s);
      }
      if (alive) umma_commit(bar_tfull);
    }
  } else {
    // ============================ epilogue, part 1: wait for the accumulator ============================
    if (nkb > 0) {
      bool ok = true;
      if (lane == 0) ok = wait_mbar(bar_tfull, 0u, p.timeout_ns, kTimeoutTmemFull, piece);
      acc_ready = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      tc_fence_after();
    }
  }
  __syncwarp();
  prof_acc.stop(kProfEpiTmemWait);
  ProfTimer prof_epi(prof && threadIdx.x == 64);

  const int q = warp & 3;             // TMEM lane quarter of an epilogue warp (warps 2..5 -> 2, 3, 0, 1)
  const int row = q * 32 + lane;      // weight row within the tile = TMEM lane
  const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  if (split > 1) {
    // every CTA of the cluster has finished reading its ring (its epilogue warps arrive only after
    // the accumulator is complete): the leader's ring may now be overwritten
    cluster_sync_all();
    if (piece != 0 && warp >= 2) {
      // partial sums of piece s live at [s-1][token][weight row] in the leader's ring
      const uint32_t base = map_to_cta(ring + ((piece - 1) * kDecTok * kBlockM + row) * 4, 0);
#pragma unroll 1
      for (int c0 = 0; c0 < kDecTok && c0 < p.M; c0 += 32) {
        uint32_t raw[32];
        if (acc_ready) {
          tmem_ld_32x32(t_lane + c0, raw);
          tmem_ld_wait();
        }
#pragma unroll
        for (int c = 0; c < 32; ++c)
          st_shared_cluster_f32(base + (c0 + c) * kBlockM * 4, acc_ready ? __uint_as_float(raw[c]) : 0.f);
      }
    }
    cluster_sync_all();
  }
  if (piece == 0 && warp >= 2) {
#pragma unroll 1
    for (int c0 = 0; c0 < kDecTok && c0 < p.M; c0 += 32) {
      uint32_t raw[32];
      float v[32];
      if (acc_ready) {
        tmem_ld_32x32(t_lane + c0, raw);
        tmem_ld_wait();
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = acc_ready ? __uint_as_float(raw[c]) : 0.f;
      for (int s = 1; s < split; ++s) {  // fixed order: the result does not depend on timing
        const uint32_t base = ring + ((s - 1) * kDecTok * kBlockM + row) * 4;
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] += ld_shared_f32(base + (c0 + c) * kBlockM * 4);
      }
      // transposed store: for one token the warp's 32 weight rows are 64 contiguous bytes
      if (n0 + row < p.N && acc_ready) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + n0 + row;
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c0 + c < p.M) out[static_cast<int64_t>(c0 + c) * p.ld_out] = __float2bfloat16_rn(v[c]);
      }
    }
  }

  prof_epi.stop(kProfEpiTotal);
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kDecTok);
  }
  prof_kernel.stop(kProfKernelTotal);
  if (prof && threadIdx.x == 0) atomicAdd(&g_prof[kProfCtas], 1ull);
}

}  // namespace edm
