// One-shot all-reduce for decode-sized outputs (EDM_OP_GEMM_AR with `one_shot`).
//
// The fused GEMM + all-reduce pays two flag round trips: partial tiles travel to their owner, the
// owner adds them up and stores the result into every rank's output.  With a few rows that cost
// is all latency.  Here every rank's plain GEMM writes its partial [M, N] into its own symmetric
// window; this kernel then raises one flag at every peer, waits for the peers' flags and adds up
// all W partials itself, reading the W-1 remote ones over NVLink: one flag round trip, (W-1) times
// the partial as link reads per rank, nothing stored remotely.  The sum runs over the ranks in
// rank order in fp32, like the owner's reduction of the fused kernel, so both give the same bits
// and every rank holds identical output.
//
// Buffer reuse: windows and flags alternate between two banks by call parity.  A rank that starts
// call e+2 has finished call e+1, in which it saw every peer's flag e+1; a peer raises that flag
// after its own call e has completed on its stream, so nobody still reads bank e when it is
// overwritten.
#pragma once
#include "tp_gemm.cuh"

namespace edm {

constexpr int kOneShotThreads = 256;
constexpr int kOneShotMaxRanks = 8;

struct OneShotRank {
  const char* part[kOneShotMaxRanks];  // every rank's partial [M, N] (dense, this call's bank) as mapped here
  uint32_t* flags[kOneShotMaxRanks];   // every rank's flag bank
  void* out;
  int64_t ld_out;                      // elements
  int32_t M, N;
  int32_t rank, world;
  uint32_t epoch;
  int32_t out_bytes;                   // 2 (bf16) or 4 (fp32)
};
struct OneShotParams {
  int32_t num_vranks;      // 1 on real multi-GPU runs; > 1: ranks emulated inside one cooperative launch
  int32_t ctas_per_vrank;
  uint64_t timeout_ns;
  OneShotRank r[kOneShotMaxRanks];
};

template <int kW, int kOutBytes>
__device__ __forceinline__ void one_shot_sum(const OneShotRank& P, int cta_in_rank, int ctas) {
  constexpr int kPerVec = 16 / kOutBytes;
  constexpr int kU = kW <= 2 ? 4 : 2;  // 8 to 16 loads of 16 B in flight per thread
  const int64_t row_vecs = static_cast<int64_t>(P.N) * kOutBytes / 16;
  const int64_t n_vecs = static_cast<int64_t>(P.M) * row_vecs;
  const int64_t stride = static_cast<int64_t>(ctas) * kOneShotThreads;
  const int64_t ld_bytes = P.ld_out * kOutBytes;
  for (int64_t v0 = static_cast<int64_t>(cta_in_rank) * kOneShotThreads + threadIdx.x; v0 < n_vecs; v0 += stride * kU) {
    uint4 x[kU][kW];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = v0 + u * stride;
#pragma unroll
      for (int src = 0; src < kW; ++src)
        x[u][src] = (v < n_vecs && EDM_ADDR_OK(P.part[src] + v * 16, 16, 30u)) ? ld_cg_v4(P.part[src] + v * 16)
                                                                            : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= n_vecs) break;
      float sum[kPerVec];
#pragma unroll
      for (int e = 0; e < kPerVec; ++e) sum[e] = 0.f;
#pragma unroll
      for (int src = 0; src < kW; ++src) {
        if constexpr (kOutBytes == 2) {
          OutPack<__nv_bfloat16>::add16B(sum, x[u][src]);
        } else {
          sum[0] += __uint_as_float(x[u][src].x); sum[1] += __uint_as_float(x[u][src].y);
          sum[2] += __uint_as_float(x[u][src].z); sum[3] += __uint_as_float(x[u][src].w);
        }
      }
      uint4 o;
      if constexpr (kOutBytes == 2) {
        o = OutPack<__nv_bfloat16>::pack8(sum);
      } else {
        o.x = __float_as_uint(sum[0]); o.y = __float_as_uint(sum[1]);
        o.z = __float_as_uint(sum[2]); o.w = __float_as_uint(sum[3]);
      }
      const int64_t row = v / row_vecs, col = v - row * row_vecs;
      char* dst = static_cast<char*>(P.out) + row * ld_bytes + col * 16;
      if (EDM_ADDR_OK(dst, 16, 31u)) st_global_v4(dst, o);
    }
  }
}

__global__ void __launch_bounds__(kOneShotThreads)
ar_one_shot_kernel(const __grid_constant__ OneShotParams lp) {
  const int vr = blockIdx.x / lp.ctas_per_vrank;
  const int cta_in_rank = blockIdx.x - vr * lp.ctas_per_vrank;
  const OneShotRank& P = lp.r[vr];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ int all_here;

  // "my partial is complete" to every peer: the GEMM that wrote it finished before this kernel
  // started; the fence makes that visible system-wide before the flag
  if (cta_in_rank == 0 && warp == 1 && lane < P.world && lane != P.rank) {
    fence_acq_rel_sys();
    if (EDM_ADDR_OK(P.flags[lane] + P.rank, 4, 32u)) st_relaxed_sys(P.flags[lane] + P.rank, P.epoch);
  }
  if (warp == 0) {
    bool here = true;
    if (lane < P.world && lane != P.rank)
      here = wait_flag(P.flags[P.rank] + lane, P.epoch, lp.timeout_ns, kTimeoutOneShotFlag, lane);
    here = __all_sync(0xffffffffu, here);
    if (lane == 0) all_here = here ? 1 : 0;
  }
  __syncthreads();
  if (!all_here) return;  // a peer never arrived (status word says which): nothing is added up

  auto run = [&](auto wtag) {
    constexpr int kW = decltype(wtag)::value;
    if (P.out_bytes == 2) one_shot_sum<kW, 2>(P, cta_in_rank, lp.ctas_per_vrank);
    else one_shot_sum<kW, 4>(P, cta_in_rank, lp.ctas_per_vrank);
  };
  switch (P.world) {
    case 2: run(IntTag<2>{}); break;
    case 3: run(IntTag<3>{}); break;
    case 4: run(IntTag<4>{}); break;
    case 5: run(IntTag<5>{}); break;
    case 6: run(IntTag<6>{}); break;
    case 7: run(IntTag<7>{}); break;
    default: run(IntTag<8>{}); break;
  }
}

}  // namespace edm
