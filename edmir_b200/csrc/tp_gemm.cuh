// Persistent, warp-specialised tcgen05 GEMM for sm_100a with the tensor-parallel exchange
// fused into it.  One kernel covers four modes:
//
//   PLAIN  D[M,N] = A[M,K] * B[N,K]^T
//   RS     every rank computes a full partial of every tile and ships it -- its own tiles
//          included -- into the window of the rank that owns the tile's rows; the owner's
//          reducer warps add the W copies up (GEMM + reduce-scatter)
//   AR     like RS with tiles dealt round-robin to owners; the owner stores the reduced tile
//          into every rank's output (GEMM + all-reduce)
//   AG     the row shards of X arrive in this rank's gather buffer -- pushed by the peers'
//          warps or by copy engines -- and the tile loop consumes each shard once its chunk
//          flags are up (all-gather + GEMM)
//
// Both operands are K-major (the reference's "TN" convention, EDM-IR/ir/c-extension/mma.cu:24-25).
//
// Roles per CTA (384 threads = 12 warps):
//   warp 0      TMA producer (operand ring)
//   warp 1      MMA issuer (one thread)
//   warps 2,3   all-gather pushes (sm transport) or reduction of received tiles (RS/AR);
//               warp 2 also allocates and frees TMEM
//   warps 4-7   epilogue: TMEM -> registers -> shared-memory staging -> global / peer window
//   warp 8      signaller
//   warps 9-11  more pushes / reduction
// A system-scope release costs on the order of ten microseconds while remote writes are queued
// (it drains the SM), so no working warp ever executes one: they post "this data has landed"
// notes into shared-memory mailboxes and the signaller turns batches of notes into one fence plus
// relaxed flag stores.
// Tiles are dealt round-robin to the CTAs (pairs); the tiles of an incomplete last wave -- or all
// tiles, when there are fewer than CTAs -- are cut along K into pieces that free CTAs claim from a
// counter and whose partial sums they exchange through scratch tiles (TailSplit, tail_piece).
// Accumulators are double buffered in TMEM (2 x 256 columns) so the epilogue of tile i, which
// is where the NVLink traffic is issued, overlaps the MMAs of tile i+1.
//
// Every wait (mbarrier or peer flag) is bounded: on expiry the kernel records a status code and
// all remaining waits fall through, so the launch always terminates and frees its TMEM.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <climits>
#include <cstdint>
#include "ptx.cuh"

namespace edm {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;  // widest tile (the TMEM double buffer holds 2 x 256 columns); a 32-wide variant serves tiny M
constexpr int kBlockKBytes = 128;  // one 128B swizzle row of K per stage
constexpr int kPipeBytes = 192 * 1024;  // operand ring: 4 stages of 48 KiB, or 6 of 32 KiB for CTA pairs
constexpr int kThreads = 384;  // 12 warps, see the role list above (registers are granted per 4 warps)
constexpr int kMaxRanks = 8;
constexpr int kMaxVirtualRanks = 4;
constexpr int kTmemCols = 512;
constexpr int kStageABytes = kBlockM * kBlockKBytes;  // 16 KiB
constexpr int kMaxStages = 9;
constexpr int kEpiRowBytes = 256;                      // staging row per pass
constexpr int kEpiWarpBytes = 32 * kEpiRowBytes;       // 8 KiB per epilogue warp
constexpr int kSmemBytes = kPipeBytes + 4 * kEpiWarpBytes + 1024 /*align*/ + 256;

enum Mode : int32_t { kPlain = 0, kRS = 1, kAR = 2, kAG = 3 };

// Status codes written to g_status[0]; g_status[1..7] carry details of the first failure.
enum Status : uint32_t {
  kOk = 0,
  kTimeoutFullBar = 1,
  kTimeoutEmptyBar = 2,
  kTimeoutTmemFull = 3,
  kTimeoutTmemEmpty = 4,
  kTimeoutPartialFlag = 5,   // RS/AR: a peer's partial tile never arrived
  kTimeoutResultFlag = 6,    // AR: an owner's reduced tile never arrived
  kTimeoutGatherFlag = 7,    // AG: a peer's shard chunk never arrived
  kTimeoutTailFlag = 8,      // split last wave: another CTA's partial sum never arrived
  kBoundsFault = 9,          // checking build only: an address outside every range the launch may touch
  kTimeoutPushCount = 10,    // AG with pusher CTAs: this rank's own pushers never finished a chunk
  kTimeoutOneShotFlag = 11,  // one-shot AR: a peer's "partial complete" flag never arrived
};

__device__ uint32_t g_status[16];

// Optional device-side accounting (LaunchParams::profile): nanoseconds, summed over CTAs, that
// each role spent waiting or working.  Slot meanings: see ProfSlot.
enum ProfSlot : int {
  kProfProducerGatherWait = 0, kProfProducerEmptyWait = 1, kProfMmaFullWait = 2, kProfMmaTmemWait = 3,
  kProfEpiTmemWait = 4, kProfEpiStagingWait = 5, kProfEpiFlagWait = 6, kProfEpiTotal = 7,
  kProfReducerFlagWait = 8, kProfReducerTotal = 9, kProfPushLoadWait = 10, kProfPushBufferWait = 11,
  kProfPushPublish = 12, kProfPushTotal = 13, kProfKernelTotal = 14, kProfCtas = 15,
  kProfEpiFence = 16, kProfEpiIssue = 17, kProfEpiTmemLoad = 18, kProfPushFence = 19,
  kProfProducerFlagPoll = 20, kProfProducerProxyFence = 21, kProfEpiTileLoop = 22, kProfEpiFinalNotes = 23,
};
__device__ unsigned long long g_prof[24];

struct ProfTimer {
  bool on;
  uint64_t t0;
  __device__ __forceinline__ explicit ProfTimer(bool enabled) : on(enabled), t0(enabled ? globaltimer_ns() : 0) {}
  __device__ __forceinline__ void stop(int slot) {
    if (on) atomicAdd(&g_prof[slot], static_cast<unsigned long long>(globaltimer_ns() - t0));
  }
};

struct alignas(64) RankParams {
  CUtensorMap tmap_a[2];  // [0] main A (AG: local gather buffer); [1] 3xTF32 low part / AG local shard
  CUtensorMap tmap_b[2];  // [0] main B; [1] 3xTF32 low part
  int32_t M, N, K;        // GEMM extents on this rank (AG: M is the gathered row count)
  int32_t rank, world;
  int32_t mode;
  int32_t passes;          // 1, or 3 for the split-fp32 path
  uint32_t epoch;          // value a flag must reach in this call
  int32_t max_owned;       // slots per source rank in a window
  uint32_t partial_flag_off, result_flag_off, gather_flag_off;  // offsets in u32 into flags[]
  int32_t ag_chunks;       // chunks per shard
  int32_t ag_local_direct; // 1: own shard is read in place through tmap_a[1]
  void* out;               // PLAIN/AG/AR: [M,N]; RS: [M/world,N]
  int64_t ld_out;          // elements
  const void* x_local;     // AG: this rank's shard [M/world,K]
  int64_t ld_x;            // elements
  uint32_t* counters;      // AG: local arrival counters [world*ag_chunks], bank of this call's epoch parity
  uint32_t* counters_next; // AG: the other bank; the publisher zeroes it for the next call
  float* scratch;          // split-fp32: running fp32 sums, one kBlockM x kBlockN tile per CTA
  int32_t seg_kblocks;     // split-fp32: K blocks accumulated in TMEM before folding into scratch (0 = all)
  int32_t ag_external;     // AG: shards and chunk flags are delivered by copy engines, not by this kernel
  int32_t ag_ce_lo;        // AG: shards for peers rank-d with d >= ag_ce_lo come by copy engine, nearer ones are pushed by this kernel
  // Grouped GEMM (PLAIN mode only; the experts of a mixture-of-experts layer): row block j of the
  // walk reads A and writes D at row group_table[4j], reads B from row group_table[4j+1] on, and
  // holds group_table[4j+2] valid rows; *group_count row blocks exist.  Both live in device memory
  // and are written by an earlier kernel on the stream (how many rows each expert received is not
  // known on the host).  M then only bounds the number of row blocks.
  const int32_t* group_table;
  const int32_t* group_count;
  void* peer_out[kMaxRanks];   // AR: every rank's output as mapped here
  char* win[kMaxRanks];        // every rank's window (parity half already selected)
  uint32_t* flags[kMaxRanks];  // every rank's flag array
  void* gather[kMaxRanks];     // AG: every rank's gather buffer [M,K]
};

struct LaunchParams {
  int32_t num_vranks;     // 1 on real multi-GPU runs; >1 = ranks emulated inside one launch
  int32_t ctas_per_vrank;
  uint64_t timeout_ns;
  int32_t profile;        // 1: accumulate per-role wait times into g_prof
  int32_t stage_limit;    // experiments: use at most this many ring stages (0 = all)
  int32_t push_stride;    // all-gather: only CTAs whose index is a multiple of this push the shard
  int32_t band;           // row blocks per band of the tile walk (0 = default)
  int32_t band_cols;      // column blocks per super-tile of a band (0 = the whole width)
  int32_t pusher_ctas;    // all-gather: the last CTAs of every rank only push the shard (no tiles); 0 = push warps inside the GEMM CTAs
  int32_t tail_split;     // most pieces a tile of an incomplete last wave is cut into along K (< 2: none)
  uint32_t tail_epoch;    // value the partial-sum flags of this launch carry
  RankParams r[kMaxVirtualRanks];
};

// ------------------------------------------------------------------ bounded waits
__device__ __forceinline__ void report(uint32_t code, uint32_t a, uint32_t b, uint32_t c) {
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = threadIdx.x;
    g_status[3] = a;
    g_status[4] = b;
    g_status[5] = c;
    __threadfence();
  }
}
__device__ __forceinline__ bool aborted() {
  return *reinterpret_cast<volatile uint32_t*>(&g_status[0]) != 0u;
}

// ------------------------------------------------------------------ checking build
// Compiled with -DEDM_DEBUG_BOUNDS every global-memory address the kernel computes itself (output
// and window stores, bulk copies, flag words, scratch tiles; TMA loads are bounded by their tensor
// maps) is looked up in a table of the ranges the launch may touch, which the host fills before
// the launch.  An address outside all of them is recorded in the status words
// {kBoundsFault, CTA, thread, site, address high, address low} and the access is skipped, so a
// wrong index shows up as a status code instead of a fault.  The ordinary build compiles the
// checks away.
#ifdef EDM_DEBUG_BOUNDS
constexpr int kDbgMaxRanges = 64;
__device__ unsigned long long g_dbg_lo[kDbgMaxRanges], g_dbg_hi[kDbgMaxRanges];
__device__ int g_dbg_n;
__device__ __noinline__ bool addr_ok(const void* p, size_t n, uint32_t site) {
  const unsigned long long a = reinterpret_cast<unsigned long long>(p);
  for (int i = 0; i < g_dbg_n; ++i)
    if (a >= g_dbg_lo[i] && a + n <= g_dbg_hi[i]) return true;
  report(kBoundsFault, site, static_cast<uint32_t>(a >> 32), static_cast<uint32_t>(a));
  return false;
}
#define EDM_ADDR_OK(p, n, site) addr_ok((p), (n), (site))
#else
#define EDM_ADDR_OK(p, n, site) true
#endif

// prof_slot >= 0: add the time spent here to that accounting slot (only the slow path pays for it)
// Both waits return true when what they waited for has happened and false when they gave up
// (their own limit ran out, or another wait anywhere on the device already had).  A role that gets
// false stops issuing work -- no further loads, MMAs or copies -- and goes to the tear-down, so
// that what is still in flight when the CTA exits is bounded by what the pipeline normally holds.
__device__ __noinline__ bool wait_mbar_slow(uint32_t bar, uint32_t parity, uint64_t timeout_ns,
                                            uint32_t code, uint32_t info, int prof_slot) {
  const uint64_t start = prof_slot >= 0 ? globaltimer_ns() : 0;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  bool ok = true;
  while (!mbar_try_wait(bar, parity)) {
    if ((spins++ & 15u) == 0u) {
      if (aborted()) { ok = false; break; }
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) { report(code, info, parity, bar); ok = false; break; }
    }
  }
  if (prof_slot >= 0) atomicAdd(&g_prof[prof_slot], static_cast<unsigned long long>(globaltimer_ns() - start));
  return ok;
}
__device__ __forceinline__ bool wait_mbar(uint32_t bar, uint32_t parity, uint64_t timeout_ns,
                                          uint32_t code, uint32_t info, int prof_slot = -1) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_mbar_slow(bar, parity, timeout_ns, code, info, prof_slot);
}

// Wait until *flag (written by another GPU / CTA with release.sys) has reached `epoch`.
__device__ __noinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                                       uint32_t code, uint32_t info) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  if (!EDM_ADDR_OK(flag, 4, 1u)) return false;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
    if ((spins++ & 31u) == 0u) {
      if (aborted()) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) { report(code, info, epoch, ld_relaxed_sys(flag)); return false; }
    }
    __nanosleep(64);
  }
  return true;
}

// ------------------------------------------------------------------ tile enumeration
struct Tile {
  int m_blk, n_blk;
  int owner;      // rank that ends up holding / reducing this tile
  int owned_idx;  // index of the tile among the owner's tiles (slot / flag index)
  int linear;     // m_blk * n_blocks + n_blk
  bool valid;     // false for a hole in the walk (all-reduce with a tile count not divisible by world)
};

// Walk an (mb x nb) grid in bands of kBand row-blocks so that concurrently running CTAs share
// A and B panels in L2 (taller bands re-read B less often; 16 measured best on the layer's shapes).
// With kCols > 0 a band is further cut into super-tiles of kCols column blocks that are finished one
// after the other: the tiles in flight at any time then cover about kBand x kCols blocks, i.e.
// kBand panels of A and kCols panels of B, instead of kBand panels of A and a sliver of B.
__host__ __device__ __forceinline__ void band_order(int i, int mb, int nb, int& m, int& n, int kBand = 8,
                                                    int kCols = 0) {
  const int per_band = kBand * nb;
  const int band = i / per_band;
  const int first = band * kBand;
  const int rows = min(kBand, mb - first);
  const int j = i - band * per_band;
  if (kCols <= 0 || kCols >= nb) {
    m = first + j % rows;
    n = j / rows;
    return;
  }
  const int per_super = rows * kCols;  // every super-tile before the last one of a band is full
  const int sup = j / per_super;
  const int jj = j - sup * per_super;
  m = first + jj % rows;
  n = sup * kCols + jj / rows;
}

struct TileWalk {
  int mode, rank, world;
  int m_blocks, n_blocks, total;
  int positions;    // length of the walk (>= total when it has holes)
  int mb_per_rank;  // RS / AG-rotated: row blocks per rank, 0 if rows do not split on block edges
  int band;         // row blocks per band of the walk
  int band_cols;    // column blocks per super-tile of a band (0: the whole width)
  int ag_own_blocks;                 // all-gather: the own shard is a band of its own (nothing of it has to arrive)
  int ag_head_blocks, ag_head_band;  // all-gather: the next row blocks are walked in lower bands
  int rounds;       // RS/AR: rounds of the owner round-robin (= most tiles any rank owns)
  int defer;        // RS/AR: own tiles of the last `defer` rounds are computed at the very end

  // tile_m = rows of one scheduling tile: 128, or 256 when a CTA pair shares a tile
  // units = CTAs (or CTA pairs) walking the tiles concurrently
  __device__ TileWalk(const RankParams& p, int rows, int tile_m, int tile_n, int band_rows, int units, int cols)
      : TileWalk(p.mode, p.rank, p.world, rows, p.N, tile_m, tile_n, band_rows, units, cols) {}
  __host__ __device__ TileWalk(int mode_, int rank_, int world_, int M, int N, int tile_m, int tile_n,
                               int band_rows, int units, int cols = 0) {
    mode = mode_; rank = rank_; world = world_;
    band = band_rows > 0 ? band_rows : 16;  // 16 x 256 rows of A stay in L2 while B streams through once per band
    band_cols = cols > 0 ? cols : 0;
    m_blocks = (M + tile_m - 1) / tile_m;
    n_blocks = (N + tile_n - 1) / tile_n;
    total = m_blocks * n_blocks;
    const int rows_per_rank = M / max(world, 1);
    mb_per_rank = (world > 1 && rows_per_rank * world == M && rows_per_rank % tile_m == 0)
                      ? rows_per_rank / tile_m : 0;
    // all-gather: shards arrive one after the other, about twice as fast as they are consumed.
    // A band must not reach further ahead than what has arrived when its first wave starts.  At
    // the start nothing has: the own shard is a band of its own (a band is walked column by
    // column, so a first band of own + next shard would put half of the first wave on rows that
    // are still on the wire).  Then two shards per band over the next four shards, then the full
    // band height.
    ag_own_blocks = 0;
    ag_head_blocks = 0;
    ag_head_band = band;
    if (mode == kAG && mb_per_rank > 0 && band_rows <= 0) {
      if (mb_per_rank < band) ag_own_blocks = mb_per_rank;
      if (2 * mb_per_rank < band) {
        ag_head_blocks = min(m_blocks - ag_own_blocks, 4 * mb_per_rank);
        ag_head_band = 2 * mb_per_rank;
      }
    }
    positions = (mode == kAR && world > 1) ? (total + world - 1) / world * world : total;
    rounds = world > 1 ? positions / world : 0;
    // about one wave of own tiles goes last: while it is computed nothing has to cross the link
    // any more, the peers already hold every partial of this rank and reduce during that wave,
    // and what is left after the last MMA is one local copy and one local reduction
    defer = min(rounds, units);
  }

  // tiles owned by `r`
  __host__ __device__ int owned_count(int r) const {
    if (mode == kRS) return mb_per_rank * n_blocks;
    if (mode == kAR && world > 1) return (total - r + world - 1) / world;
    return total;
  }
  // coordinates of the idx-th tile owned by `r`
  __host__ __device__ void owned_tile(int r, int idx, int& m_blk, int& n_blk) const {
    if (mode == kRS) {
      int lm;
      band_order(idx, mb_per_rank, n_blocks, lm, n_blk, band);
      m_blk = r * mb_per_rank + lm;
    } else {
      const int lin = idx * world + r;
      m_blk = lin / n_blocks;
      n_blk = lin - m_blk * n_blocks;
    }
  }

  __host__ __device__ Tile at(int i) const {
    Tile t;
    t.valid = true;
    if ((mode == kRS || mode == kAR) && world > 1) {
      // Round R = i / world: this rank computes tile R of every owner (rank+1, rank+2, ..., rank,
      // starting at a rotating position).  Pushes therefore leave at a steady rate towards every
      // peer for the whole launch, and every owner receives the partials of its tile R from all
      // ranks at about the same time.
      // The own tiles of the last `defer` rounds are taken out of their rounds and appended.
      // Inside a round the order of the owners is rotated by the round number.  Units take
      // positions i, i + units, i + 2 units, ...; with a fixed order and an even number of units a
      // unit would meet only the owners of one parity class -- at two ranks half of the units
      // would ship every tile over the link and the other half none.
      const int full = (rounds - defer) * world;        // positions of the undisturbed rounds
      const int thin = defer * (world - 1);             // positions of the rounds without own tile
      int round, d;
      if (i < full) { round = i / world; d = (i - round * world + round) % world; }
      else if (i < full + thin) {
        const int j = i - full;
        round = rounds - defer + j / (world - 1);
        d = (j - (j / (world - 1)) * (world - 1) + round) % (world - 1);  // 0 .. world-2: never this rank
      } else { round = rounds - defer + (i - full - thin); d = world - 1; }
      t.owner = (rank + 1 + d) % world;
      t.owned_idx = round;
      t.valid = round < owned_count(t.owner);
      owned_tile(t.owner, round, t.m_blk, t.n_blk);
    } else if (mode == kAG && mb_per_rank > 0) {
      int pm, n;
      const int own_tiles = ag_own_blocks * n_blocks;
      const int head_tiles = ag_head_blocks * n_blocks;
      if (i < own_tiles) {
        band_order(i, ag_own_blocks, n_blocks, pm, n, ag_own_blocks);
      } else if (i < own_tiles + head_tiles) {
        band_order(i - own_tiles, ag_head_blocks, n_blocks, pm, n, ag_head_band);
        pm += ag_own_blocks;
      } else {
        band_order(i - own_tiles - head_tiles, m_blocks - ag_own_blocks - ag_head_blocks, n_blocks, pm, n, band, band_cols);
        pm += ag_own_blocks + ag_head_blocks;
      }
      t.m_blk = (rank * mb_per_rank + pm) % m_blocks;  // own shard first, then rank+1, ...
      t.n_blk = n;
      t.owner = rank;
      t.owned_idx = 0;
    } else {
      band_order(i, m_blocks, n_blocks, t.m_blk, t.n_blk, band, band_cols);
      t.owner = rank;
      t.owned_idx = 0;
    }
    t.linear = t.m_blk * n_blocks + t.n_blk;
    return t;
  }
};

// ------------------------------------------------------------------ split of the last wave
// `units` CTAs (or pairs) take tiles round-robin, so when the tile count is not a multiple of
// `units` the last wave leaves most of them idle for a whole tile time (160 tiles on 74 pairs: the
// third wave has 12; a decode-sized GEMM has fewer tiles than units to begin with).  Those `tiles`
// tail tiles are instead cut along K into `parts` pieces that run side by side.  Pieces are not assigned in advance: a unit that has finished its whole tiles
// claims the next piece from a counter, piece index = tile * parts + piece, so the pieces of one
// tile go to units that became free at about the same time (units drift apart by tens of
// microseconds over a launch) and the slowest units get none.  The pieces of a tile exchange fp32
// partial sums through scratch tiles and each finishes its share of the tile's columns (see
// tail_piece in the kernel).
constexpr int kTailMinKBlocks = 4;    // a piece is at least this many K blocks
constexpr int kTailMinTileKBlocks = 32;  // shorter tiles are not cut: the exchange (~7 us) would cost more than it saves
constexpr int kTailMaxParts = 8;
constexpr int kTailMaxCtas = 160;     // CTAs the static scratch below has room for
struct TailSplit {
  int first;   // tiles (walk positions) below this are computed whole, round-robin
  int tiles;   // tail tiles
  int parts;   // pieces per tail tile (1: nothing is split)
  // max_parts: most pieces per tile (a power of two up to kTailMaxParts; < 2 switches the split off)
  __host__ __device__ TailSplit(int positions, int units, int k_blocks, int max_parts) {
    first = positions; tiles = 0; parts = 1;
    const int full = units > 0 ? positions / units * units : 0;
    const int rest = positions - full;
    // (full == 0: fewer tiles than units, e.g. a decode-sized GEMM; every tile is a tail tile then
    // and the launch is a split-K GEMM over otherwise idle CTAs)
    if (max_parts >= 2 && rest > 0 && k_blocks >= kTailMinTileKBlocks) {
      int s = units / rest;
      if (s > k_blocks / kTailMinKBlocks) s = k_blocks / kTailMinKBlocks;
      if (s > kTailMaxParts) s = kTailMaxParts;
      if (s > max_parts) s = max_parts;
      while (s & (s - 1)) s &= s - 1;  // a power of two: each piece finishes whole 32-column chunks
      if (s >= 2) { first = full; tiles = rest; parts = s; }
    }
  }
  __host__ __device__ int pieces() const { return parts > 1 ? tiles * parts : 0; }
  // claimed piece -> position in the tile walk, piece of the tile and its K-block range
  __host__ __device__ void piece(int idx, int k_blocks, int& pos, int& part, int& k_lo, int& k_hi) const {
    const int r = idx / parts;
    part = idx - r * parts;
    pos = first + r;
    k_lo = static_cast<int>(static_cast<int64_t>(k_blocks) * part / parts);
    k_hi = static_cast<int>(static_cast<int64_t>(k_blocks) * (part + 1) / parts);
  }
};
// One work item of a CTA: a whole tile (n_parts == 1) or a piece of a tail tile.
struct Work {
  int pos;            // position in the tile walk
  int part, n_parts;  // piece of the tile
  int k_lo, k_hi;     // K blocks
  int piece;          // claimed piece index (slot of its scratch tile and flags)
};
// Scratch tiles and flags of the pieces (one fp32 tile and one flag per epilogue warp per piece
// and CTA of a pair), the claim counter per (virtual) rank, and the word through which the warp
// that claimed tells the other warps of its CTA pair: launch epoch << 32 | piece index.
__device__ float g_tail_scratch[static_cast<size_t>(kTailMaxCtas) * kBlockM * kBlockN];
__device__ uint32_t g_tail_flags[kTailMaxCtas * 4];
__device__ uint32_t g_tail_next[kMaxVirtualRanks];
__device__ unsigned long long g_tail_claim[kTailMaxCtas];

// ------------------------------------------------------------------ descriptors
// K-major operand tile in shared memory, 128B rows, 128B swizzle, 8-row groups 1024B apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;            // leading byte offset: unused with swizzled K-major
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}
template <int kCG, int kBN, bool kTf32>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  const uint32_t fmt = kTf32 ? 2u : 1u;  // 1 = BF16, 2 = TF32
  return (1u << 4)                        // D format F32
         | (fmt << 7) | (fmt << 10)       // A, B formats; both K-major (bits 15,16 = 0)
         | (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>((kBlockM * kCG) >> 4) << 24);
}

template <int V> struct IntTag { static constexpr int value = V; };

// ------------------------------------------------------------------ mailboxes to the signaller
// One single-producer ring per posting warp: epilogue warps -> 0-3, warps 2-3 -> 4-5, warps 9-11 -> 6-8.
constexpr int kMailboxes = 9;
constexpr int kMailboxDepth = 16;
enum NoteKind : uint64_t {
  kNoteFlag = 0,     // payload = address of a flag word: store the epoch there
  kNoteResult = 1,   // payload = result-flag index: store the epoch into every peer's result flag
  kNoteChunk = 2,    // payload = peer << 24 | chunk: count this warp's share of an all-gather chunk
};
struct Mailbox {
  uint32_t ready;    // notes posted
  uint32_t done;     // notes published
  uint32_t closed;   // poster has finished
  uint32_t pad;
  uint64_t note[kMailboxDepth];
};
__device__ __forceinline__ uint64_t make_note(uint64_t kind, uint64_t payload) { return (kind << 60) | payload; }

// Called by one lane of the posting warp.  Everything the note vouches for must already be
// complete from this lane's point of view.
__device__ __forceinline__ void mailbox_post(Mailbox* mb, uint64_t note, uint64_t timeout_ns) {
  volatile Mailbox* v = mb;
  const uint32_t r = v->ready;
  if (r - v->done >= kMailboxDepth) {
    const uint64_t t0 = globaltimer_ns();
    while (r - v->done >= kMailboxDepth) {
      if (aborted() || globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(100);
    }
  }
  v->note[r % kMailboxDepth] = note;
  __threadfence_block();
  v->ready = r + 1;
}
__device__ __forceinline__ void mailbox_close(Mailbox* mb) {
  __threadfence_block();
  reinterpret_cast<volatile Mailbox*>(mb)->closed = 1;
}

// ------------------------------------------------------------------ output conversion
template <typename OutT> struct OutPack;
template <> struct OutPack<__nv_bfloat16> {
  static constexpr int kColsPerPass = kEpiRowBytes / 2;  // 128
  // 8 fp32 -> one 16B vector
  __device__ static __forceinline__ uint4 pack8(const float* v) {
    uint4 o;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
    return o;
  }
  __device__ static __forceinline__ void add16B(float* acc, uint4 w) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += __uint_as_float(u[i] << 16);
      acc[2 * i + 1] += __uint_as_float(u[i] & 0xFFFF0000u);
    }
  }
};
template <> struct OutPack<float> {
  static constexpr int kColsPerPass = kEpiRowBytes / 4;  // 64
};

// ------------------------------------------------------------------ the kernel
// kCG = 1: one CTA per 128x256 tile.  kCG = 2: a CTA pair (cluster of 2) shares a 256x256 tile;
// each CTA loads its 128 rows of A and its 128-row half of the B tile, the even CTA issues
// cta_group::2 MMAs that read both CTAs' shared memory, and each CTA's TMEM receives its own
// 128 accumulator rows, so the epilogue is the same per-CTA code in both variants.
// kBN = tile width: 256, or 32 for decode-sized M (one row block): 128x32 tiles give every SM a
// slab of the weights to stream instead of leaving most SMs idle (plain GEMM only; for long K the
// host prefers 256-wide tiles cut along K over the idle CTAs, see TailSplit).
template <int kCG, int kBN, bool kTf32, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_kernel(const __grid_constant__ LaunchParams lp) {
  static_assert(kBN == 256 || (kBN == 32 && kCG == 1), "tile width");
  constexpr int kStageBBytes = (kBN / kCG) * kBlockKBytes;  // 32 KiB, 16 KiB per CTA of a pair, or 4 KiB
  constexpr int kStageBytes = kStageABytes + kStageBBytes;
  constexpr int kStages = kPipeBytes / kStageBytes;             // 4, 6 or 9
  static_assert(kStages <= kMaxStages, "barrier array too small");
  constexpr int kElemBytes = kTf32 ? 4 : 2;
  constexpr int kBlockK = kBlockKBytes / kElemBytes;   // elements of K per stage
  constexpr int kOutBytes = sizeof(OutT);
  constexpr int kTileOutBytes = kBlockM * kBN * kOutBytes;
  constexpr int kColsPerPass = kEpiRowBytes / kOutBytes;   // 128 (bf16) / 64 (fp32)
  constexpr int kPasses = kBN >= kColsPerPass ? kBN / kColsPerPass : 1;               // 2 / 4 (1 for the narrow tile)
  constexpr int kChunksPerPass = (kBN >= kColsPerPass ? kColsPerPass : kBN) / 32;     // 4 / 2 (1)
  constexpr int kOutPerVec = 16 / kOutBytes;               // 8 / 4

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[2 * kMaxStages + 8];
  __shared__ uint32_t tmem_base_slot;
  __shared__ Mailbox mbox[kMailboxes];
  __shared__ uint32_t reduce_next;  // next (half-tile, quarter) unit of the reduction

  const int vr = blockIdx.x / lp.ctas_per_vrank;
  const int cta_in_rank = blockIdx.x - vr * lp.ctas_per_vrank;
  const RankParams& P = lp.r[vr];
  // all-gather with dedicated pushers: the last pusher_ctas CTAs (whole pairs) of every rank take
  // no tiles; they only move this rank's shard into the peers' gather buffers
  const int pusher_ctas = (P.mode == kAG && P.world > 1 && !P.ag_external) ? lp.pusher_ctas : 0;
  const int gemm_ctas = lp.ctas_per_vrank - pusher_ctas;
  const bool is_pusher = cta_in_rank >= gemm_ctas;
  // scheduling unit: a CTA, or a CTA pair (ctas_per_vrank is even then and pairs never straddle ranks)
  const int cta = cta_in_rank / kCG;
  const int num_ctas = gemm_ctas / kCG;
  const uint32_t pr = kCG == 2 ? cluster_ctarank() : 0u;  // position in the pair; 0 issues the MMAs
  const uint64_t timeout_ns = lp.timeout_ns;
  const bool prof = lp.profile != 0;
  ProfTimer prof_kernel(prof && threadIdx.x == 0);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_epi = smem_base + kStages * kStageBytes;
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kStages]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * kStages]);
  const uint32_t bar_tempty = smem_u32(&bars[2 * kStages + 2]);
  const uint32_t bar_tail = smem_u32(&bars[2 * kMaxStages + 4]);  // one per epilogue warp: partial sums have landed
  // all-gather with the sm transport: warps 2, 3 and 9-11 push this rank's shard to the peers
  const bool ag_push = P.mode == kAG && P.world > 1 && !P.ag_external && pusher_ctas == 0;
  constexpr int kPusherWarps = 6;        // warps of a pusher CTA that drive copies (one lane each)
  constexpr int kPushDepth = 4;          // staging buffers per such warp
  constexpr uint32_t kPushBytes = 8192;  // bytes per copy: kPusherWarps * kPushDepth * kPushBytes = the operand ring
  static_assert(kPusherWarps * kPushDepth * kPushBytes <= kPipeBytes, "pusher staging exceeds the ring");
  static_assert(kPusherWarps * kPushDepth <= 2 * kMaxStages + 8, "not enough barriers for the pusher staging");
  uint32_t stages = kStages;
  if (lp.stage_limit > 0 && static_cast<uint32_t>(lp.stage_limit) < stages) stages = lp.stage_limit;

  if (threadIdx.x == 32) reduce_next = 0;
  if (threadIdx.x < kMailboxes) {
    mbox[threadIdx.x].ready = 0; mbox[threadIdx.x].done = 0; mbox[threadIdx.x].closed = 0;
  }
  if (threadIdx.x == 0) {
    if (is_pusher) {
      // one barrier per staging buffer: a local bulk load has landed
      for (int i = 0; i < kPusherWarps * kPushDepth; ++i) mbar_init(smem_u32(&bars[i]), 1);
    } else {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(bar_full + 8 * s, 1);
        mbar_init(bar_empty + 8 * s, 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(bar_tfull + 8 * a, 1);
        mbar_init(bar_tempty + 8 * a, 4 * kCG);  // every epilogue warp of the pair
      }
      for (int w = 0; w < 4; ++w) mbar_init(bar_tail + 8 * w, 1);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 2 && !is_pusher) {
    tmem_alloc<kCG>(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish<kCG>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kCG == 2) cluster_sync_all();  // partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_base_slot);

  // grouped: as many row blocks as the table holds (read once; an earlier kernel wrote it)
  const bool grouped = P.group_table != nullptr;
  const int walk_rows = grouped ? min(__ldg(P.group_count) * kBlockM * kCG, P.M) : P.M;
  const TileWalk walk(P, walk_rows, kBlockM * kCG, kBN, lp.band, num_ctas, lp.band_cols);
  // first row of A / D, first row of B and valid rows of the 128-row half `half` of row block m_blk
  auto block_rows = [&](int m_blk, int half, int& row0, int& b_row0, int& rows) {
    if (grouped) {
      const int4 e = __ldg(reinterpret_cast<const int4*>(P.group_table) + m_blk);
      row0 = e.x + half * kBlockM;
      b_row0 = e.y;
      rows = max(0, min(kBlockM, e.z - half * kBlockM));
    } else {
      row0 = (m_blk * kCG + half) * kBlockM;
      b_row0 = 0;
      rows = min(kBlockM, P.M - row0);
    }
  };
  const int num_kb_pass = (P.K + kBlockK - 1) / kBlockK;
  // The tensor core adds into its fp32 accumulator with truncation, so a long accumulation
  // drifts.  The split-fp32 path therefore accumulates `seg_kb` K blocks at a time in TMEM and
  // folds each segment into a running sum kept with ordinary fp32 adds.
  const int seg_kb = (P.seg_kblocks > 0 && P.seg_kblocks < num_kb_pass) ? P.seg_kblocks : num_kb_pass;
  const int num_segs = (num_kb_pass + seg_kb - 1) / seg_kb;
  const int rows_per_rank = P.world > 0 ? P.M / P.world : P.M;
  // only launches that write their tiles in place split the last wave (fused reductions end on
  // local tiles anyway; the split-fp32 path already uses its accumulator segments)
  const TailSplit tail(walk.positions, num_ctas, num_kb_pass,
                       (kBN == 256 && (P.mode == kPlain || P.mode == kAG) && P.passes == 1 && num_segs == 1 &&
                        !grouped && gridDim.x <= kTailMaxCtas) ? lp.tail_split : 0);

  // Work items of this CTA, in order: its whole tiles, then at most one claimed piece of a tail
  // tile.  `claim` is called once, when the whole tiles are done: the producer thread of the
  // unit's first CTA takes the next piece index from the counter and publishes it; every other
  // role waits for that word.
  const int first_cta_of_unit = static_cast<int>(blockIdx.x) - static_cast<int>(pr);
  auto claim_piece = [&]() -> int {
    const uint32_t got = atomicAdd(&g_tail_next[vr], 1u);
    // every unit claims exactly once per launch: the last one leaves the counter at zero
    if (got == static_cast<uint32_t>(num_ctas) - 1u) atomicExch(&g_tail_next[vr], 0u);
    if (EDM_ADDR_OK(&g_tail_claim[first_cta_of_unit], 8, 19u))
      *reinterpret_cast<volatile unsigned long long*>(&g_tail_claim[first_cta_of_unit]) =
          (static_cast<unsigned long long>(lp.tail_epoch) << 32) | got;
    return static_cast<int>(got);
  };
  auto await_piece = [&]() -> int {
    const volatile unsigned long long* word = &g_tail_claim[first_cta_of_unit];
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
      const unsigned long long v = *word;
      if (static_cast<uint32_t>(v >> 32) == lp.tail_epoch) return static_cast<int>(v & 0xFFFFFFFFull);
      if ((spins++ & 31u) == 0u) {
        if (aborted()) return INT_MAX;
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > timeout_ns) { report(kTimeoutTailFlag, 0xFFFFu, lp.tail_epoch, static_cast<uint32_t>(v >> 32)); return INT_MAX; }
      }
      __nanosleep(64);
    }
  };
  // advances (i, tail_taken); false when this CTA has nothing left
  auto next_work = [&](int& i, bool& tail_taken, bool claims, Work& w) -> bool {
    if (i < tail.first) {
      w.pos = i; w.part = 0; w.n_parts = 1; w.k_lo = 0; w.k_hi = num_kb_pass; w.piece = -1;
      i += num_ctas;
      return true;
    }
    if (tail.parts == 1 || tail_taken) return false;
    tail_taken = true;
    const int idx = claims ? claim_piece() : await_piece();
    if (idx >= tail.pieces()) return false;
    tail.piece(idx, num_kb_pass, w.pos, w.part, w.k_lo, w.k_hi);
    w.n_parts = tail.parts;
    w.piece = idx;
    return true;
  };

  // ------------------------------------------------------------------ all-gather pushes
  // Five warps per CTA (2, 3, 9, 10, 11) copy the local shard into every peer's gather buffer with
  // plain 16-byte loads and stores; the TMA queue stays reserved for the operand ring, which a
  // back-pressured remote bulk store would otherwise hold up.  The stores need no completion
  // wait: a warp posts "my part of chunk c for peer p is issued" and the signaller's
  // system-scope fence orders those stores before the flag.
  constexpr int kPushWarps = 5;
  auto push_shard = [&](int pw, Mailbox* note_box) {
    const bool pprof = prof && lane == 0 && pw == 0;
    ProfTimer push_total(pprof);
    // pushing CTAs: every push_stride-th one (remote stores that queue up behind a busy link also
    // delay the operand loads of the SM that issued them, so the duty is kept to a subset)
    const int stride = max(lp.push_stride, 1);
    if (cta_in_rank % stride != 0) return;
    const int pushers = (lp.ctas_per_vrank + stride - 1) / stride;
    const int gw = (cta_in_rank / stride) * kPushWarps + pw;
    const int total_warps = pushers * kPushWarps;
    const int chunk_rows = (rows_per_rank + P.ag_chunks - 1) / P.ag_chunks;
    const int64_t row_vecs = static_cast<int64_t>(P.K) * kElemBytes / 16;  // 16B vectors per row
    const int64_t src_ld = P.ld_x * kElemBytes;
    const int64_t dst_ld = static_cast<int64_t>(P.K) * kElemBytes;
    const int64_t dst_row0 = static_cast<int64_t>(P.rank) * rows_per_rank;
    const int first_d = P.ag_local_direct ? 1 : 0;
    const int d_hi = min(P.world, P.ag_ce_lo);  // farther peers get the shard from copy engines
    // peer-major: the whole shard goes to rank-1 first (it consumes this shard right after its
    // own), then to rank-2, ...: every GPU sends to and receives from one peer at a time
    for (int d = first_d; d < d_hi; ++d) {
      const int peer = (P.rank - d + P.world) % P.world;
      const char* src = static_cast<const char*>(P.x_local);
      char* dst = static_cast<char*>(P.gather[peer]);
      for (int c = 0; c < P.ag_chunks; ++c) {
        const int r_lo = c * chunk_rows;
        const int r_hi = min(r_lo + chunk_rows, rows_per_rank);
        const int64_t nvec = static_cast<int64_t>(max(r_hi - r_lo, 0)) * row_vecs;
        constexpr int kUnroll = 8;
        for (int64_t v0 = static_cast<int64_t>(gw) * 32 * kUnroll; v0 < nvec;
             v0 += static_cast<int64_t>(total_warps) * 32 * kUnroll) {
          uint4 buf[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int64_t v = v0 + u * 32 + lane;
            if (v < nvec) {
              const int64_t row = v / row_vecs, col = v - row * row_vecs;
              if (EDM_ADDR_OK(src + (r_lo + row) * src_ld + col * 16, 16, 2u))
                buf[u] = ld_cg_v4(src + (r_lo + row) * src_ld + col * 16);
            }
          }
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int64_t v = v0 + u * 32 + lane;
            if (v < nvec) {
              const int64_t row = v / row_vecs, col = v - row * row_vecs;
              if (EDM_ADDR_OK(dst + (dst_row0 + r_lo + row) * dst_ld + col * 16, 16, 3u))
                st_global_v4(dst + (dst_row0 + r_lo + row) * dst_ld + col * 16, buf[u]);
            }
          }
        }
        __syncwarp();
        if (lane == 0)
          mailbox_post(note_box, make_note(kNoteChunk, (static_cast<uint64_t>(peer) << 24) | c), timeout_ns);
      }
    }
    push_total.stop(kProfPushTotal);
  };

  // ------------------------------------------------------------------ reduction of owned tiles
  // Adds up the W partial copies of a 128-row half-tile this rank owns (fp32, fixed rank order,
  // so the result is deterministic) and writes the result to the local output (reduce-scatter)
  // or to every rank's output (all-reduce).  Work units are (half-tile, row quarter); warps take
  // them from a shared counter: the two reducer warps from the start, the epilogue warps once
  // their tiles are done.  None of this holds up the MMA pipeline.
  const bool fused_reduce = (P.mode == kRS || P.mode == kAR) && P.world > 1;
  auto reduce_units = [&](Mailbox* note_box, bool rprof) {
    const int W = P.world;
    const int n_items = walk.owned_count(P.rank) * kCG;  // half-tiles owned by this rank
    const int my_items = n_items > cta_in_rank ? (n_items - cta_in_rank + lp.ctas_per_vrank - 1) / lp.ctas_per_vrank : 0;
    while (true) {
      uint32_t u = 0;
      if (lane == 0) u = atomicAdd(&reduce_next, 1u);
      u = __shfl_sync(0xffffffffu, u, 0);
      if (u >= static_cast<uint32_t>(my_items) * 4u) break;
      const int item = cta_in_rank + static_cast<int>(u >> 2) * lp.ctas_per_vrank;
      const int qq = static_cast<int>(u & 3u);
      const int idx = item / kCG, hp = item - idx * kCG;  // owned tile, half within the pair tile
      int m_blk, n_blk;
      walk.owned_tile(P.rank, idx, m_blk, n_blk);
      const int m0 = (m_blk * kCG + hp) * kBlockM, n0 = n_blk * kBN;
      const int valid_rows = min(kBlockM, P.M - m0), valid_cols = min(kBN, P.N - n0);
      const int64_t out_row0 = P.mode == kRS ? m0 - P.rank * rows_per_rank : m0;
      const int64_t ld_bytes = P.ld_out * kOutBytes;
      const char* slot0 = P.win[P.rank] + static_cast<int64_t>(item) * kTileOutBytes;
      const int64_t src_stride = static_cast<int64_t>(P.max_owned) * kTileOutBytes;
      {
        ProfTimer rf(rprof);
        bool arrived = true;
        if (lane < W)
          arrived = wait_flag(P.flags[P.rank] + P.partial_flag_off +
                                  (static_cast<uint32_t>(lane) * P.max_owned + item) * 4 + qq,
                              P.epoch, timeout_ns, kTimeoutPartialFlag, (lane << 24) | item);
        arrived = __all_sync(0xffffffffu, arrived);
        rf.stop(kProfReducerFlagWait);
        if (!arrived) return;  // a partial never came: nothing more to add up in this launch
#pragma unroll 1
        for (int h = 0; h < kPasses; ++h) {
          const char* blk = slot0 + (h * 4 + qq) * kEpiWarpBytes;  // 512 vectors of 16 B
          // kW sources x kU vectors per lane are loaded before any is used (12 to 20 loads of
          // 16 B in flight per lane whatever the group size), then summed in rank order
          auto run = [&](auto wtag) {
            constexpr int kW = decltype(wtag)::value;
            constexpr int kVecs = kEpiWarpBytes / 16 / 32;  // 16 vectors per lane per block
            constexpr int kU = kW == 2 ? 8 : (kW <= 5 ? 4 : 2);  // divides kVecs; 12 to 20 loads in flight
#pragma unroll 1
            for (int it = 0; it < kVecs; it += kU) {
              uint4 x[kU][kW];
#pragma unroll
              for (int u = 0; u < kU; ++u)
#pragma unroll
                for (int src = 0; src < kW; ++src)
                  x[u][src] = EDM_ADDR_OK(blk + src * src_stride + ((it + u) * 32 + lane) * 16, 16, 4u)
                                  ? ld_cg_v4(blk + src * src_stride + ((it + u) * 32 + lane) * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
              for (int u = 0; u < kU; ++u) {
                float sum[kOutPerVec];
#pragma unroll
                for (int e = 0; e < kOutPerVec; ++e) sum[e] = 0.f;
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
                // undo the staging layout: vector -> (row, logical 16B vector)
                const int vec = (it + u) * 32 + lane;
                const int r = vec >> 4, lv = (vec & 15) ^ (r & 7);
                const int trow = qq * 32 + r, col = h * kColsPerPass + lv * kOutPerVec;
                if (trow < valid_rows && col < valid_cols) {
                  const int64_t off = (out_row0 + trow) * ld_bytes + static_cast<int64_t>(n0 + col) * kOutBytes;
                  if (P.mode == kRS) {
                    if (EDM_ADDR_OK(static_cast<char*>(P.out) + off, 16, 5u))
                      st_global_v4(static_cast<char*>(P.out) + off, o);
                  } else {
#pragma unroll
                    for (int d = 0; d < kW; ++d)
                      if (EDM_ADDR_OK(static_cast<char*>(P.peer_out[(P.rank + d) % kW]) + off, 16, 6u))
                        st_global_v4(static_cast<char*>(P.peer_out[(P.rank + d) % kW]) + off, o);
                  }
                }
              }
            }
          };
          switch (W) {
            case 2: run(IntTag<2>{}); break;
            case 3: run(IntTag<3>{}); break;
            case 4: run(IntTag<4>{}); break;
            case 5: run(IntTag<5>{}); break;
            case 6: run(IntTag<6>{}); break;
            case 7: run(IntTag<7>{}); break;
            default: run(IntTag<8>{}); break;
          }
        }
        if (P.mode == kAR) {
          // this quarter of the reduced half-tile has been stored to every rank's output
          __syncwarp();
          if (lane == 0) {
            const int lin = idx * W + P.rank;
            mailbox_post(&*note_box, make_note(kNoteResult, static_cast<uint32_t>(lin * kCG + hp) * 4 + qq),
                         timeout_ns);
          }
        }
      }
    }
  };

  // ------------------------------------------------------------------ dedicated pusher CTAs
  // One lane of each of kPusherWarps warps moves 8 KiB segments of the shard: bulk load from local
  // memory into one of its kPushDepth staging buffers, bulk store from there into the peer's gather
  // buffer.  Loads run kPushDepth - 1 segments ahead of the stores.  Segments are dealt round-robin
  // over all pusher warps of the rank; a warp counts every (peer, chunk) -- also when it moved
  // nothing of it -- once its copies of that chunk have been written: one relaxed add on the
  // chunk's arrival counter and no fence (a system-scope fence on an SM with remote writes queued
  // costs tens of microseconds; the completed bulk groups have performed their writes).  The flag
  // at the peer is raised by the publisher below, on an SM that pushes nothing.  Waiting for
  // "written" right after the last copy of a chunk would drain the warp's pipeline, so the count
  // goes out kPushDepth segments later, when the bulk-group count alone proves the copies complete.
  auto pusher_role = [&](int w) {
    if (lane != 0) return;
    ProfTimer push_total(prof && w == 0);
    const int T = pusher_ctas * kPusherWarps;
    const int gw = (cta_in_rank - gemm_ctas) * kPusherWarps + w;
    const int first_d = P.ag_local_direct ? 1 : 0;
    const int d_hi = min(P.world, P.ag_ce_lo);
    const int chunk_rows = (rows_per_rank + P.ag_chunks - 1) / P.ag_chunks;
    const int64_t row_bytes = static_cast<int64_t>(P.K) * kElemBytes;
    const int64_t src_ld = P.ld_x * kElemBytes;
    const bool flat = src_ld == row_bytes;  // contiguous shard: segments ignore row boundaries
    const int64_t segs_per_row = (row_bytes + kPushBytes - 1) / kPushBytes;
    const int64_t dst_row0 = static_cast<int64_t>(P.rank) * rows_per_rank;
    const uint32_t buf0 = smem_base + static_cast<uint32_t>(w) * kPushDepth * kPushBytes;
    const uint32_t bar0 = smem_u32(&bars[w * kPushDepth]);

    struct Cursor { int d, c, r_lo, r_hi; int64_t s, nseg, rot; };
    auto open_chunk = [&](Cursor& u) {
      u.r_lo = u.c * chunk_rows;
      u.r_hi = min(u.r_lo + chunk_rows, rows_per_rank);
      const int64_t rows = max(u.r_hi - u.r_lo, 0);
      u.nseg = flat ? (rows * row_bytes + kPushBytes - 1) / kPushBytes : rows * segs_per_row;
      u.s = ((gw - u.rot) % T + T) % T;  // continues the round-robin where the previous chunk stopped
    };
    // next item of this warp's sequence: 0 = a segment, 1 = a chunk is finished (note), 2 = the end
    auto advance = [&](Cursor& u, const char*& src, char*& dst, uint32_t& bytes, uint64_t& note) -> int {
      if (u.d >= d_hi) return 2;
      const int peer = (P.rank - u.d + P.world) % P.world;
      if (u.s < u.nseg) {
        int64_t so, dof;
        if (flat) {
          const int64_t off = u.s * kPushBytes, total = static_cast<int64_t>(u.r_hi - u.r_lo) * row_bytes;
          bytes = static_cast<uint32_t>(min(static_cast<int64_t>(kPushBytes), total - off));
          so = u.r_lo * row_bytes + off;
          dof = (dst_row0 + u.r_lo) * row_bytes + off;
        } else {
          const int64_t row = u.s / segs_per_row, off = (u.s - row * segs_per_row) * kPushBytes;
          bytes = static_cast<uint32_t>(min(static_cast<int64_t>(kPushBytes), row_bytes - off));
          so = (u.r_lo + row) * src_ld + off;
          dof = (dst_row0 + u.r_lo + row) * row_bytes + off;
        }
        src = static_cast<const char*>(P.x_local) + so;
        dst = static_cast<char*>(P.gather[peer]) + dof;
        u.s += T;
        return 0;
      }
      note = static_cast<uint64_t>(peer * P.ag_chunks + u.c);  // index of the chunk's arrival counter
      u.rot = (u.rot + u.nseg) % T;
      if (++u.c == P.ag_chunks) { u.c = 0; ++u.d; }
      if (u.d < d_hi) open_chunk(u);
      return 1;
    };

    auto count_chunk = [&](uint64_t idx) {
      uint32_t* ctr = P.counters + idx;
      if (EDM_ADDR_OK(ctr, 4, 20u)) atomicAdd(ctr, 1u);
    };
    Cursor lc{first_d, 0, 0, 0, 0, 0, 0};
    if (first_d < d_hi) open_chunk(lc);
    Cursor sc = lc;
    uint32_t loads = 0, stores = 0;  // segments whose load / store has been issued
    auto issue_load = [&]() -> bool {
      const char* src = nullptr; char* dst = nullptr; uint32_t bytes = 0; uint64_t note = 0;
      int k;
      while ((k = advance(lc, src, dst, bytes, note)) == 1) {}
      if (k == 2) return false;
      const uint32_t b = loads % kPushDepth;
      mbar_arrive_expect_tx(bar0 + 8 * b, bytes);
      if (EDM_ADDR_OK(src, bytes, 7u)) bulk_load(buf0 + b * kPushBytes, src, bytes, bar0 + 8 * b);
      else mbar_complete_tx(bar0 + 8 * b, bytes);  // checking build: keep the barrier's byte count whole
      ++loads;
      return true;
    };
    for (int i = 0; i < kPushDepth - 1; ++i)
      if (!issue_load()) break;
    bool pending = false;  // a finished chunk whose note has not been posted yet
    uint64_t pending_note = 0;
    uint32_t since = 0;    // copies issued since that chunk ended
    while (true) {
      const char* src = nullptr; char* dst = nullptr; uint32_t bytes = 0; uint64_t note = 0;
      const int k = advance(sc, src, dst, bytes, note);
      if (k == 2) break;
      if (k == 1) {
        if (pending) {
          bulk_wait_pending<0>();
          count_chunk(pending_note);
        }
        pending = true; pending_note = note; since = 0;
        continue;
      }
      const uint32_t b = stores % kPushDepth;
      if (!wait_mbar(bar0 + 8 * b, (stores / kPushDepth) & 1u, timeout_ns, kTimeoutFullBar,
                     0x8000u | static_cast<uint32_t>(w)))
        break;  // a local load never landed: stop copying (what is in flight is awaited below)
      if (EDM_ADDR_OK(dst, bytes, 8u)) bulk_store(dst, buf0 + b * kPushBytes, bytes);
      bulk_commit();
      ++stores;
      // the load that runs kPushDepth - 1 ahead reuses the buffer of the previous store: wait
      // until that store has read it
      bulk_wait_read_pending<1>();
      issue_load();
      if (pending && ++since >= static_cast<uint32_t>(kPushDepth)) {
        bulk_wait_pending<kPushDepth>();  // everything older than the last kPushDepth copies is written
        count_chunk(pending_note);
        pending = false;
      }
    }
    bulk_wait_pending<0>();
    if (pending && !aborted()) count_chunk(pending_note);
    push_total.stop(kProfPushTotal);
  };

  // ------------------------------------------------------------------ publisher (pusher CTAs)
  // One lane of the first tile CTA of the rank -- an SM that issues no remote stores, so its
  // system-scope fence is cheap -- walks the (peer, chunk) pairs in the order the pushers finish
  // them, waits until all pusher warps have counted a chunk, and raises the chunk's flag at the
  // peer.  A counter is re-armed as soon as it has been consumed; the counters of the other bank
  // (epoch parity) are zeroed as well, so that a launch that gave up part-way does not leave stale
  // counts to the call after the next.
  auto publisher_role = [&]() {
    if (lane != 0) return;
    const int first_d = P.ag_local_direct ? 1 : 0;
    const int d_hi = min(P.world, P.ag_ce_lo);
    const uint32_t target = static_cast<uint32_t>(pusher_ctas * kPusherWarps);
    for (int i = 0; i < P.world * P.ag_chunks; ++i)
      if (EDM_ADDR_OK(P.counters_next + i, 4, 21u)) P.counters_next[i] = 0u;
    for (int d = first_d; d < d_hi; ++d) {
      const int peer = (P.rank - d + P.world) % P.world;
      for (int c = 0; c < P.ag_chunks; ++c) {
        const uint32_t* ctr = P.counters + peer * P.ag_chunks + c;
        if (!EDM_ADDR_OK(ctr, 4, 22u)) return;
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (ld_acquire_gpu(ctr) < target) {
          if ((spins++ & 31u) == 0u) {
            if (aborted()) return;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > timeout_ns) { report(kTimeoutPushCount, (peer << 16) | c, target, ld_acquire_gpu(ctr)); return; }
          }
          __nanosleep(100);
        }
        *reinterpret_cast<volatile uint32_t*>(P.counters + peer * P.ag_chunks + c) = 0u;  // re-armed for a later call
        fence_acq_rel_sys();
        uint32_t* flag = P.flags[peer] + P.gather_flag_off + P.rank * P.ag_chunks + c;
        if (EDM_ADDR_OK(flag, 4, 23u)) st_relaxed_sys(flag, P.epoch);
      }
    }
  };

  // ------------------------------------------------------------------ signaller
  // Lane w serves mailbox w.  A batch of notes costs one system-scope fence; the flag stores
  // after it are relaxed (the fence already orders the landed data before them).
  auto signaller_role = [&]() {
    // (nothing is ever posted without an exchange, nor by the tile CTAs of a launch with dedicated
    // pushers: stay off the issue slots then)
    if (lane < kMailboxes && P.world > 1 && P.mode != kPlain && !(P.mode == kAG && P.ag_external) &&
        !(pusher_ctas > 0 && !is_pusher)) {
      volatile Mailbox* mb = &mbox[lane];
      uint32_t done = 0;
      uint64_t idle_since = 0;
      const int total_push_warps = pusher_ctas > 0 ? pusher_ctas * kPusherWarps
          : (lp.ctas_per_vrank + max(lp.push_stride, 1) - 1) / max(lp.push_stride, 1) * kPushWarps;
      while (true) {
        const uint32_t ready = mb->ready;
        if (ready != done) {
          __threadfence_block();
          fence_acq_rel_sys();
          for (; done != ready; ++done) {
            const uint64_t note = mb->note[done % kMailboxDepth];
            const uint64_t kind = note >> 60, payload = note & ((1ull << 60) - 1);
            if (kind == kNoteFlag) {
              if (EDM_ADDR_OK(reinterpret_cast<uint32_t*>(payload), 4, 9u))
                st_relaxed_sys(reinterpret_cast<uint32_t*>(payload), P.epoch);
            } else if (kind == kNoteResult) {
              for (int peer = 0; peer < P.world; ++peer)
                if (peer != P.rank && EDM_ADDR_OK(P.flags[peer] + P.result_flag_off + static_cast<uint32_t>(payload), 4, 10u))
                  st_relaxed_sys(P.flags[peer] + P.result_flag_off + static_cast<uint32_t>(payload), P.epoch);
            } else {
              const int peer = static_cast<int>(payload >> 24), c = static_cast<int>(payload & 0xFFFFFF);
              uint32_t* ctr = P.counters + peer * P.ag_chunks + c;
              if (!EDM_ADDR_OK(ctr, 4, 11u) ||
                  !EDM_ADDR_OK(P.flags[peer] + P.gather_flag_off + P.rank * P.ag_chunks + c, 4, 12u)) continue;
              if (atomicAdd(ctr, 1u) == static_cast<uint32_t>(total_push_warps - 1)) {
                // last push warp of this GPU: every piece of the chunk has been written
                *reinterpret_cast<volatile uint32_t*>(ctr) = 0u;
                fence_acq_rel_sys();
                st_relaxed_sys(P.flags[peer] + P.gather_flag_off + P.rank * P.ag_chunks + c, P.epoch);
              }
            }
          }
          mb->done = done;
          idle_since = 0;
        } else if (mb->closed) {
          if (mb->ready == done) break;
        } else {
          __nanosleep(1000);
          if (aborted()) break;
          const uint64_t now = globaltimer_ns();
          if (idle_since == 0) idle_since = now;
          else if (now - idle_since > 4 * timeout_ns) break;  // posters are bounded; this is a backstop
        }
      }
    }
  };

  if (is_pusher) {
    // ============================ pusher CTA ============================
    if (warp < kPusherWarps) pusher_role(warp);
  } else if (warp == 0) {
    // ============================ TMA producer ============================
    if (lane == 0) {
      tma_prefetch_desc(&P.tmap_a[0]);
      tma_prefetch_desc(&P.tmap_b[0]);
      uint32_t it = 0, s = 0, ph = 0;  // ring position: stage and the phase bit of its current use
      uint64_t seen_chunks = 0;        // all-gather chunks whose flag this CTA has already acquired
      const int prof_empty = prof ? kProfProducerEmptyWait : -1;
      Work w;
      bool tail_taken = false;
      bool alive = true;  // false once a wait gave up: no further loads are issued
      for (int i = cta; alive && next_work(i, tail_taken, pr == 0, w);) {
        const int k_lo = w.k_lo, k_hi = w.k_hi;
        const Tile t = walk.at(w.pos);
        if (!t.valid) continue;
        int m0, b_row0, rows_unused;  // this CTA's rows of A
        block_rows(t.m_blk, static_cast<int>(pr), m0, b_row0, rows_unused);
        const int n0 = b_row0 + t.n_blk * kBN + static_cast<int>(pr) * (kBN / kCG);  // its rows of B
        const CUtensorMap* amap = &P.tmap_a[0];
        int a_row = m0;
        if (P.mode == kAG) {
          // wait for every shard chunk this row block touches
          const int m1 = min(m0 + kBlockM, P.M);
          const int chunk_rows = (rows_per_rank + P.ag_chunks - 1) / P.ag_chunks;
          const int s_lo = m0 / rows_per_rank, s_hi = (m1 - 1) / rows_per_rank;
          if (P.ag_local_direct && s_lo == P.rank) {
            amap = &P.tmap_a[1];
            a_row = m0 - P.rank * rows_per_rank;
          } else {
            ProfTimer pt(prof);
            bool fresh = false;  // some chunk is seen for the first time by this CTA
            for (int s = s_lo; s <= s_hi; ++s) {
              const int lo = max(m0, s * rows_per_rank) - s * rows_per_rank;
              const int hi = min(m1, (s + 1) * rows_per_rank) - s * rows_per_rank;
              for (int c = lo / chunk_rows; c <= (hi - 1) / chunk_rows; ++c) {
                const int id = s * P.ag_chunks + c;
                if (id < 64 && ((seen_chunks >> id) & 1ull)) continue;  // acquired earlier
                ProfTimer pa(prof);
                alive = alive && wait_flag(P.flags[P.rank] + P.gather_flag_off + id, P.epoch,
                                           timeout_ns, kTimeoutGatherFlag, (s << 16) | c);
                pa.stop(kProfProducerFlagPoll);
                if (id < 64) seen_chunks |= 1ull << id;
                fresh = true;
              }
            }
            // rows written by a peer (generic proxy) are read by TMA (async proxy) next
            if (fresh) {
              ProfTimer pf(prof);
              fence_proxy_async_global();
              pf.stop(kProfProducerProxyFence);
            }
            pt.stop(kProfProducerGatherWait);
          }
        }
        for (int seg = 0; alive && seg < num_segs; ++seg) {
          const int j0 = k_lo + seg * seg_kb, j1 = min(j0 + seg_kb, k_hi);
          for (int pass = 0; alive && pass < P.passes; ++pass) {
            // split fp32: (lo,hi), (hi,lo), then (hi,hi) so the small terms meet a small accumulator
            const CUtensorMap* am = (P.passes == 3 && pass == 0) ? &P.tmap_a[1] : amap;
            const CUtensorMap* bm = (P.passes == 3 && pass == 1) ? &P.tmap_b[1] : &P.tmap_b[0];
            for (int j = j0; j < j1; ++j, ++it, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0)) {
              if (!wait_mbar(bar_empty + 8 * s, ph ^ 1u, timeout_ns, kTimeoutEmptyBar, it, prof_empty)) {
                alive = false;
                break;
              }
              const uint32_t sa = smem_base + s * kStageBytes;
              if constexpr (kCG == 1) {
                mbar_arrive_expect_tx(bar_full + 8 * s, kStageBytes);
                tma_load_2d(sa, am, j * kBlockK, a_row, bar_full + 8 * s);
                tma_load_2d(sa + kStageABytes, bm, j * kBlockK, n0, bar_full + 8 * s);
              } else {
                // both CTAs' loads complete on the even CTA's barrier, which expects both stages
                if (pr == 0) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * kStageBytes);
                const uint32_t fb = map_to_cta(bar_full + 8 * s, 0);
                tma_load_2d_pair(sa, am, j * kBlockK, a_row, fb);
                tma_load_2d_pair(sa + kStageABytes, bm, j * kBlockK, n0, fb);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0 && pr == 0) {
      constexpr uint32_t idesc = make_idesc<kCG, kBN, kTf32>();
      uint32_t it = 0, unit = 0;  // unit = (tile, K segment): one TMEM accumulator each
      uint32_t s = 0, ph = 0;     // ring position: stage and the phase bit of its current use
      const uint64_t adesc0 = make_smem_desc(smem_base);
      const int prof_full = prof ? kProfMmaFullWait : -1, prof_tmem = prof ? kProfMmaTmemWait : -1;
      Work w;
      bool tail_taken = false;
      bool alive = true;  // false once a wait gave up: no further MMAs are issued
      for (int i = cta; alive && next_work(i, tail_taken, false, w);) {
        const int k_lo = w.k_lo, k_hi = w.k_hi;
        if (!walk.at(w.pos).valid) continue;
        for (int seg = 0; alive && seg < num_segs; ++seg, ++unit) {
          const uint32_t acc = unit & 1u;
          if (!wait_mbar(bar_tempty + 8 * acc, ((unit >> 1) & 1u) ^ 1u, timeout_ns, kTimeoutTmemEmpty, unit, prof_tmem)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * kBN;
          const int nkb = (min(k_lo + (seg + 1) * seg_kb, k_hi) - (k_lo + seg * seg_kb)) * P.passes;
          for (int kb = 0; kb < nkb; ++kb, ++it, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0)) {
            if (!wait_mbar(bar_full + 8 * s, ph, timeout_ns, kTimeoutFullBar, it, prof_full)) {
              alive = false;
              break;
            }
            tc_fence_after();
            // stage s sits s * kStageBytes further on: only the address field (16-byte units) moves
            const uint64_t adesc = adesc0 + s * (kStageBytes >> 4);
            const uint64_t bdesc = adesc + (kStageABytes >> 4);
#pragma unroll
            for (int k = 0; k < kBlockKBytes / 32; ++k) {
              // each MMA consumes 32 bytes of K; descriptors advance in 16-byte units
              umma_ss<kCG, kTf32>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if constexpr (kCG == 1) umma_commit(bar_empty + 8 * s);
            else umma_commit_pair(bar_empty + 8 * s, 3);
          }
          if (!alive) break;
          if constexpr (kCG == 1) umma_commit(bar_tfull + 8 * acc);
          else umma_commit_pair(bar_tfull + 8 * acc, 3);
        }
      }
    }
  } else if (warp < 4) {
    // ============================ all-gather pushes ============================
    if (ag_push) push_shard(warp - 2, &mbox[4 + (warp - 2)]);
    if (fused_reduce) {
      // ============================ reducer ============================
      const bool rprof = prof && lane == 0 && warp == 2;
      ProfTimer red_total(rprof);
      reduce_units(&mbox[4 + (warp - 2)], rprof);
      red_total.stop(kProfReducerTotal);
    }
    __syncwarp();
    if (lane == 0) mailbox_close(&mbox[4 + (warp - 2)]);
  } else if (warp < 8) {
    // ============================ epilogue ============================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool eprof = prof && lane == 0 && q == 0;
    ProfTimer epi_total(eprof);
    const uint32_t stage_smem = smem_epi + q * kEpiWarpBytes;
    const int row = q * 32 + lane;  // row within the tile owned by this thread
    uint32_t unit = 0;  // (tile, K segment) counter, in step with the MMA warp
    bool bulk_pending = false;  // a bulk copy out of this warp's staging rows may still be reading them
    uint32_t* pend_old = nullptr;  // flags of the (up to two) shipped tiles whose copies may be in flight
    uint32_t* pend_new = nullptr;
    // a tile of >= 32 K blocks takes longer than a remote copy needs to land (see settle_early use)
    const bool settle_early = num_kb_pass * P.passes >= 32;
    const bool fused = (P.mode == kRS || P.mode == kAR) && P.world > 1;
    // running fp32 sums of this thread's row: [chunk][row][32 floats], private to the CTA
    float* my_scratch = P.scratch == nullptr ? nullptr
        : P.scratch + (static_cast<size_t>(blockIdx.x) * kBlockM * kBlockN + static_cast<size_t>(row) * 32);
    // partial sums of a piece of a split tail tile: this thread's row in this CTA's scratch tile
    // scratch tile / flags of piece `idx` for this CTA's half of the tile
    auto tail_slot = [&](int idx) { return vr * lp.ctas_per_vrank + idx * kCG + static_cast<int>(pr); };
    // accumulator `u` -> fp32 tile at dst ([32-column chunk][row][32 floats]), optionally added to what is there
    // (returns false when the accumulator never became ready: the caller stops)
    auto dump_accumulator = [&](uint32_t u, float* dst, bool add) -> bool {
      const uint32_t sacc = u & 1u;
      uint32_t ready = 1u;
      if (lane == 0)
        ready = wait_mbar(bar_tfull + 8 * sacc, (u >> 1) & 1u, timeout_ns, kTimeoutTmemFull, u) ? 1u : 0u;
      if (!__shfl_sync(0xffffffffu, ready, 0)) return false;
      tc_fence_after();
      const uint32_t staddr = tmem_base + sacc * kBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(staddr + c * 32, raw);
        tmem_ld_wait();
        float4* sp = reinterpret_cast<float4*>(dst + static_cast<size_t>(c) * kBlockM * 32);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          float4 x = make_float4(__uint_as_float(raw[4 * w]), __uint_as_float(raw[4 * w + 1]),
                                 __uint_as_float(raw[4 * w + 2]), __uint_as_float(raw[4 * w + 3]));
          if (add) {
            const float4 y = sp[w];
            x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
          }
          sp[w] = x;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCG == 1) mbar_arrive(bar_tempty + 8 * sacc);
        else mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * sacc, 0));
      }
      return true;
    };
    // One of the `n_parts` pieces (K ranges) of a split tail tile.  The pieces run at the same time
    // on different CTAs and finish the tile together: piece p owns the 32-column chunks
    // [p, p+1) * 8 / n_parts of the tile.  It leaves its partial sums of all other chunks in its
    // scratch tile, raises its flag, waits for the other pieces' flags, adds their partial sums of
    // its own chunks to its accumulator and writes those columns of the output.
    auto tail_piece = [&](const Tile& t, const Work& wk, uint32_t u) {
      const int part = wk.part, n_parts = wk.n_parts;
      const int my_slot = tail_slot(wk.piece), slot0 = tail_slot(wk.piece - part);  // own, and piece 0 of the tile
      // A scratch tile is 32 blocks of 4 KiB, block (chunk c, warp q) = the warp's 32 rows x 32
      // columns as [8 vectors][32 rows] x 16 bytes: a warp writes and reads 512 contiguous bytes
      // per instruction, and a block moves with one bulk copy.
      constexpr uint32_t kBlk = 4096;
      constexpr size_t kTileBytes = static_cast<size_t>(kBlockM) * kBlockN * 4;
      char* const scratch = reinterpret_cast<char*>(g_tail_scratch);
      const uint32_t acc = u & 1u;
      // (accounting slots of the reducer and of the fused epilogue double for the pieces' exchange)
      ProfTimer piece_total(eprof);
      if (lane == 0) {
        ProfTimer pt(eprof);
        wait_mbar(bar_tfull + 8 * acc, (u >> 1) & 1u, timeout_ns, kTimeoutTmemFull, u);
        pt.stop(kProfEpiTmemWait);
      }
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
      ProfTimer pdump(eprof);
      const int per = (kBN / 32) / n_parts, c_lo = part * per, c_hi = c_lo + per;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        if (c >= c_lo && c < c_hi) continue;
        uint32_t raw[32];
        tmem_ld_32x32(taddr + c * 32, raw);
        tmem_ld_wait();
        char* blk = scratch + my_slot * kTileBytes + static_cast<size_t>(c * 4 + q) * kBlk + lane * 16;
#pragma unroll
        for (int w = 0; w < 8; ++w)
          if (EDM_ADDR_OK(blk + w * 512, 16, 13u))
            st_global_v4(blk + w * 512, make_uint4(raw[4 * w], raw[4 * w + 1], raw[4 * w + 2], raw[4 * w + 3]));
      }
      pdump.stop(kProfEpiIssue);
      ProfTimer pfence(eprof);
      __threadfence();
      __syncwarp();
      pfence.stop(kProfEpiFence);
      if (lane == 0 && EDM_ADDR_OK(&g_tail_flags[my_slot * 4 + q], 4, 14u))
        st_relaxed_sys(&g_tail_flags[my_slot * 4 + q], lp.tail_epoch);
      ProfTimer pwait(eprof);
      if (lane < n_parts && lane != part)
        wait_flag(&g_tail_flags[(slot0 + lane * kCG) * 4 + q], lp.tail_epoch, timeout_ns,
                  kTimeoutTailFlag, lane);
      __syncwarp();
      // The other pieces' partial sums of this piece's chunks come in with bulk copies, all in
      // flight at once, into operand-ring space (the ring is idle: this piece was the CTA's last
      // work and its MMAs have completed).  At most 7 blocks per warp.
      const uint32_t land = smem_base + static_cast<uint32_t>(q) * 7u * kBlk;
      const uint32_t my_bar = bar_tail + 8 * q;
      if (lane == 0) {
        fence_proxy_async_global();  // written with ordinary stores by the peers, read by a bulk copy here
        mbar_arrive_expect_tx(my_bar, static_cast<uint32_t>((n_parts - 1) * per) * kBlk);
        uint32_t dst = land;
        for (int p = 0; p < n_parts; ++p) {
          if (p == part) continue;
          for (int c = c_lo; c < c_hi; ++c, dst += kBlk) {
            const char* from = scratch + (slot0 + p * kCG) * kTileBytes + static_cast<size_t>(c * 4 + q) * kBlk;
            if (EDM_ADDR_OK(from, kBlk, 15u) && dst + kBlk <= smem_base + kPipeBytes) bulk_load(dst, from, kBlk, my_bar);
            else mbar_complete_tx(my_bar, kBlk);
          }
        }
      }
      wait_mbar(my_bar, 0u, timeout_ns, kTimeoutTailFlag, 0x100u | static_cast<uint32_t>(q));
      pwait.stop(kProfReducerFlagWait);
      const int m0 = (t.m_blk * kCG + static_cast<int>(pr)) * kBlockM, n0 = t.n_blk * kBN;
      char* out_row = static_cast<char*>(P.out) + (static_cast<int64_t>(m0 + row) * P.ld_out + n0) * kOutBytes;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(taddr + c * 32, raw);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
#pragma unroll 1
        for (int k = 0; k < n_parts - 1; ++k) {
          const uint32_t blk = land + static_cast<uint32_t>(k * per + (c - c_lo)) * kBlk + lane * 16;
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const uint4 y = ld_shared_v4(blk + w * 512);
            v[4 * w] += __uint_as_float(y.x); v[4 * w + 1] += __uint_as_float(y.y);
            v[4 * w + 2] += __uint_as_float(y.z); v[4 * w + 3] += __uint_as_float(y.w);
          }
        }
        if (m0 + row < P.M) {
#pragma unroll
          for (int w = 0; w < 32 / kOutPerVec; ++w) {
            uint4 o;
            if constexpr (kOutBytes == 2) {
              o = OutPack<__nv_bfloat16>::pack8(&v[w * 8]);
            } else {
              o.x = __float_as_uint(v[w * 4 + 0]); o.y = __float_as_uint(v[w * 4 + 1]);
              o.z = __float_as_uint(v[w * 4 + 2]); o.w = __float_as_uint(v[w * 4 + 3]);
            }
            const int col = c * 32 + w * kOutPerVec;
            if (n0 + col < P.N && EDM_ADDR_OK(out_row + col * kOutBytes, 16, 16u)) st_global_v4(out_row + col * kOutBytes, o);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCG == 1) mbar_arrive(bar_tempty + 8 * acc);
        else mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
      }
      piece_total.stop(kProfReducerTotal);
    };
    Work w;
    bool tail_taken = false;
    for (int i = cta; next_work(i, tail_taken, false, w);) {
      const Tile t = walk.at(w.pos);
      if (!t.valid) continue;
      if (w.n_parts > 1) {
        tail_piece(t, w, unit++);
        continue;
      }
      // this CTA's 128-row half of the tile: its slot / flag index at the owner
      const int slot_idx = t.owned_idx * kCG + static_cast<int>(pr);
      // every segment but the last is only folded into the running sum
      bool segs_ok = true;
      for (int seg = 0; segs_ok && seg + 1 < num_segs; ++seg, ++unit) segs_ok = dump_accumulator(unit, my_scratch, seg > 0);
      if (!segs_ok) break;
      const uint32_t tile_iter = unit++;
      const uint32_t acc = tile_iter & 1u;
      uint32_t tile_ready = 1u;
      if (lane == 0) {
        ProfTimer pt(eprof);
        tile_ready = wait_mbar(bar_tfull + 8 * acc, (tile_iter >> 1) & 1u, timeout_ns, kTimeoutTmemFull, tile_iter) ? 1u : 0u;
        pt.stop(kProfEpiTmemWait);
        if (tile_ready && settle_early && pend_new != nullptr) {
          // Long tiles: the previous tile's copies were issued a whole tile time ago and have
          // landed by now, so its flag can go out one tile (not two) after the data.
          ProfTimer pw(eprof);
          bulk_wait_pending<0>();
          pw.stop(kProfEpiFlagWait);
          mailbox_post(&mbox[q], make_note(kNoteFlag, reinterpret_cast<uint64_t>(pend_new)), timeout_ns);
          pend_new = nullptr;
        }
      }
      // (the shuffle also re-converges the warp) an accumulator that never became ready ends this
      // warp's tile loop: nothing more is read from TMEM or shipped
      if (!__shfl_sync(0xffffffffu, tile_ready, 0)) break;
      tc_fence_after();
      // Where the tile goes.  Fused modes: every tile -- this rank's own included -- is shipped
      // as a partial into the owner's window slot [source rank][slot]; the owner's reducer warps
      // add the slots up.  Otherwise it is written to the output in place.
      int m0, b_row_unused, valid_rows;
      block_rows(t.m_blk, static_cast<int>(pr), m0, b_row_unused, valid_rows);
      const int n0 = t.n_blk * kBN;
      const int valid_cols = min(kBN, P.N - n0);
      char* dst_base;
      if (fused)
        dst_base = P.win[t.owner] + (static_cast<int64_t>(P.rank) * P.max_owned + slot_idx) * kTileOutBytes;
      else
        dst_base = static_cast<char*>(P.out) + (static_cast<int64_t>(m0) * P.ld_out + n0) * kOutBytes;
      const int64_t dst_ld = P.ld_out * kOutBytes;

      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int h = 0; h < kPasses; ++h) {
#pragma unroll
        for (int j = 0; j < kChunksPerPass; ++j) {
          const int c = h * kChunksPerPass + j;  // 32-column chunk of the tile
          uint32_t raw[32];
          ProfTimer ptl(eprof);
          tmem_ld_32x32(taddr + c * 32, raw);
          tmem_ld_wait();
          ptl.stop(kProfEpiTmemLoad);
          if (c == kBN / 32 - 1) {
            // accumulator fully read: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (kCG == 1) mbar_arrive(bar_tempty + 8 * acc);
              else mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
            }
          }
          float v[32];
          if (num_segs > 1) {
            // add the running sum of the earlier K segments (written by this same thread)
            const float4* sp = reinterpret_cast<const float4*>(my_scratch + static_cast<size_t>(c) * kBlockM * 32);
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              const float4 y = sp[w];
              v[4 * w] = __uint_as_float(raw[4 * w]) + y.x;
              v[4 * w + 1] = __uint_as_float(raw[4 * w + 1]) + y.y;
              v[4 * w + 2] = __uint_as_float(raw[4 * w + 2]) + y.z;
              v[4 * w + 3] = __uint_as_float(raw[4 * w + 3]) + y.w;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
          }
          if (j == 0 && bulk_pending) {
            // the previous pass's bulk copy may still be reading the staging rows
            if (lane == 0) {
              ProfTimer pt(eprof);
              bulk_wait_read_all();
              pt.stop(kProfEpiStagingWait);
            }
            __syncwarp();
            bulk_pending = false;
          }
          // registers -> staging: thread owns row `lane`; 16B vectors XOR-swizzled by row
#pragma unroll
          for (int w = 0; w < 32 / kOutPerVec; ++w) {
            uint4 o;
            if constexpr (kOutBytes == 2) {
              o = OutPack<__nv_bfloat16>::pack8(&v[w * 8]);
            } else {
              o.x = __float_as_uint(v[w * 4 + 0]); o.y = __float_as_uint(v[w * 4 + 1]);
              o.z = __float_as_uint(v[w * 4 + 2]); o.w = __float_as_uint(v[w * 4 + 3]);
            }
            const int lv = j * (32 / kOutPerVec) + w;  // logical 16B vector within the staged row
            st_shared_v4(stage_smem + lane * kEpiRowBytes + ((lv ^ (lane & 7)) << 4), o);
          }
        }
        if (fused) {
          // ship the warp's 8 KiB of staged rows as they are with one bulk copy; a slot keeps the
          // staging layout [pass][warp][row][swizzled 16B vectors]
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            ProfTimer pi(eprof);
            if (EDM_ADDR_OK(dst_base + (h * 4 + q) * kEpiWarpBytes, kEpiWarpBytes, 17u))
              bulk_store(dst_base + (h * 4 + q) * kEpiWarpBytes, stage_smem, kEpiWarpBytes);
            bulk_commit();
            pi.stop(kProfEpiIssue);
          }
          bulk_pending = true;
          continue;
        }
        __syncwarp();
        // staging -> global: two full 256B rows per warp instruction
        const int col0 = h * kColsPerPass;  // first tile column of this pass
#pragma unroll 4
        for (int itr = 0; itr < 16; ++itr) {
          const int lr = itr * 2 + (lane >> 4);  // row within the warp's 32 rows
          const int lv = lane & 15;
          const uint4 x = ld_shared_v4(stage_smem + lr * kEpiRowBytes + ((lv ^ (lr & 7)) << 4));
          const int col = col0 + lv * kOutPerVec;
          if (q * 32 + lr < valid_rows && col < valid_cols &&
              EDM_ADDR_OK(dst_base + static_cast<int64_t>(q * 32 + lr) * dst_ld + col * kOutBytes, 16, 18u))
            st_global_v4(dst_base + static_cast<int64_t>(q * 32 + lr) * dst_ld + col * kOutBytes, x);
        }
        __syncwarp();
      }

      if (fused && lane == 0) {
        // Two shipped tiles may be in flight per warp.  When a third has been issued, the oldest
        // is certainly older than the 2 * kPasses newest copy groups, so waiting for "all but
        // those" settles it without draining the link; then the signaller gets its flag.
        if (pend_old != nullptr) {
          ProfTimer pt(eprof);
          bulk_wait_pending<2 * kPasses>();
          pt.stop(kProfEpiFlagWait);
          mailbox_post(&mbox[q], make_note(kNoteFlag, reinterpret_cast<uint64_t>(pend_old)), timeout_ns);
        }
        pend_old = pend_new;
        pend_new = P.flags[t.owner] + P.partial_flag_off +
                   (static_cast<uint32_t>(P.rank) * P.max_owned + slot_idx) * 4 + q;
      }
    }
    if (eprof) atomicAdd(&g_prof[kProfEpiTileLoop], static_cast<unsigned long long>(globaltimer_ns() - epi_total.t0));
    if (lane == 0) {
      ProfTimer pfn(eprof);
      bulk_wait_pending<0>();  // nothing of this warp's staging may be in flight when the CTA exits
      if (pend_new != nullptr) {
        if (pend_old != nullptr)
          mailbox_post(&mbox[q], make_note(kNoteFlag, reinterpret_cast<uint64_t>(pend_old)), timeout_ns);
        mailbox_post(&mbox[q], make_note(kNoteFlag, reinterpret_cast<uint64_t>(pend_new)), timeout_ns);
      }
      pfn.stop(kProfEpiFinalNotes);
    }
    __syncwarp();
    if (fused_reduce) reduce_units(&mbox[q], false);  // tiles done: help add up the owned tiles
    __syncwarp();
    if (lane == 0) mailbox_close(&mbox[q]);
    __syncwarp();
    epi_total.stop(kProfEpiTotal);

    if (P.mode == kAR && fused) {
      // the call is complete on this rank only when every other owner's tiles have arrived
      const int gw = cta_in_rank * 4 + q;
      const int total_warps = lp.ctas_per_vrank * 4;
      const int nflags = walk.total * kCG * 4;  // (tile half, quarter) pairs
      for (int base = gw * 32; base < nflags; base += total_warps * 32) {
        const int idx = base + lane;
        if (idx < nflags && ((idx >> 2) / kCG) % P.world != P.rank)
          wait_flag(P.flags[P.rank] + P.result_flag_off + idx, P.epoch, timeout_ns,
                    kTimeoutResultFlag, idx);
      }
    }
  }

  else if (warp == 8) {
    // ============================ signaller / publisher ============================
    if (pusher_ctas > 0) { if (cta_in_rank == 0) publisher_role(); }
    else signaller_role();
  } else {
    // ============================ extra reducers / push warps (warps 9-11) ============================
    if (fused_reduce) reduce_units(&mbox[6 + (warp - 9)], false);
    if (ag_push) push_shard(2 + (warp - 9), &mbox[6 + (warp - 9)]);
    __syncwarp();
    if (lane == 0) mailbox_close(&mbox[6 + (warp - 9)]);
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  prof_kernel.stop(kProfKernelTotal);
  if (prof && threadIdx.x == 0) atomicAdd(&g_prof[kProfCtas], 1ull);
  if (aborted()) __nanosleep(200000);  // let loads that are still in flight land before smem goes away
  // a pair leaves together: the partner may still signal this CTA's barriers or read its smem
  if constexpr (kCG == 2) cluster_sync_all();
  if (warp == 2 && !is_pusher) {
    tc_fence_after();
    tmem_dealloc<kCG>(tmem_base, kTmemCols);
  }
}

// Split fp32 into a tf32-representable high part and the (tf32-rounded) remainder.
__global__ void split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                  float* __restrict__ lo, int64_t rows, int64_t cols, int64_t ld) {
  const int64_t n = rows * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const float v = x[r * ld + c];
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    const float rem = v - __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rem));
    hi[i] = __uint_as_float(h);
    lo[i] = __uint_as_float(l);
  }
}

// ------------------------------------------------------------------ link probe
// Copies `bytes` from local memory into a peer's window, with the store mechanisms the fused
// kernels use, so the host can measure what the link sustains (calibration of the schedule
// selector's transfer term).  mode 0: 16-byte loads and stores from every thread; mode 1: every
// warp stages 8 KiB in shared memory and ships it with one bulk copy; modes 2 and 3: the pusher
// CTAs' mechanism -- bulk load into shared memory, bulk store from there, one lane per warp --
// with 16 KiB (6 warps x 2 buffers) and 32 KiB (3 warps x 2 buffers) per copy.
__global__ void __launch_bounds__(256, 1)
p2p_probe_kernel(const char* __restrict__ src, char* __restrict__ dst, size_t bytes, int mode) {
  extern __shared__ uint8_t probe_smem[];
  __shared__ uint64_t probe_bars[12];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (mode == 0) {
    const size_t nvec = bytes / 16;
    constexpr int kU = 8;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * kU;
    for (size_t v0 = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x - lane) * kU; v0 < nvec; v0 += stride) {
      uint4 buf[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const size_t v = v0 + u * 32 + lane;
        if (v < nvec) buf[u] = ld_cg_v4(src + v * 16);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const size_t v = v0 + u * 32 + lane;
        if (v < nvec) st_global_v4(dst + v * 16, buf[u]);
      }
    }
  } else if (mode == 1) {
    constexpr uint32_t kChunk = 8192;
    const uint32_t base = (smem_u32(probe_smem) + 127u) & ~127u;
    const uint32_t buf0 = base + warp * 2 * kChunk;
    const size_t nchunks = bytes / kChunk;
    const size_t gw = static_cast<size_t>(blockIdx.x) * 8 + warp, tw = static_cast<size_t>(gridDim.x) * 8;
    int b = 0;
    for (size_t c = gw; c < nchunks; c += tw, b ^= 1) {
      const uint32_t sb = buf0 + b * kChunk;
      // the bulk copy issued two iterations ago out of this buffer must have read it
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 16; ++u)
        st_shared_v4(sb + (u * 32 + lane) * 16, ld_cg_v4(src + c * kChunk + (u * 32 + lane) * 16));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        bulk_store(dst + c * kChunk, sb, kChunk);
        bulk_commit();
      }
    }
    if (lane == 0) bulk_wait_all();
  } else {
    const uint32_t chunk = mode == 2 ? 16384u : 32768u;
    const int warps = mode == 2 ? 6 : 3;
    if (threadIdx.x == 0) {
      for (int i = 0; i < 12; ++i) mbar_init(smem_u32(&probe_bars[i]), 1);
      mbar_fence_init();
      fence_proxy_async_smem();
    }
    __syncthreads();
    if (warp >= warps || lane != 0) return;
    const uint32_t base = (smem_u32(probe_smem) + 127u) & ~127u;
    const uint32_t buf0 = base + warp * 2 * chunk;
    const uint32_t bar0 = smem_u32(&probe_bars[warp * 2]);
    const size_t nchunks = bytes / chunk;
    const size_t gw = static_cast<size_t>(blockIdx.x) * warps + warp, tw = static_cast<size_t>(gridDim.x) * warps;
    uint32_t n = 0;
    size_t next = gw;
    if (next < nchunks) {  // one load ahead of the stores
      mbar_arrive_expect_tx(bar0, chunk);
      bulk_load(buf0, src + next * chunk, chunk, bar0);
    }
    for (size_t c = gw; c < nchunks; c += tw, ++n) {
      const uint32_t b = n & 1u;
      uint32_t spins = 0;
      while (!mbar_try_wait(bar0 + 8 * b, (n >> 1) & 1u))
        if (++spins > (1u << 24)) return;  // bounded: a load that never lands ends the probe
      bulk_store(dst + c * chunk, buf0 + b * chunk, chunk);
      bulk_commit();
      const size_t nx = c + tw;
      if (nx < nchunks) {
        // the other buffer was read by the store before this one
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        mbar_arrive_expect_tx(bar0 + 8 * (b ^ 1u), chunk);
        bulk_load(buf0 + (b ^ 1u) * chunk, src + nx * chunk, chunk, bar0 + 8 * (b ^ 1u));
      }
    }
    bulk_wait_all();
  }
}

}  // namespace edm
