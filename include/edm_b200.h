/* C ABI of the B200 backend for EDM-IR's tensor-parallel linear layer.
 *
 * Everything is plain C: raw device pointers, sizes in elements, a CUDA stream passed as
 * void*, integer status returns.  Nothing here allocates on the launch path; the caller owns
 * every tensor, the library owns only what edm_comm_create() hands out.
 *
 * Operand convention (all GEMM entry points): A is [M,K] row-major, B is [N,K] row-major
 * (both K-major, "TN"), D is [M,N] row-major.  This is the convention of the reference's only
 * GEMM operator, tiled_mma_bf16_bf16_bf16_fp32 (EDM-IR/ir/c-extension/mma.cu:24-25, :175).
 * Leading dimensions are in elements and must make every row start 16-byte aligned.
 *
 * The reference has no collective, window or selector code; where an entry point has no
 * reference counterpart its comment says which reference concept it serves instead.
 *
 * Threads and devices: the library keeps a little state per device (function attributes,
 * occupancy, the address of its static scratch, the event that keeps launches sharing its
 * K-split scratch apart) in tables indexed by the current device and guarded by locks or
 * atomics, so entry points may be called from several host threads and a process may drive
 * several GPUs.  A context (edm_comm_t) and the launches on it belong to one thread at a time.
 * edm_set_timeout_ms / edm_profile_enable are process-wide settings.
 *
 * A checking variant of the library (built with -DEDM_DEBUG_BOUNDS, `python -m edmir_b200.build
 * --checked`) validates every global address the kernels compute against the ranges the launch
 * may touch and reports a violation as status code 9 (address in the status words) instead of
 * performing the access; it synchronises around every launch and refuses stream capture.
 */
#ifndef EDM_B200_H_
#define EDM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define EDM_OK 0
#define EDM_ERR_BAD_ARG 1        /* shape / alignment / null pointer */
#define EDM_ERR_CUDA 2           /* a CUDA call failed; see edm_last_cuda_error() */
#define EDM_ERR_DEVICE_TIMEOUT 3 /* a bounded device-side wait expired; see edm_status_read() */
#define EDM_ERR_CAPACITY 4       /* window / flag / heap space too small for this shape */
#define EDM_ERR_NOT_SYMMETRIC 5  /* all-reduce output does not live in the symmetric heap */
#define EDM_ERR_UNSUPPORTED 6

#define EDM_DTYPE_BF16 0 /* bf16 in, fp32 accumulate, bf16 out */
#define EDM_DTYPE_FP32 1 /* fp32 in/out through three tf32 tensor-core passes (hi*hi+lo*hi+hi*lo) */

#define EDM_OP_GEMM 0    /* D = A * B^T */
#define EDM_OP_GEMM_RS 1 /* row-parallel linear + reduce-scatter: rank r gets rows r*M/W.. of sum_r A_r B_r^T */
#define EDM_OP_GEMM_AR 2 /* row-parallel linear + all-reduce: every rank gets sum_r A_r B_r^T */
#define EDM_OP_AG_GEMM 3 /* all-gather of token-sharded X, then D_r = X * W_r^T */

/* How the shards of an all-gather travel.  SM: warps of the GEMM kernel store them into the peers'
 * windows.  COPY_ENGINE: the library's side stream copies them (cudaMemcpy2DAsync) and raises the
 * chunk flags with stream-ordered 32-bit writes; the kernel only waits for the flags.  The copy
 * engines do not compete with the GEMM for the SMs' memory pipelines. */
#define EDM_TRANSPORT_SM 0
#define EDM_TRANSPORT_COPY_ENGINE 1
/* HYBRID: the `ce_peers` farthest peers (rank-d for the largest d; their consumers need the shard
 * last) are served by copy engines, the nearer ones by the kernel. */
#define EDM_TRANSPORT_HYBRID 2
/* COPY_ENGINE_STRIPED: copy engines only, but the chunks of one shard are dealt over the side
 * streams, so all engines serve the same peer at a time (every GPU sends to one peer and receives
 * from one peer at any moment) instead of one peer per stream.  Wants chunks >= side_streams. */
#define EDM_TRANSPORT_COPY_ENGINE_STRIPED 3

#define EDM_MAX_RANKS 8
#define EDM_IPC_HANDLE_BYTES 64

/* Library/ABI version, and the last cudaError_t seen by any entry point on this thread's device
 * (replaces the reference wrapper's throw of std::runtime_error, mma.cu:248-252). */
int edm_version(void);
int edm_last_cuda_error(void);

/* Device-side status words of the current device: out[0] = 0 or a timeout code, out[1..7] =
 * CTA, thread and wait details of the first failure.  Synchronises the device.
 * edm_status_clear() re-arms it.  (The reference exits the process on errors,
 * mma.cu:119-136; here errors are returned, never fatal.) */
int edm_status_read(uint32_t out[16]);
int edm_status_clear(void);
/* Synchronises the device and returns EDM_ERR_DEVICE_TIMEOUT if a bounded wait has expired since
 * the last edm_status_clear(), EDM_OK otherwise.  The launch entry points themselves are
 * asynchronous and cannot report it: after an expiry every later wait of every later launch falls
 * through (so nothing ever hangs), which leaves outputs undefined until edm_status_clear(). */
int edm_status_check(void);

/* Device-side accounting for tracing (the reference times phases with CUDA events only,
 * EDM-IR/ir/trace.py:38-43; this looks inside a launch).  While enabled, every launch adds the
 * nanoseconds each role spent waiting or working, summed over CTAs, to 24 counters:
 * 0 producer waiting for gathered shards, 1 producer waiting for a free stage, 2 MMA waiting for
 * operands, 3 MMA waiting for an accumulator, 4 epilogue waiting for an accumulator, 5 epilogue
 * waiting to reuse staging, 6 epilogue waiting for pushed tiles to land, 7 epilogue total,
 * 8 reducer waiting for partial tiles, 9 reducer total, 10 push warps waiting for local loads,
 * 11 push warps waiting for a buffer, 12 push warps publishing chunks, 13 push warps total,
 * 14 kernel total, 15 number of CTAs counted, 16 epilogue flag fences, 17 epilogue copy issue,
 * 18 epilogue accumulator loads, 19 push-warp flag fences, 20 producer polling chunk flags,
 * 21 producer proxy fences, 22 epilogue tile loop (start to last tile shipped), 23 epilogue waiting
 * for its last copies.
 * edm_profile_read synchronises the device. */
int edm_profile_enable(int on);
int edm_profile_read(uint64_t out[24], int reset);

/* Upper bound for every device-side wait, in milliseconds (default 2000). */
int edm_set_timeout_ms(uint32_t ms);

/* ---- single-GPU GEMM ---------------------------------------------------------------
 * Replaces run_tiled_mma / tiled_mma_bf16_bf16_bf16_fp32 (EDM-IR/ir/c-extension/mma.cu:168-271)
 * for arbitrary M, N, K.  Asynchronous on `stream`.  May be issued under stream capture (captured
 * launches use a schedule without cross-CTA K-splitting, whose flags depend on a host-side launch
 * counter). */
int edm_gemm_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
                  int64_t M, int64_t N, int64_t K, void* stream);

/* fp32 GEMM with fp32-level accuracy on the tensor cores.  `workspace` holds the tf32 high/low
 * splits of A and B and must be at least edm_gemm_fp32_workspace_bytes(M,N,K) bytes. */
size_t edm_gemm_fp32_workspace_bytes(int64_t M, int64_t N, int64_t K);
int edm_gemm_fp32(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
                  int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                  void* stream);

/* fp32 GEMM that allocates nothing and needs no workspace argument.  (No counterpart in the
 * reference.)  It is meant for callers that cannot call cudaMalloc or hand over a scratch
 * buffer at the point where they need the product -- code running inside another framework's
 * allocator-owned region, plugin callbacks with a fixed signature, or start-up paths that run
 * before an allocator exists.  Same arithmetic and accuracy as edm_gemm_fp32; its scratch is a
 * 12 MiB device array built into the library (held by every GPU that loads the library until the
 * process exits), which bounds the problem: 8 * (M*K + N*K) bytes (each term rounded up to 256)
 * must not exceed 8 MiB, otherwise EDM_ERR_CAPACITY is returned and nothing is launched.  The
 * launch uses at most 32 CTAs, so it is slower than edm_gemm_fp32 on large outputs.
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call before any stream capture begins.  All calls share the one array and it
 * keeps whatever the last call left; every call rewrites all of it that it reads, but two calls
 * that overlap on the GPU (different streams, or different threads' streams) race on it. */
int edm_gemm_fp32_static(const void* a, int64_t lda, const void* b, int64_t ldb, void* d, int64_t ldd,
                         int64_t M, int64_t N, int64_t K, void* stream);

/* ---- symmetric memory and peer windows ---------------------------------------------
 * No reference counterpart: the reference only names collectives as op strings
 * (EDM-IR/ir/ops.py:32-35) and records `backend` as free text (EDM-IR/ir/uop.py:49).
 * One context per rank.  It owns a single device allocation, laid out identically on every rank:
 * flag words, a double-buffered window for in-flight tiles / gathered shards, and a bump heap
 * for tensors that peers write directly (all-reduce outputs). */
typedef struct edm_comm edm_comm_t;

int edm_comm_create(int rank, int world, size_t window_bytes, size_t heap_bytes, edm_comm_t** out);
int edm_comm_destroy(edm_comm_t* comm);
/* Exchange: export this rank's allocation as a 64-byte IPC handle; import every peer's. */
int edm_comm_export(edm_comm_t* comm, void* handle64);
int edm_comm_import(edm_comm_t* comm, int peer, const void* handle64);
/* Same-process peers (several contexts on one GPU, or on GPUs with peer access enabled). */
int edm_comm_link_local(edm_comm_t* comm, int peer, edm_comm_t* peer_comm);
/* Bump allocation from the symmetric heap; every rank must make the same sequence of calls. */
int edm_comm_heap_alloc(edm_comm_t* comm, size_t bytes, void** out);
int edm_comm_heap_reset(edm_comm_t* comm);
/* Debugging aid (no reference counterpart): fills this rank's window (both halves: tile slots and
 * gather buffers, not the flag words) with `byte_value`, asynchronously on `stream`.  With 0xFF
 * every bf16 / fp32 element there is a NaN, so a launch that reads a slot or a gathered row before
 * its sender wrote it shows up in the output instead of silently re-using the previous call's
 * data.  Every rank must have finished its previous launch (no copies in flight). */
int edm_comm_poison(edm_comm_t* comm, int byte_value, void* stream);
/* Link probe for calibration: copies `bytes` (a multiple of 32768, at most half the window) from
 * this rank's window into `peer`'s with mode 0 = 16-byte stores from every thread, mode 1 =
 * 8 KiB bulk copies staged through shared memory by all lanes, modes 2 / 3 = the pusher CTAs'
 * bulk-load-then-bulk-store pipeline with 16 / 32 KiB per copy.  The caller times it with CUDA events; the
 * figures feed the selector's transfer term ("calibrated from ... P2P tests",
 * paper/mlsys-2027/model.md:111).  Both ranks of a pair may probe each other at once. */
int edm_comm_p2p_probe(edm_comm_t* comm, int peer, size_t bytes, int mode, void* stream);
/* The order in which one rank's CTAs take the output tiles of a launch (host-side evaluation of
 * the enumeration the kernel uses; no device work).  tile_m is 128, or 256 when a CTA pair shares
 * a tile; tile_n 256 (32 for decode-sized plain GEMMs); band_rows 0 = default; band_cols = column
 * blocks per super-tile of a band (0 = the whole width); units = CTAs (or pairs) of the launch.  Writes *positions = length of the walk and, when `out` is not NULL and
 * holds `capacity` >= *positions entries, four int32 per position: row block, column block (both
 * -1 for a hole of the all-reduce walk), owner rank, index among the owner's tiles.  No
 * reference counterpart (the reference has no multi-tile launch, ir/c-extension/mma.cu:168-176);
 * used by the CPU tests to check that every tile is produced exactly once per rank and that all
 * ranks agree on owners and slots. */
int edm_tile_walk(int op, int rank, int world, int64_t M, int64_t N, int tile_m, int tile_n, int band_rows,
                  int band_cols, int units, int32_t* out, int64_t capacity, int64_t* positions);
/* How a launch of `tiles` output tiles on `units` CTAs (or CTA pairs) with `k_blocks` blocks of 128
 * bytes along K treats an incomplete last wave (host-side evaluation, no device work):
 * out[0] = tiles computed whole, out[1] = tiles of the last wave that are split along K,
 * out[2] = pieces per split tile (1 = nothing is split).  Piece p of a split tile covers K blocks
 * [k_blocks * p / pieces, k_blocks * (p + 1) / pieces); CTAs claim pieces from a device counter as
 * they finish their whole tiles.
 * Applies to EDM_OP_GEMM and EDM_OP_AG_GEMM in bf16 with 256-wide tiles.  No reference
 * counterpart; used by the CPU tests. */
int edm_tail_split(int64_t tiles, int units, int64_t k_blocks, int32_t out[3]);
/* What edm_gemm_bf16 would launch for an [M, N, K] problem on a GPU with `sms` SMs (host-side
 * evaluation of the launch heuristics, no device work): out[0] = CTAs per tile (1, or 2 for CTA
 * pairs on 256-row tiles), out[1] = tile width (256 or 32), out[2] = CTAs launched, out[3] = pieces
 * a tile of an incomplete last wave (or every tile, when there are fewer tiles than CTAs) is cut
 * into along K (1 = none).  No reference counterpart; used by the CPU tests. */
int edm_gemm_plan(int64_t M, int64_t N, int64_t K, int sms, int32_t out[4]);
int edm_comm_rank(const edm_comm_t* comm);
int edm_comm_world(const edm_comm_t* comm);

/* ---- fused tensor-parallel linear ----------------------------------------------------
 * These are the launches a lowering of compute.gemm + comm.reduce_scatter / comm.all_reduce /
 * comm.all_gather node pairs (EDM-IR/ir/ops.py:29,32-34) turns into.  Every rank of the
 * context calls the same entry point with the same shape, in the same order. */
typedef struct {
  int32_t op;    /* EDM_OP_* */
  int32_t dtype; /* EDM_DTYPE_* */
  const void* a; /* GEMM_RS / GEMM_AR: A_r [M, K]; AG_GEMM: X_r [M/world, K] */
  int64_t lda;
  const void* b; /* B_r [N, K] */
  int64_t ldb;
  void* d; /* GEMM_RS: [M/world, N]; GEMM_AR: [M, N] in the symmetric heap; AG_GEMM: [M, N] */
  int64_t ldd;
  int64_t M, N, K; /* per-rank GEMM extents; for AG_GEMM M counts the gathered rows */
  int32_t chunks;  /* AG_GEMM: chunks per shard (>= 1); ignored otherwise */
  int32_t transport; /* AG_GEMM: EDM_TRANSPORT_*; ignored otherwise */
  void* workspace; /* EDM_DTYPE_FP32 only: tf32 split scratch */
  size_t workspace_bytes;
  /* Schedule fields (what the selector chooses besides `chunks` and `transport`); 0 = default. */
  int32_t pusher_ctas;  /* AG_GEMM, kernel-side pushes: this many CTAs (rounded down to whole CTA pairs)
                           take no tiles and only move the shard, with bulk copies staged through
                           their shared memory; 0 = warps inside every GEMM CTA push with 16-byte stores */
  int32_t ce_peers;     /* AG_GEMM, EDM_TRANSPORT_HYBRID: peers served by copy engines (0 .. world-1) */
  int32_t side_streams; /* AG_GEMM, copy engines: streams the copies are spread over (1 .. 4; 0 = 2) */
  int32_t band_rows;    /* tile walk: row blocks per band (0 = default) */
  int32_t band_cols;    /* tile walk: column blocks per super-tile of a band (0 = the whole width) */
  int32_t one_shot;     /* GEMM_AR: 1 = plain GEMM into the window, then a one-shot all-reduce (every rank reads
                           all partials: for decode-sized M; d may be any device memory); 0 = fused kernel */
} edm_tp_call_t;

/* Not capturable: the flags of the exchange carry the context's call counter, which a graph replay
 * would repeat; with world > 1 a launch on a capturing stream returns EDM_ERR_UNSUPPORTED. */
int edm_tp_launch(edm_comm_t* comm, const edm_tp_call_t* call, void* stream);

/* Runs n ranks' calls as ONE cooperative launch on the current device (rank i uses 1/n of the
 * SMs).  This is how the multi-rank protocol is exercised on a single GPU: kernels that wait on
 * one another must not be separate launches on one device. */
int edm_tp_launch_emulated(edm_comm_t* const* comms, const edm_tp_call_t* calls, int n, void* stream);

/* Convenience wrappers over edm_tp_launch for the bf16 layer ops. */
int edm_gemm_rs_bf16(edm_comm_t* comm, const void* a, int64_t lda, const void* b, int64_t ldb,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream);
int edm_gemm_ar_bf16(edm_comm_t* comm, const void* a, int64_t lda, const void* b, int64_t ldb,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, void* stream);
int edm_ag_gemm_bf16(edm_comm_t* comm, const void* x, int64_t ldx, const void* w, int64_t ldw,
                     void* d, int64_t ldd, int64_t M, int64_t N, int64_t K, int32_t chunks,
                     void* stream);

/* ---- expert-parallel mixture-of-experts layer ------------------------------------------
 * No reference counterpart: the reference names the exchange (comm.all_to_all, EDM-IR/ir/ops.py:35)
 * and tags nodes with ep_rank (EDM-IR/ir/uop.py:106); a dispatch/combine study is planned
 * (experiments/deepep-vs-nccl-ep-h100/README.md:19-57).  One call runs, for the `tokens` tokens of
 * this rank: top-2 routing from the router logits, dispatch of every (token, choice) row to the
 * rank that holds its expert (stores into symmetric peer windows plus flag words, like the tile
 * pushes of the fused linears), per-expert down(silu(gate(x)) * up(x)) as two grouped tensor-core
 * GEMMs, return of the rows and the combination weighted by the softmax of the two selected
 * logits.  Expert e lives on rank e / (experts / world); every rank of the context makes the same
 * call.  The context's window must hold edm_moe_window_bytes(); `workspace` (256-byte aligned,
 * edm_moe_workspace_bytes(), owned by the caller) holds the routing results, the row-block tables
 * and the intermediate activations.  Like the fused linears the call cannot be stream-captured. */
typedef struct {
  int32_t tokens, hidden, ffn, experts; /* T per rank, H, F, E in total (E <= 64, E % world == 0) */
  const void* x;       /* [T, H] bf16 */
  int64_t ldx;
  const float* logits; /* [T, E] fp32 router logits (any bias already added) */
  int64_t ld_logits;
  const void* w1;      /* [E/world * 2F, H] bf16: per local expert the gate rows, then the up rows */
  int64_t ldw1;
  const void* w2;      /* [E/world * H, F] bf16 */
  int64_t ldw2;
  void* out;           /* [T, H] bf16 */
  int64_t ldo;
  void* workspace;
  size_t workspace_bytes;
} edm_moe_call_t;
size_t edm_moe_window_bytes(int64_t tokens, int64_t hidden, int64_t experts, int world);
size_t edm_moe_workspace_bytes(int64_t tokens, int64_t hidden, int64_t ffn, int64_t experts, int world);
/* Byte offsets inside the workspace of the routing results of the last call: out[0] selected
 * experts (int32 [T,2]), out[1] their weights (fp32 [T,2]), out[2] the slot of every (token,
 * choice) among this rank's rows for the same expert (int32 [T,2]). */
int edm_moe_routing_offsets(int64_t tokens, int64_t hidden, int64_t ffn, int64_t experts, int world, size_t out[3]);
int edm_moe_forward(edm_comm_t* comm, const edm_moe_call_t* call, void* stream);
/* n ranks of a group on ONE device: every stage is a single launch over all ranks. */
int edm_moe_forward_emulated(edm_comm_t* const* comms, const edm_moe_call_t* calls, int n, void* stream);

/* ---- schedule selector -----------------------------------------------------------------
 * Integer restatement of the reference's cost evaluation: a chunked GEMM->collective pipeline
 * is scored exactly as analyze_critical_path (EDM-IR/ir/analysis.py:36-65) scores the graph
 * EDMBuilder (EDM-IR/ir/builder.py:22-110) builds for it, with the alpha-beta communication
 * term of paper/mlsys-2027/model.md:98 and the split overheads of model.md:161-168.
 * All durations are integers (nanoseconds or any other unit) so the result is bit-exact. */
typedef struct {
  int64_t gemm_total;      /* duration of the unchunked GEMM */
  int64_t comm_bytes;      /* bytes the unchunked collective moves per GPU */
  int64_t alpha;           /* fixed cost per collective launch / chunk */
  int64_t beta_num;        /* transfer cost = ceil(bytes * beta_num / beta_den) */
  int64_t beta_den;
  int64_t split_overhead;  /* added to every GEMM chunk when chunks > 1 */
  int32_t comm_first;      /* 0: GEMM chunk feeds collective chunk (RS/AR); 1: collective feeds GEMM (AG) */
  int32_t reserved;
} edm_cost_params_t;

typedef struct {
  int64_t makespan;        /* critical-path duration of the candidate */
  int64_t exposed_comm;    /* summed duration of comm nodes on the critical path */
  int64_t total_comm;
  int64_t gemm_chunk;      /* duration of one GEMM chunk */
  int64_t comm_chunk;      /* duration of one collective chunk */
} edm_candidate_cost_t;

/* Score one candidate. */
int edm_schedule_cost(const edm_cost_params_t* p, int32_t chunks, edm_candidate_cost_t* out);
/* Score candidates[0..n) and return the index of the smallest makespan (ties: lowest index) in
 * *chosen; costs may be NULL. */
int edm_select_schedule(const edm_cost_params_t* p, const int32_t* candidates, int32_t n,
                        edm_candidate_cost_t* costs, int32_t* chosen);

/* The same evaluation for an arbitrary graph (the candidates of the all-gather and reduce-scatter
 * schedules have one GEMM node per shard or tile round, pushes per peer, a final reduction; they
 * are built with the EDMBuilder API and scored here).  Nodes are 0 .. n_nodes-1 in id order with
 * integer durations, the end timestamps that take part in tie-breaking, and a flag for comm.*
 * nodes; edges are (src, dst) in insertion order.  Returns the critical-path duration, the summed
 * duration of comm nodes on it and, when `path` is not NULL, the node ids of the path
 * (*path_len: capacity in, length out).  A cycle or an edge to an unknown node is EDM_ERR_BAD_ARG.
 * Bit-exact with analyze_critical_path / analyze_exposure (EDM-IR/ir/analysis.py:36-65, :89-123)
 * for integer durations. */
int edm_graph_cost(int32_t n_nodes, const int64_t* dur, const int64_t* end, const uint8_t* is_comm,
                   int32_t n_edges, const int32_t* src, const int32_t* dst, int64_t* makespan,
                   int64_t* exposed_comm, int32_t* path, int32_t* path_len);

#ifdef __cplusplus
}
#endif
#endif /* EDM_B200_H_ */
