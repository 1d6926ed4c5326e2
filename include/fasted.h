/* C ABI of the B200 epsilon self-join library (libfasted.so, also loadable
 * under the reference's file name main.so).
 *
 * Two layers:
 *   1. The four entry points of the reference's shared library, with the same
 *      names, argument meaning and by-value Results struct, so that the
 *      reference's ctypes driver loads this library unchanged.
 *   2. A context API with plain pointers and sizes for callers that own their
 *      buffers (tests, benchmarks, multi-GPU band sharding).
 *
 * All functions are host functions; none is thread-safe with respect to the
 * same context.  Every wait inside a kernel gives up after 2 s of wall time
 * (the GPU's global timer, not SM cycles) and the call then fails with
 * FASTED_EKERNEL: on a GPU that is time-sliced with other processes a long
 * preemption counts toward that limit, so give the library a GPU of its own.  Functions of layer 2 return 0 on success and a negative
 * FASTED_E* code on failure; fasted_last_error() gives the message.
 * There is no CPU fallback: without a usable sm_100 device every compute call
 * fails.
 */
#ifndef FASTED_H_
#define FASTED_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------
 * Layer 1: drop-in for the reference's shared-library interface
 * ---------------------------------------------------------------------- */

/* Replaces Mma::mmaShape, source/ptxMma.cuh:27-31. */
typedef struct mmaShape {
    int m, n, k;
} mmaShape;

/* Replaces SimSearch::Results, source/findPairs.cuh:37-46 (56 bytes, returned
 * by value; mirrored by results/scripts/experiment/find_pairs.py:24-50).
 * totalTime: wall seconds from entry to after sort + device-to-host copy.
 * TFLOPS: 2*N*N*D / kernel seconds / 1e12 over the un-padded N and D, kernel
 * seconds = row-norm kernel + join kernel (source/findPairs.cuh:728-748).
 * pairsFound counts every hit, self pairs and both orientations included;
 * pairsStored counts those that fitted in the pair buffer. */
typedef struct Results {
    double totalTime;
    double TFLOPS;
    unsigned long long pairsFound;
    unsigned long long pairsStored;
    mmaShape inputProblemShape;
    mmaShape paddedProblemShape;
} Results;

/* Replaces runFromExponentialDataset, source/main.cu:66-67 (declaration) and
 * :251-261 (definition).  Generates the seeded synthetic dataset
 * (source/DataLoader/ExponentialPointGenerator.hpp), uploads it and joins.
 * maxValue is the rejection upper bound of the generator. */
Results runFromExponentialDataset(int size, int dimensionality, double lambda, double maxValue, double epsilon,
                                  bool savePairs);

/* Replaces runFromFile, source/main.cu:53 and :263-273.  CSV: one point per
 * line, comma separated, no header; the first row fixes the dimension. */
Results runFromFile(const char* filename, double epsilon, bool savePairs);

/* Replaces reRun, source/main.cu:43 and :275-278: joins the resident dataset
 * again with another epsilon.  Calling it before a runFrom* call is an error
 * (the reference leaves that case undefined). */
Results reRun(double epsilon, bool savePairs);

/* Replaces releaseResources, source/main.cu:73 and :280 (whose body recurses
 * forever in the reference; the intent, SimSearch::releaseGlobalMemory at
 * source/findPairs.cuh:766-776, is what is implemented). */
void releaseResources(void);

/* Errors in layer 1 follow the reference (source/main.cu:244-247,
 * source/utils.cuh:22-29): message on stdout, then exit(EXIT_FAILURE).
 *
 * Environment switches of layer 1 (all optional):
 *   FASTED_OUTPUT_DIR   directory for "<dataset>_<eps>.pairs" when savePairs
 *                       is true (default /scratch/bc2497/pairsData/, the path
 *                       hard-wired at source/main.cu:214-215)
 *   FASTED_DEVICE       CUDA device ordinal (default 0, source/findPairs.cuh:622)
 *   FASTED_NUM_GPUS     number of GPUs this one process drives (default 1; "all" = every visible
 *                       device): the dataset is uploaded once and replicated by one NCCL broadcast
 *                       (peer copies where NCCL is absent), GPU g joins the g-th band of query rows
 *                       against all candidates, the sorted band lists are concatenated on the host
 *                       in band order
 *   FASTED_WRITE_DIST   "1": third text column sqrt(d2) in the .pairs file
 *   FASTED_SYMMETRIC    "1": each unordered pair is computed once and both orientations are emitted
 *                       (identical output in about half the time; "Estimated TFLOPS" still divides
 *                       2*N*N*D by the time, and a "Schedule:" line on stdout says which one ran).
 *                       Default: all N x N entries are computed, like the reference.
 *   FASTED_EXACT_NORMS  "1": correctly rounded row norms (option "exact_norms" of the context API)
 */

/* ------------------------------------------------------------------------
 * Layer 2: context API
 * ---------------------------------------------------------------------- */

typedef struct fasted_ctx fasted_ctx;

enum {
    FASTED_OK = 0,
    FASTED_EINVAL = -1,   /* bad argument */
    FASTED_ECUDA = -2,    /* CUDA runtime / driver error */
    FASTED_ENODEV = -3,   /* no sm_100 device */
    FASTED_ESTATE = -4,   /* call out of order (e.g. join before points) */
    FASTED_EKERNEL = -5,  /* a device-side wait ran out; status bits in the message */
    FASTED_EIO = -6       /* file error */
};

enum {
    FASTED_JOIN_DIST2 = 1,       /* also record the FP32 squared distance of every stored pair */
    FASTED_JOIN_NO_SORT = 2,     /* leave stored pairs in device order (count-only / timing runs) */
    FASTED_JOIN_KEEP_NORMS = 4,  /* reuse row norms computed by an earlier call on the same points */
    FASTED_JOIN_RAW_DOT = 16,    /* diagnostic, with FASTED_JOIN_DIST2: the distance array receives the raw FP32
                                    Gram entry a_ij of every stored pair instead of d2 (to study the tensor
                                    core's accumulate) */
    FASTED_JOIN_SYMMETRIC = 8    /* full self-join only: compute each unordered pair once (d2(i,j) == d2(j,i))
                                    and emit both orientations; same output, about half the tensor work */
};

typedef struct fasted_join_stats {
    unsigned long long pairs_found;
    unsigned long long pairs_stored;
    double norms_ms;   /* row-norm kernel, device time (0 where a small join overlapped it: join_ms then covers both) */
    double join_ms;    /* join kernel, device time */
    double kernel_ms;  /* start of norms to end of join (the reference's TFLOPS interval) */
    double sort_ms;    /* sort + unpack, device time (fasted_join_stream: the sum over the chunks) */
    unsigned long long status;  /* device status bits, 0 = clean */
    int tiles_m, tiles_n;
    int grid;
    unsigned long long cta0_cycles;  /* SM cycles CTA 0 of the join kernel ran (0 for the CTA-pair kernel) */
    unsigned long long cta0_tiles;   /* tiles CTA 0 computed */
    unsigned long long cta0_setup_cycles;    /* SM cycles CTA 0 spent before its first tile (barriers, TMEM allocation) */
    unsigned long long cta0_release_cycles;  /* SM cycles CTA 0 spent releasing its TMEM at the end */
    unsigned long long cta0_feed_wait_cycles;  /* SM cycles CTA 0's MMA thread waited for operand stages (TMA) */
    unsigned long long cta0_acc_wait_cycles;   /* ... and for a free accumulator (the epilogue two tiles back) */
    int chunks;      /* join launches of this call (1 except for fasted_join_stream / fasted_join_stream_shared, where
                        join_ms is the device time of those launches without the sorts that ran between them) */
    double tail_ms;  /* fasted_join_stream: device time of the last chunk's sort plus whatever of its copy to the
                        host was left after the last join launch (what the egress pipeline could not hide) */
} fasted_join_stats;

const char* fasted_last_error(void);

/* Creates a context on CUDA device `device` (must be compute capability 10.x). */
int fasted_create(int device, fasted_ctx** out);
void fasted_destroy(fasted_ctx* ctx);

/* Uses `stream` (a cudaStream_t) for all work of this context; default is a
 * stream the context creates. */
int fasted_set_stream(fasted_ctx* ctx, void* stream);

/* Dataset, replaces TransferPointsToGMem / allocateTransferPoints,
 * source/findPairs.cuh:560-590 (one device copy instead of two: query and
 * candidate sets are the same matrix).
 * host: n rows of binary16 values, row stride ld_host elements (>= d).
 * The device copy has row stride = d rounded up to a multiple of 64, zero
 * padded (source/main.cu:207, source/DataLoader/PointListBuilder.hpp:34-39). */
int fasted_set_points_host_f16(fasted_ctx* ctx, const uint16_t* host, int64_t n, int64_t d, int64_t ld_host);

/* Borrow a device matrix (e.g. one received by an NCCL broadcast).  dev must
 * be 16-byte aligned and ld a multiple of 8 elements; columns [d, ld) must be
 * zero if ld > d.  The caller keeps ownership and must keep it alive. */
int fasted_set_points_device_f16(fasted_ctx* ctx, const void* dev, int64_t n, int64_t d, int64_t ld);

/* Replicate the resident dataset of `src` (another GPU of the same process) into `dst` with one
 * device-to-device copy over NVLink / PCIe; dst owns its copy.  For one process driving several
 * GPUs (layer 1 with FASTED_NUM_GPUS); one process per GPU uses an NCCL broadcast instead. */
int fasted_copy_points_from(fasted_ctx* dst, fasted_ctx* src);

/* Replicate the resident dataset of ctxs[0] into ctxs[1 .. count) -- contexts of this process on
 * `count` distinct GPUs -- with ONE NCCL broadcast over NVLink (communicators from ncclCommInitAll,
 * kept for the life of the process).  The reference is single-GPU (cudaSetDevice(0),
 * source/findPairs.cuh:622) and has no counterpart; one process per GPU uses the broadcast of its
 * own process group instead (fasted_b200/dist.py).  NCCL is bound at run time: without libnccl.so.2
 * the call fails with FASTED_ENODEV and fasted_copy_points_from remains.  *ms_out (optional): wall
 * time of the collective. */
int fasted_broadcast_points(fasted_ctx* const* ctxs, int count, double* ms_out);

/* Allocate an n x d dataset on the device and fill it with the counter-based
 * Exponential(lambda) generator (values rejected to [0, max_value], rounded
 * double -> float -> half).  For benchmark shapes too large for the reference's
 * sequential host generator. */
int fasted_generate_exponential(fasted_ctx* ctx, int64_t n, int64_t d, double lambda, double max_value,
                                uint64_t seed);

/* Fill a caller-owned device matrix (n rows, row stride ld, ld a multiple of 8,
 * 16-byte aligned) with the same generator; columns [d, ld) are zeroed.  Does
 * not change the resident dataset. */
int fasted_fill_exponential_device(fasted_ctx* ctx, void* dev, int64_t n, int64_t d, int64_t ld, double lambda,
                                   double max_value, uint64_t seed);

/* Device pointer / shape of the resident dataset. */
int fasted_points_info(fasted_ctx* ctx, void** dev, int64_t* n, int64_t* d, int64_t* ld);
/* Copy the resident dataset to the host (row stride ld_host >= d). */
int fasted_get_points_host_f16(fasted_ctx* ctx, uint16_t* host, int64_t ld_host);

/* Copy selected rows of the resident dataset to the host (row i of the output = row rows[i]). */
int fasted_get_rows_host_f16(fasted_ctx* ctx, const int64_t* rows, int64_t count, uint16_t* host, int64_t ld_host);

/* Row norms, replaces SumSqd::ComputeSquaredSums, source/sumSquared.cuh:84-118.
 * Result stays on the device; ms (optional) receives the kernel time. */
int fasted_row_norms(fasted_ctx* ctx, double* ms);
int fasted_get_norms(fasted_ctx* ctx, float* host_out);

/* The join, replaces SimSearch::FindPairs, source/findPairs.cuh:615-764, for
 * query rows [q_begin, q_end) against all n candidates (q_end = -1 means n).
 * capacity = pair-buffer size in pairs (0: the reference's n*256 rule capped by
 * free device memory, source/findPairs.cuh:642-647, source/pair.cuh:69-91).
 * Results stay on the device, sorted row-major unless FASTED_JOIN_NO_SORT. */
int fasted_join(fasted_ctx* ctx, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                fasted_join_stats* stats);

/* The join with pipelined egress: sort + device-to-host copy overlap the join itself.  Replaces the
 * reference's serial tail Pairs::sort -> Pairs::getPairs after the kernel (source/pair.cuh:139-158,
 * source/findPairs.cuh:699-716).  The query range is cut into chunks of whole raster bands (one join
 * launch each, all enqueued at once); as soon as a chunk's launch retires its records are sorted,
 * unpacked and copied to the host on separate streams while the GPU joins the next chunks.  Chunks are
 * ascending ranges of query rows, so the chunks' lists laid end to end are the global row-major order
 * of source/pair.cuh:39-45: the output is identical to fasted_join + fasted_get_pairs.
 *
 * pairs_host (optional): room for host_capacity (query, candidate) int32 records; record i of the
 * whole list lands at pairs_host[2*i], records beyond host_capacity are not copied.  Pinned (or
 * registered) memory is written by DMA while the join runs; pageable memory goes through the
 * context's pinned staging buffers.  dist2_host (optional, needs FASTED_JOIN_DIST2): the distances.
 * on_chunk (optional): called on the calling thread for consecutive runs of records, in order, once a
 * run is on the host: pairs / dist2 point at the run (inside pairs_host / dist2_host when those are
 * given, else into a staging buffer that is valid during the call only), first = index of the run's
 * first record in the whole list.  A non-zero return value stops the delivery (the call then fails
 * with FASTED_EINVAL after the GPU work has drained).
 * flags: FASTED_JOIN_DIST2, FASTED_JOIN_KEEP_NORMS.  Afterwards fasted_get_pairs works as after
 * fasted_join.  Option "stream_chunk_bands" (fasted_set_option) fixes the raster bands per chunk. */
typedef int (*fasted_chunk_fn)(void* user, const int32_t* pairs, const float* dist2, uint64_t first, uint64_t count);
int fasted_join_stream(fasted_ctx* ctx, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                       int32_t* pairs_host, float* dist2_host, uint64_t host_capacity, fasted_chunk_fn on_chunk,
                       void* user, fasted_join_stats* stats);

/* The streamed join over the GPUs of one node, one process (or context) per GPU, all holding the same
 * dataset: the ranks do not own fixed bands of query rows but TAKE chunks of whole raster bands from a
 * common counter, each whenever its join stream has room for another launch.  A GPU that runs faster
 * (every GPU sits under its own power cap) takes more chunks, so all ranks finish within one small chunk
 * of each other; and because chunk k's place in the global list is the sum of the record counts of the
 * chunks before it -- published by their ranks at about the time chunk k retires -- every rank copies
 * its sorted chunks straight to their FINAL position in one host buffer that all ranks share, while
 * the join is still running.  The result in that buffer is the reference's single row-major list
 * (source/pair.cuh:39-45); the reference itself is single-GPU (source/findPairs.cuh:622).
 *
 * The table lives in memory that every rank maps (e.g. a shared file mapping) and is the only thing
 * the ranks exchange during the join: no collective.  One rank sizes it with
 * fasted_shared_chunks_bytes(max_chunks) -- q rows / 128 + 1, plus one per band for a plan by bands (below), is
 * always enough for max_chunks -- and fills
 * it with fasted_shared_chunks_init (plan from that rank's context: identical on all ranks, which hold
 * the same dataset and options) BEFORE the others are let in (a barrier); then every rank calls
 * fasted_join_stream_shared with its own context and the SAME host buffer (pairs_host = the buffer's
 * first record in this process's mapping; page-locked memory is written by DMA).  flags:
 * FASTED_JOIN_KEEP_NORMS, FASTED_JOIN_NO_SORT (count only: no sort, no copy -- a timing or counting
 * run with the same load balance).  A rank that fails marks the table; the others stop waiting and
 * fail with FASTED_ESTATE.  After a barrier, fasted_shared_chunks_totals gives the job's totals.
 * stats: this rank's share (its launches, its records).
 * The lower-level calls (init_plan / take / publish / offset / fail) are the table's primitives, for
 * schedulers of the caller's own and for tests; none of them touches a GPU. */
size_t fasted_shared_chunks_bytes(uint64_t max_chunks);
int fasted_shared_chunks_init(fasted_ctx* ctx, void* mem, size_t bytes, double eps, int64_t q_begin, int64_t q_end,
                              int ranks, uint64_t* chunks_out);
int fasted_join_stream_shared(fasted_ctx* ctx, double eps, uint64_t capacity, unsigned flags, void* shared_mem,
                              int32_t* pairs_host, uint64_t host_capacity, fasted_join_stats* stats);
int fasted_shared_chunks_totals(const void* mem, unsigned long long* found_total, unsigned long long* stored_total,
                                unsigned long long* failed);
/* group_rows = 0: chunk k is rows [q_begin + k * chunk_rows, ...).  group_rows > 0 (needs q_begin = 0): the rows
 * are cut into groups of group_rows rows, every group into chunks from its own first row, and the first lead_chunks
 * chunks of every group are not handed out by take (see fasted_join_stream_arriving). */
int fasted_shared_chunks_init_plan(void* mem, size_t bytes, int64_t q_begin, int64_t q_end, int64_t chunk_rows,
                                   int64_t group_rows, int lead_chunks, uint64_t* chunks_out);
int fasted_shared_chunks_range(const void* mem, uint64_t chunk, int64_t* begin, int64_t* end); /* rows of a chunk */
int64_t fasted_shared_chunks_take(void* mem);                /* next chunk nobody has taken, -1 when none is left */
int fasted_shared_chunks_publish(void* mem, uint64_t chunk, uint64_t stored, uint64_t found);
int fasted_shared_chunks_offset(void* mem, uint64_t chunk, double timeout_ms, uint64_t* offset_out);
void fasted_shared_chunks_fail(void* mem);

/* The same join started while the dataset is still ARRIVING on the GPUs.  The loader this is made for: G ranks,
 * rank g holds rows [g * B, (g + 1) * B) on its host (B = group_rows), uploads them in P pieces and all-gathers
 * every piece as soon as it has landed, so piece p -- rows [g * B + p * B / P, g * B + (p + 1) * B / P) of EVERY
 * band g -- is complete on every GPU at about (p + 1) / P of the load.  Without this call the join's first launch
 * waits for the whole load.  With it, every rank first joins a few chunks of its OWN band (the "lead": rows of its
 * own first piece, resident from the start) against piece 0, then against piece 1, ... each launch behind the
 * event that says the piece is complete (a launch takes candidate rows of one piece only; row norms are computed
 * piece by piece in front of it); when the last piece is in, the remaining chunks are dealt out as in
 * fasted_join_stream_shared.  The result is the same list in the same shared buffer.
 *   pieces, groups, group_rows: P, G, B; B a multiple of 256 * P, G * B >= n (rows beyond n do not exist).
 *   own_begin: first row of the calling rank's band (g * B); every band needs exactly one rank that calls.
 *   lead_rows: for fasted_shared_chunks_init_arriving only: rows of the lead (rounded down to whole chunks, at
 *              most one piece); 0 = the library's choice.
 *   events:    P cudaEvent_t handles; events[p] completes when piece p of every band is resident on THIS GPU.
 *              The join stream waits for them in order (cudaStreamWaitEvent); NULL, or a NULL entry = resident
 *              already.  They must have been recorded before the call.
 * fasted_shared_chunks_init_arriving plans the table for this (one rank, before the others are let in). */
typedef struct fasted_arrival {
    int pieces, groups;
    int64_t group_rows, own_begin, lead_rows;
    void* const* events;
} fasted_arrival;
int fasted_shared_chunks_init_arriving(fasted_ctx* ctx, void* mem, size_t bytes, double eps, int ranks,
                                       const fasted_arrival* arrival, uint64_t* chunks_out);
int fasted_join_stream_arriving(fasted_ctx* ctx, double eps, uint64_t capacity, unsigned flags, void* shared_mem,
                                const fasted_arrival* arrival, int32_t* pairs_host, uint64_t host_capacity,
                                fasted_join_stats* stats);

/* One shard of the symmetric schedule for a self-join split over shard_world GPUs that all hold the
 * dataset: shard r computes the raster bands r, 2G-1-r, 2G+r, ... (G = shard_world) of the upper
 * triangle and emits both orientations of every hit, so the union of the shards' outputs is the
 * full join's output, each pair exactly once.  A shard's output is sorted but not a contiguous
 * query range (the mirrored records belong to other rows): see fasted_b200/dist.py for the exchange
 * that gives every rank a contiguous range. */
int fasted_join_symmetric_shard(fasted_ctx* ctx, double eps, int shard_rank, int shard_world, uint64_t capacity,
                                unsigned flags, fasted_join_stats* stats);

/* Epsilon whose mean neighbour count per point (self pair excluded) is about `target`, estimated
 * on `sample_rows` query rows (up to 8 bands spread over the dataset; 0 = 4096) against all
 * candidates by bisection with count-only band joins; stops within rel_tol (0 = 1 %) of the target.
 * Replaces the search the reference's driver runs with full reRun calls
 * (results/scripts/experiment/experiments.py:153-281: doubling, then bisection on selectivity):
 * a probe costs sample_rows/n of a full join.  *achieved_out (optional) is the sample's mean. */
int fasted_estimate_epsilon(fasted_ctx* ctx, double target_mean_neighbours, int64_t sample_rows, double rel_tol,
                            double* eps_out, double* achieved_out);

/* Copy stored pairs [first, first + count) of the last join to the host as
 * (query, candidate) int32 records, replaces Pairs::getPairs,
 * source/pair.cuh:139-146.  dist2_out may be null. */
int fasted_get_pairs(fasted_ctx* ctx, uint64_t first, uint64_t count, int32_t* pairs_out, float* dist2_out);

/* Device pointers of the last join's results (int2 records, float distances). */
int fasted_pairs_device(fasted_ctx* ctx, void** pairs_dev, void** dist2_dev);

/* FP64 brute-force check on the device (accuracy reporting): for each of the
 * n_samples query rows counts the candidates with FP64 d2 <= eps*eps. */
int fasted_brute_force_f64(fasted_ctx* ctx, const int32_t* sample_rows, int n_samples, double eps,
                           unsigned long long* counts_out);

/* Join of all n points with no memory allocation of any kind.  (This entry point has no
 * counterpart in the reference.)
 *
 * Who needs it: host programs in which this library is a guest.  A database or a tensor
 * framework usually claims nearly all of the GPU's memory for its own pool at start-up and hands
 * out pieces of it; inside such a host a cudaMalloc from a plug-in fails or steals from the pool,
 * and cudaMalloc/cudaFree also stall every stream of the device, which a caller on a latency
 * budget cannot accept.  Such a caller passes buffers carved from its own pool and calls this.
 *
 * The caller passes the input (points_dev: n rows of binary16 on the device, row stride ld, ld a
 * multiple of 8, 16-byte aligned, columns [d, ld) zero) and the output (keys_out_dev: room for
 * `capacity` 64-bit records on the device).  Each record is (query << 32) | candidate, in the
 * order the GPU found them (not sorted: sorting needs scratch proportional to the output).
 * *pairs_found counts all hits, *pairs_stored those written (at most capacity), as in fasted_join.
 *
 * What the join needs besides that - the row norms and its counters - lives in an area built into
 * the library: 4 MiB + 256 bytes of device memory, one instance per process and GPU, held from the
 * moment the CUDA runtime loads this library's module on that GPU until the process exits.  It is
 * sized for n <= 1,048,576 points; a larger n is rejected with FASTED_EINVAL (use fasted_join).
 * Every call on a GPU shares the area: it still holds the previous call's contents on entry (the
 * function re-zeroes its counters and recomputes the norms every time), and two calls of one
 * process whose GPU work overlaps - different streams or host threads - race on it.  Run them one
 * after the other.  (Another process has its own CUDA context and therefore its own instance.)
 *
 * When the memory is taken: with CUDA's default lazy module loading, the kernels and the built-in
 * area are placed on a GPU by the first call of ANY function of this library that touches that GPU.
 * If that first call is this one, it is the one call that does take device memory (the area plus
 * the kernel images, a few MiB) and it fails with FASTED_ECUDA if the host has left none.  A guest
 * should therefore make one warm-up call (n = 1, capacity = 0 is enough) before its host claims the
 * pool, or run with CUDA_MODULE_LOADING=EAGER so that loading the library does it.  Every later
 * call leaves the amount of free device memory exactly as it found it.
 *
 * Works on the current CUDA device and on `stream` (a cudaStream_t, may be 0); it returns after
 * the stream has drained.  Each call looks up the device address of the built-in area and sets
 * the kernels' shared-memory limits (table look-ups, nothing is cached between calls); make the
 * first call on a device outside any stream capture.  No cudaMalloc, cudaFree, event, stream or
 * library allocation is made. */
int fasted_join_static_scratch(const void* points_dev, int64_t n, int64_t d, int64_t ld, double eps,
                               unsigned long long* keys_out_dev, uint64_t capacity, void* stream,
                               unsigned long long* pairs_found, unsigned long long* pairs_stored);

/* Same check, also returning the neighbours themselves: keys_out receives up to `capacity`
 * records (query << 32) | candidate in no particular order, *n_keys_out the number found. */
int fasted_brute_force_f64_pairs(fasted_ctx* ctx, const int32_t* sample_rows, int n_samples, double eps,
                                 unsigned long long* counts_out, unsigned long long* keys_out, uint64_t capacity,
                                 unsigned long long* n_keys_out);

/* Host-side dataset builders (no GPU involved), the loaders behind layer 1.
 * Exponential: replaces SimSearch::ExponentialPointGenerator,
 * source/DataLoader/ExponentialPointGenerator.hpp:22-52, plus the
 * double -> float -> half rounding of source/DataLoader/PointListBuilder.hpp:57-66.
 * CSV: replaces SimSearch::FilePointGenerator, source/DataLoader/FilePointGenerator.hpp:20-56,
 * with the shape rule of PointListBuilder.hpp:154-163 (ragged rows are FASTED_EINVAL,
 * unreadable files FASTED_EIO).  out rows have stride ld_out >= d; columns
 * [d, ld_out) are zeroed. */
int fasted_dataset_exponential_f16(int64_t n, int64_t d, double lambda, double max_value, uint16_t* out,
                                   int64_t ld_out);
int fasted_dataset_csv_shape(const char* path, int64_t* n, int64_t* d);
int fasted_dataset_csv_f16(const char* path, uint16_t* out, int64_t n, int64_t d, int64_t ld_out);

/* The tile schedule of the join kernel, evaluated on the host (no GPU): the (tile row, tile
 * column) sequence that CTA `cta` of `grid` walks for query rows [q_begin, q_end) of n points.
 * tile_m is 128 (single-CTA kernel) or 256 (CTA pairs; cta then counts pairs); tile columns are 256
 * candidates wide.  Replaces OnDemandRasterizer::nextChunk, source/rasterizer/onDemandRasterizer.cuh:78-108.
 * tiles_out (optional) receives up to max_tiles (tm, tn) int32 pairs, *count_out the full count. */
int fasted_tile_schedule(int64_t n, int64_t q_begin, int64_t q_end, int tile_m, int band_tiles, int symmetric,
                         int shard_rank, int shard_world, int grid, int cta, int32_t* tiles_out, int64_t max_tiles,
                         int64_t* count_out);

/* The same for the query-stationary kernel that joins short rows (d <= 512): bands of rows_per_band
 * 128-row tile rows (at most `grid`); in a band of r rows CTA b takes row b % r and the tile columns
 * b / r, b / r + grid / r, ...  (tm, tn) pairs as above. */
int fasted_tile_schedule_stationary(int64_t n, int64_t q_begin, int64_t q_end, int rows_per_band, int symmetric, int grid,
                                    int cta, int32_t* tiles_out, int64_t max_tiles, int64_t* count_out);

/* Self-test of the failure path every device-side wait of this library has: a one-block kernel
 * waits, with a limit of limit_ms (at most 1000), on a barrier that nothing completes.  The wait
 * must give up, the kernel must return normally, *status_out must carry the wait's status bits
 * (non-zero), and the context must stay usable.  Nothing faults, traps or hangs.  (The reference
 * has no counterpart: its CUDA errors exit the process, source/utils.cuh:22-29.) */
int fasted_selftest_wait_timeout(fasted_ctx* ctx, double limit_ms, unsigned long long* status_out,
                                 double* waited_ms_out);

/* Tuning knobs: "band_tiles" (128-row tile rows per raster band, 0 = automatic: 16, fewer for rows wider than 8 KB), "grid" (CTAs,
 * 0 = one per SM), "cta_pair" (1 = the CTA-pair kernel: 256 x 256 tiles computed by two CTAs with
 * tcgen05 cta_group::2; same results bit for bit; default 0 because it sustains less under the
 * power cap on B200), "exact_norms" (1 = correctly rounded row norms (FP64 sum, one rounding)
 * instead of the reference's round-toward-zero chain: NOT the reference's numerics, but closer to an
 * FP64 join on this hardware, whose tensor-core accumulate does not truncate; default 0),
 * "query_stationary" (-1 = automatic: for rows of at most 512 values a CTA keeps its 128 query rows in
 * shared memory and streams candidate rows only; 0 = never, 1 = the same rule as automatic; same results
 * bit for bit), "stream_chunk_bands" (raster bands per chunk of fasted_join_stream, 0 = automatic), "stream_key32" (1 = default:
 * 32-bit chunk-relative records in fasted_join_stream where they fit and the output is dense), "stream_sort_batch" (16 =
 * default: where the output is sparse, one sort takes the records of up to this many consecutive chunks; 1 = one sort
 * per chunk), "dependent_launch" (1 = default: a small join is
 * launched as a programmatic dependent of the row-norm kernel and overlaps it). */
int fasted_set_option(fasted_ctx* ctx, const char* name, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* FASTED_H_ */
