// Device kernels of the epsilon self-join for sm_100a.
//
//   row_norms_kernel   FP16 rows -> FP32 squared norms (HBM-bound, TMA-staged)
//   join_kernel        persistent TMA + tcgen05.mma pipeline with the fused
//                      distance / threshold / pair-compaction epilogue
//   join_pair_kernel   the same on CTA pairs (tcgen05 cta_group::2), optional
//   unpack_pairs_kernel, gen_exponential_kernel, brute_f64_kernel  (helpers)
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace fasted {

// ---------------------------------------------------------------------------
// Shared constants
// ---------------------------------------------------------------------------

constexpr int kTileK = 64;     // halfs per pipeline stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;     // K of one tcgen05.mma kind::f16
constexpr int kTileM = 128;    // query rows per CTA tile = TMEM lanes
constexpr int kTileN = 256;    // candidate rows per tile = TMEM columns per accumulator
constexpr int kStages = 4;     // TMA -> MMA ring depth
constexpr int kTmemCols = 512; // two accumulator buffers of kTileN columns

constexpr int kEpiWarps = 8;       // two per TMEM lane quarter, each taking half of the tile's columns
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kJoinThreads = 64 + kEpiThreads;  // warp 0: TMA, warp 1: MMA issue + TMEM, warps 2..9: epilogue
constexpr int kEpiCols = kTileN / (kEpiWarps / 4);  // accumulator columns handled by one epilogue warp

constexpr uint32_t kStageBytesA = kTileM * kTileK * 2;  // 16 KiB
constexpr uint32_t kStageBytesB = kTileN * kTileK * 2;  // 32 KiB
constexpr uint32_t kStageBytes = kStageBytesA + kStageBytesB;

// Wait limit of every device-side wait.  A legitimate wait lasts at most one
// tile main loop (tens of microseconds); after the limit the kernel records
// an error and returns.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Status word bits (counters[2]).
constexpr unsigned long long kErrProducerWait = 1ull;
constexpr unsigned long long kErrMmaWait = 2ull;
constexpr unsigned long long kErrEpilogueWait = 4ull;
constexpr unsigned long long kErrNormWait = 8ull;

struct JoinParams {
    const float* norms;            // [n] row norms
    int norms_vec4;                // 1: norms is 16-byte aligned (vector loads allowed)
    unsigned long long* counters;  // [0] pairs found, [1] unused (stored = min(found, capacity)), [2] status bits,
                                   // CTA 0 of the single-CTA kernels: [4] SM cycles on its tiles, [5] set-up,
                                   // [6] TMEM release, [7] cycles its MMA thread waited for operands, [8] ... for a
                                   // free accumulator
    unsigned long long* keys;      // pair buffer: (query << 32) | candidate
    float* dist2;                  // optional squared distances, parallel to keys (may be null)
    unsigned long long capacity;   // pair buffer capacity
    float eps2;                    // threshold on the squared distance (inclusive)
    int n;                         // real number of points (candidates are rows [0, n))
    int q_begin, q_end;            // query rows handled by this launch
    int k_steps;                   // ceil(d / kTileK)
    int tiles_m, tiles_n;          // tile grid of this launch
    int band_tiles;                // tile rows per raster band
    long long total_tiles;         // upper bound of the tiles walked (grid sizing only)
    int tile_m;                    // query rows per tile (kTileM, or 2 * kTileM for CTA pairs)
    int raw_dot;                   // 1 (diagnostic): record the raw accumulator a_ij instead of d2
    int symmetric;                 // 1: walk only tiles that touch j >= i and emit (i,j) and (j,i)
    int shard_rank, shard_world;   // symmetric mode over several GPUs: this launch takes the raster bands
                                   // r, 2G-1-r, 2G+r, 4G-1-r, ... (a snake over the G shards, which evens out
                                   // the shrinking band lengths of the triangle); 0, 1 = everything
    int astat_rows;                // query-stationary kernel: tile rows per band (at most the grid size)
    int astat_stages;              // query-stationary kernel: depth of its candidate ring
    int key_shift, key_qbase;      // record = ((query - key_qbase) << key_shift) | candidate.  32 and 0 give the
                                   // plain (query << 32) | candidate; a launch over one chunk of query rows can
                                   // pack tighter, so that the chunk's sort has fewer significant bits to look at
    int cand_t, cand_group_rows, cand_base;  // candidate subset of this launch.  cand_t = 0: all rows, tile column tn
                                   // covers candidates [tn * 256, +256).  Else the launch joins against G groups of
                                   // cand_t tile columns each: tile column tn covers the 256 rows that start at
                                   // (tn / cand_t) * cand_group_rows + cand_base + (tn % cand_t) * 256 (a piece of the
                                   // matrix that has arrived from every rank while the rest is still on its way)
    int key32;                     // 1: the packed record fits 32 bits and `keys` is an array of uint32_t (half the
                                   // bytes to write, to sort and to read back)
};

// First candidate row of tile column tn (see JoinParams::cand_t).
__device__ __forceinline__ int cand_row0(const JoinParams& p, int tn) {
    if (p.cand_t == 0) return tn * kTileN;
    const int g = tn / p.cand_t;
    return g * p.cand_group_rows + p.cand_base + (tn - g * p.cand_t) * kTileN;
}

__device__ __forceinline__ unsigned long long pack_record(const JoinParams& p, unsigned long long q,
                                                          unsigned long long c) {
    return ((q - static_cast<unsigned long long>(p.key_qbase)) << p.key_shift) | c;
}

__device__ __forceinline__ void store_record(const JoinParams& p, unsigned long long slot, unsigned long long q,
                                             unsigned long long c) {
    const unsigned long long rec = pack_record(p, q, c);
    if (p.key32)
        reinterpret_cast<uint32_t*>(p.keys)[slot] = static_cast<uint32_t>(rec);
    else
        p.keys[slot] = rec;
}

// Persistent static schedule: CTA (or CTA pair) b handles tiles b, b + grid, b + 2*grid, ... of a
// linear order that walks bands of `band_tiles` tile rows; inside a band the tile row is the fastest
// index, so the CTAs that run together cover a band_tiles x (grid / band_tiles) block of the tile
// grid and the query rows of a band stay L2-resident while the band sweeps over the candidates.
// (Replaces the reference's atomic work queue and its 8 x 8 super-tiles,
// source/rasterizer/onDemandRasterizer.cuh:78-108.)
//
// Symmetric mode: d2(i,j) == d2(j,i), so only elements with j >= i are computed.  A band then
// starts at the first candidate tile that reaches its diagonal, and tiles that lie entirely below
// the diagonal are skipped.  All roles of a CTA walk the same sequence.
struct TileIter {
    long long rem;        // index of the current tile inside the current band
    long long band_size;  // tiles in the current band
    long long step;
    int band, nbands;     // index into this launch's bands, and how many it has
    int pband;            // the current band in the global numbering
    int rows;             // tile rows in the current band
    int tn0;              // first candidate tile of the current band
    int col, row;         // position of the current tile inside the band (rem == col * rows + row)
    int step_col, step_row;  // step / rows and step % rows of the current band
    int tm, tn;
    bool valid;

    // Raster band (in the global numbering) behind this launch's k-th band.
    __host__ __device__ __forceinline__ int physical_band(const JoinParams& p, int k) const {
        const int g = p.shard_world > 1 ? p.shard_world : 1;
        const int r = p.shard_world > 1 ? p.shard_rank : 0;
        return (k >> 1) * (2 * g) + ((k & 1) ? (2 * g - 1 - r) : r);
    }
    __host__ __device__ __forceinline__ void load_band(const JoinParams& p) {
        pband = physical_band(p, band);
        const int first_row = pband * p.band_tiles;
        rows = p.tiles_m - first_row < p.band_tiles ? p.tiles_m - first_row : p.band_tiles;
        tn0 = 0;
        if (p.symmetric) {
            const int r0 = p.q_begin + first_row * p.tile_m;
            tn0 = r0 >= kTileN ? (r0 - (kTileN - 1)) / kTileN : 0;
            if (tn0 > p.tiles_n) tn0 = p.tiles_n;
        }
        band_size = static_cast<long long>(rows) * (p.tiles_n - tn0);
        const unsigned s32 = static_cast<unsigned>(step), r32 = static_cast<unsigned>(rows);
        step_col = static_cast<int>(s32 / r32);
        step_row = static_cast<int>(s32 % r32);
    }
    __host__ __device__ __forceinline__ bool below_diagonal(const JoinParams& p) const {
        return p.symmetric && tn * kTileN + (kTileN - 1) < p.q_begin + tm * p.tile_m;
    }
    // Position from rem by division: at the start and when a band ends (once per band).
    __host__ __device__ __forceinline__ void settle(const JoinParams& p) {
        for (;;) {
            while (band < nbands && rem >= band_size) {
                rem -= band_size;
                if (++band < nbands) load_band(p);
            }
            if (band >= nbands) {
                valid = false;
                return;
            }
            col = static_cast<int>(rem / rows);
            row = static_cast<int>(rem - static_cast<long long>(col) * rows);
            tn = tn0 + col;
            tm = pband * p.band_tiles + row;
            if (!below_diagonal(p)) {
                valid = true;
                return;
            }
            rem += step;  // tile entirely below the diagonal: nothing to do
        }
    }
    __host__ __device__ __forceinline__ void init(const JoinParams& p, long long first, long long stride) {
        step = stride;
        rem = first;
        band = 0;
        const int total_bands = (p.tiles_m + p.band_tiles - 1) / p.band_tiles;
        nbands = 0;
        while (physical_band(p, nbands) < total_bands) ++nbands;  // physical_band grows with k
        valid = false;
        if (nbands > 0) {
            load_band(p);
            settle(p);
        }
    }
    // The next tile of this CTA: inside a band the position moves by (step_col, step_row) with one
    // carry, no division (the kernel's three roles all walk the schedule, once per tile).
    __host__ __device__ __forceinline__ void advance(const JoinParams& p) {
        for (;;) {
            rem += step;
            if (rem >= band_size) {
                settle(p);
                return;
            }
            col += step_col;
            row += step_row;
            if (row >= rows) {
                row -= rows;
                ++col;
            }
            tn = tn0 + col;
            tm = pband * p.band_tiles + row;
            if (!below_diagonal(p)) return;
        }
    }
};

// ---------------------------------------------------------------------------
// Row norms
// ---------------------------------------------------------------------------
//
// s_i = sequential round-toward-zero sum, over column pairs in ascending k, of
// RZ(x_k^2 + x_{k+1}^2) with exact FP32 squares: the reduction of
// source/sumSquared.cuh:34-40 and :59-72 of the reference, bit for bit.
//
// The reference runs one thread per point reading 4 bytes at a time.  Here a
// CTA owns 128 rows; thread 0 streams [128 rows x 64 halfs] boxes through a
// ring of TMA stages (128-byte swizzle, so that thread r reading row r's 16-byte
// chunks is bank-conflict free) and thread r walks row r's chain.  The chain
// is serial per row by definition, but 128 rows x several CTAs per SM keep the
// loads far ahead of it: the kernel is bound by HBM.

constexpr int kNormRows = 128;
constexpr int kNormStages = 4;
constexpr int kNormBoxesPerStage = 1;  // 128 contiguous bytes per row per stage; 64 KiB ring -> 3 blocks per SM
constexpr uint32_t kNormBoxBytes = kNormRows * kTileK * 2;
constexpr uint32_t kNormStageBytes = kNormBoxBytes * kNormBoxesPerStage;
constexpr int kNormSmemBytes = kNormStages * kNormStageBytes + 1024 + 64;

// kExact = false: the reference's chain above.  kExact = true (an option, not the reference's
// numerics): the same squares summed in FP64 and rounded once to FP32, i.e. the correctly rounded
// norm, which matches the near-exact accumulation of tcgen05.mma better than the chain's
// round-toward-zero bias does (the chain exists to match the truncating accumulate of the
// reference's A100).
// (Measured at D = 4096, |p|^2 ~ 5.1: d2(i,i) is -2.3e-4 with the chain and +2.3e-4 with exact norms, so
// tcgen05.mma's accumulate does lose low bits, about as much as the chain, in the other direction for
// d2.  A chain truncated once per 16-wide slice leaves +1.8e-4, so it is not a simple per-instruction
// truncation and no norm variant cancels it exactly.)
template <int kExact>
__global__ void __launch_bounds__(kNormRows)
row_norms_kernel(const __grid_constant__ CUtensorMap map, float* __restrict__ norms, int n, int k_boxes,
                 int row_blocks, int row_block_begin, unsigned long long* __restrict__ status) {
    // (row blocks [row_block_begin, row_block_begin + row_blocks) of 128 rows each: the whole matrix, or
    // the rows of a piece that has just arrived)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + kNormStages * kNormStageBytes;  // kNormStages full barriers
    __shared__ int abort_flag;

    const int tid = threadIdx.x;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kNormStages; ++s) ptx::mbar_init(bars + 8 * s, 1);
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&map);
    }
    __syncthreads();
    // The join that follows may be scheduled now: its prologue and its first tiles' loads and MMAs need
    // nothing of this kernel's; its epilogue waits for the norms (grid_dependency_wait).
    ptx::launch_dependents();

    const int steps_per_block = (k_boxes + kNormBoxesPerStage - 1) / kNormBoxesPerStage;
    // Work items of this CTA: (row block, k step) pairs in order.
    const int my_blocks = (row_blocks - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                          static_cast<int>(gridDim.x);
    const long long total_items = static_cast<long long>(my_blocks) * steps_per_block;

    auto issue = [&](long long item) {
        const int blk = static_cast<int>(item / steps_per_block);
        const int step = static_cast<int>(item - static_cast<long long>(blk) * steps_per_block);
        const int row0 = (row_block_begin + static_cast<int>(blockIdx.x) + blk * static_cast<int>(gridDim.x)) * kNormRows;
        const int s = static_cast<int>(item % kNormStages);
        const uint32_t bar = bars + 8 * s;
        const int nb = min(kNormBoxesPerStage, k_boxes - step * kNormBoxesPerStage);
        ptx::mbar_expect_tx(bar, nb * kNormBoxBytes);
        for (int b = 0; b < nb; ++b)
            ptx::tma_load_2d(base + s * kNormStageBytes + b * kNormBoxBytes, &map, bar,
                             (step * kNormBoxesPerStage + b) * kTileK, row0);
    };

    if (tid == 0) {
        const long long pre = total_items < kNormStages ? total_items : kNormStages;
        for (long long i = 0; i < pre; ++i) issue(i);
    }

    float acc = 0.0f;
    double acc64 = 0.0;
    bool ok = true;
    for (long long item = 0; item < total_items; ++item) {
        const int blk = static_cast<int>(item / steps_per_block);
        const int step = static_cast<int>(item - static_cast<long long>(blk) * steps_per_block);
        const int s = static_cast<int>(item % kNormStages);
        const uint32_t parity = static_cast<uint32_t>((item / kNormStages) & 1);
        if (step == 0) {
            acc = 0.0f;
            acc64 = 0.0;
        }
        ok = ptx::mbar_wait_bounded(bars + 8 * s, parity, &abort_flag, kWaitLimitNs);
        if (ok) {
            const int nb = min(kNormBoxesPerStage, k_boxes - step * kNormBoxesPerStage);
            for (int b = 0; b < nb; ++b) {
                const uint8_t* box =
                    smem_raw + (base - ptx::smem_u32(smem_raw)) + s * kNormStageBytes + b * kNormBoxBytes;
                const uint8_t* row = box + tid * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 q = *reinterpret_cast<const uint4*>(row + ((c ^ (tid & 7)) << 4));
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                        if constexpr (kExact != 0) {
                            // f.x^2 + f.y^2 is formed exactly in FP64 (22-bit products), then accumulated.
                            acc64 += static_cast<double>(f.x) * static_cast<double>(f.x) +
                                     static_cast<double>(f.y) * static_cast<double>(f.y);
                        } else {
                            acc = __fadd_rz(acc, __fadd_rz(f.x * f.x, f.y * f.y));
                        }
                    }
                }
            }
            if (step == steps_per_block - 1) {
                const int r = (row_block_begin + static_cast<int>(blockIdx.x) + blk * static_cast<int>(gridDim.x)) * kNormRows + tid;
                if (r < n) norms[r] = kExact == 1 ? static_cast<float>(acc64) : acc;
            }
        }
        // Every thread is done with stage s.  The same barrier carries the outcome of the waits, so
        // that all threads leave the loop together if any of them gave up.
        if (__syncthreads_or(ok ? 0 : 1)) {
            ok = false;
            break;
        }
        if (tid == 0 && item + kNormStages < total_items) issue(item + kNormStages);
    }
    if (!ok) {
        // Give loads that are still in flight a bounded chance to land before the CTA exits.
        if (tid == 0) {
            atomicOr(status, kErrNormWait);
            const uint64_t t0 = ptx::globaltimer_ns();
            for (int s = 0; s < kNormStages; ++s)
                for (int ph = 0; ph < 2; ++ph)
                    while (!ptx::mbar_try_wait(bars + 8 * s, ph) && ptx::globaltimer_ns() - t0 < 20000000ull) {
                    }
        }
    }
}

// ---------------------------------------------------------------------------
// The join
// ---------------------------------------------------------------------------
//
// Replaces, for one band of query rows against all candidates, the reference's
// FindPairsKernel (source/findPairs.cuh:360-546): tile hand-out
// (source/rasterizer/onDemandRasterizer.cuh:78-108), global->shared staging
// (findPairs.cuh:182-218), ldmatrix + mma.sync (source/ptxMma.cuh:95-191,
// source/warpMma.cuh:131-190), the distance test (warpMma.cuh:220-273) and the
// pair append (source/pair.cuh:123-133).
//
// Warp roles (320 threads, one CTA per SM):
//   warp 0      one lane issues the TMA loads of A (128 x 64) and B (256 x 64)
//               FP16 boxes into a 4-stage ring of 128B-swizzled shared memory
//   warp 1      allocates TMEM; one lane issues 4 tcgen05.mma (M128 N256 K16)
//               per stage into one of two 256-column FP32 accumulators and
//               commits stage-release / accumulator-ready mbarriers
//   warps 2..9  epilogue: two warps per TMEM lane quarter, each taking 128 of
//               the 256 accumulator columns: tcgen05.ld.16x256b (a thread holds
//               2 rows x 16 columns per chunk), a conservative fast reject, the
//               exact d2 = (s_q + s_c) - 2a <= eps2 where it does not reject,
//               a warp scan and one atomicAdd per warp and tile, packed pairs
//               written one tile later.  The warps never meet at a barrier:
//               each stages its own norms.
// The epilogue of tile t overlaps the main loop of tile t+1 through the two
// accumulator buffers.

// Epilogue of one accumulator for one warp: its TMEM lane quarter (32 query rows) x kEpiCols
// candidate columns.  The accumulator comes in four tcgen05.ld.16x256b.x8 chunks (16 rows x 64
// columns each): a thread then holds 2 rows x 16 columns per chunk, so over the tile it needs
// only 4 query norms and 32 candidate norms (a thread that owned one whole row would need all
// kEpiCols candidate norms: four times the shared-memory traffic).
//
// Exact test: d2 = (s_q + s_c) - 2a as the reference's inspectResults
// (source/warpMma.cuh:239-242), inclusive compare (:257); rows and columns that are padding carry
// +inf norms and can never hit (:259).
//
// Fast reject, per chunk and row: with u_j = fma(a_j, -2, s_cj) (one packed FMA per two elements)
// and lo = min_j u_j (one three-input min per two elements), no column of the row can hit when
// lo + s_q > eps2 + slack * (s_q + max s_c + eps2).  The slack covers the rounding differences
// between this expression and the exact one: both differ from the real s_q + s_c - 2a by at most
// 2^-21 * (s_q + s_c + eps2) in total when the exact d2 is <= eps2 (two roundings to nearest each,
// of values bounded by 3 * (s_q + s_c) + 2 * eps2 in magnitude; a much larger a makes both sums
// negative, which never rejects); 2^-19 is used.  A row that is not rejected takes the exact path,
// so the result is the exact test's, bit for bit.  NaNs drop out of the min and the reject is
// written as !(x > thr), so a NaN can only send a chunk to the exact path.
//
// Pass 1 turns the warp's share of the tile into hit bit masks (4 chunks x 32 elements per
// thread).  Only if some thread of the warp has a hit does pass 2 run: one warp scan of the
// per-thread counts, ONE atomicAdd on the found counter per warp and tile, then every thread writes
// its records to consecutive slots -- the reference does two atomics per pair
// (source/pair.cuh:123-133).  Overflow keeps its rule: found counts everything, records beyond the
// capacity are dropped (the host derives stored = min(found, capacity)).
//
// Symmetric mode keeps columns c >= q and emits, for c > q, the mirrored record (c, q) as well.
//
// taddr: TMEM address of (first lane of the quarter, first column of the warp's share);
// wcn: the warp's kEpiCols candidate norms in shared memory; sq_lane: the query norm of row
// (q0 + lane); q0 / c0: global index of the quarter's first row / the share's first column.
constexpr float kRejectSlack = 1.9073486328125e-6f;  // 2^-19

__device__ __forceinline__ float finite_or_zero(float x) { return x < __int_as_float(0x7f800000) ? x : 0.0f; }

__device__ __forceinline__ uint32_t epi_chunk_taddr(uint32_t taddr, int k) {
    // chunk k: row block k & 1 (16 lanes each), column half k >> 1 (64 columns each)
    return taddr + (static_cast<uint32_t>((k & 1) * 16) << 16) + static_cast<uint32_t>((k >> 1) * 64);
}

// Hits of one warp in one tile, kept in registers between the test and the writing of the records.
struct EpiHits {
    uint32_t hit[kEpiCols / 32];
    uint32_t mir[kEpiCols / 32];
    uint32_t cnt;    // this thread's records (hits + mirrored hits)
    uint32_t excl;   // records of the lower lanes
    unsigned long long base;  // lane 0: first slot of the warp's reservation
    int q0, c0;
    bool any;        // warp-uniform: some thread has a record
};

// Test of one chunk (this thread's 2 rows x 16 columns): fast reject, else the exact test.
// sc2: the candidate norms of the chunk's column half; d0 = column - row of element 0.
__device__ __forceinline__ void epi_test_chunk(const JoinParams& p, const uint32_t (&v)[32], const uint64_t (&sc2)[8],
                                               float scmax, float sqA, float sqB, int d0, uint32_t& mask,
                                               uint32_t& mirror) {
    const float inf = __int_as_float(0x7f800000);
    const uint64_t m2 = ptx::pack_f32x2(-2.0f, -2.0f);
    float loA0 = inf, loA1 = inf, loB0 = inf, loB1 = inf;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint64_t aA = ptx::pack_f32x2(__uint_as_float(v[4 * g + 0]), __uint_as_float(v[4 * g + 1]));
        const uint64_t aB = ptx::pack_f32x2(__uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3]));
        float x0, x1, y0, y1;
        ptx::unpack_f32x2(ptx::fma_f32x2(aA, m2, sc2[g]), x0, x1);
        ptx::unpack_f32x2(ptx::fma_f32x2(aB, m2, sc2[g]), y0, y1);
        if (g & 1) {
            loA1 = ptx::min3_f32(loA1, x0, x1);
            loB1 = ptx::min3_f32(loB1, y0, y1);
        } else {
            loA0 = ptx::min3_f32(loA0, x0, x1);
            loB0 = ptx::min3_f32(loB0, y0, y1);
        }
    }
    const float base = scmax + p.eps2;
    const float thrA = fmaf(kRejectSlack, finite_or_zero(sqA) + base, p.eps2);
    const float thrB = fmaf(kRejectSlack, finite_or_zero(sqB) + base, p.eps2);
    const bool rejA = (fminf(loA0, loA1) + sqA) > thrA;
    const bool rejB = (fminf(loB0, loB1) + sqB) > thrB;
    mask = 0;
    mirror = 0;
    if (!(rejA && rejB)) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float s0, s1;
            ptx::unpack_f32x2(sc2[i >> 2], s0, s1);
            const float d2 = (((i & 2) ? sqB : sqA) + ((i & 1) ? s1 : s0)) - 2.0f * __uint_as_float(v[i]);
            if (d2 <= p.eps2) mask |= (1u << i);
        }
        if (p.symmetric && mask) {
            // element i lies at column - row = d0 + 8 * (i >> 2) + (i & 1) - ((i & 2) ? 8 : 0)
            if (d0 - 8 > 0) {
                mirror = mask;  // the whole chunk lies above the diagonal
            } else {
                uint32_t m = mask;
                while (m) {
                    const int i = __ffs(m) - 1;
                    m &= m - 1;
                    const int delta = d0 + 8 * (i >> 2) + (i & 1) - ((i & 2) ? 8 : 0);
                    if (delta < 0) mask &= ~(1u << i);
                    if (delta > 0) mirror |= (1u << i);
                }
            }
        }
    }
}

// This thread's candidate norms of one 64-column half (columns c2, c2 + 1 of each 8-column unit)
// and the largest finite one.
__device__ __forceinline__ float epi_load_cand(const float* wcn_half, uint64_t (&sc2)[8]) {
    float mx = 0.0f;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const float2 x = reinterpret_cast<const float2*>(wcn_half)[4 * g];
        sc2[g] = ptx::pack_f32x2(x.x, x.y);
        mx = fmaxf(mx, fmaxf(finite_or_zero(x.x), finite_or_zero(x.y)));
    }
    return mx;
}

// Pass 1: test the warp's share of the tile, leave the hit masks in `out`, return this thread's
// record count.
__device__ __forceinline__ uint32_t epilogue_scan(const JoinParams& p, uint32_t taddr, const float* wcn, float sq_lane,
                                                  int q0, int c0, int lane, float (&sq)[4], EpiHits& out) {
    static_assert(kEpiCols == 128, "four chunks: two row blocks x two 64-column halves");
    const int r4 = lane >> 2;        // row inside an 8-row group
    const int c2 = (lane & 3) * 2;   // first of this thread's two columns inside an 8-column unit
    // Query norms of this thread's four rows (r4 + 8i of the quarter).
#pragma unroll
    for (int i = 0; i < 4; ++i) sq[i] = __shfl_sync(0xffffffffu, sq_lane, r4 + 8 * i);
    uint32_t cnt = 0;
    // Two register buffers: while chunk k is tested, the load of chunk k + 1 is in flight.
    constexpr int kChunks = kEpiCols / 32;
    uint32_t va[32], vb[32];
    ptx::tmem_ld_16x256b_x8(taddr, va);
    uint64_t sc2[8];
    float scmax = 0.0f;
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
        const int b = k & 1, h = k >> 1;
        uint32_t(&v)[32] = (k & 1) ? vb : va;
        uint32_t(&w)[32] = (k & 1) ? va : vb;
        ptx::tmem_ld_wait_for(v);
        if (k + 1 < kChunks) ptx::tmem_ld_16x256b_x8(epi_chunk_taddr(taddr, k + 1), w);
        if (b == 0) scmax = epi_load_cand(wcn + h * 64 + c2, sc2);
        const int d0 = (c0 + h * 64 + c2) - (q0 + 16 * b + r4);
        epi_test_chunk(p, v, sc2, scmax, sq[2 * b], sq[2 * b + 1], d0, out.hit[k], out.mir[k]);
        cnt += __popc(out.hit[k]) + __popc(out.mir[k]);
    }
    return cnt;
}

// Pass 2a: if the warp has records, reserve their slots with ONE atomicAdd (lane 0).  The returned
// base is not touched here, so the caller can let a whole tile pass before it needs the value.
__device__ __forceinline__ void epilogue_reserve(const JoinParams& p, uint32_t cnt, int q0, int c0, int lane, EpiHits& h) {
    h.any = __any_sync(0xffffffffu, cnt != 0);
    if (!h.any) return;
    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    h.cnt = cnt;
    h.excl = incl - cnt;
    h.q0 = q0;
    h.c0 = c0;
    h.base = 0;
    if (lane == 0) h.base = atomicAdd(p.counters + 0, static_cast<unsigned long long>(total));
}

// Element i of chunk k: row q0 + 16 * (k & 1) + r4 + ((i & 2) ? 8 : 0),
// column c0 + 64 * (k >> 1) + c2 + 8 * (i >> 2) + (i & 1).

// Pass 2b, records only: every thread writes its records to consecutive slots.
__device__ __forceinline__ void epilogue_emit(const JoinParams& p, EpiHits& h, int lane) {
    constexpr int kChunks = kEpiCols / 32;
    unsigned long long slot = __shfl_sync(0xffffffffu, h.base, 0) + h.excl;
    const int q_thread = h.q0 + (lane >> 2);
    const int c_thread = h.c0 + (lane & 3) * 2;
#pragma unroll 1
    for (int k = 0; k < kChunks; ++k) {
        // (dynamic register indexing is avoided by rotating the arrays)
        uint32_t m = h.hit[0], r = h.mir[0];
#pragma unroll
        for (int j = 0; j + 1 < kChunks; ++j) {
            h.hit[j] = h.hit[j + 1];
            h.mir[j] = h.mir[j + 1];
        }
        const uint32_t qk = static_cast<uint32_t>(q_thread + 16 * (k & 1));
        const uint32_t ck = static_cast<uint32_t>(c_thread + 64 * (k >> 1));
        while (m) {
            const int i = __ffs(m) - 1;
            m &= m - 1;
            const unsigned long long q = qk + ((i & 2) ? 8u : 0u);
            const unsigned long long c = ck + 8u * (i >> 2) + (i & 1);
            if (slot < p.capacity) store_record(p, slot, q, c);
            ++slot;
        }
        while (r) {
            const int i = __ffs(r) - 1;
            r &= r - 1;
            const unsigned long long q = qk + ((i & 2) ? 8u : 0u);
            const unsigned long long c = ck + 8u * (i >> 2) + (i & 1);
            if (slot < p.capacity) store_record(p, slot, c, q);
            ++slot;
        }
    }
}

// Pass 2b with distances: read the accumulator chunk again where the warp has hits (the caller
// still owns the TMEM buffer).
__device__ __forceinline__ void epilogue_emit_dist(const JoinParams& p, const EpiHits& h, uint32_t taddr, const float* wcn,
                                                   const float (&sq)[4], int lane) {
    constexpr int kChunks = kEpiCols / 32;
    unsigned long long slot = __shfl_sync(0xffffffffu, h.base, 0) + h.excl;
    const int q_thread = h.q0 + (lane >> 2);
    const int c2 = (lane & 3) * 2;
    const int c_thread = h.c0 + c2;
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
        const uint32_t m = h.hit[k], r = h.mir[k];
        if (!__any_sync(0xffffffffu, (m | r) != 0)) continue;
        uint32_t v[32];
        ptx::tmem_ld_16x256b_x8(epi_chunk_taddr(taddr, k), v);
        ptx::tmem_ld_wait_for(v);
        const uint32_t qk = static_cast<uint32_t>(q_thread + 16 * (k & 1));
        const uint32_t ck = static_cast<uint32_t>(c_thread + 64 * (k >> 1));
        const float* scp = wcn + (k >> 1) * 64 + c2;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if ((m | r) & (1u << i)) {
                const float sqr = sq[2 * (k & 1) + ((i >> 1) & 1)];
                const float d2 = p.raw_dot ? __uint_as_float(v[i])
                                           : (sqr + scp[8 * (i >> 2) + (i & 1)]) - 2.0f * __uint_as_float(v[i]);
                const unsigned long long q = qk + ((i & 2) ? 8u : 0u);
                const unsigned long long c = ck + 8u * (i >> 2) + (i & 1);
                if (m & (1u << i)) {
                    if (slot < p.capacity) {
                        store_record(p, slot, q, c);
                        p.dist2[slot] = d2;
                    }
                    ++slot;
                }
                if (r & (1u << i)) {
                    if (slot < p.capacity) {
                        store_record(p, slot, c, q);
                        p.dist2[slot] = d2;
                    }
                    ++slot;
                }
            }
        }
    }
}

// One tile of one epilogue warp.  After pass 1 the accumulator goes back to the MMA warp at once
// (`release`), the slots of THIS tile's records are reserved, and only then are the records of the
// PREVIOUS tile written (`pend`): the atomic's round trip to L2 and back, about a microsecond and
// otherwise paid by nearly every tile that has a hit, hides behind a whole tile.  The caller
// writes out the last `pend` after its loop.  With distances the accumulator is read again, so
// that mode reserves and writes before it releases.
template <class Release>
__device__ __forceinline__ void epilogue_tile(const JoinParams& p, uint32_t taddr, const float* wcn, float sq_lane,
                                              int q0, int c0, int lane, EpiHits& pend, Release release) {
    float sq[4];
    EpiHits cur;
    cur.any = false;
    const uint32_t cnt = epilogue_scan(p, taddr, wcn, sq_lane, q0, c0, lane, sq, cur);
    if (p.dist2 != nullptr) {
        epilogue_reserve(p, cnt, q0, c0, lane, cur);
        if (cur.any) epilogue_emit_dist(p, cur, taddr, wcn, sq, lane);
        release();
        return;
    }
    release();
    if (pend.any) epilogue_emit(p, pend, lane);
    // (the masks are copied, the atomic's result lands in pend.base itself: no instruction waits for it
    // before the next tile's epilogue_emit)
#pragma unroll
    for (int k = 0; k < kEpiCols / 32; ++k) {
        pend.hit[k] = cur.hit[k];
        pend.mir[k] = cur.mir[k];
    }
    epilogue_reserve(p, cnt, q0, c0, lane, pend);
}

// The norms one epilogue warp needs for a tile, fetched one tile ahead (their global-memory
// latency hides behind the previous tile): lane l takes the candidate norms of columns
// c_first + 4l .. + 3 (the warp's kEpiCols columns, staged through the warp's own shared-memory
// row, so the epilogue warps never meet at a barrier) and the query norm of row q_first + l.
// Padding rows and columns get +inf and can never hit.
__device__ __forceinline__ void fetch_warp_norms(const JoinParams& p, int c_first, int q_first, int lane, float4& cand,
                                                 float& query) {
    static_assert(kEpiCols == 128, "four candidate norms per lane");
    const float inf = __int_as_float(0x7f800000);
    const int c = c_first + 4 * lane;
    // (plain loads, not the read-only path: when the join overlaps the norm kernel -- dependent launch --
    // the norms are written during this kernel's lifetime, before grid_dependency_wait() returns)
    if (c + 3 < p.n && p.norms_vec4) {
        cand = *reinterpret_cast<const float4*>(p.norms + c);
    } else {
        cand.x = (c + 0 < p.n) ? p.norms[c + 0] : inf;
        cand.y = (c + 1 < p.n) ? p.norms[c + 1] : inf;
        cand.z = (c + 2 < p.n) ? p.norms[c + 2] : inf;
        cand.w = (c + 3 < p.n) ? p.norms[c + 3] : inf;
    }
    const int q = q_first + lane;
    query = (q < p.q_end) ? p.norms[q] : inf;
}

struct JoinSmemAux {
    unsigned long long full_bar[kStages];
    unsigned long long empty_bar[kStages];
    unsigned long long acc_full_bar[2];
    unsigned long long acc_empty_bar[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float warp_cand[kEpiWarps][kEpiCols];  // each epilogue warp stages its own candidate norms
};

constexpr int kJoinSmemBytes = kStages * kStageBytes + 1024 + static_cast<int>(sizeof(JoinSmemAux)) + 64;

__global__ void __launch_bounds__(kJoinThreads, 1)
join_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const JoinParams p) {
    const long long clock_entry = clock64();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
    const uint32_t tiles_u32 = (raw_u32 + 1023u) & ~1023u;
    JoinSmemAux* aux = reinterpret_cast<JoinSmemAux*>(smem_raw + (tiles_u32 - raw_u32) + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &aux->abort_flag;

    if (threadIdx.x == 0) {
        aux->abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&aux->full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&aux->acc_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->acc_empty_bar[b]), kEpiWarps);  // one arrive per epilogue warp
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&map_a);
        ptx::prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(&aux->tmem_base), kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = aux->tmem_base;

    const long long first_tile = blockIdx.x;
    const long long tile_step = gridDim.x;
    const long long clock_start = clock64();

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long issued = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p)) {
                const int tm = ti.tm, tn = ti.tn;
                const int row_a = p.q_begin + tm * kTileM;
                const int row_b = cand_row0(p, tn);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->empty_bar[stage]), phase ^ 1u, abort_flag,
                                                kWaitLimitNs);
                    if (!ok) break;
                    const uint32_t bar = ptx::smem_u32(&aux->full_bar[stage]);
                    const uint32_t dst = tiles_u32 + stage * kStageBytes;
                    ptx::mbar_expect_tx(bar, kStageBytes);
                    ptx::tma_load_2d(dst, &map_a, bar, ks * kTileK, row_a);
                    ptx::tma_load_2d(dst + kStageBytesA, &map_b, bar, ks * kTileK, row_b);
                    ++issued;
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                atomicOr(p.counters + 2, kErrProducerWait);
                // Bounded wait for the loads still in flight (at most kStages of them).
                const uint64_t t0 = ptx::globaltimer_ns();
                const long long pending = issued < kStages ? issued : kStages;
                int s = stage;
                uint32_t ph = phase;
                for (long long i = 0; i < pending; ++i) {
                    if (--s < 0) {
                        s = kStages - 1;
                        ph ^= 1u;
                    }
                    while (!ptx::mbar_try_wait(ptx::smem_u32(&aux->full_bar[s]), ph) &&
                           ptx::globaltimer_ns() - t0 < 20000000ull) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer ---------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_f16_idesc(kTileM, kTileN);
            long long feed_wait = 0, acc_wait = 0;  // cycles this thread waited for operands / for a free accumulator
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long it = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p), ++it) {
                const int buf = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                const long long w0 = clock64();
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_empty_bar[buf]), acc_phase ^ 1u, abort_flag,
                                            kWaitLimitNs);
                acc_wait += clock64() - w0;
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    const long long f0 = clock64();
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->full_bar[stage]), phase, abort_flag,
                                                kWaitLimitNs);
                    feed_wait += clock64() - f0;
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = tiles_u32 + stage * kStageBytes;
                    const uint64_t desc_a = ptx::make_kmajor_sw128_desc(a_addr);
                    const uint64_t desc_b = ptx::make_kmajor_sw128_desc(a_addr + kStageBytesA);
#pragma unroll
                    for (int k = 0; k < kTileK / kUmmaK; ++k) {
                        // Advance 16 halfs = 32 bytes inside the 128-byte swizzle row: +2 in the >>4 address field.
                        ptx::umma_f16_ss<1>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc,
                                            (ks > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::umma_commit_1cta(ptx::smem_u32(&aux->empty_bar[stage]));
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::umma_commit_1cta(ptx::smem_u32(&aux->acc_full_bar[buf]));
            }
            if (!ok) atomicOr(p.counters + 2, kErrMmaWait);
            if (blockIdx.x == 0) {
                p.counters[7] = static_cast<unsigned long long>(feed_wait);
                p.counters[8] = static_cast<unsigned long long>(acc_wait);
            }
        }
    } else {
        // ------------------------- Epilogue -----------------------------
        const int quarter = warp & 3;               // TMEM lane quarter this warp may access
        const int ewarp = warp - 2;
        const int col_off = (ewarp >> 2) * kEpiCols;  // this warp's share of the tile's columns
        float* wcn = aux->warp_cand[ewarp];
        bool ok = true;
        long long it = 0;
        TileIter ti;
        ti.init(p, first_tile, tile_step);
        float4 next_cand;
        float next_query;
        EpiHits pend;
        pend.any = false;
        ptx::grid_dependency_wait();  // the row norms come from the kernel before this one
        if (ti.valid)
            fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kTileM + quarter * 32, lane, next_cand,
                             next_query);
        for (; ti.valid; ++it) {
            const int buf = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const int q0 = p.q_begin + ti.tm * kTileM + quarter * 32;
            const int c0 = cand_row0(p, ti.tn) + col_off;
            __syncwarp();  // every lane is done with the previous tile's norms
            reinterpret_cast<float4*>(wcn)[lane] = next_cand;
            const float sq_lane = next_query;
            __syncwarp();
            ti.advance(p);
            if (ti.valid)
                fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kTileM + quarter * 32, lane,
                                 next_cand, next_query);
            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_full_bar[buf]), acc_phase, abort_flag,
                                                kWaitLimitNs);
            if (!ok) continue;  // walk the schedule to its end, do nothing else
            ptx::tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN + col_off);
            epilogue_tile(p, taddr, wcn, sq_lane, q0, c0, lane, pend, [&] {
                // Hand the accumulator back to the MMA warp.
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&aux->acc_empty_bar[buf]));
            });
        }
        if (pend.any) epilogue_emit(p, pend, lane);
        if (!ok && lane == 0) atomicOr(p.counters + 2, kErrEpilogueWait);
    }

    // Teardown: everyone meets, then the allocating warp frees TMEM.
    ptx::tc_fence_before_sync();
    __syncthreads();
    // SM cycles CTA 0 spent on its share of the tiles: lets the host derive the mean SM clock of the
    // launch (cycles / device time) and the share of those cycles the tensor pipe had work for.
    const long long clock_end = clock64();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.counters[4] = static_cast<unsigned long long>(clock_end - clock_start);
        p.counters[5] = static_cast<unsigned long long>(clock_start - clock_entry);  // set-up: barriers, TMEM allocation
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
        if (blockIdx.x == 0 && lane == 0) p.counters[6] = static_cast<unsigned long long>(clock64() - clock_end);  // TMEM release
    }
}

// ---------------------------------------------------------------------------
// The join for short rows: query tile stationary in shared memory
// ---------------------------------------------------------------------------
//
// For d <= 512 (at most 8 K steps) the main loop of join_kernel is bound by the L2 -> SM operand
// feed, not by the tensor pipe: every K step brings 16 KB of query rows and 32 KB of candidate rows
// for 512 clocks of MMA work, and every tile fetches its query rows again although a CTA's 128 x d
// query tile is only 16 KB per K step.  Here a CTA keeps its query tile resident and sweeps along
// its tile ROW: per K step only the 32 KB candidate box moves (one third less traffic into the SM),
// and the shared memory the query stages occupied becomes a deeper candidate ring.
//
// Schedule (AStatIter): the tile rows are cut into bands of R rows (R = 37 for 148 CTAs).  In a
// band of `rows` rows, C = grid / rows CTAs share each row: CTA b takes row b % rows and the tile
// columns (b / rows), (b / rows) + C, ...  CTAs with consecutive indices sit on the two SMs of a TPC
// and walk neighbouring rows through the SAME columns at the same time, so their candidate boxes
// are fetched from L2 once per TPC; a band's sweep reads every candidate row from DRAM once.
// Roles, epilogue, barriers and the bounded waits are those of join_kernel; in addition a_full /
// a_empty hand the resident query tile between the TMA thread and the MMA thread once per row.
constexpr int kAStatMaxStages = 6;
constexpr int kAStatMaxK = 8;

struct AStatIter {
    int grid, cta;
    int band_start;  // first tile row of the current band
    int rows, cper;  // tile rows in the current band, CTAs per row
    int tm, tn;
    bool valid;
    bool new_row;    // the current tile is this CTA's first of a new tile row: load the query tile

    __host__ __device__ __forceinline__ void enter_band(const JoinParams& p) {
        for (;;) {
            if (band_start >= p.tiles_m) {
                valid = false;
                return;
            }
            rows = p.tiles_m - band_start < p.astat_rows ? p.tiles_m - band_start : p.astat_rows;
            cper = grid / rows;  // >= 1: astat_rows <= grid
            const int r = cta % rows, c = cta / rows;
            if (c < cper) {
                tm = band_start + r;
                tn = c;
                if (p.symmetric) {
                    // tile (tm, tn) lies entirely below the diagonal iff tn * kTileN + kTileN - 1 < first row
                    const int tn0 = (p.q_begin + tm * kTileM) / kTileN;
                    if (tn0 > tn) tn += (tn0 - tn + cper - 1) / cper * cper;
                }
                if (tn < p.tiles_n) {
                    valid = true;
                    new_row = true;
                    return;
                }
            }
            band_start += p.astat_rows;  // nothing for this CTA in this band
        }
    }
    __host__ __device__ __forceinline__ void init(const JoinParams& p, int cta_, int grid_) {
        grid = grid_;
        cta = cta_;
        band_start = 0;
        valid = false;
        new_row = false;
        enter_band(p);
    }
    __host__ __device__ __forceinline__ void advance(const JoinParams& p) {
        tn += cper;
        new_row = false;
        if (tn >= p.tiles_n) {
            band_start += p.astat_rows;
            enter_band(p);
        }
    }
};

struct AStatSmemAux {
    unsigned long long full_bar[kAStatMaxStages];
    unsigned long long empty_bar[kAStatMaxStages];
    unsigned long long a_full_bar, a_empty_bar;
    unsigned long long acc_full_bar[2];
    unsigned long long acc_empty_bar[2];
    uint32_t tmem_base;
    int abort_flag;
    // Candidate norms of the tile, one row per half of its columns, double-buffered by tile parity.  The
    // four epilogue warps of a column half all write the same values (harmless) after the tile's
    // accumulator is ready: by then every warp has released the tile two back, the last reader of this buffer.
    alignas(16) float cand[2][kEpiWarps / 4][kEpiCols];
};

// The shared-memory budget is what decides the depth of the candidate ring (six K steps of query tile plus
// four 32 KB candidate stages are 224 of the 227 KB a block may have), so nothing is spent on alignment
// slack: the dynamic shared memory of this kernel is declared 1024-byte aligned (the 128-byte swizzle's
// requirement), and the kernel checks that before it touches anything.
__host__ __device__ constexpr int astat_smem_bytes(int k_steps, int stages) {
    return k_steps * static_cast<int>(kStageBytesA) + stages * static_cast<int>(kStageBytesB) +
           static_cast<int>(sizeof(AStatSmemAux)) + 16;
}

constexpr unsigned long long kErrSmemAlign = 16ull;  // status bit: dynamic shared memory was not 1024-byte aligned

__global__ void __launch_bounds__(kJoinThreads, 1)
join_astat_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const JoinParams p) {
    const long long clock_entry = clock64();
    extern __shared__ __align__(1024) uint8_t smem_astat[];
    const uint32_t a_u32 = ptx::smem_u32(smem_astat);                        // resident query tile: k_steps boxes
    const uint32_t b_u32 = a_u32 + static_cast<uint32_t>(p.k_steps) * kStageBytesA;  // candidate ring
    const int stages = p.astat_stages;
    AStatSmemAux* aux = reinterpret_cast<AStatSmemAux*>(smem_astat + static_cast<uint32_t>(p.k_steps) * kStageBytesA +
                                                        static_cast<uint32_t>(stages) * kStageBytesB);
    if ((a_u32 & 1023u) != 0) {  // would corrupt every swizzled tile: report and leave (uniform over the CTA)
        if (threadIdx.x == 0) atomicOr(p.counters + 2, kErrSmemAlign);
        return;
    }

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &aux->abort_flag;

    if (threadIdx.x == 0) {
        aux->abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&aux->full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->empty_bar[s]), 1);
        }
        ptx::mbar_init(ptx::smem_u32(&aux->a_full_bar), 1);
        ptx::mbar_init(ptx::smem_u32(&aux->a_empty_bar), 1);
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&aux->acc_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->acc_empty_bar[b]), kEpiWarps);
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&map_a);
        ptx::prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(&aux->tmem_base), kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = aux->tmem_base;
    const long long clock_start = clock64();
    const int cta = static_cast<int>(blockIdx.x), grid = static_cast<int>(gridDim.x);

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, a_rows_loaded = 0;
            bool ok = true;
            long long issued = 0;
            AStatIter ti;
            for (ti.init(p, cta, grid); ti.valid && ok; ti.advance(p)) {
                if (ti.new_row) {
                    // the MMAs that read the previous row's query tile are complete (first row: a fresh
                    // barrier counts as released)
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->a_empty_bar), (a_rows_loaded & 1u) ^ 1u, abort_flag,
                                                kWaitLimitNs);
                    if (!ok) break;
                    const uint32_t bar = ptx::smem_u32(&aux->a_full_bar);
                    ptx::mbar_expect_tx(bar, static_cast<uint32_t>(p.k_steps) * kStageBytesA);
                    for (int ks = 0; ks < p.k_steps; ++ks)
                        ptx::tma_load_2d(a_u32 + static_cast<uint32_t>(ks) * kStageBytesA, &map_a, bar, ks * kTileK,
                                         p.q_begin + ti.tm * kTileM);
                    ++a_rows_loaded;
                }
                const int row_b = cand_row0(p, ti.tn);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->empty_bar[stage]), phase ^ 1u, abort_flag,
                                                kWaitLimitNs);
                    if (!ok) break;
                    const uint32_t bar = ptx::smem_u32(&aux->full_bar[stage]);
                    ptx::mbar_expect_tx(bar, kStageBytesB);
                    ptx::tma_load_2d(b_u32 + static_cast<uint32_t>(stage) * kStageBytesB, &map_b, bar, ks * kTileK, row_b);
                    ++issued;
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                atomicOr(p.counters + 2, kErrProducerWait);
                // Bounded wait for the loads still in flight (the query tile and at most `stages` boxes).
                const uint64_t t0 = ptx::globaltimer_ns();
                if (a_rows_loaded > 0)
                    while (!ptx::mbar_try_wait(ptx::smem_u32(&aux->a_full_bar), (a_rows_loaded - 1u) & 1u) &&
                           ptx::globaltimer_ns() - t0 < 20000000ull) {
                    }
                const long long pending = issued < stages ? issued : stages;
                int s = stage;
                uint32_t ph = phase;
                for (long long i = 0; i < pending; ++i) {
                    if (--s < 0) {
                        s = stages - 1;
                        ph ^= 1u;
                    }
                    while (!ptx::mbar_try_wait(ptx::smem_u32(&aux->full_bar[s]), ph) &&
                           ptx::globaltimer_ns() - t0 < 20000000ull) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer ---------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_f16_idesc(kTileM, kTileN);
            long long feed_wait = 0, acc_wait = 0;  // cycles this thread waited for operands / for a free accumulator
            int stage = 0;
            uint32_t phase = 0, a_rows_seen = 0;
            bool ok = true;
            long long it = 0;
            AStatIter ti;
            for (ti.init(p, cta, grid); ti.valid && ok; ti.advance(p), ++it) {
                if (ti.new_row) {
                    // everything issued so far read the previous query tile: release it, then wait for the new one
                    if (a_rows_seen > 0) ptx::umma_commit_1cta(ptx::smem_u32(&aux->a_empty_bar));
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->a_full_bar), a_rows_seen & 1u, abort_flag, kWaitLimitNs);
                    if (!ok) break;
                    ++a_rows_seen;
                    ptx::tc_fence_after_sync();
                }
                const int buf = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                const long long w0 = clock64();
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_empty_bar[buf]), acc_phase ^ 1u, abort_flag,
                                            kWaitLimitNs);
                acc_wait += clock64() - w0;
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    const long long f0 = clock64();
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->full_bar[stage]), phase, abort_flag, kWaitLimitNs);
                    feed_wait += clock64() - f0;
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint64_t desc_a = ptx::make_kmajor_sw128_desc(a_u32 + static_cast<uint32_t>(ks) * kStageBytesA);
                    const uint64_t desc_b =
                        ptx::make_kmajor_sw128_desc(b_u32 + static_cast<uint32_t>(stage) * kStageBytesB);
#pragma unroll
                    for (int k = 0; k < kTileK / kUmmaK; ++k)
                        ptx::umma_f16_ss<1>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, (ks > 0 || k > 0) ? 1u : 0u);
                    ptx::umma_commit_1cta(ptx::smem_u32(&aux->empty_bar[stage]));
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) ptx::umma_commit_1cta(ptx::smem_u32(&aux->acc_full_bar[buf]));
            }
            if (!ok) atomicOr(p.counters + 2, kErrMmaWait);
            if (blockIdx.x == 0) {
                p.counters[7] = static_cast<unsigned long long>(feed_wait);
                p.counters[8] = static_cast<unsigned long long>(acc_wait);
            }
        }
    } else {
        // ------------------------- Epilogue -----------------------------
        const int quarter = warp & 3;
        const int ewarp = warp - 2;
        const int col_off = (ewarp >> 2) * kEpiCols;
        bool ok = true;
        long long it = 0;
        AStatIter ti;
        ti.init(p, cta, grid);
        float4 next_cand;
        float next_query;
        EpiHits pend;
        pend.any = false;
        ptx::grid_dependency_wait();  // the row norms come from the kernel before this one
        if (ti.valid)
            fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kTileM + quarter * 32, lane, next_cand,
                             next_query);
        for (; ti.valid; ++it) {
            const int buf = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const int q0 = p.q_begin + ti.tm * kTileM + quarter * 32;
            const int c0 = cand_row0(p, ti.tn) + col_off;
            const float4 cand_now = next_cand;
            const float sq_lane = next_query;
            ti.advance(p);
            if (ti.valid)
                fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kTileM + quarter * 32, lane,
                                 next_cand, next_query);
            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_full_bar[buf]), acc_phase, abort_flag,
                                                kWaitLimitNs);
            if (!ok) continue;
            ptx::tc_fence_after_sync();
            float* wcn = aux->cand[buf][ewarp >> 2];
            reinterpret_cast<float4*>(wcn)[lane] = cand_now;
            __syncwarp();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN + col_off);
            epilogue_tile(p, taddr, wcn, sq_lane, q0, c0, lane, pend, [&] {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&aux->acc_empty_bar[buf]));
            });
        }
        if (pend.any) epilogue_emit(p, pend, lane);
        if (!ok && lane == 0) atomicOr(p.counters + 2, kErrEpilogueWait);
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    const long long clock_end = clock64();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.counters[4] = static_cast<unsigned long long>(clock_end - clock_start);
        p.counters[5] = static_cast<unsigned long long>(clock_start - clock_entry);  // set-up: barriers, TMEM allocation
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
        if (blockIdx.x == 0 && lane == 0) p.counters[6] = static_cast<unsigned long long>(clock64() - clock_end);  // TMEM release
    }
}

// ---------------------------------------------------------------------------
// The join on CTA pairs (tcgen05 cta_group::2)
// ---------------------------------------------------------------------------
//
// Same algorithm, same roles, same epilogue as join_kernel, but two CTAs on neighbouring SMs
// (a cluster of 2) share one 256 x 256 tile: each CTA holds 128 query rows (its half of A and its
// 128 x 256 FP32 accumulator in its own TMEM) and loads only HALF of the candidate rows of the
// tile (128 x 64 per stage); one tcgen05.mma.cta_group::2 (M256 N256 K16), issued by the leader
// CTA, reads A from each CTA's own shared memory and the two halves of B from both.  Per stage a
// CTA therefore moves 32 KB from L2 instead of 48 KB and the tensor core reads B from shared memory
// once per pair instead of once per CTA: the L2 -> SM path and the shared-memory reads are what the
// single-CTA kernel spends its power on.  No multicast load is used: each CTA fetches its own boxes.
//
// Barriers: full[s] lives in the leader (one expect_tx of 64 KB by the leader's producer, completion
// bytes from both CTAs' loads); empty[s] and acc_full[b] live in both CTAs and are signalled by two
// commits of the leader's MMA thread (own CTA + peer); acc_empty[b] lives in the leader and counts
// the eight epilogue warps of the pair.

constexpr int kPairStages = 6;
constexpr uint32_t kPairStageBytesA = kTileM * kTileK * 2;        // 16 KiB: 128 query rows
constexpr uint32_t kPairStageBytesB = (kTileN / 2) * kTileK * 2;  // 16 KiB: 128 of the 256 candidate rows
constexpr uint32_t kPairStageBytes = kPairStageBytesA + kPairStageBytesB;
constexpr int kPairTileM = 2 * kTileM;  // query rows per CTA pair

struct PairSmemAux {
    unsigned long long full_bar[kPairStages];
    unsigned long long empty_bar[kPairStages];
    unsigned long long acc_full_bar[2];
    unsigned long long acc_empty_bar[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float warp_cand[kEpiWarps][kEpiCols];  // each epilogue warp stages its own candidate norms
};

constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + static_cast<int>(sizeof(PairSmemAux)) + 64;

__global__ void __launch_bounds__(kJoinThreads, 1)
join_pair_kernel(const __grid_constant__ CUtensorMap map, const JoinParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
    const uint32_t tiles_u32 = (raw_u32 + 1023u) & ~1023u;
    PairSmemAux* aux = reinterpret_cast<PairSmemAux*>(smem_raw + (tiles_u32 - raw_u32) + kPairStages * kPairStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_cta_rank();  // 0 = leader of the pair
    const bool leader = rank == 0;
    volatile int* abort_flag = &aux->abort_flag;

    if (threadIdx.x == 0) {
        aux->abort_flag = 0;
        for (int s = 0; s < kPairStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&aux->full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&aux->acc_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&aux->acc_empty_bar[b]), 2 * kEpiWarps);  // epilogue warps of both CTAs
        }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&map);
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(ptx::smem_u32(&aux->tmem_base), kTmemCols);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();  // both CTAs' barriers exist before anything remote touches them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = aux->tmem_base;

    const long long first_tile = blockIdx.x >> 1;
    const long long tile_step = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------- TMA producer (both CTAs) -------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long issued = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p)) {
                const int tm = ti.tm, tn = ti.tn;
                const int row_a = p.q_begin + tm * kPairTileM + static_cast<int>(rank) * kTileM;
                const int row_b = cand_row0(p, tn) + static_cast<int>(rank) * (kTileN / 2);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->empty_bar[stage]), phase ^ 1u, abort_flag,
                                                kWaitLimitNs);
                    if (!ok) break;
                    const uint32_t bar_local = ptx::smem_u32(&aux->full_bar[stage]);
                    const uint32_t bar_leader = ptx::mapa_u32(bar_local, 0);
                    const uint32_t dst = tiles_u32 + stage * kPairStageBytes;
                    if (leader) ptx::mbar_expect_tx(bar_local, 2 * kPairStageBytes);
                    ptx::tma_load_2d_pair(dst, &map, bar_leader, ks * kTileK, row_a);
                    ptx::tma_load_2d_pair(dst + kPairStageBytesA, &map, bar_leader, ks * kTileK, row_b);
                    ++issued;
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // Tail: do not leave while the leader's MMA thread may still signal this CTA's empty
            // barriers (or, on failure, while loads are in flight): walk one more lap of the ring.
            // (Stages never used pass at once: a fresh barrier counts as released.)
            const uint64_t t0 = ptx::globaltimer_ns();
            for (int i = 0; i < kPairStages && issued > 0; ++i) {
                while (!ptx::mbar_try_wait(ptx::smem_u32(&aux->empty_bar[stage]), phase ^ 1u) &&
                       ptx::globaltimer_ns() - t0 < (ok ? kWaitLimitNs : 20000000ull)) {
                }
                if (++stage == kPairStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) atomicOr(p.counters + 2, kErrProducerWait);
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer (leader CTA only) ----------------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = ptx::make_f16_idesc(kPairTileM, kTileN);
            long long acc_wait = 0;  // (kept for symmetry with the single-CTA kernels; not reported)
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long it = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p), ++it) {
                const int buf = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                const long long w0 = clock64();
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_empty_bar[buf]), acc_phase ^ 1u, abort_flag,
                                            kWaitLimitNs);
                acc_wait += clock64() - w0;
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->full_bar[stage]), phase, abort_flag, kWaitLimitNs);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = tiles_u32 + stage * kPairStageBytes;
                    const uint64_t desc_a = ptx::make_kmajor_sw128_desc(a_addr);
                    const uint64_t desc_b = ptx::make_kmajor_sw128_desc(a_addr + kPairStageBytesA);
#pragma unroll
                    for (int k = 0; k < kTileK / kUmmaK; ++k)
                        ptx::umma_f16_ss<2>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, (ks > 0 || k > 0) ? 1u : 0u);
                    const uint32_t eb = ptx::smem_u32(&aux->empty_bar[stage]);
                    ptx::umma_commit_pair(ptx::mapa_u32(eb, 0));
                    ptx::umma_commit_pair(ptx::mapa_u32(eb, 1));
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {
                    const uint32_t fb = ptx::smem_u32(&aux->acc_full_bar[buf]);
                    ptx::umma_commit_pair(ptx::mapa_u32(fb, 0));
                    ptx::umma_commit_pair(ptx::mapa_u32(fb, 1));
                }
            }
            if (!ok) atomicOr(p.counters + 2, kErrMmaWait);
        }
    } else {
        // ------------------------- Epilogue (both CTAs) ------------------------------
        const int quarter = warp & 3;
        const int ewarp = warp - 2;
        const int col_off = (ewarp >> 2) * kEpiCols;
        const int row_off = static_cast<int>(rank) * kTileM + quarter * 32;  // inside the pair's 256-row tile
        float* wcn = aux->warp_cand[ewarp];
        bool ok = true;
        long long it = 0;
        TileIter ti;
        ti.init(p, first_tile, tile_step);
        float4 next_cand;
        float next_query;
        EpiHits pend;
        pend.any = false;
        ptx::grid_dependency_wait();  // the row norms come from the kernel before this one
        if (ti.valid)
            fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kPairTileM + row_off, lane, next_cand,
                             next_query);
        for (; ti.valid; ++it) {
            const int buf = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const int q0 = p.q_begin + ti.tm * kPairTileM + row_off;
            const int c0 = cand_row0(p, ti.tn) + col_off;
            __syncwarp();
            reinterpret_cast<float4*>(wcn)[lane] = next_cand;
            const float sq_lane = next_query;
            __syncwarp();
            ti.advance(p);
            if (ti.valid)
                fetch_warp_norms(p, cand_row0(p, ti.tn) + col_off, p.q_begin + ti.tm * kPairTileM + row_off, lane,
                                 next_cand, next_query);

            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_full_bar[buf]), acc_phase, abort_flag,
                                                kWaitLimitNs);
            if (!ok) continue;
            ptx::tc_fence_after_sync();

            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN + col_off);
            epilogue_tile(p, taddr, wcn, sq_lane, q0, c0, lane, pend, [&] {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive_cluster_addr(ptx::mapa_u32(ptx::smem_u32(&aux->acc_empty_bar[buf]), 0));
            });
        }
        if (pend.any) epilogue_emit(p, pend, lane);
        if (!ok && lane == 0) atomicOr(p.counters + 2, kErrEpilogueWait);
    }

    // Teardown: neither CTA may leave (or free TMEM) while its peer can still touch it.
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait
// ---------------------------------------------------------------------------
//
// Waits, with the given limit, on an mbarrier that nothing will ever complete, the way a join
// role would wait for a peer that never answers.  The wait must give up after the limit, raise the
// CTA's abort flag, record its status bit and let the kernel return normally: no trap, no hang,
// the context stays usable.  Thread 1 waits on the same barrier and must leave through the abort
// flag raised by thread 0's timeout (or its own).
__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns, unsigned long long* status,
                                             unsigned long long* waited_ns) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x < 2) {
        const uint64_t t0 = ptx::globaltimer_ns();
        const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0, &abort_flag, limit_ns);
        const uint64_t t1 = ptx::globaltimer_ns();
        if (!ok) atomicOr(status, threadIdx.x == 0 ? kErrProducerWait : kErrMmaWait);
        if (threadIdx.x == 0) *waited_ns = t1 - t0;
    }
}

// ---------------------------------------------------------------------------
// Helpers
// ---------------------------------------------------------------------------

// Packed records -> {int query; int candidate}, the reference's Pair layout (source/pair.cuh:27-30).
// Record = ((query - qbase) << shift) | candidate (see JoinParams::key_shift).  keys and out may be the
// same buffer (every thread reads its record before it writes it).
__global__ void unpack_pairs_kernel(const unsigned long long* keys, int2* out, unsigned long long count, int shift,
                                    int qbase) {
    const unsigned long long mask = shift >= 64 ? ~0ull : ((1ull << shift) - 1ull);
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += stride) {
        const unsigned long long k = keys[i];
        out[i] = make_int2(static_cast<int>(k >> shift) + qbase, static_cast<int>(k & mask));
    }
}

// The same for 32-bit records (JoinParams::key32); keys and out must not overlap.
__global__ void unpack_pairs32_kernel(const uint32_t* __restrict__ keys, int2* __restrict__ out, unsigned long long count,
                                      int shift, int qbase) {
    const uint32_t mask = shift >= 32 ? ~0u : ((1u << shift) - 1u);
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += stride) {
        const uint32_t k = keys[i];
        out[i] = make_int2(static_cast<int>(k >> shift) + qbase, static_cast<int>(k & mask));
    }
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Counter-based synthetic data: coordinate (i, k) = Exponential(lambda) drawn
// from a hash of (seed, i*d + k), rejected to [0, max_value], rounded
// double -> float -> half like the reference's loader.  Used for the large
// benchmark shapes, where the reference's sequential host generator
// (source/DataLoader/ExponentialPointGenerator.hpp:42-52) would take minutes;
// the distribution is the same, the stream is not.
__global__ void gen_exponential_kernel(__half* __restrict__ out, long long n, int d, int ld, double lambda,
                                       double max_value, unsigned long long seed) {
    const long long chunks_per_row = ld / 8;
    const long long total = n * chunks_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += stride) {
        const long long row = g / chunks_per_row;
        const int k0 = static_cast<int>(g - row * chunks_per_row) * 8;
        __align__(16) __half h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = k0 + j;
            float f = 0.0f;
            if (k < d) {
                const uint64_t ctr = static_cast<uint64_t>(row) * static_cast<uint64_t>(d) + static_cast<uint64_t>(k);
                double v;
                uint64_t attempt = 0;
                do {
                    const uint64_t r = mix64(mix64(seed ^ (attempt * 0xd1342543de82ef95ull)) + ctr);
                    const double u = (static_cast<double>(r >> 11) + 0.5) * (1.0 / 9007199254740992.0);
                    v = -log(u) / lambda;
                    ++attempt;
                } while (v > max_value && attempt < 64);
                f = static_cast<float>(v);
            }
            h[j] = __float2half_rn(f);
        }
        *reinterpret_cast<uint4*>(out + row * ld + k0) = *reinterpret_cast<const uint4*>(h);
    }
}

// FP64 brute-force squared distances of sampled query rows against all
// candidates (accuracy reporting only; plain CUDA cores).  One CTA per
// (sample, candidate block); counts, per sample, the candidates with
// d2 <= eps2 and optionally records them.
__global__ void brute_f64_kernel(const __half* __restrict__ pts, int n, int d, int ld,
                                 const int* __restrict__ sample_rows, int n_samples, double eps2,
                                 unsigned long long* __restrict__ counts, unsigned long long* __restrict__ keys,
                                 unsigned long long capacity, unsigned long long* __restrict__ n_keys) {
    extern __shared__ float qrow[];
    const int s = blockIdx.y;
    const int q = sample_rows[s];
    for (int k = threadIdx.x; k < d; k += blockDim.x) qrow[k] = __half2float(pts[static_cast<long long>(q) * ld + k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    unsigned long long local = 0;
    for (int c = blockIdx.x * nwarps + warp; c < n; c += gridDim.x * nwarps) {
        const __half* row = pts + static_cast<long long>(c) * ld;
        double acc = 0.0;
        for (int k = lane; k < d; k += 32) {
            const double t = static_cast<double>(qrow[k]) - static_cast<double>(__half2float(row[k]));
            acc += t * t;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0 && acc <= eps2) {
            ++local;
            if (keys && capacity) {
                const unsigned long long slot = atomicAdd(n_keys, 1ull);
                if (slot < capacity)
                    keys[slot] = (static_cast<unsigned long long>(static_cast<uint32_t>(q)) << 32) |
                                 static_cast<unsigned long long>(static_cast<uint32_t>(c));
            }
        }
    }
    if (lane == 0 && local) atomicAdd(counts + s, local);
}

}  // namespace fasted
