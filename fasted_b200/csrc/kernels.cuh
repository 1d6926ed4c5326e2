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
    unsigned long long* counters;  // [0] pairs found, [1] unused (stored = min(found, capacity)), [2] status bits,
                                   // [4] SM cycles of CTA 0 (single-CTA kernel)
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
};

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
    }
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
            const int col = static_cast<int>(rem / rows);
            tn = tn0 + col;
            tm = pband * p.band_tiles + static_cast<int>(rem - static_cast<long long>(col) * rows);
            if (!p.symmetric || tn * kTileN + (kTileN - 1) >= p.q_begin + tm * p.tile_m) {
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
    __host__ __device__ __forceinline__ void advance(const JoinParams& p) {
        rem += step;
        settle(p);
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
                 int row_blocks, unsigned long long* __restrict__ status) {
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

    const int steps_per_block = (k_boxes + kNormBoxesPerStage - 1) / kNormBoxesPerStage;
    // Work items of this CTA: (row block, k step) pairs in order.
    const int my_blocks = (row_blocks - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                          static_cast<int>(gridDim.x);
    const long long total_items = static_cast<long long>(my_blocks) * steps_per_block;

    auto issue = [&](long long item) {
        const int blk = static_cast<int>(item / steps_per_block);
        const int step = static_cast<int>(item - static_cast<long long>(blk) * steps_per_block);
        const int row0 = (static_cast<int>(blockIdx.x) + blk * static_cast<int>(gridDim.x)) * kNormRows;
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
        if (!ok) break;
        const int nb = min(kNormBoxesPerStage, k_boxes - step * kNormBoxesPerStage);
        for (int b = 0; b < nb; ++b) {
            const uint8_t* box = smem_raw + (base - ptx::smem_u32(smem_raw)) + s * kNormStageBytes + b * kNormBoxBytes;
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
            const int r = (static_cast<int>(blockIdx.x) + blk * static_cast<int>(gridDim.x)) * kNormRows + tid;
            if (r < n) norms[r] = kExact == 1 ? static_cast<float>(acc64) : acc;
        }
        __syncthreads();  // every thread is done with stage s
        if (tid == 0 && item + kNormStages < total_items) issue(item + kNormStages);
    }
    if (!ok) {
        // Give loads that are still in flight a bounded chance to land before the CTA exits.
        __syncthreads();
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
//               the 256 accumulator columns: tcgen05.ld (thread = query row),
//               d2 = (s_q + s_c) - 2a, compare with eps2, compact the hits with
//               a warp scan and one atomicAdd per warp, store packed pairs.
// The epilogue of tile t overlaps the main loop of tile t+1 through the two
// accumulator buffers.

// Epilogue of one accumulator (128 lanes x kTileN columns) for one warp: thread = query row q
// (TMEM lane), 32 columns per tcgen05.ld.  d2 = (s_q + s_c) - 2a exactly as the reference's
// inspectResults (source/warpMma.cuh:239-242), inclusive compare (:257); rows and columns that are
// padding carry +inf norms and can never hit (:259).
//
// Pass 1 turns the warp's share of the tile row into hit bit masks (4 chunks x 32 columns per thread).  Only if
// some thread of the warp has a hit does pass 2 run: one warp scan of the per-thread counts, ONE
// atomicAdd on the found counter per warp and tile, then every thread writes its records to
// consecutive slots -- the reference does two atomics per pair (source/pair.cuh:123-133).  Overflow
// keeps its rule: found counts everything, records beyond the capacity are dropped (the host
// derives stored = min(found, capacity)).
//
// Symmetric mode keeps columns c >= q and emits, for c > q, the mirrored record (c, q) as well.
__device__ __forceinline__ void epilogue_tile(const JoinParams& p, uint32_t taddr, const float* cn, float sq, int q,
                                              int c_base, int lane) {
    // taddr, cn and c_base already point at this warp's first column.
    constexpr int kChunks = kEpiCols / 32;
    uint32_t hit[kChunks];
    uint32_t mir[kChunks];
    uint32_t cnt = 0;
    // Two register buffers: while chunk ch is tested, the load of chunk ch + 1 is in flight.
    uint32_t va[32], vb[32];
    ptx::tmem_ld_32x32b_x32(taddr, va);
#pragma unroll
    for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t(&v)[32] = (ch & 1) ? vb : va;
        uint32_t(&w)[32] = (ch & 1) ? va : vb;
        ptx::tmem_ld_wait_for(v);
        if (ch + 1 < kChunks) ptx::tmem_ld_32x32b_x32(taddr + (ch + 1) * 32, w);
        // Fast reject: the smallest d2 of the chunk; the candidate norms come as 16-byte broadcast
        // loads.  NaNs drop out of fminf, so a NaN never hits.
        const float4* cn4 = reinterpret_cast<const float4*>(cn + ch * 32);
        float lo = __int_as_float(0x7f800000);
        const uint64_t sq2 = ptx::pack_f32x2(sq, sq);
        const uint64_t m2 = ptx::pack_f32x2(-2.0f, -2.0f);
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
            // two elements per instruction: t = s_q + s_c, d2 = fma(a, -2, t) (== t - 2a: 2a is exact)
            const float4 c4 = cn4[j4];
            const uint64_t t01 = ptx::add_f32x2(sq2, ptx::pack_f32x2(c4.x, c4.y));
            const uint64_t t23 = ptx::add_f32x2(sq2, ptx::pack_f32x2(c4.z, c4.w));
            const uint64_t a01 = ptx::pack_f32x2(__uint_as_float(v[4 * j4 + 0]), __uint_as_float(v[4 * j4 + 1]));
            const uint64_t a23 = ptx::pack_f32x2(__uint_as_float(v[4 * j4 + 2]), __uint_as_float(v[4 * j4 + 3]));
            float d0, d1, d2, d3;
            ptx::unpack_f32x2(ptx::fma_f32x2(a01, m2, t01), d0, d1);
            ptx::unpack_f32x2(ptx::fma_f32x2(a23, m2, t23), d2, d3);
            lo = ptx::min3_f32(ptx::min3_f32(lo, d0, d1), d2, d3);
        }
        uint32_t mask = 0;
        if (lo <= p.eps2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float d2 = (sq + cn[ch * 32 + j]) - 2.0f * __uint_as_float(v[j]);
                if (d2 <= p.eps2) mask |= (1u << j);
            }
        }
        uint32_t mirror = 0;
        if (p.symmetric) {
            const int rel = q - (c_base + ch * 32);  // column index inside the chunk that equals q
            const uint32_t keep = rel <= 0 ? 0xffffffffu : (rel >= 32 ? 0u : (0xffffffffu << rel));
            const uint32_t above = rel < 0 ? 0xffffffffu : (rel >= 31 ? 0u : (0xffffffffu << (rel + 1)));
            mirror = mask & above;
            mask &= keep;
        }
        hit[ch] = mask;
        mir[ch] = mirror;
        cnt += __popc(mask) + __popc(mirror);
    }
    if (!__any_sync(0xffffffffu, cnt != 0)) return;

    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    unsigned long long base = 0;
    if (lane == 0) base = atomicAdd(p.counters + 0, static_cast<unsigned long long>(total));
    base = __shfl_sync(0xffffffffu, base, 0);
    unsigned long long slot = base + (incl - cnt);
    const unsigned long long qkey = static_cast<unsigned long long>(static_cast<uint32_t>(q)) << 32;
    const unsigned long long qlow = static_cast<unsigned long long>(static_cast<uint32_t>(q));

    if (p.dist2 == nullptr) {
#pragma unroll 1
        for (int ch = 0; ch < kChunks; ++ch) {
            // (dynamic register indexing is avoided by rotating the arrays)
            uint32_t m = hit[0], r = mir[0];
#pragma unroll
            for (int k = 0; k + 1 < kChunks; ++k) {
                hit[k] = hit[k + 1];
                mir[k] = mir[k + 1];
            }
            const uint32_t c0 = static_cast<uint32_t>(c_base + ch * 32);
            while (m) {
                const int j = __ffs(m) - 1;
                m &= m - 1;
                if (slot < p.capacity) p.keys[slot] = qkey | static_cast<unsigned long long>(c0 + j);
                ++slot;
            }
            while (r) {
                const int j = __ffs(r) - 1;
                r &= r - 1;
                if (slot < p.capacity) p.keys[slot] = (static_cast<unsigned long long>(c0 + j) << 32) | qlow;
                ++slot;
            }
        }
    } else {
        // Distances wanted too: read the accumulator chunk again where the warp has hits.
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
            const uint32_t m = hit[ch], r = mir[ch];
            if (!__any_sync(0xffffffffu, (m | r) != 0)) continue;
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(taddr + ch * 32, v);
            ptx::tmem_ld_wait_for(v);
            const uint32_t c0 = static_cast<uint32_t>(c_base + ch * 32);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if ((m | r) & (1u << j)) {
                    const float d2 = p.raw_dot ? __uint_as_float(v[j])
                                               : (sq + cn[ch * 32 + j]) - 2.0f * __uint_as_float(v[j]);
                    if (m & (1u << j)) {
                        if (slot < p.capacity) {
                            p.keys[slot] = qkey | static_cast<unsigned long long>(c0 + j);
                            p.dist2[slot] = d2;
                        }
                        ++slot;
                    }
                    if (r & (1u << j)) {
                        if (slot < p.capacity) {
                            p.keys[slot] = (static_cast<unsigned long long>(c0 + j) << 32) | qlow;
                            p.dist2[slot] = d2;
                        }
                        ++slot;
                    }
                }
            }
        }
    }
}

struct JoinSmemAux {
    unsigned long long full_bar[kStages];
    unsigned long long empty_bar[kStages];
    unsigned long long acc_full_bar[2];
    unsigned long long acc_empty_bar[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float cand_norms[2][kTileN];
};

constexpr int kJoinSmemBytes = kStages * kStageBytes + 1024 + static_cast<int>(sizeof(JoinSmemAux)) + 64;

__global__ void __launch_bounds__(kJoinThreads, 1)
join_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const JoinParams p) {
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
                const int row_b = tn * kTileN;
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
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long it = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p), ++it) {
                const int buf = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_empty_bar[buf]), acc_phase ^ 1u, abort_flag,
                                            kWaitLimitNs);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kTileN);
                for (int ks = 0; ks < p.k_steps; ++ks) {
                    ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->full_bar[stage]), phase, abort_flag,
                                                kWaitLimitNs);
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
        }
    } else {
        // ------------------------- Epilogue -----------------------------
        const int quarter = warp & 3;               // TMEM lane quarter this warp may access
        const int col_off = ((warp - 2) >> 2) * kEpiCols;  // this warp's share of the tile's columns
        const int row_in_tile = quarter * 32 + lane;
        const int epi_tid = threadIdx.x - 64;       // 0..255
        const float inf = __int_as_float(0x7f800000);
        bool ok = true;
        long long it = 0;
        // The tile's norms (one candidate norm per epilogue thread, this thread's query norm) are
        // fetched one tile ahead, so their global-memory latency hides behind the previous tile.
        // Padding rows and columns get +inf and can never hit.
        static_assert(kEpiThreads == kTileN, "one candidate norm per epilogue thread");
        auto fetch_norms = [&](const TileIter& t, float& cand, float& query) {
            const int c = t.tn * kTileN + epi_tid;
            const int qq = p.q_begin + t.tm * kTileM + row_in_tile;
            cand = (c < p.n) ? __ldg(p.norms + c) : inf;
            query = (qq < p.q_end) ? __ldg(p.norms + qq) : inf;
        };
        TileIter ti;
        ti.init(p, first_tile, tile_step);
        float next_cand = inf, next_query = inf;
        if (ti.valid) fetch_norms(ti, next_cand, next_query);
        for (; ti.valid; ++it) {
            const int tm = ti.tm, tn = ti.tn;
            const int buf = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const int q = p.q_begin + tm * kTileM + row_in_tile;
            const int c_base = tn * kTileN;

            float* cn = aux->cand_norms[buf];
            cn[epi_tid] = next_cand;
            const float sq = next_query;
            ptx::named_bar_sync(1, kEpiThreads);
            ti.advance(p);
            if (ti.valid) fetch_norms(ti, next_cand, next_query);

            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_full_bar[buf]), acc_phase, abort_flag,
                                                kWaitLimitNs);
            if (!ok) continue;  // keep taking part in the named barrier, do nothing else
            ptx::tc_fence_after_sync();

            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN);
            epilogue_tile(p, taddr + col_off, cn + col_off, sq, q, c_base + col_off, lane);
            // Hand the accumulator back to the MMA warp.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&aux->acc_empty_bar[buf]));
        }
        if (!ok && lane == 0) atomicOr(p.counters + 2, kErrEpilogueWait);
    }

    // Teardown: everyone meets, then the allocating warp frees TMEM.
    ptx::tc_fence_before_sync();
    __syncthreads();
    // SM cycles CTA 0 spent on its share of the tiles: lets the host derive the mean SM clock of the
    // launch (cycles / device time) and the share of those cycles the tensor pipe had work for.
    if (blockIdx.x == 0 && threadIdx.x == 0) p.counters[4] = static_cast<unsigned long long>(clock64() - clock_start);
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
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
    alignas(16) float cand_norms[2][kTileN];
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
                const int row_b = tn * kTileN + static_cast<int>(rank) * (kTileN / 2);
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
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long it = 0;
            TileIter ti;
            for (ti.init(p, first_tile, tile_step); ti.valid && ok; ti.advance(p), ++it) {
                const int buf = static_cast<int>(it & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_empty_bar[buf]), acc_phase ^ 1u, abort_flag,
                                            kWaitLimitNs);
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
        const int col_off = ((warp - 2) >> 2) * kEpiCols;
        const int row_in_tile = quarter * 32 + lane;
        const int epi_tid = threadIdx.x - 64;
        const float inf = __int_as_float(0x7f800000);
        bool ok = true;
        long long it = 0;
        // The tile's norms (one candidate norm per epilogue thread, this thread's query norm) are
        // fetched one tile ahead, so their global-memory latency hides behind the previous tile.
        // Padding rows and columns get +inf and can never hit.
        static_assert(kEpiThreads == kTileN, "one candidate norm per epilogue thread");
        auto fetch_norms = [&](const TileIter& t, float& cand, float& query) {
            const int c = t.tn * kTileN + epi_tid;
            const int qq = p.q_begin + t.tm * kPairTileM + static_cast<int>(rank) * kTileM + row_in_tile;
            cand = (c < p.n) ? __ldg(p.norms + c) : inf;
            query = (qq < p.q_end) ? __ldg(p.norms + qq) : inf;
        };
        TileIter ti;
        ti.init(p, first_tile, tile_step);
        float next_cand = inf, next_query = inf;
        if (ti.valid) fetch_norms(ti, next_cand, next_query);
        for (; ti.valid; ++it) {
            const int tm = ti.tm, tn = ti.tn;
            const int buf = static_cast<int>(it & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const int q = p.q_begin + tm * kPairTileM + static_cast<int>(rank) * kTileM + row_in_tile;
            const int c_base = tn * kTileN;

            float* cn = aux->cand_norms[buf];
            cn[epi_tid] = next_cand;
            const float sq = next_query;
            ptx::named_bar_sync(1, kEpiThreads);
            ti.advance(p);
            if (ti.valid) fetch_norms(ti, next_cand, next_query);

            if (ok) ok = ptx::mbar_wait_bounded(ptx::smem_u32(&aux->acc_full_bar[buf]), acc_phase, abort_flag,
                                                kWaitLimitNs);
            if (!ok) continue;
            ptx::tc_fence_after_sync();

            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN);
            epilogue_tile(p, taddr + col_off, cn + col_off, sq, q, c_base + col_off, lane);
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster_addr(ptx::mapa_u32(ptx::smem_u32(&aux->acc_empty_bar[buf]), 0));
        }
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

// Sorted packed keys -> {int query; int candidate} records, the reference's
// Pair layout (source/pair.cuh:27-30).
__global__ void unpack_pairs_kernel(const unsigned long long* __restrict__ keys, int2* __restrict__ out,
                                    unsigned long long count) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += stride) {
        const unsigned long long k = keys[i];
        out[i] = make_int2(static_cast<int>(k >> 32), static_cast<int>(k & 0xffffffffull));
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
