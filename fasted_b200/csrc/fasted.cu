// Context API of the B200 epsilon self-join (layer 2 of include/fasted.h):
// device memory, TMA tensor maps, kernel launches, timing, sort and egress.
#include "fasted.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <sched.h>

#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <string>
#include <vector>

#include <dlfcn.h>
#include <nccl.h>  // types and prototypes only: the library is bound at run time (see NcclApi)

#include <cub/device/device_radix_sort.cuh>

#include "kernels.cuh"

#include "error.hpp"

namespace fasted {
thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}
}  // namespace fasted

namespace {
using fasted::fail;

#define CU_TRY(expr)                                                                                 \
    do {                                                                                             \
        cudaError_t e_ = (expr);                                                                     \
        if (e_ != cudaSuccess)                                                                       \
            return fail(FASTED_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, \
                        __LINE__);                                                                   \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

}  // namespace

struct fasted_ctx {
    int device = 0;
    int num_sms = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;

    // dataset
    __half* points = nullptr;
    bool owns_points = false;
    int64_t n = 0, d = 0, ld = 0;
    float* norms = nullptr;
    int64_t norms_cap = 0;
    bool norms_valid = false;
    CUtensorMap map_a{}, map_b{};

    // results
    unsigned long long* counters = nullptr;  // found, stored, status, spare
    unsigned long long* keys = nullptr;      // device-order packed pairs
    unsigned long long* keys_alt = nullptr;  // sort double buffer; reused for the unpacked records
    float* dist = nullptr;
    float* dist_alt = nullptr;
    uint64_t capacity = 0;
    bool have_dist_buf = false;
    void* sort_tmp = nullptr;
    size_t sort_tmp_bytes = 0;
    uint64_t stored = 0;
    void* result_pairs = nullptr;  // int2 records of the last join
    bool unpack_pending = false;   // the last join left packed records in `keys` (device order); they are
                                   // turned into int2 records when somebody asks for them
    unsigned long long* counters_host = nullptr;  // pinned mirror of the counter block
    float* result_dist = nullptr;
    bool result_sorted = false;

    cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};

    // egress pipeline of fasted_join_stream: a chunk's sort and its device-to-host copy run on
    // streams of their own (highest priority) while the next chunks are being joined
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> chunk_ev;            // end of each chunk's join launch
    std::vector<cudaEvent_t> sorted_ev;           // end of each chunk's sort + unpack
    std::vector<cudaEvent_t> copied_ev;           // end of each chunk's device-to-host copy
    std::vector<cudaEvent_t> sort_t0, sort_t1;    // timing brackets of the sorts
    cudaEvent_t ev_tail = nullptr, ev_copied[2] = {nullptr, nullptr};
    int stream_key32 = 1;                          // option: 32-bit records where they fit
    double density_hint = 0.0;                     // records per query row of the last join ...
    int64_t hint_n = 0, hint_d = 0;                // ... on a dataset of this shape (a re-upload of the same shape keeps it)
    unsigned long long* chunk_end_host = nullptr;  // pinned: the found counter after each chunk
    size_t chunk_end_cap = 0;
    int stream_chunk_bands = 0;                    // option: raster bands per chunk (0 = automatic)
    int stream_sort_batch = 16;                    // option: chunks whose records one sort may take together
    int query_stationary = -1;                     // option: -1 automatic, 0 never, 1 whenever the rows are short enough
    int use_pdl = 1;                               // option: let the join start while the norm kernel still runs

    // pinned staging for transfers from / to pageable host memory
    void* stage_buf[2] = {nullptr, nullptr};
    cudaEvent_t stage_ev[2] = {nullptr, nullptr};

    // options
    int band_tiles = 0;  // 0 = chosen per dataset (default_band_tiles)
    int grid = 0;
    int cta_pair = 0;  // 1: CTA-pair kernel (256 x 256 tiles on 2-CTA clusters)
    int exact_norms = 0;  // 1: correctly rounded norms instead of the reference's round-toward-zero chain
    int max_pair_clusters = 0;
};

constexpr int kCounterWords = 16;  // found, -, status, self-test, and CTA 0's cycle counters (see JoinParams::counters)

struct JoinPlan {
    fasted::JoinParams p;
    int grid;
    bool pair;
    bool astat;      // query-stationary kernel (short rows)
    int smem_bytes;  // its dynamic shared memory
};

namespace {

constexpr int kMaxDynamicSmem = 227 * 1024;  // per-block limit of sm_100
constexpr int kAStatAutoMinStages = 3;       // automatic choice: query-stationary when its ring has at least this depth

// Depth of the query-stationary kernel's candidate ring for rows of k_steps K steps (0: does not fit).
int astat_stages_for(int k_steps) {
    if (k_steps > fasted::kAStatMaxK) return 0;
    int s = fasted::kAStatMaxStages;
    while (s > 0 && fasted::astat_smem_bytes(k_steps, s) > kMaxDynamicSmem) --s;
    return s;
}

int make_map(fasted_ctx* c, CUtensorMap* map, int box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(FASTED_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(c->d), static_cast<cuuint64_t>(c->n)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(c->ld) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(fasted::kTileK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, c->points, gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FASTED_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FASTED_OK;
}

void release_points(fasted_ctx* c) {
    if (c->owns_points && c->points) cudaFree(c->points);
    c->points = nullptr;
    c->owns_points = false;
    c->n = c->d = c->ld = 0;
    c->norms_valid = false;
}

int adopt_points(fasted_ctx* c, __half* dev, bool owns, int64_t n, int64_t d, int64_t ld) {
    c->points = dev;
    c->owns_points = owns;
    c->n = n;
    c->d = d;
    c->ld = ld;
    c->norms_valid = false;
    c->stored = 0;
    c->result_pairs = nullptr;
    c->unpack_pending = false;
    if (c->norms_cap < n) {
        if (c->norms) cudaFree(c->norms);
        c->norms = nullptr;
        c->norms_cap = 0;
        CU_TRY(cudaMalloc(&c->norms, static_cast<size_t>(n) * sizeof(float)));
        c->norms_cap = n;
    }
    int rc = make_map(c, &c->map_a, fasted::kTileM);
    if (rc) return rc;
    return make_map(c, &c->map_b, fasted::kTileN);
}

// Tile rows (128 query rows each) per raster band.  16 rows x 9.25 columns is the near-square block of
// 148 concurrent tiles that touches the fewest distinct bytes per K step.  Measured under the power cap:
// on 1,000,000 x 4096 (6.5 s joins, alternating) 16 -> 1298, 24 -> 1259, 32 -> 1235 TFLOPS, although 32
// halves the DRAM traffic; on 262144 x 4096 (0.4 s joins, alternating) 16 -> 1345, 32 -> 1385, 36 -> 1405,
// 37 -> 1209 (148 CTAs = 37 x 4: every wave starts on a column boundary and all CTAs miss at once).
// The long-run optimum is kept; for rows wider than 8 KB the band shrinks so that its query rows stay
// within 16 MB of L2.
int default_band_tiles(int64_t ld) {
    const int64_t row_block_bytes = 128 * ld * 2;
    const int64_t fit = (int64_t(17) << 20) / std::max<int64_t>(row_block_bytes, 1);
    return static_cast<int>(std::max<int64_t>(4, std::min<int64_t>(16, fit)));
}

int check_shape(int64_t n, int64_t d) {
    if (n <= 0 || d <= 0) return fail(FASTED_EINVAL, "n and d must be positive (n=%lld d=%lld)", (long long)n, (long long)d);
    if (n > 0x7fffffffLL - 1024 || d > 0x7fffffffLL - 1024)
        return fail(FASTED_EINVAL, "n and d must fit a 32-bit index (n=%lld d=%lld)", (long long)n, (long long)d);
    return FASTED_OK;
}

void free_pair_buffers(fasted_ctx* c) {
    if (c->keys) cudaFree(c->keys);
    if (c->keys_alt) cudaFree(c->keys_alt);
    if (c->dist) cudaFree(c->dist);
    if (c->dist_alt) cudaFree(c->dist_alt);
    if (c->sort_tmp) cudaFree(c->sort_tmp);
    c->keys = c->keys_alt = nullptr;
    c->dist = c->dist_alt = nullptr;
    c->sort_tmp = nullptr;
    c->sort_tmp_bytes = 0;
    c->capacity = 0;
    c->have_dist_buf = false;
    c->stored = 0;
    c->result_pairs = nullptr;
    c->result_dist = nullptr;
    c->unpack_pending = false;
}

// ---- transfers through pinned staging ---------------------------------------------------------
//
// A cudaMemcpy from or to pageable memory is staged by the driver chunk by chunk without overlap.
// Here two pinned 64 MiB buffers alternate: while the DMA engine moves one, the host threads fill or
// drain the other (the reference copies straight from its std::vector, source/findPairs.cuh:578-579,
// and straight into one, source/pair.cuh:139-146).  Pinned or registered user memory skips all this.
constexpr size_t kStageBytes = size_t(64) << 20;

bool host_is_pinned(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeManaged;
}

cudaError_t ensure_staging(fasted_ctx* c) {
    for (int i = 0; i < 2; ++i) {
        if (!c->stage_buf[i]) {
            cudaError_t e = cudaMallocHost(&c->stage_buf[i], kStageBytes);
            if (e != cudaSuccess) return e;
        }
        if (!c->stage_ev[i]) {
            cudaError_t e = cudaEventCreateWithFlags(&c->stage_ev[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

void parallel_copy(void* dst, const void* src, size_t bytes) {
    const size_t piece = size_t(4) << 20;
    const long long pieces = static_cast<long long>((bytes + piece - 1) / piece);
#pragma omp parallel for schedule(static) if (pieces > 1)
    for (long long i = 0; i < pieces; ++i) {
        const size_t off = static_cast<size_t>(i) * piece;
        std::memcpy(static_cast<char*>(dst) + off, static_cast<const char*>(src) + off, std::min(piece, bytes - off));
    }
}

// rows x row_bytes from host (pitch src_pitch) to device (pitch dst_pitch).
cudaError_t upload_rows(fasted_ctx* c, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                        size_t rows) {
    // (a single row wider than a staging buffer also takes the plain copy)
    if (host_is_pinned(src) || rows * row_bytes < (size_t(8) << 20) || row_bytes > kStageBytes)
        return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyHostToDevice, c->stream);
    cudaError_t e = ensure_staging(c);
    if (e != cudaSuccess) return e;
    const size_t rows_per_chunk = kStageBytes / row_bytes;  // >= 1: wider rows took the plain copy above
    int which = 0;
    for (size_t r0 = 0; r0 < rows; r0 += rows_per_chunk, which ^= 1) {
        const size_t nr = std::min(rows_per_chunk, rows - r0);
        e = cudaEventSynchronize(c->stage_ev[which]);  // the DMA that last read this buffer is done
        if (e != cudaSuccess) return e;
        const char* s = static_cast<const char*>(src) + r0 * src_pitch;
        if (src_pitch == row_bytes) {
            parallel_copy(c->stage_buf[which], s, nr * row_bytes);
        } else {
#pragma omp parallel for schedule(static)
            for (long long r = 0; r < static_cast<long long>(nr); ++r)
                std::memcpy(static_cast<char*>(c->stage_buf[which]) + static_cast<size_t>(r) * row_bytes,
                            s + static_cast<size_t>(r) * src_pitch, row_bytes);
        }
        e = cudaMemcpy2DAsync(static_cast<char*>(dst) + r0 * dst_pitch, dst_pitch, c->stage_buf[which], row_bytes,
                              row_bytes, nr, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) return e;
        e = cudaEventRecord(c->stage_ev[which], c->stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// bytes from device to host; returns after the data is in dst.
cudaError_t download_bytes(fasted_ctx* c, void* dst, const void* src, size_t bytes, cudaStream_t stream) {
    if (host_is_pinned(dst) || bytes < (size_t(8) << 20)) {
        cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream);
        return e != cudaSuccess ? e : cudaStreamSynchronize(stream);
    }
    cudaError_t e = ensure_staging(c);
    if (e != cudaSuccess) return e;
    const size_t chunks = (bytes + kStageBytes - 1) / kStageBytes;
    for (size_t i = 0; i <= chunks; ++i) {
        if (i < chunks) {  // start chunk i
            const size_t off = i * kStageBytes, nb = std::min(kStageBytes, bytes - off);
            e = cudaMemcpyAsync(c->stage_buf[i & 1], static_cast<const char*>(src) + off, nb, cudaMemcpyDeviceToHost,
                                stream);
            if (e != cudaSuccess) return e;
            e = cudaEventRecord(c->stage_ev[i & 1], stream);
            if (e != cudaSuccess) return e;
        }
        if (i > 0) {  // drain chunk i - 1 while chunk i is on its way
            const size_t off = (i - 1) * kStageBytes, nb = std::min(kStageBytes, bytes - off);
            e = cudaEventSynchronize(c->stage_ev[(i - 1) & 1]);
            if (e != cudaSuccess) return e;
            parallel_copy(static_cast<char*>(dst) + off, c->stage_buf[(i - 1) & 1], nb);
        }
    }
    return cudaSuccess;
}

// Device memory for a new dataset.  Pair buffers only ever grow, so if the dataset does not fit
// beside them they are released (the next join sizes them again) and the allocation is retried.
cudaError_t alloc_points(fasted_ctx* c, __half** dev, size_t bytes) {
    cudaError_t e = cudaMalloc(dev, bytes);
    if (e == cudaErrorMemoryAllocation && c->capacity > 0) {
        cudaGetLastError();
        free_pair_buffers(c);
        e = cudaMalloc(dev, bytes);
    }
    return e;
}

int ensure_pair_buffers(fasted_ctx* c, uint64_t capacity, bool want_dist) {
    // Buffers only grow: probes with a tiny capacity (epsilon search) must not throw away the
    // buffers of the full join that follows.
    if (c->capacity >= capacity && (!want_dist || c->have_dist_buf)) return FASTED_OK;
    const uint64_t cap = std::max<uint64_t>(std::max<uint64_t>(capacity, c->capacity), 1);
    free_pair_buffers(c);
    CU_TRY(cudaMalloc(&c->keys, cap * 8));
    CU_TRY(cudaMalloc(&c->keys_alt, cap * 8));
    if (want_dist) {
        CU_TRY(cudaMalloc(&c->dist, cap * 4));
        CU_TRY(cudaMalloc(&c->dist_alt, cap * 4));
    }
    c->capacity = cap;
    c->have_dist_buf = want_dist;
    return FASTED_OK;
}

}  // namespace

extern "C" {

const char* fasted_last_error(void) { return fasted::g_last_error.c_str(); }

int fasted_create(int device, fasted_ctx** out) {
    if (!out) return fail(FASTED_EINVAL, "out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(FASTED_ENODEV, "no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(FASTED_EINVAL, "device %d out of range (%d devices)", device, count);
    cudaDeviceProp prop;
    CU_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(FASTED_ENODEV, "device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major,
                    prop.minor);
    CU_TRY(cudaSetDevice(device));
    fasted_ctx* c = new fasted_ctx();
    c->device = device;
    c->num_sms = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete c;
        return fail(FASTED_ECUDA, "cudaStreamCreate failed");
    }
    c->owns_stream = true;
    for (auto& ev : c->ev) {
        if (cudaEventCreate(&ev) != cudaSuccess) {
            ev = nullptr;
            fasted_destroy(c);
            return fail(FASTED_ECUDA, "cudaEventCreate failed");
        }
    }
    if (cudaMalloc(&c->counters, kCounterWords * sizeof(unsigned long long)) != cudaSuccess ||
        cudaMallocHost(&c->counters_host, kCounterWords * sizeof(unsigned long long)) != cudaSuccess) {
        fasted_destroy(c);
        return fail(FASTED_ECUDA, "allocation of the counters failed");
    }
    cudaFuncSetAttribute(fasted::join_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fasted::kJoinSmemBytes);
    cudaFuncSetAttribute(fasted::row_norms_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         fasted::kNormSmemBytes);
    cudaFuncSetAttribute(fasted::row_norms_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         fasted::kNormSmemBytes);
    cudaFuncSetAttribute(fasted::join_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         fasted::kPairSmemBytes);
    cudaFuncSetAttribute(fasted::join_astat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
    // All kernels of a join ask for the same split of the SM's L1 / shared memory (all of it shared): a
    // kernel that needs another split than its predecessor makes every SM drain and reconfigure first,
    // which a 30-microsecond join cannot afford between its norm kernel, its join kernel and the next call.
    cudaFuncSetAttribute(fasted::join_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::join_astat_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::join_pair_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::row_norms_kernel<0>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::row_norms_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::unpack_pairs_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(fasted::unpack_pairs32_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    {
        // How many 2-CTA clusters of the pair kernel the device can hold at once.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * c->num_sms);
        cfg.blockDim = dim3(fasted::kJoinThreads);
        cfg.dynamicSmemBytes = fasted::kPairSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, fasted::join_pair_kernel, &cfg) == cudaSuccess && clusters > 0)
            c->max_pair_clusters = clusters;
        else
            c->max_pair_clusters = c->num_sms / 2;
        cudaGetLastError();
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        fasted_destroy(c);
        return fail(FASTED_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    }
    *out = c;
    return FASTED_OK;
}

void fasted_destroy(fasted_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    release_points(c);
    free_pair_buffers(c);
    if (c->norms) cudaFree(c->norms);
    if (c->counters) cudaFree(c->counters);
    if (c->counters_host) cudaFreeHost(c->counters_host);
    for (auto& ev : c->ev)
        if (ev) cudaEventDestroy(ev);
    for (int i = 0; i < 2; ++i) {
        if (c->stage_buf[i]) cudaFreeHost(c->stage_buf[i]);
        if (c->stage_ev[i]) cudaEventDestroy(c->stage_ev[i]);
    }
    for (auto* list : {&c->chunk_ev, &c->sorted_ev, &c->copied_ev, &c->sort_t0, &c->sort_t1})
        for (cudaEvent_t ev : *list)
            if (ev) cudaEventDestroy(ev);
    if (c->ev_tail) cudaEventDestroy(c->ev_tail);
    for (auto& ev : c->ev_copied)
        if (ev) cudaEventDestroy(ev);
    if (c->chunk_end_host) cudaFreeHost(c->chunk_end_host);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->owns_stream && c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

int fasted_set_stream(fasted_ctx* c, void* stream) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    if (c->owns_stream && c->stream) {
        cudaStreamSynchronize(c->stream);
        cudaStreamDestroy(c->stream);
    }
    c->stream = static_cast<cudaStream_t>(stream);
    c->owns_stream = false;
    return FASTED_OK;
}

int fasted_set_option(fasted_ctx* c, const char* name, int64_t value) {
    if (!c || !name) return fail(FASTED_EINVAL, "null argument");
    if (!strcmp(name, "band_tiles")) {
        if (value < 0 || value > 4096) return fail(FASTED_EINVAL, "band_tiles out of range");
        c->band_tiles = static_cast<int>(value);
    } else if (!strcmp(name, "exact_norms")) {
        if (value != 0 && value != 1) return fail(FASTED_EINVAL, "exact_norms must be 0 or 1");
        if (c->exact_norms != static_cast<int>(value)) c->norms_valid = false;
        c->exact_norms = static_cast<int>(value);
    } else if (!strcmp(name, "cta_pair")) {
        if (value != 0 && value != 1) return fail(FASTED_EINVAL, "cta_pair must be 0 or 1");
        c->cta_pair = static_cast<int>(value);
    } else if (!strcmp(name, "dependent_launch")) {
        if (value != 0 && value != 1) return fail(FASTED_EINVAL, "dependent_launch must be 0 or 1");
        c->use_pdl = static_cast<int>(value);
    } else if (!strcmp(name, "query_stationary")) {
        if (value < -1 || value > 1) return fail(FASTED_EINVAL, "query_stationary must be -1, 0 or 1");
        c->query_stationary = static_cast<int>(value);
    } else if (!strcmp(name, "stream_key32")) {
        if (value != 0 && value != 1) return fail(FASTED_EINVAL, "stream_key32 must be 0 or 1");
        c->stream_key32 = static_cast<int>(value);
    } else if (!strcmp(name, "stream_sort_batch")) {
        if (value < 1 || value > 1024) return fail(FASTED_EINVAL, "stream_sort_batch must be 1..1024");
        c->stream_sort_batch = static_cast<int>(value);
    } else if (!strcmp(name, "stream_chunk_bands")) {
        if (value < 0 || value > (1 << 20)) return fail(FASTED_EINVAL, "stream_chunk_bands out of range");
        c->stream_chunk_bands = static_cast<int>(value);
    } else if (!strcmp(name, "grid")) {
        if (value < 0 || value > 65535) return fail(FASTED_EINVAL, "grid out of range");
        c->grid = static_cast<int>(value);
    } else {
        return fail(FASTED_EINVAL, "unknown option '%s'", name);
    }
    return FASTED_OK;
}

int fasted_set_points_host_f16(fasted_ctx* c, const uint16_t* host, int64_t n, int64_t d, int64_t ld_host) {
    if (!c || !host) return fail(FASTED_EINVAL, "null argument");
    int rc = check_shape(n, d);
    if (rc) return rc;
    if (ld_host < d) return fail(FASTED_EINVAL, "ld_host (%lld) < d (%lld)", (long long)ld_host, (long long)d);
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    const int64_t ld = (d + fasted::kTileK - 1) / fasted::kTileK * fasted::kTileK;
    __half* dev = nullptr;
    if (c->owns_points && c->points && c->n * c->ld == n * ld) {
        // Same footprint as the resident dataset (the run / run-again cycle of a parameter sweep):
        // keep the allocation, cudaFree + cudaMalloc would stall the whole device for nothing.
        dev = c->points;
        c->points = nullptr;
        c->owns_points = false;
    }
    release_points(c);
    if (!dev) CU_TRY(alloc_points(c, &dev, static_cast<size_t>(n) * ld * 2));
    cudaError_t e = cudaSuccess;
    if (ld != d) e = cudaMemsetAsync(dev, 0, static_cast<size_t>(n) * ld * 2, c->stream);
    if (e == cudaSuccess)
        e = upload_rows(c, dev, static_cast<size_t>(ld) * 2, host, static_cast<size_t>(ld_host) * 2,
                        static_cast<size_t>(d) * 2, static_cast<size_t>(n));
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return fail(FASTED_ECUDA, "upload of points failed: %s", cudaGetErrorString(e));
    }
    return adopt_points(c, dev, true, n, d, ld);
}

int fasted_set_points_device_f16(fasted_ctx* c, const void* dev, int64_t n, int64_t d, int64_t ld) {
    if (!c || !dev) return fail(FASTED_EINVAL, "null argument");
    int rc = check_shape(n, d);
    if (rc) return rc;
    if (ld < d || (ld % 8) != 0) return fail(FASTED_EINVAL, "ld (%lld) must be >= d and a multiple of 8", (long long)ld);
    if (reinterpret_cast<uintptr_t>(dev) % 16 != 0) return fail(FASTED_EINVAL, "device pointer must be 16-byte aligned");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    release_points(c);
    return adopt_points(c, static_cast<__half*>(const_cast<void*>(dev)), false, n, d, ld);
}

int fasted_copy_points_from(fasted_ctx* dst, fasted_ctx* src) {
    if (!dst || !src || dst == src) return fail(FASTED_EINVAL, "bad argument");
    if (!src->points) return fail(FASTED_ESTATE, "the source context has no dataset");
    CU_TRY(cudaSetDevice(dst->device));
    CU_TRY(cudaStreamSynchronize(dst->stream));
    release_points(dst);
    if (dst->device != src->device) {
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, dst->device, src->device) == cudaSuccess && can) {
            cudaError_t pe = cudaDeviceEnablePeerAccess(src->device, 0);
            if (pe != cudaSuccess) cudaGetLastError();  // already enabled is fine; the copy works either way
        }
    }
    const size_t bytes = static_cast<size_t>(src->n) * src->ld * 2;
    __half* dev = nullptr;
    CU_TRY(alloc_points(dst, &dev, bytes));
    cudaError_t e = cudaMemcpyPeerAsync(dev, dst->device, src->points, src->device, bytes, dst->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dst->stream);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return fail(FASTED_ECUDA, "peer copy of points failed: %s", cudaGetErrorString(e));
    }
    return adopt_points(dst, dev, true, src->n, src->d, src->ld);
}

// ---------------------------------------------------------------------------
// Replication of the dataset over the GPUs of one process: one NCCL broadcast
// ---------------------------------------------------------------------------
//
// The candidate set is the only thing the GPUs share, and it is replicated by one collective: a
// broadcast from the GPU that holds it (a ring / tree over NVLink moves every byte out of the root
// once, where G - 1 peer copies that all read the root would queue on its egress links).  NCCL is
// bound at run time (dlopen of libnccl.so.2) so that the library still loads, and every single-GPU
// path still works, where NCCL is not installed; a process that already holds an NCCL (the one a
// Python framework bundles) gets that same copy.  The communicators are created once per set of
// devices with ncclCommInitAll (one process, several GPUs) and kept for the life of the process.
namespace {
struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclCommInitAll) CommInitAll = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclBroadcast) Broadcast = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
};

NcclApi& nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (api.handle) {
            api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(dlsym(api.handle, "ncclCommInitAll"));
            api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(dlsym(api.handle, "ncclGroupStart"));
            api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(dlsym(api.handle, "ncclGroupEnd"));
            api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(dlsym(api.handle, "ncclBroadcast"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
            api.ok = api.CommInitAll && api.GroupStart && api.GroupEnd && api.Broadcast && api.GetErrorString;
        }
    }
    return api;
}

struct NcclGroup {
    std::vector<int> devices;
    std::vector<ncclComm_t> comms;
};
std::vector<NcclGroup> g_nccl_groups;  // one per distinct device list, never destroyed
}  // namespace

int fasted_broadcast_points(fasted_ctx* const* ctxs, int count, double* ms_out) {
    if (!ctxs || count < 1) return fail(FASTED_EINVAL, "bad argument");
    for (int g = 0; g < count; ++g)
        if (!ctxs[g]) return fail(FASTED_EINVAL, "context %d is null", g);
    fasted_ctx* src = ctxs[0];
    if (!src->points) return fail(FASTED_ESTATE, "the first context has no dataset");
    if (ms_out) *ms_out = 0.0;
    if (count == 1) return FASTED_OK;
    std::vector<int> devices(count);
    for (int g = 0; g < count; ++g) {
        devices[g] = ctxs[g]->device;
        for (int h = 0; h < g; ++h)
            if (devices[h] == devices[g])
                return fail(FASTED_EINVAL, "contexts %d and %d share device %d: a broadcast needs one GPU per context", h, g,
                            devices[g]);
    }
    NcclApi& api = nccl_api();
    if (!api.ok) return fail(FASTED_ENODEV, "NCCL (libnccl.so.2) is not available: %s", api.handle ? "symbols missing" : dlerror());
    NcclGroup* grp = nullptr;
    for (auto& g : g_nccl_groups)
        if (g.devices == devices) grp = &g;
    if (!grp) {
        NcclGroup ng;
        ng.devices = devices;
        ng.comms.resize(count);
        ncclResult_t r = api.CommInitAll(ng.comms.data(), count, devices.data());
        if (r != ncclSuccess) return fail(FASTED_ECUDA, "ncclCommInitAll failed: %s", api.GetErrorString(r));
        g_nccl_groups.push_back(std::move(ng));
        grp = &g_nccl_groups.back();
    }
    const size_t bytes = static_cast<size_t>(src->n) * src->ld * 2;
    std::vector<__half*> dst(count, nullptr);
    dst[0] = src->points;
    for (int g = 1; g < count; ++g) {
        CU_TRY(cudaSetDevice(ctxs[g]->device));
        CU_TRY(cudaStreamSynchronize(ctxs[g]->stream));
        release_points(ctxs[g]);
        cudaError_t e = alloc_points(ctxs[g], &dst[g], bytes);
        if (e != cudaSuccess) {
            for (int h = 1; h < g; ++h) {
                cudaSetDevice(ctxs[h]->device);
                cudaFree(dst[h]);
            }
            return fail(FASTED_ECUDA, "allocation of the replica on device %d failed: %s", ctxs[g]->device,
                        cudaGetErrorString(e));
        }
    }
    CU_TRY(cudaSetDevice(src->device));
    CU_TRY(cudaStreamSynchronize(src->stream));
    const double t0 = [] {
        timespec ts;
        clock_gettime(CLOCK_MONOTONIC, &ts);
        return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
    }();
    ncclResult_t r = api.GroupStart();
    for (int g = 0; g < count && r == ncclSuccess; ++g) {
        cudaSetDevice(ctxs[g]->device);
        r = api.Broadcast(dst[g], dst[g], bytes, ncclUint8, 0, grp->comms[g], ctxs[g]->stream);
    }
    const ncclResult_t r2 = api.GroupEnd();
    if (r == ncclSuccess) r = r2;
    cudaError_t e = cudaSuccess;
    for (int g = 0; g < count; ++g) {
        cudaSetDevice(ctxs[g]->device);
        const cudaError_t eg = cudaStreamSynchronize(ctxs[g]->stream);
        if (e == cudaSuccess) e = eg;
    }
    if (r != ncclSuccess || e != cudaSuccess) {
        for (int g = 1; g < count; ++g) {
            cudaSetDevice(ctxs[g]->device);
            cudaFree(dst[g]);
        }
        return r != ncclSuccess ? fail(FASTED_ECUDA, "ncclBroadcast failed: %s", api.GetErrorString(r))
                                : fail(FASTED_ECUDA, "broadcast of the points failed: %s", cudaGetErrorString(e));
    }
    if (ms_out) {
        timespec ts;
        clock_gettime(CLOCK_MONOTONIC, &ts);
        *ms_out = ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6 - t0;
    }
    for (int g = 1; g < count; ++g) {
        CU_TRY(cudaSetDevice(ctxs[g]->device));
        int rc = adopt_points(ctxs[g], dst[g], true, src->n, src->d, src->ld);
        if (rc) return rc;
    }
    return FASTED_OK;
}

int fasted_generate_exponential(fasted_ctx* c, int64_t n, int64_t d, double lambda, double max_value, uint64_t seed) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    int rc = check_shape(n, d);
    if (rc) return rc;
    if (!(lambda > 0) || !(max_value > 0)) return fail(FASTED_EINVAL, "lambda and max_value must be positive");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    release_points(c);
    const int64_t ld = (d + fasted::kTileK - 1) / fasted::kTileK * fasted::kTileK;
    __half* dev = nullptr;
    CU_TRY(alloc_points(c, &dev, static_cast<size_t>(n) * ld * 2));
    fasted::gen_exponential_kernel<<<c->num_sms * 8, 256, 0, c->stream>>>(dev, n, static_cast<int>(d),
                                                                          static_cast<int>(ld), lambda, max_value, seed);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return fail(FASTED_ECUDA, "generator kernel failed: %s", cudaGetErrorString(e));
    }
    return adopt_points(c, dev, true, n, d, ld);
}

int fasted_fill_exponential_device(fasted_ctx* c, void* dev, int64_t n, int64_t d, int64_t ld, double lambda,
                                   double max_value, uint64_t seed) {
    if (!c || !dev) return fail(FASTED_EINVAL, "null argument");
    int rc = check_shape(n, d);
    if (rc) return rc;
    if (ld < d || (ld % 8) != 0 || reinterpret_cast<uintptr_t>(dev) % 16 != 0)
        return fail(FASTED_EINVAL, "ld must be >= d and a multiple of 8, dev 16-byte aligned");
    if (!(lambda > 0) || !(max_value > 0)) return fail(FASTED_EINVAL, "lambda and max_value must be positive");
    CU_TRY(cudaSetDevice(c->device));
    fasted::gen_exponential_kernel<<<c->num_sms * 8, 256, 0, c->stream>>>(
        static_cast<__half*>(dev), n, static_cast<int>(d), static_cast<int>(ld), lambda, max_value, seed);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(c->stream));
    return FASTED_OK;
}

int fasted_points_info(fasted_ctx* c, void** dev, int64_t* n, int64_t* d, int64_t* ld) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (dev) *dev = c->points;
    if (n) *n = c->n;
    if (d) *d = c->d;
    if (ld) *ld = c->ld;
    return FASTED_OK;
}

int fasted_get_points_host_f16(fasted_ctx* c, uint16_t* host, int64_t ld_host) {
    if (!c || !host) return fail(FASTED_EINVAL, "null argument");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (ld_host < c->d) return fail(FASTED_EINVAL, "ld_host < d");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaMemcpy2DAsync(host, static_cast<size_t>(ld_host) * 2, c->points, static_cast<size_t>(c->ld) * 2,
                             static_cast<size_t>(c->d) * 2, static_cast<size_t>(c->n), cudaMemcpyDeviceToHost,
                             c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    return FASTED_OK;
}

int fasted_get_rows_host_f16(fasted_ctx* c, const int64_t* rows, int64_t count, uint16_t* host, int64_t ld_host) {
    if (!c || !rows || !host || count < 0) return fail(FASTED_EINVAL, "bad argument");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (ld_host < c->d) return fail(FASTED_EINVAL, "ld_host < d");
    CU_TRY(cudaSetDevice(c->device));
    for (int64_t i = 0; i < count; ++i) {
        if (rows[i] < 0 || rows[i] >= c->n) return fail(FASTED_EINVAL, "row %lld out of range", (long long)rows[i]);
        CU_TRY(cudaMemcpyAsync(host + i * ld_host, c->points + rows[i] * c->ld, static_cast<size_t>(c->d) * 2,
                               cudaMemcpyDeviceToHost, c->stream));
    }
    CU_TRY(cudaStreamSynchronize(c->stream));
    return FASTED_OK;
}

// Row norms of rows [row_begin, row_end) (row_begin a multiple of 128; the whole matrix by default).
static int launch_norms(fasted_ctx* c, int64_t row_begin = 0, int64_t row_end = -1) {
    if (row_end < 0 || row_end > c->n) row_end = c->n;
    if (row_begin >= row_end) return FASTED_OK;
    const int first_block = static_cast<int>(row_begin / fasted::kNormRows);
    const int row_blocks = static_cast<int>((row_end + fasted::kNormRows - 1) / fasted::kNormRows) - first_block;
    const int k_boxes = static_cast<int>((c->d + fasted::kTileK - 1) / fasted::kTileK);
    const int grid = std::min(row_blocks, c->num_sms * 3);
    if (c->exact_norms)
        fasted::row_norms_kernel<1><<<grid, fasted::kNormRows, fasted::kNormSmemBytes, c->stream>>>(
            c->map_a, c->norms, static_cast<int>(c->n), k_boxes, row_blocks, first_block, c->counters + 2);
    else
        fasted::row_norms_kernel<0><<<grid, fasted::kNormRows, fasted::kNormSmemBytes, c->stream>>>(
            c->map_a, c->norms, static_cast<int>(c->n), k_boxes, row_blocks, first_block, c->counters + 2);
    CU_TRY(cudaGetLastError());
    return FASTED_OK;
}

int fasted_row_norms(fasted_ctx* c, double* ms) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaMemsetAsync(c->counters, 0, kCounterWords * sizeof(unsigned long long), c->stream));
    CU_TRY(cudaEventRecord(c->ev[0], c->stream));
    int rc = launch_norms(c);
    if (rc) return rc;
    CU_TRY(cudaEventRecord(c->ev[1], c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    unsigned long long status = 0;
    CU_TRY(cudaMemcpy(&status, c->counters + 2, 8, cudaMemcpyDeviceToHost));
    if (status) return fail(FASTED_EKERNEL, "row-norm kernel gave up a wait (status 0x%llx)", status);
    if (ms) {
        float t = 0;
        cudaEventElapsedTime(&t, c->ev[0], c->ev[1]);
        *ms = t;
    }
    c->norms_valid = true;
    return FASTED_OK;
}

int fasted_get_norms(fasted_ctx* c, float* host_out) {
    if (!c || !host_out) return fail(FASTED_EINVAL, "null argument");
    if (!c->norms_valid) return fail(FASTED_ESTATE, "row norms have not been computed");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaMemcpyAsync(host_out, c->norms, static_cast<size_t>(c->n) * 4, cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    return FASTED_OK;
}

// ---------------------------------------------------------------------------
// The join: planning, launch, results
// ---------------------------------------------------------------------------

// The reference's sizing rule for the pair buffer: n * 256 pairs, reduced to what fits in free
// memory (source/findPairs.cuh:642-647, source/pair.cuh:69-91).
static int default_capacity(fasted_ctx* c, bool want_dist, uint64_t* out) {
    uint64_t capacity = static_cast<uint64_t>(c->n) * 256ull;
    if (c->capacity < capacity) {
        size_t free_b = 0, total_b = 0;
        CU_TRY(cudaMemGetInfo(&free_b, &total_b));
        free_b += c->capacity * (c->have_dist_buf ? 24 : 16);
        const uint64_t per_pair = want_dist ? 24 + 2 : 16 + 2;  // keys x2 (+ dist x2) + sort scratch slack
        const uint64_t fit = static_cast<uint64_t>(free_b * 0.9) / per_pair;
        if (capacity > fit) capacity = fit;
    }
    *out = capacity;
    return FASTED_OK;
}

// Kernel parameters and grid of one launch over query rows [q_begin, q_end).
static int plan_join(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                     int shard_rank, int shard_world, JoinPlan* out, int cand_tile_columns = 0) {
    // cand_tile_columns > 0: the launch joins against that many 256-row candidate tiles (a subset of the rows
    // that the caller describes with JoinParams::cand_t and its companions) instead of all ceil(n / 256)
    const bool want_dist = (flags & FASTED_JOIN_DIST2) != 0;
    fasted::JoinParams p{};
    p.norms = c->norms;
    p.norms_vec4 = (reinterpret_cast<uintptr_t>(p.norms) & 15u) == 0 ? 1 : 0;
    p.counters = c->counters;
    p.keys = c->keys;
    p.dist2 = want_dist ? c->dist : nullptr;
    p.capacity = capacity;
    const double e2 = eps * eps;
    p.eps2 = e2 > FLT_MAX ? FLT_MAX : static_cast<float>(e2);
    p.n = static_cast<int>(c->n);
    p.q_begin = static_cast<int>(q_begin);
    p.q_end = static_cast<int>(q_end);
    p.k_steps = static_cast<int>((c->d + fasted::kTileK - 1) / fasted::kTileK);
    const bool pair = c->cta_pair != 0;
    const int tile_m = pair ? fasted::kPairTileM : fasted::kTileM;
    const bool symmetric = (flags & FASTED_JOIN_SYMMETRIC) != 0;
    if (symmetric && (q_begin != 0 || q_end != c->n))
        return fail(FASTED_EINVAL, "FASTED_JOIN_SYMMETRIC needs the full query range [0, n)");
    p.tile_m = tile_m;
    p.symmetric = symmetric ? 1 : 0;
    p.shard_rank = shard_rank;
    p.shard_world = shard_world;
    p.raw_dot = (flags & FASTED_JOIN_RAW_DOT) && want_dist ? 1 : 0;
    p.key_shift = 32;
    p.key_qbase = 0;
    p.key32 = 0;
    if (shard_world > 1 && !symmetric) return fail(FASTED_EINVAL, "band snakes are for the symmetric schedule only");
    p.tiles_m = static_cast<int>((q_end - q_begin + tile_m - 1) / tile_m);
    p.tiles_n = cand_tile_columns > 0 ? cand_tile_columns : static_cast<int>((c->n + fasted::kTileN - 1) / fasted::kTileN);
    // band_tiles counts 128-row tile rows; a pair tile is two of them.
    const int band_opt = c->band_tiles > 0 ? c->band_tiles : default_band_tiles(c->ld);
    const int band = pair ? std::max(1, band_opt / 2) : band_opt;
    p.band_tiles = std::max(1, std::min(band, std::max(p.tiles_m, 1)));
    p.total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    int grid;
    out->astat = false;
    out->smem_bytes = 0;
    if (pair) {
        int clusters = c->grid > 0 ? std::max(1, c->grid / 2) : c->max_pair_clusters;
        if (p.total_tiles < clusters) clusters = static_cast<int>(std::max<long long>(p.total_tiles, 1));
        grid = 2 * clusters;
    } else {
        grid = c->grid > 0 ? c->grid : c->num_sms;
        if (p.total_tiles < grid) grid = static_cast<int>(std::max<long long>(p.total_tiles, 1));
        // Short rows: keep the query tile in shared memory and stream candidates only (join_astat_kernel).
        const int stages = astat_stages_for(p.k_steps);
        const bool want = c->query_stationary == 1 || (c->query_stationary < 0 && stages >= kAStatAutoMinStages);
        if (want && stages >= 2 && shard_world <= 1) {
            out->astat = true;
            out->smem_bytes = fasted::astat_smem_bytes(p.k_steps, stages);
            p.astat_stages = stages;
            // rows per band: the largest divisor of the grid up to 40 (37 for 148 CTAs: 37 rows x 4 CTAs each)
            int r = std::min(grid, 40);
            while (grid % r != 0) --r;
            p.astat_rows = r;
        }
    }
    out->p = p;
    out->grid = grid;
    out->pair = pair;
    return FASTED_OK;
}

// after_norms: the launch directly follows the row-norm kernel in the stream; it is then allowed to start
// while that kernel is still running (programmatic dependent launch), its epilogue waits for the norms.
static int launch_join(fasted_ctx* c, const JoinPlan& pl, bool after_norms = false) {
    if (pl.p.total_tiles <= 0) return FASTED_OK;
    if (!pl.pair && after_norms && c->use_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(pl.grid);
        cfg.blockDim = dim3(fasted::kJoinThreads);
        cfg.dynamicSmemBytes = pl.astat ? pl.smem_bytes : fasted::kJoinSmemBytes;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (pl.astat)
            CU_TRY(cudaLaunchKernelEx(&cfg, fasted::join_astat_kernel, c->map_a, c->map_b, pl.p));
        else
            CU_TRY(cudaLaunchKernelEx(&cfg, fasted::join_kernel, c->map_a, c->map_b, pl.p));
        return FASTED_OK;
    }
    if (pl.pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(pl.grid);
        cfg.blockDim = dim3(fasted::kJoinThreads);
        cfg.dynamicSmemBytes = fasted::kPairSmemBytes;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        CU_TRY(cudaLaunchKernelEx(&cfg, fasted::join_pair_kernel, c->map_a, pl.p));
    } else if (pl.astat) {
        fasted::join_astat_kernel<<<pl.grid, fasted::kJoinThreads, pl.smem_bytes, c->stream>>>(c->map_a, c->map_b, pl.p);
        CU_TRY(cudaGetLastError());
    } else {
        fasted::join_kernel<<<pl.grid, fasted::kJoinThreads, fasted::kJoinSmemBytes, c->stream>>>(c->map_a, c->map_b,
                                                                                                 pl.p);
        CU_TRY(cudaGetLastError());
    }
    return FASTED_OK;
}

static int check_join_args(fasted_ctx* c, double eps, int64_t q_begin, int64_t* q_end) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (*q_end < 0) *q_end = c->n;
    if (q_begin < 0 || q_begin > *q_end || *q_end > c->n)
        return fail(FASTED_EINVAL, "query band [%lld, %lld) outside [0, %lld)", (long long)q_begin, (long long)*q_end,
                    (long long)c->n);
    // Only eps*eps is used, as in the reference (source/findPairs.cuh:678): a negative epsilon
    // means the same as its absolute value; NaN is refused.
    if (eps != eps) return fail(FASTED_EINVAL, "epsilon is NaN");
    return FASTED_OK;
}

static void fill_stats(fasted_ctx* c, const JoinPlan& pl, const unsigned long long* h, uint64_t stored,
                       fasted_join_stats* stats) {
    if (!stats) return;
    float t01 = 0, t12 = 0, t02 = 0, t34 = 0;
    cudaEventElapsedTime(&t01, c->ev[0], c->ev[1]);
    cudaEventElapsedTime(&t12, c->ev[1], c->ev[2]);
    cudaEventElapsedTime(&t02, c->ev[0], c->ev[2]);
    cudaEventElapsedTime(&t34, c->ev[3], c->ev[4]);
    stats->pairs_found = h[0];
    stats->pairs_stored = stored;
    stats->norms_ms = t01;
    stats->join_ms = t12;
    stats->kernel_ms = t02;
    stats->sort_ms = t34;
    stats->status = h[2];
    stats->tiles_m = pl.p.tiles_m;
    stats->tiles_n = pl.p.tiles_n;
    stats->grid = pl.grid;
    stats->cta0_cycles = pl.pair ? 0 : h[4];
    stats->cta0_setup_cycles = pl.pair ? 0 : h[5];
    stats->cta0_release_cycles = pl.pair ? 0 : h[6];
    stats->cta0_feed_wait_cycles = pl.pair ? 0 : h[7];
    stats->cta0_acc_wait_cycles = pl.pair ? 0 : h[8];
    stats->cta0_tiles = 0;
    stats->chunks = 1;
    stats->tail_ms = 0;
    if (pl.astat && pl.p.total_tiles > 0) {
        fasted::AStatIter ti;
        for (ti.init(pl.p, 0, pl.grid); ti.valid; ti.advance(pl.p)) ++stats->cta0_tiles;
    } else if (!pl.pair && pl.p.total_tiles > 0) {
        fasted::TileIter ti;
        for (ti.init(pl.p, 0, pl.grid); ti.valid; ti.advance(pl.p)) ++stats->cta0_tiles;
    }
}

static bool symmetric_flag(unsigned flags) { return (flags & FASTED_JOIN_SYMMETRIC) != 0; }

static void set_density_hint(fasted_ctx* c, double records_per_row) {
    c->density_hint = records_per_row;
    c->hint_n = c->n;
    c->hint_d = c->d;
}

static int unpack_blocks(fasted_ctx* c, uint64_t count) {
    return static_cast<int>(std::min<uint64_t>((count + 255) / 256, static_cast<uint64_t>(c->num_sms) * 16));
}

static int join_impl(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                     int shard_rank, int shard_world, fasted_join_stats* stats) {
    int rc = check_join_args(c, eps, q_begin, &q_end);
    if (rc) return rc;
    CU_TRY(cudaSetDevice(c->device));
    const bool want_dist = (flags & FASTED_JOIN_DIST2) != 0;
    if (capacity == 0) {
        rc = default_capacity(c, want_dist, &capacity);
        if (rc) return rc;
    }
    rc = ensure_pair_buffers(c, capacity, want_dist);
    if (rc) return rc;
    JoinPlan pl;
    rc = plan_join(c, eps, q_begin, q_end, capacity, flags, shard_rank, shard_world, &pl);
    if (rc) return rc;

    CU_TRY(cudaMemsetAsync(c->counters, 0, kCounterWords * sizeof(unsigned long long), c->stream));
    CU_TRY(cudaEventRecord(c->ev[0], c->stream));
    // Small joins (a few tiles per CTA) are launch-bound: the join is then launched as a programmatic
    // dependent of the norm kernel, with nothing between the two in the stream, so that its prologue and
    // first tiles overlap the norm kernel.  The two kernels' times can then not be told apart: norms_ms is
    // reported as 0 and join_ms covers both.
    const bool need_norms = !(flags & FASTED_JOIN_KEEP_NORMS) || !c->norms_valid;
    const bool overlap = need_norms && c->use_pdl && !pl.pair && pl.p.total_tiles > 0 &&
                         pl.p.total_tiles <= 8LL * pl.grid;
    if (overlap) CU_TRY(cudaEventRecord(c->ev[1], c->stream));
    if (need_norms) {
        rc = launch_norms(c);
        if (rc) return rc;
    }
    if (!overlap) CU_TRY(cudaEventRecord(c->ev[1], c->stream));
    rc = launch_join(c, pl, overlap);
    if (rc) return rc;
    CU_TRY(cudaEventRecord(c->ev[2], c->stream));
    unsigned long long h[kCounterWords] = {};
    c->stored = 0;
    c->result_pairs = nullptr;
    c->result_dist = nullptr;
    c->unpack_pending = false;

    if (flags & FASTED_JOIN_NO_SORT) {
        // Device order is the result.  The call needs the host once, at its end: the counters come back
        // through a pinned mirror, and the packed records are turned into (query, candidate) records
        // only when somebody asks for them (what a sweep of small joins pays per call is launch and
        // synchronisation latency, not kernel time).
        CU_TRY(cudaEventRecord(c->ev[3], c->stream));
        CU_TRY(cudaEventRecord(c->ev[4], c->stream));
        CU_TRY(cudaMemcpyAsync(c->counters_host, c->counters, sizeof(h), cudaMemcpyDeviceToHost, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
        std::memcpy(h, c->counters_host, sizeof(h));
        c->norms_valid = (h[2] & fasted::kErrNormWait) == 0;
        if (h[2]) return fail(FASTED_EKERNEL, "a device-side wait ran out (status 0x%llx)", h[2]);
        const uint64_t stored = std::min<uint64_t>(h[0], capacity);
        c->stored = stored;
        if (q_end > q_begin && !symmetric_flag(flags)) set_density_hint(c, static_cast<double>(h[0]) / static_cast<double>(q_end - q_begin));
        c->unpack_pending = true;
        c->result_dist = want_dist ? c->dist : nullptr;
        c->result_sorted = false;
        fill_stats(c, pl, h, stored, stats);
        return FASTED_OK;
    }

    CU_TRY(cudaMemcpyAsync(c->counters_host, c->counters, sizeof(h), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    std::memcpy(h, c->counters_host, sizeof(h));
    c->norms_valid = (h[2] & fasted::kErrNormWait) == 0;
    if (h[2]) return fail(FASTED_EKERNEL, "a device-side wait ran out (status 0x%llx)", h[2]);
    // Every record with a slot below the capacity is written, the others are dropped.
    const uint64_t stored = std::min<uint64_t>(h[0], capacity);

    CU_TRY(cudaEventRecord(c->ev[3], c->stream));
    const unsigned long long* sorted_keys = c->keys;
    float* sorted_dist = c->dist;
    if (stored > 1) {
        // Row-major order of (query, candidate) == numeric order of the packed key
        // (replaces thrust::sort with Pair::operator<, source/pair.cuh:39-45, 151-158).
        int end_bit = 33;
        while (end_bit < 64 && (static_cast<uint64_t>(c->n) >> (end_bit - 32)) != 0) ++end_bit;
        cub::DoubleBuffer<unsigned long long> kb(c->keys, c->keys_alt);
        cub::DoubleBuffer<float> vb(c->dist, c->dist_alt);
        size_t need = 0;
        if (want_dist)
            CU_TRY(cub::DeviceRadixSort::SortPairs(nullptr, need, kb, vb, stored, 0, end_bit, c->stream));
        else
            CU_TRY(cub::DeviceRadixSort::SortKeys(nullptr, need, kb, stored, 0, end_bit, c->stream));
        if (need > c->sort_tmp_bytes) {
            if (c->sort_tmp) cudaFree(c->sort_tmp);
            c->sort_tmp = nullptr;
            c->sort_tmp_bytes = 0;
            CU_TRY(cudaMalloc(&c->sort_tmp, need));
            c->sort_tmp_bytes = need;
        }
        if (want_dist)
            CU_TRY(cub::DeviceRadixSort::SortPairs(c->sort_tmp, need, kb, vb, stored, 0, end_bit, c->stream));
        else
            CU_TRY(cub::DeviceRadixSort::SortKeys(c->sort_tmp, need, kb, stored, 0, end_bit, c->stream));
        if (kb.Current() != c->keys) std::swap(c->keys, c->keys_alt);
        if (want_dist && vb.Current() != c->dist) std::swap(c->dist, c->dist_alt);
        sorted_keys = c->keys;
        sorted_dist = c->dist;
    }
    if (stored > 0) {
        fasted::unpack_pairs_kernel<<<unpack_blocks(c, stored), 256, 0, c->stream>>>(
            sorted_keys, reinterpret_cast<int2*>(c->keys_alt), stored, 32, 0);
        CU_TRY(cudaGetLastError());
    }
    CU_TRY(cudaEventRecord(c->ev[4], c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    c->stored = stored;
    if (q_end > q_begin && !symmetric_flag(flags)) set_density_hint(c, static_cast<double>(h[0]) / static_cast<double>(q_end - q_begin));
    c->result_pairs = c->keys_alt;
    c->result_dist = want_dist ? sorted_dist : nullptr;
    c->result_sorted = true;
    fill_stats(c, pl, h, stored, stats);
    return FASTED_OK;
}

int fasted_join(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                fasted_join_stats* stats) {
    return join_impl(c, eps, q_begin, q_end, capacity, flags, 0, 1, stats);
}

int fasted_join_symmetric_shard(fasted_ctx* c, double eps, int shard_rank, int shard_world, uint64_t capacity,
                                unsigned flags, fasted_join_stats* stats) {
    if (shard_world < 1 || shard_rank < 0 || shard_rank >= shard_world) return fail(FASTED_EINVAL, "bad shard");
    return join_impl(c, eps, 0, -1, capacity, flags | FASTED_JOIN_SYMMETRIC, shard_rank, shard_world, stats);
}

// ---------------------------------------------------------------------------
// The join with pipelined egress
// ---------------------------------------------------------------------------
//
// The reference sorts the whole pair list after its kernel and then copies it to the host
// (source/findPairs.cuh:699-716, source/pair.cuh:139-158): three serial phases.  Here the query range
// is cut into chunks of whole raster bands, one join launch per chunk.  The launches share one found
// counter, so chunk k's records occupy the slots between the counter's value after chunk k-1 and
// after chunk k; and because chunks are contiguous, ascending ranges of query rows, the chunks' sorted
// lists laid end to end ARE the global row-major order.
//
// Stream order on the join stream:  join(0) join(1) sort(0) join(2) sort(1) join(3) ...
// The host stays two launches ahead: when chunk k's launch retires (an event and a pinned copy of the
// counter tell it how many records the chunk has) it enqueues sort(k) -- a radix sort over only the
// slice's significant bits, then the unpacking to (query, candidate) records -- behind join(k+1),
// which is already running, and then join(k+2).  The sort of a chunk therefore runs on an otherwise
// idle GPU between two launches (a persistent join CTA fills its SM, nothing fits beside it), costs
// what a sort of that slice costs and nothing more, and the GPU never waits for the host.  The
// device-to-host copy of chunk k runs on a copy stream while the GPU joins chunk k+2.  When the last
// launch retires, only the last chunk's sort and copy are still to come.
//
// Records are packed relative to the chunk: ((query - first row of the chunk) << bits(n)) |
// candidate.  Where that fits 32 bits (n up to a few million points with chunks of a thousand rows
// and more) the kernel writes 32-bit records: half the bytes to write, sort and read back.

static int ensure_stream_pipeline(fasted_ctx* c, size_t chunks) {
    if (!c->copy_stream) {
        int lo = 0, hi = 0;
        CU_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        CU_TRY(cudaStreamCreateWithPriority(&c->copy_stream, cudaStreamNonBlocking, hi));
        CU_TRY(cudaEventCreate(&c->ev_tail));
        for (auto& ev : c->ev_copied) CU_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    }
    while (c->chunk_ev.size() < chunks) {
        cudaEvent_t ev = nullptr, sorted = nullptr, copied = nullptr, t0 = nullptr, t1 = nullptr;
        CU_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        CU_TRY(cudaEventCreateWithFlags(&sorted, cudaEventDisableTiming));
        CU_TRY(cudaEventCreateWithFlags(&copied, cudaEventDisableTiming));
        c->copied_ev.push_back(copied);
        CU_TRY(cudaEventCreate(&t0));
        CU_TRY(cudaEventCreate(&t1));
        c->chunk_ev.push_back(ev);
        c->sorted_ev.push_back(sorted);
        c->sort_t0.push_back(t0);
        c->sort_t1.push_back(t1);
    }
    if (c->chunk_end_cap < chunks + kCounterWords) {
        if (c->chunk_end_host) cudaFreeHost(c->chunk_end_host);
        c->chunk_end_host = nullptr;
        c->chunk_end_cap = 0;
        CU_TRY(cudaMallocHost(&c->chunk_end_host, (chunks + kCounterWords) * sizeof(unsigned long long)));
        c->chunk_end_cap = chunks + kCounterWords;
    }
    return FASTED_OK;
}

static int bits_of(uint64_t v) {  // number of bits needed to write v (at least 1)
    int b = 1;
    while (b < 64 && (v >> b) != 0) ++b;
    return b;
}

// The chunk plan of a streamed join over query rows [q_begin, q_end): chunks of whole raster bands.
// min_chunks = 0: about 64 chunks, each at least about a millisecond of tensor work (one GPU).  A
// larger min_chunks (ranks that share the chunks want many small ones, so that the last chunk a rank
// takes is a small part of its work) is honoured down to one band per chunk.  Never more rows than
// 32-bit records can number, where one band's rows can be.
struct ChunkPlan {
    int64_t band_rows, chunk_rows;
    uint64_t chunks;
    int key_shift;
    bool fits32;  // a chunk's rows can be numbered by a 32-bit record
};

static int plan_chunks(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t min_chunks, ChunkPlan* out) {
    JoinPlan whole;
    int rc = plan_join(c, eps, q_begin, q_end, 1, 0, 0, 1, &whole);
    if (rc) return rc;
    const int64_t band_rows = whole.astat ? static_cast<int64_t>(whole.p.astat_rows) * whole.p.tile_m
                                          : static_cast<int64_t>(whole.p.band_tiles) * whole.p.tile_m;
    const int64_t rows = q_end - q_begin;
    const int64_t total_bands = std::max<int64_t>(1, (rows + band_rows - 1) / band_rows);
    const int key_shift = bits_of(static_cast<uint64_t>(std::max<int64_t>(c->n - 1, 1)));
    const int64_t rows32 = key_shift < 32 ? (int64_t(1) << (32 - key_shift)) : 0;
    int64_t bands_per_chunk = c->stream_chunk_bands;
    if (bands_per_chunk <= 0) {
        const double min_rows = 2e12 / (2.0 * static_cast<double>(c->n) * static_cast<double>(c->ld));
        const int64_t want_chunks = std::max<int64_t>(64, static_cast<int64_t>(min_chunks));
        bands_per_chunk = (total_bands + want_chunks - 1) / want_chunks;
        if (min_chunks == 0)
            bands_per_chunk = std::max<int64_t>(bands_per_chunk,
                                                static_cast<int64_t>(std::ceil(min_rows / static_cast<double>(band_rows))));
        // Dense outputs (the last join on this dataset stored 128 records per row or more): chunks small
        // enough for 32-bit records, which halve the sort's traffic.  Sparse outputs: fewer, larger chunks,
        // because a sort of a small slice is all launch overhead.
        if (rows32 >= band_rows && c->density_hint >= 128.0 && c->hint_n == c->n && c->hint_d == c->d)
            bands_per_chunk = std::min<int64_t>(bands_per_chunk, rows32 / band_rows);
    }
    bands_per_chunk = std::max<int64_t>(1, std::min<int64_t>(bands_per_chunk, total_bands));
    out->band_rows = band_rows;
    out->chunk_rows = bands_per_chunk * band_rows;
    out->chunks = static_cast<uint64_t>((rows + out->chunk_rows - 1) / out->chunk_rows);
    out->key_shift = key_shift;
    out->fits32 = out->chunk_rows <= rows32;
    return FASTED_OK;
}

// ---- chunks shared by the ranks of one node ----------------------------------------------------
//
// One process per GPU, all holding the same dataset: instead of giving every rank one fixed band of
// query rows, the ranks take CHUNKS from a common counter, each whenever its join stream has room for
// another launch.  A GPU that runs faster (each sits under its own power cap) simply takes more
// chunks, so all ranks finish within one chunk of each other; and since chunk k's place in the global
// list is the sum of the record counts of chunks 0 .. k-1 -- which other ranks publish at about the
// time chunk k itself retires -- every rank can copy its chunks straight to their final position in
// one shared host buffer while the join is still running.  The table lives in memory that all ranks
// map (a shared file mapping); it is the only thing the ranks exchange during the join: no collective.
struct SharedChunks {
    uint64_t magic;
    int64_t q_begin, q_end, chunk_rows;
    // One group: chunk k is rows [q_begin + k * chunk_rows, ...).  Several groups (the bands in which the
    // matrix reaches the GPUs, one per rank): every group is cut into chunks_per_group chunks from its own
    // first row, and the first lead_chunks chunks of group g are not handed out: rank g joins them itself,
    // piece by piece, while the rest of the matrix is still arriving (their rows are the first it holds).
    int64_t group_rows;
    uint64_t groups, chunks_per_group, lead_chunks;
    uint64_t chunks;               // ids: groups * chunks_per_group, ascending with the rows they cover
    std::atomic<uint64_t> next;    // chunks handed out so far (only those that are handed out count)
    std::atomic<uint64_t> failed;  // a rank gave up: everybody stops waiting
    std::atomic<uint64_t> found_total, stored_total;
    std::atomic<uint64_t> count[1];  // records stored for chunk k; kUnknownCount until its rank publishes it
};
constexpr uint64_t kSharedMagic = 0x46615354454464ull;
constexpr uint64_t kUnknownCount = ~0ull;
static_assert(sizeof(std::atomic<uint64_t>) == sizeof(uint64_t), "lock-free 64-bit atomics expected");

// Rows of chunk `id` (an empty range, begin == end, lies beyond the data).
static void shared_chunk_range(const SharedChunks* t, uint64_t id, int64_t* begin, int64_t* end) {
    const uint64_t g = id / t->chunks_per_group, i = id % t->chunks_per_group;
    const int64_t base = t->groups > 1 ? static_cast<int64_t>(g) * t->group_rows : t->q_begin;
    const int64_t group_end = t->groups > 1 ? std::min<int64_t>(t->q_end, base + t->group_rows) : t->q_end;
    const int64_t b = base + static_cast<int64_t>(i) * t->chunk_rows;
    *begin = std::min<int64_t>(b, std::max<int64_t>(group_end, std::min<int64_t>(base, t->q_end)));
    *end = std::max<int64_t>(*begin, std::min<int64_t>(group_end, b + t->chunk_rows));
}

int64_t fasted_shared_chunks_take(void* mem);
int fasted_shared_chunks_publish(void* mem, uint64_t chunk, uint64_t stored, uint64_t found);

static int join_stream_core(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                            int32_t* pairs_host, float* dist2_host, uint64_t host_capacity, fasted_chunk_fn on_chunk,
                            void* user, SharedChunks* shared, const fasted_arrival* arr, fasted_join_stats* stats) {
    int rc = check_join_args(c, eps, q_begin, &q_end);
    if (rc) return rc;
    if (arr && (!shared || arr->pieces < 1 || arr->groups < 1 || arr->group_rows <= 0 ||
                arr->group_rows % (256 * static_cast<int64_t>(arr->pieces)) != 0 || arr->own_begin < 0 ||
                arr->own_begin % arr->group_rows != 0 ||
                static_cast<int64_t>(arr->groups) * arr->group_rows < c->n))
        return fail(FASTED_EINVAL, "bad arrival description (groups x group_rows must cover the matrix, group_rows a "
                                   "multiple of 256 x pieces, own_begin the first row of a group)");
    const bool count_only = shared != nullptr && (flags & FASTED_JOIN_NO_SORT) != 0;
    if (flags & (FASTED_JOIN_SYMMETRIC | FASTED_JOIN_RAW_DOT | (shared ? FASTED_JOIN_DIST2 : FASTED_JOIN_NO_SORT)))
        return fail(FASTED_EINVAL, shared ? "the shared-chunk join takes FASTED_JOIN_NO_SORT and FASTED_JOIN_KEEP_NORMS only"
                                          : "fasted_join_stream takes FASTED_JOIN_DIST2 and FASTED_JOIN_KEEP_NORMS only");
    const bool want_dist = (flags & FASTED_JOIN_DIST2) != 0;
    if (dist2_host && !want_dist) return fail(FASTED_EINVAL, "dist2_host given without FASTED_JOIN_DIST2");
    CU_TRY(cudaSetDevice(c->device));
    if (capacity == 0) {
        rc = default_capacity(c, want_dist, &capacity);
        if (rc) return rc;
    }
    rc = ensure_pair_buffers(c, capacity, want_dist);
    if (rc) return rc;

    JoinPlan whole;
    rc = plan_join(c, eps, q_begin, q_end, capacity, flags & ~FASTED_JOIN_NO_SORT, 0, 1, &whole);
    if (rc) return rc;
    ChunkPlan cp;
    rc = plan_chunks(c, eps, q_begin, q_end, 0, &cp);
    if (rc) return rc;
    if (shared) {
        // the plan every rank follows is the one in the table (made by fasted_shared_chunks_init)
        if (shared->magic != kSharedMagic || shared->q_begin != q_begin || shared->q_end != q_end ||
            shared->chunk_rows <= 0 || shared->chunk_rows % cp.band_rows != 0)
            return fail(FASTED_EINVAL, "the shared chunk table does not belong to this join");
        cp.chunk_rows = shared->chunk_rows;
        cp.chunks = shared->chunks;
        const int64_t rows32 = cp.key_shift < 32 ? (int64_t(1) << (32 - cp.key_shift)) : 0;
        cp.fits32 = cp.chunk_rows <= rows32;
        if (arr && shared->groups > 1 && (shared->group_rows != arr->group_rows || shared->groups != static_cast<uint64_t>(arr->groups)))
            return fail(FASTED_EINVAL, "the shared chunk table was planned for other groups than the arrival describes");
    }
    const int key_shift = cp.key_shift;
    const int64_t chunk_rows = cp.chunk_rows;
    const size_t chunks = static_cast<size_t>(cp.chunks);  // chunks of the whole join (all ranks')
    // The rows this rank joins while the matrix is still arriving: the first lead chunks of its own group,
    // as ONE launch sequence (one launch per arriving piece), hence one slice of records.
    int64_t lead_begin = 0, lead_end = 0;
    uint64_t lead_id = 0;
    if (arr && shared->lead_chunks > 0) {
        lead_id = static_cast<uint64_t>(arr->own_begin / arr->group_rows) * shared->chunks_per_group;
        int64_t b0, e0, b1, e1;
        shared_chunk_range(shared, lead_id, &b0, &e0);
        shared_chunk_range(shared, lead_id + shared->lead_chunks - 1, &b1, &e1);
        lead_begin = b0;
        lead_end = e1;
        if (lead_end - lead_begin > arr->group_rows / arr->pieces)
            return fail(FASTED_EINVAL, "the lead chunks must lie inside the first piece of the rank's own band");
    } else if (shared && shared->lead_chunks > 0) {
        return fail(FASTED_EINVAL, "this chunk table sets lead chunks aside: every rank has to join with its arrival description");
    }
    const int64_t max_rows = std::max<int64_t>(chunk_rows, lead_end - lead_begin);
    const int64_t rows32_all = key_shift < 32 ? (int64_t(1) << (32 - key_shift)) : 0;
    // Two ways to keep the sorts cheap.  Dense output (the last join on this dataset stored 128 records per row
    // or more): one sort per chunk over 32-bit chunk-relative records, half the bytes.  Otherwise a chunk holds so
    // few records that its sort is all launch overhead (and each sort drains the join stream once): records
    // carry absolute rows, and one sort takes the records of up to stream_sort_batch consecutive chunks of this
    // rank, which ascend with the rows, so every chunk's sorted run comes out where its unsorted records were.
    const bool fits_key32 = c->stream_key32 != 0 && cp.fits32 && max_rows <= rows32_all;
    const bool dense = c->density_hint >= 128.0 && c->hint_n == c->n && c->hint_d == c->d;
    const size_t batch_max = (c->stream_sort_batch > 1 && !(dense && fits_key32)) ? static_cast<size_t>(c->stream_sort_batch) : 1;
    const bool key32 = fits_key32 && batch_max == 1;  // one record width per call
    constexpr uint64_t kBatchRecords = 2u << 20;      // a batch is closed early once it holds this many records
    rc = ensure_stream_pipeline(c, chunks + 1);
    if (rc) return rc;
    const int sort_bits = std::min(key32 ? 32 : 64,
                                   key_shift + bits_of(static_cast<uint64_t>(std::max<int64_t>(
                                                   (batch_max > 1 ? static_cast<int64_t>(c->n) : max_rows) - 1, 1))));
    // 32-bit records: both halves of the sort's double buffer live in `keys` (capacity 64-bit words hold
    // 2 x capacity 32-bit ones), the unpacked (query, candidate) records go to `keys_alt`.
    uint32_t* const ping32 = reinterpret_cast<uint32_t*>(c->keys);
    uint32_t* const pong32 = ping32 + capacity;

    // Sort scratch for the largest slice a chunk can have (the library sort's scratch is bounded: it
    // works through long inputs in portions), allocated before anything is enqueued.
    if (!count_only) {
        size_t need = 0;
        cub::DoubleBuffer<float> vb(c->dist, c->dist_alt);
        if (key32) {
            cub::DoubleBuffer<uint32_t> kb(ping32, pong32);
            if (want_dist)
                CU_TRY(cub::DeviceRadixSort::SortPairs(nullptr, need, kb, vb, capacity, 0, sort_bits, c->stream));
            else
                CU_TRY(cub::DeviceRadixSort::SortKeys(nullptr, need, kb, capacity, 0, sort_bits, c->stream));
        } else {
            cub::DoubleBuffer<unsigned long long> kb(c->keys, c->keys_alt);
            if (want_dist)
                CU_TRY(cub::DeviceRadixSort::SortPairs(nullptr, need, kb, vb, capacity, 0, sort_bits, c->stream));
            else
                CU_TRY(cub::DeviceRadixSort::SortKeys(nullptr, need, kb, capacity, 0, sort_bits, c->stream));
        }
        if (need > c->sort_tmp_bytes) {
            if (c->sort_tmp) cudaFree(c->sort_tmp);
            c->sort_tmp = nullptr;
            c->sort_tmp_bytes = 0;
            CU_TRY(cudaMalloc(&c->sort_tmp, need));
            c->sort_tmp_bytes = need;
        }
    }
    if (on_chunk && !pairs_host) {
        cudaError_t e = ensure_staging(c);
        if (e != cudaSuccess) return fail(FASTED_ECUDA, "pinned staging: %s", cudaGetErrorString(e));
    }
    const bool host_pinned = pairs_host && host_is_pinned(pairs_host) && (!dist2_host || host_is_pinned(dist2_host));

    c->stored = 0;
    c->result_pairs = nullptr;
    c->result_dist = nullptr;
    c->unpack_pending = false;
    CU_TRY(cudaMemsetAsync(c->counters, 0, kCounterWords * sizeof(unsigned long long), c->stream));
    CU_TRY(cudaEventRecord(c->ev[0], c->stream));
    if (!arr && (!(flags & FASTED_JOIN_KEEP_NORMS) || !c->norms_valid)) {
        rc = launch_norms(c);
        if (rc) return rc;
    }
    CU_TRY(cudaEventRecord(c->ev[1], c->stream));

    // Launch sequence j of this rank joins rows [begin, end) = chunk `id`: the next in order (one GPU), or the
    // next one nobody has taken yet (chunks shared by several ranks), or this rank's lead chunks.
    struct Entry {
        size_t id;
        int64_t begin, end;
        int64_t qbase;  // the row its records count from
    };
    std::vector<Entry> ids;
    bool has_lead = false;  // ids[0] is this rank's lead
    auto snapshot = [&](size_t j) -> int {
        // (pinned destination: a copy into pageable memory would hold the host until the GPU gets here)
        CU_TRY(cudaMemcpyAsync(c->chunk_end_host + j, c->counters, sizeof(unsigned long long), cudaMemcpyDeviceToHost,
                               c->stream));
        CU_TRY(cudaEventRecord(c->chunk_ev[j], c->stream));
        return FASTED_OK;
    };
    auto enqueue_next_join = [&]() -> int {
        size_t id = ids.size();
        int64_t b = 0, e = 0;
        for (;;) {
            if (shared) {
                const int64_t taken = fasted_shared_chunks_take(shared);
                if (taken < 0) return FASTED_OK;
                id = static_cast<size_t>(taken);
                shared_chunk_range(shared, id, &b, &e);
                if (b < e) break;
                fasted_shared_chunks_publish(shared, id, 0, 0);  // a chunk beyond the data: nothing to join
            } else {
                if (id >= chunks) return FASTED_OK;
                b = q_begin + static_cast<int64_t>(id) * chunk_rows;
                e = std::min<int64_t>(q_end, b + chunk_rows);
                break;
            }
        }
        JoinPlan pl;
        int r = plan_join(c, eps, b, e, capacity, flags & ~FASTED_JOIN_NO_SORT, 0, 1, &pl);
        if (r) return r;
        const int64_t qbase = batch_max > 1 ? 0 : b;
        pl.p.key_shift = key_shift;
        pl.p.key_qbase = static_cast<int>(qbase);
        pl.p.key32 = key32 ? 1 : 0;
        r = launch_join(c, pl);
        if (r) return r;
        r = snapshot(ids.size());
        if (r) return r;
        ids.push_back(Entry{id, b, e, qbase});
        return FASTED_OK;
    };

    if (arr && shared->lead_chunks > 0) {
        // the lead chunks are joined as one sequence: its records are counted under the first id
        for (uint64_t k = lead_end > lead_begin ? 1 : 0; k < shared->lead_chunks; ++k)
            fasted_shared_chunks_publish(shared, lead_id + k, 0, 0);
    }
    if (arr) {
        // The matrix arrives in pieces (piece p = rows [g * B + p * B / P, ...) of every group g).  As soon as a
        // piece is there: its rows' norms, then the lead rows against exactly those candidates.  The launches
        // of the lead sequence are consecutive on the stream, so its records are one slice like any chunk's.
        const int64_t piece_rows = arr->group_rows / arr->pieces;
        for (int pc = 0; pc < arr->pieces; ++pc) {
            if (arr->events && arr->events[pc])
                CU_TRY(cudaStreamWaitEvent(c->stream, static_cast<cudaEvent_t>(arr->events[pc]), 0));
            for (int g = 0; g < arr->groups; ++g) {
                const int64_t r0 = static_cast<int64_t>(g) * arr->group_rows + static_cast<int64_t>(pc) * piece_rows;
                rc = launch_norms(c, r0, r0 + piece_rows);
                if (rc) return rc;
            }
            if (lead_end > lead_begin) {
                JoinPlan pl;
                const int cand_t = static_cast<int>(piece_rows / fasted::kTileN);
                rc = plan_join(c, eps, lead_begin, lead_end, capacity, flags & ~FASTED_JOIN_NO_SORT, 0, 1, &pl,
                               arr->groups * cand_t);
                if (rc) return rc;
                pl.p.key_shift = key_shift;
                pl.p.key_qbase = static_cast<int>(lead_begin);
                pl.p.key32 = key32 ? 1 : 0;
                pl.p.cand_t = cand_t;
                pl.p.cand_group_rows = static_cast<int>(arr->group_rows);
                pl.p.cand_base = static_cast<int>(static_cast<int64_t>(pc) * piece_rows);
                rc = launch_join(c, pl);
                if (rc) return rc;
            }
        }
        if (lead_end > lead_begin) {
            rc = snapshot(0);
            if (rc) return rc;
            ids.push_back(Entry{static_cast<size_t>(lead_id), lead_begin, lead_end, lead_begin});
            has_lead = true;
        }
    }

    constexpr size_t kAhead = 2;  // join launches enqueued beyond the chunk the host is waiting for
    for (size_t k = 0; k < kAhead; ++k) {
        rc = enqueue_next_join();
        if (rc) return rc;
    }

    // Place of a chunk's first record in the list the host receives.  One GPU: the chunk's first slot.
    // Shared chunks: the sum of the counts of all chunks before it, as soon as their ranks have
    // published them (they retire at about the same time as this one; the wait is bounded).
    struct Scan {
        uint64_t upto = 0, prefix = 0;  // prefix = records of chunks [0, upto)
    };
    // (two scans, each moving forward only: the chunks this rank takes come in ascending order, but its lead
    // chunk -- the first thing it joins -- lies behind every chunk of the bands before its own)
    Scan scan_dealt, scan_lead;
    auto advance = [&](Scan& s, size_t id) -> bool {
        while (s.upto < id) {
            const uint64_t v = shared->count[s.upto].load(std::memory_order_acquire);
            if (v == kUnknownCount) return false;
            s.prefix += v;
            ++s.upto;
        }
        return true;
    };
    auto global_offset = [&](Scan& s, size_t id, uint64_t* off) -> int {
        timespec t0;
        clock_gettime(CLOCK_MONOTONIC, &t0);
        for (unsigned spin = 0; !advance(s, id); ++spin) {
            if (shared->failed.load(std::memory_order_acquire)) return fail(FASTED_ESTATE, "another rank gave up its join");
            if ((spin & 1023u) == 1023u) {
                timespec t1;
                clock_gettime(CLOCK_MONOTONIC, &t1);
                if (t1.tv_sec - t0.tv_sec > 120)
                    return fail(FASTED_ESTATE, "chunk %llu was not published within 120 s by the rank that took it",
                                (unsigned long long)s.upto);
                sched_yield();
            }
        }
        *off = s.prefix;
        return FASTED_OK;
    };

    // Delivery of a chunk's sorted records (device slots [a, b)) to the host; runs one chunk behind the
    // sorts so that the host never waits for a copy while it could be feeding the join stream.
    int abort_rc = FASTED_OK;
    struct Pending {
        bool any = false;
        uint64_t a = 0, b = 0;
        size_t j = 0;
        bool copy_enqueued = false;
        bool lead = false;
    } lead_pend;
    std::vector<Pending> pend, now;  // sorted runs to deliver: of the batch before, of the batch closed just now
    auto deliver = [&](const Pending& pd) -> int {
        if (!pd.any) return FASTED_OK;
        const uint64_t a = pd.a, m = pd.b - pd.a;
        const int2* src_pairs = reinterpret_cast<const int2*>(c->keys_alt) + a;
        const float* src_dist = want_dist ? c->dist_alt + a : nullptr;
        uint64_t at = a;  // index of the chunk's first record in the host list
        if (shared) {
            const int r = global_offset(pd.lead ? scan_lead : scan_dealt, ids[pd.j].id, &at);
            if (r) return r;
        }
        if (pairs_host) {
            const uint64_t hm = at < host_capacity ? std::min<uint64_t>(m, host_capacity - at) : 0;
            if (hm == 0) return FASTED_OK;
            if (host_pinned) {
                if (!pd.copy_enqueued) {
                    CU_TRY(cudaMemcpyAsync(pairs_host + 2 * at, src_pairs, hm * 8, cudaMemcpyDeviceToHost, c->copy_stream));
                    if (dist2_host)
                        CU_TRY(cudaMemcpyAsync(dist2_host + at, src_dist, hm * 4, cudaMemcpyDeviceToHost, c->copy_stream));
                    CU_TRY(cudaEventRecord(c->copied_ev[pd.j], c->copy_stream));
                }
                // with nobody to tell, the copy may finish on its own (the end of the call waits for it)
                if (on_chunk) CU_TRY(cudaEventSynchronize(c->copied_ev[pd.j]));
            } else {
                CU_TRY(download_bytes(c, pairs_host + 2 * at, src_pairs, hm * 8, c->copy_stream));
                if (dist2_host) CU_TRY(download_bytes(c, dist2_host + at, src_dist, hm * 4, c->copy_stream));
            }
            if (on_chunk && on_chunk(user, pairs_host + 2 * at, dist2_host ? dist2_host + at : nullptr, at, hm) != 0)
                return fail(FASTED_EINVAL, "the chunk callback asked to stop");
        } else if (on_chunk) {
            // No destination of the caller's: runs of records pass through the two pinned staging
            // buffers; while the callback reads one, the DMA engine fills the other.
            const uint64_t run = (kStageBytes / (want_dist ? 12 : 8)) & ~uint64_t(1023);
            const uint64_t runs = (m + run - 1) / run;
            for (uint64_t i = 0; i <= runs; ++i) {
                if (i < runs) {
                    const uint64_t off = i * run, cnt = std::min(run, m - off);
                    char* buf = static_cast<char*>(c->stage_buf[i & 1]);
                    CU_TRY(cudaMemcpyAsync(buf, src_pairs + off, cnt * 8, cudaMemcpyDeviceToHost, c->copy_stream));
                    if (want_dist)
                        CU_TRY(cudaMemcpyAsync(buf + run * 8, src_dist + off, cnt * 4, cudaMemcpyDeviceToHost,
                                               c->copy_stream));
                    CU_TRY(cudaEventRecord(c->ev_copied[i & 1], c->copy_stream));
                }
                if (i > 0) {
                    const uint64_t off = (i - 1) * run, cnt = std::min(run, m - off);
                    const char* buf = static_cast<const char*>(c->stage_buf[(i - 1) & 1]);
                    CU_TRY(cudaEventSynchronize(c->ev_copied[(i - 1) & 1]));
                    if (on_chunk(user, reinterpret_cast<const int32_t*>(buf),
                                 want_dist ? reinterpret_cast<const float*>(buf + run * 8) : nullptr, at + off, cnt) != 0)
                        return fail(FASTED_EINVAL, "the chunk callback asked to stop");
                }
            }
        }
        return FASTED_OK;
    };
    auto give_up = [&](int code) {
        if (shared) shared->failed.store(1, std::memory_order_release);
        return code;
    };

    uint64_t prev_end = 0;
    size_t sorts = 0;
    size_t batch_first = 0;  // first entry of the open batch
    for (size_t j = 0; j < ids.size(); ++j) {
        CU_TRY(cudaEventSynchronize(c->chunk_ev[j]));
        const uint64_t end_j = c->chunk_end_host[j];
        const uint64_t a = std::min<uint64_t>(prev_end, capacity), b = std::min<uint64_t>(end_j, capacity);
        if (shared) fasted_shared_chunks_publish(shared, ids[j].id, b - a, end_j - prev_end);  // later chunks can be placed
        prev_end = end_j;
        c->chunk_end_host[j] = b;  // (from here on: the entry's last slot, clipped)
        now.clear();
        // The batch [batch_first, j] is closed by its size, by the lead (a batch of its own: its rows do not
        // ascend with the chunks that follow) or by the end of this rank's entries.
        const uint64_t batch_a = batch_first == 0 ? 0 : c->chunk_end_host[batch_first - 1];
        const bool close = j + 1 - batch_first >= batch_max || b - batch_a >= kBatchRecords || (has_lead && j == 0) ||
                           j + 1 == ids.size();
        if (close) {
            if (b > batch_a && abort_rc == FASTED_OK && !count_only) {
                const uint64_t m = b - batch_a;
                const int qbase = static_cast<int>(ids[batch_first].qbase);  // (the same for every entry of a batch)
                // the sort and its unpacking, on the join stream, behind the launch that is running now
                CU_TRY(cudaEventRecord(c->sort_t0[sorts], c->stream));
                cub::DoubleBuffer<float> vb(want_dist ? c->dist + batch_a : nullptr, want_dist ? c->dist_alt + batch_a : nullptr);
                size_t need = c->sort_tmp_bytes;
                if (key32) {
                    cub::DoubleBuffer<uint32_t> kb(ping32 + batch_a, pong32 + batch_a);
                    if (m > 1) {
                        if (want_dist)
                            CU_TRY(cub::DeviceRadixSort::SortPairs(c->sort_tmp, need, kb, vb, m, 0, sort_bits, c->stream));
                        else
                            CU_TRY(cub::DeviceRadixSort::SortKeys(c->sort_tmp, need, kb, m, 0, sort_bits, c->stream));
                    }
                    fasted::unpack_pairs32_kernel<<<unpack_blocks(c, m), 256, 0, c->stream>>>(
                        kb.Current(), reinterpret_cast<int2*>(c->keys_alt + batch_a), m, key_shift, qbase);
                } else {
                    cub::DoubleBuffer<unsigned long long> kb(c->keys + batch_a, c->keys_alt + batch_a);
                    if (m > 1) {
                        if (want_dist)
                            CU_TRY(cub::DeviceRadixSort::SortPairs(c->sort_tmp, need, kb, vb, m, 0, sort_bits, c->stream));
                        else
                            CU_TRY(cub::DeviceRadixSort::SortKeys(c->sort_tmp, need, kb, m, 0, sort_bits, c->stream));
                    }
                    fasted::unpack_pairs_kernel<<<unpack_blocks(c, m), 256, 0, c->stream>>>(
                        kb.Current(), reinterpret_cast<int2*>(c->keys_alt + batch_a), m, key_shift, qbase);
                }
                CU_TRY(cudaGetLastError());
                if (want_dist && vb.Current() != c->dist_alt + batch_a)
                    CU_TRY(cudaMemcpyAsync(c->dist_alt + batch_a, vb.Current(), m * sizeof(float), cudaMemcpyDeviceToDevice,
                                           c->stream));
                CU_TRY(cudaEventRecord(c->sort_t1[sorts], c->stream));
                CU_TRY(cudaEventRecord(c->sorted_ev[j], c->stream));
                ++sorts;
                if (shared) {
                    // every chunk has its own place in the shared list
                    uint64_t ea = batch_a;
                    for (size_t i = batch_first; i <= j; ++i) {
                        const uint64_t eb = c->chunk_end_host[i];
                        if (eb > ea) {
                            Pending pd;
                            pd.any = true;
                            pd.a = ea;
                            pd.b = eb;
                            pd.j = i;
                            now.push_back(pd);
                        }
                        ea = eb;
                    }
                } else {
                    Pending pd;  // one GPU: the batch is one run of the list
                    pd.any = true;
                    pd.a = batch_a;
                    pd.b = b;
                    pd.j = j;
                    now.push_back(pd);
                }
            }
            batch_first = j + 1;
        }
        // keep the join stream fed before anything else
        if (abort_rc == FASTED_OK) {
            rc = enqueue_next_join();
            if (rc) return give_up(rc);
        }
        if (!now.empty()) {
            CU_TRY(cudaStreamWaitEvent(c->copy_stream, c->sorted_ev[j], 0));
            if (!shared && pairs_host && host_pinned) {
                // one GPU: the run's place on the host is its first slot, known already
                Pending& run = now[0];
                const uint64_t hb = std::min<uint64_t>(run.b, host_capacity);
                if (hb > run.a) {
                    CU_TRY(cudaMemcpyAsync(pairs_host + 2 * run.a, reinterpret_cast<const int2*>(c->keys_alt) + run.a,
                                           (hb - run.a) * 8, cudaMemcpyDeviceToHost, c->copy_stream));
                    if (dist2_host)
                        CU_TRY(cudaMemcpyAsync(dist2_host + run.a, c->dist_alt + run.a, (hb - run.a) * 4,
                                               cudaMemcpyDeviceToHost, c->copy_stream));
                }
                CU_TRY(cudaEventRecord(c->copied_ev[j], c->copy_stream));
                run.copy_enqueued = true;
            }
        }
        // the records of the batch before: on the host by now, or nearly
        for (const Pending& pd : pend) {
            if (abort_rc != FASTED_OK) break;
            abort_rc = deliver(pd);
            if (abort_rc != FASTED_OK) give_up(abort_rc);
        }
        pend.clear();
        if (has_lead && j == 0) {
            // The lead's place in the list is known when every chunk of the bands before this rank's has been
            // counted, which is late in the join: its records wait on the device until then, and nothing waits
            // for them (a rank that held back its own later chunks for it would hold up everybody).
            if (!now.empty()) {
                lead_pend = now[0];
                lead_pend.lead = true;
            }
            now.clear();
        }
        pend.swap(now);
        if (lead_pend.any && abort_rc == FASTED_OK && advance(scan_lead, ids[0].id)) {
            abort_rc = deliver(lead_pend);
            if (abort_rc != FASTED_OK) give_up(abort_rc);
            lead_pend.any = false;
        }
    }
    const size_t mine = ids.size();
    CU_TRY(cudaEventRecord(c->ev[2], c->stream));
    unsigned long long* h = c->chunk_end_host + chunks;
    CU_TRY(cudaMemcpyAsync(h, c->counters, kCounterWords * sizeof(unsigned long long), cudaMemcpyDeviceToHost, c->stream));
    for (const Pending& pd : pend) {
        if (abort_rc != FASTED_OK) break;
        abort_rc = deliver(pd);
        if (abort_rc != FASTED_OK) give_up(abort_rc);
    }
    if (abort_rc == FASTED_OK && lead_pend.any) {  // (every chunk this rank took is published: waiting is safe now)
        abort_rc = deliver(lead_pend);
        if (abort_rc != FASTED_OK) give_up(abort_rc);
    }
    CU_TRY(cudaEventRecord(c->ev_tail, c->copy_stream));
    CU_TRY(cudaStreamSynchronize(c->copy_stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    c->norms_valid = (h[2] & fasted::kErrNormWait) == 0;
    if (h[2]) return give_up(fail(FASTED_EKERNEL, "a device-side wait ran out (status 0x%llx)", h[2]));
    if (abort_rc != FASTED_OK) return abort_rc;
    const uint64_t stored = std::min<uint64_t>(h[0], capacity);
    c->stored = stored;
    {
        int64_t my_rows = 0;
        for (const Entry& en : ids) my_rows += en.end - en.begin;
        if (my_rows > 0) set_density_hint(c, static_cast<double>(h[0]) / static_cast<double>(my_rows));
    }
    if (count_only) {
        c->stored = 0;  // a counting run: the (chunk-relative, unsorted) records are not offered afterwards
        c->result_sorted = false;
    } else {
        c->result_pairs = c->keys_alt;  // one GPU: the whole list; shared chunks: this rank's chunks in the order it took them
        c->result_dist = want_dist ? c->dist_alt : nullptr;
        c->result_sorted = shared == nullptr;
    }
    CU_TRY(cudaEventRecord(c->ev[3], c->stream));
    CU_TRY(cudaEventRecord(c->ev[4], c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    fill_stats(c, whole, h, stored, stats);
    if (stats) {
        // ev[1] -> ev[2] spans the join launches AND the sorts that ran between them
        float sort_ms = 0.f, last_sort_ms = 0.f;
        for (size_t i = 0; i < sorts; ++i) {
            float t = 0.f;
            cudaEventElapsedTime(&t, c->sort_t0[i], c->sort_t1[i]);
            sort_ms += t;
            if (i + 1 == sorts) last_sort_ms = t;
        }
        // (what nothing can hide: the last chunk's sort, then whatever of its copy remains after ev[2])
        stats->sort_ms = sort_ms;
        stats->join_ms = std::max(0.0, stats->join_ms - static_cast<double>(sort_ms));
        stats->kernel_ms = stats->norms_ms + stats->join_ms;
        float tail = 0.f;
        if (cudaEventElapsedTime(&tail, c->ev[2], c->ev_tail) != cudaSuccess) tail = 0.f;
        stats->tail_ms = static_cast<double>(last_sort_ms) + std::max(0.f, tail);
        stats->chunks = static_cast<int>(mine);
        if (shared) {  // this rank's share of the tile rows
            int64_t my_rows = 0;
            for (const Entry& en : ids) my_rows += en.end - en.begin;
            stats->tiles_m = static_cast<int>((my_rows + whole.p.tile_m - 1) / whole.p.tile_m);
        }
        stats->cta0_cycles = 0;  // the counter holds the last launch's only
        stats->cta0_tiles = 0;
    }
    return FASTED_OK;
}

int fasted_join_stream(fasted_ctx* c, double eps, int64_t q_begin, int64_t q_end, uint64_t capacity, unsigned flags,
                       int32_t* pairs_host, float* dist2_host, uint64_t host_capacity, fasted_chunk_fn on_chunk,
                       void* user, fasted_join_stats* stats) {
    return join_stream_core(c, eps, q_begin, q_end, capacity, flags, pairs_host, dist2_host, host_capacity, on_chunk, user,
                            nullptr, nullptr, stats);
}

size_t fasted_shared_chunks_bytes(uint64_t max_chunks) {
    return sizeof(SharedChunks) + static_cast<size_t>(max_chunks) * sizeof(uint64_t);
}

int fasted_shared_chunks_init(fasted_ctx* c, void* mem, size_t bytes, double eps, int64_t q_begin, int64_t q_end,
                              int ranks, uint64_t* chunks_out) {
    if (!mem || ranks < 1) return fail(FASTED_EINVAL, "bad argument");
    int rc = check_join_args(c, eps, q_begin, &q_end);
    if (rc) return rc;
    ChunkPlan cp;
    // Many small chunks: the ranks finish within one chunk of each other, so a chunk should be a small
    // part of a rank's share (1/256 where there are bands enough; never less than one raster band, whose
    // sweep over all candidates is what keeps the DRAM traffic low).
    rc = plan_chunks(c, eps, q_begin, q_end, static_cast<uint64_t>(ranks) * 256, &cp);
    if (rc) return rc;
    if (fasted_shared_chunks_bytes(cp.chunks) > bytes)
        return fail(FASTED_EINVAL, "the table needs %zu bytes for %llu chunks, %zu were given", fasted_shared_chunks_bytes(cp.chunks),
                    (unsigned long long)cp.chunks, bytes);
    return fasted_shared_chunks_init_plan(mem, bytes, q_begin, q_end, cp.chunk_rows, 0, 0, chunks_out);
}

int fasted_shared_chunks_init_plan(void* mem, size_t bytes, int64_t q_begin, int64_t q_end, int64_t chunk_rows,
                                   int64_t group_rows, int lead_chunks, uint64_t* chunks_out) {
    if (!mem || q_begin < 0 || q_end < q_begin || chunk_rows <= 0 || group_rows < 0 || lead_chunks < 0)
        return fail(FASTED_EINVAL, "bad argument");
    if (group_rows > 0 && q_begin != 0) return fail(FASTED_EINVAL, "groups need the whole row range [0, n)");
    const int64_t rows = q_end - q_begin;
    const uint64_t groups =
        group_rows > 0 ? static_cast<uint64_t>(std::max<int64_t>(1, (rows + group_rows - 1) / group_rows)) : 1;
    const int64_t per_group = groups > 1 ? group_rows : rows;
    const uint64_t cpg = static_cast<uint64_t>(std::max<int64_t>(1, (per_group + chunk_rows - 1) / chunk_rows));
    if (groups == 1) lead_chunks = 0;
    if (static_cast<uint64_t>(lead_chunks) > cpg) return fail(FASTED_EINVAL, "more lead chunks than a group has");
    const uint64_t chunks = groups * cpg;
    if (fasted_shared_chunks_bytes(chunks) > bytes)
        return fail(FASTED_EINVAL, "the table is too small for %llu chunks", (unsigned long long)chunks);
    SharedChunks* t = static_cast<SharedChunks*>(mem);
    t->q_begin = q_begin;
    t->q_end = q_end;
    t->chunk_rows = chunk_rows;
    t->group_rows = groups > 1 ? group_rows : 0;
    t->groups = groups;
    t->chunks_per_group = cpg;
    t->lead_chunks = static_cast<uint64_t>(lead_chunks);
    t->chunks = chunks;
    t->next.store(0, std::memory_order_relaxed);
    t->failed.store(0, std::memory_order_relaxed);
    t->found_total.store(0, std::memory_order_relaxed);
    t->stored_total.store(0, std::memory_order_relaxed);
    for (uint64_t k = 0; k < chunks; ++k) t->count[k].store(kUnknownCount, std::memory_order_relaxed);
    std::atomic_thread_fence(std::memory_order_release);
    t->magic = kSharedMagic;
    if (chunks_out) *chunks_out = chunks;
    return FASTED_OK;
}

int64_t fasted_shared_chunks_take(void* mem) {
    SharedChunks* t = static_cast<SharedChunks*>(mem);
    if (!t || t->magic != kSharedMagic || t->failed.load(std::memory_order_acquire)) return -1;
    const uint64_t dealt_per_group = t->chunks_per_group - t->lead_chunks;
    const uint64_t v = t->next.fetch_add(1, std::memory_order_acq_rel);
    if (dealt_per_group == 0 || v >= t->groups * dealt_per_group) return -1;
    return static_cast<int64_t>((v / dealt_per_group) * t->chunks_per_group + t->lead_chunks + v % dealt_per_group);
}

int fasted_shared_chunks_range(const void* mem, uint64_t chunk, int64_t* begin, int64_t* end) {
    const SharedChunks* t = static_cast<const SharedChunks*>(mem);
    if (!t || t->magic != kSharedMagic || chunk >= t->chunks || !begin || !end) return fail(FASTED_EINVAL, "bad chunk");
    shared_chunk_range(t, chunk, begin, end);
    return FASTED_OK;
}

int fasted_shared_chunks_publish(void* mem, uint64_t chunk, uint64_t stored, uint64_t found) {
    SharedChunks* t = static_cast<SharedChunks*>(mem);
    if (!t || t->magic != kSharedMagic || chunk >= t->chunks) return fail(FASTED_EINVAL, "bad chunk");
    t->found_total.fetch_add(found, std::memory_order_relaxed);
    t->stored_total.fetch_add(stored, std::memory_order_relaxed);
    t->count[chunk].store(stored, std::memory_order_release);
    return FASTED_OK;
}

int fasted_shared_chunks_offset(void* mem, uint64_t chunk, double timeout_ms, uint64_t* offset_out) {
    SharedChunks* t = static_cast<SharedChunks*>(mem);
    if (!t || t->magic != kSharedMagic || chunk > t->chunks || !offset_out) return fail(FASTED_EINVAL, "bad argument");
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    uint64_t sum = 0;
    for (uint64_t k = 0; k < chunk;) {
        const uint64_t v = t->count[k].load(std::memory_order_acquire);
        if (v != kUnknownCount) {
            sum += v;
            ++k;
            continue;
        }
        if (t->failed.load(std::memory_order_acquire)) return fail(FASTED_ESTATE, "another rank gave up its join");
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        if ((t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6 > timeout_ms)
            return fail(FASTED_ESTATE, "chunk %llu was not published in time", (unsigned long long)k);
        sched_yield();
    }
    *offset_out = sum;
    return FASTED_OK;
}

void fasted_shared_chunks_fail(void* mem) {
    SharedChunks* t = static_cast<SharedChunks*>(mem);
    if (t && t->magic == kSharedMagic) t->failed.store(1, std::memory_order_release);
}

int fasted_shared_chunks_totals(const void* mem, unsigned long long* found_total, unsigned long long* stored_total,
                                unsigned long long* failed) {
    const SharedChunks* t = static_cast<const SharedChunks*>(mem);
    if (!t || t->magic != kSharedMagic) return fail(FASTED_EINVAL, "not a shared chunk table");
    if (found_total) *found_total = t->found_total.load(std::memory_order_acquire);
    if (stored_total) *stored_total = t->stored_total.load(std::memory_order_acquire);
    if (failed) *failed = t->failed.load(std::memory_order_acquire);
    return FASTED_OK;
}

int fasted_join_stream_shared(fasted_ctx* c, double eps, uint64_t capacity, unsigned flags, void* shared_mem,
                              int32_t* pairs_host, uint64_t host_capacity, fasted_join_stats* stats) {
    SharedChunks* t = static_cast<SharedChunks*>(shared_mem);
    if (!t || t->magic != kSharedMagic) return fail(FASTED_EINVAL, "not a shared chunk table");
    return join_stream_core(c, eps, t->q_begin, t->q_end, capacity, flags, pairs_host, nullptr, host_capacity, nullptr,
                            nullptr, t, nullptr, stats);
}

int fasted_shared_chunks_init_arriving(fasted_ctx* c, void* mem, size_t bytes, double eps, int ranks,
                                       const fasted_arrival* arr, uint64_t* chunks_out) {
    if (!mem || ranks < 1 || !arr || arr->pieces < 1 || arr->groups < 1 || arr->group_rows <= 0 ||
        arr->group_rows % (256 * static_cast<int64_t>(arr->pieces)) != 0 || arr->lead_rows < 0)
        return fail(FASTED_EINVAL, "bad argument");
    int64_t q_end = -1;
    int rc = check_join_args(c, eps, 0, &q_end);
    if (rc) return rc;
    if (static_cast<int64_t>(arr->groups) * arr->group_rows < q_end)
        return fail(FASTED_EINVAL, "groups x group_rows must cover the matrix");
    ChunkPlan cp;
    rc = plan_chunks(c, eps, 0, q_end, static_cast<uint64_t>(ranks) * 256, &cp);
    if (rc) return rc;
    // The lead: what a rank joins while the matrix is still on its way.  It has to lie in the first piece of
    // the rank's band (the rows it holds from the start).  By default one twelfth of the band, which outlasts
    // a load over PCIe + NVLink for long rows; where the output is dense (the last join on this dataset
    // stored 128 records per row or more) no more rows than a 32-bit record can number, because wider
    // records would cost the sorts more than the lead hides.
    const int64_t piece_rows = arr->group_rows / arr->pieces;
    int64_t lead_rows = arr->lead_rows > 0 ? arr->lead_rows : arr->group_rows / 12;
    lead_rows = std::min(lead_rows, piece_rows);
    const int64_t rows32 = cp.key_shift < 32 ? (int64_t(1) << (32 - cp.key_shift)) : 0;
    if (cp.fits32 && c->stream_key32 != 0 && c->density_hint >= 128.0 && c->hint_n == c->n && c->hint_d == c->d)
        lead_rows = std::min(lead_rows, rows32);
    const int64_t per_group = std::min<int64_t>(arr->group_rows, q_end);
    const int64_t cpg = std::max<int64_t>(1, (per_group + cp.chunk_rows - 1) / cp.chunk_rows);
    int64_t lead_chunks = arr->groups > 1 ? std::min<int64_t>(lead_rows / cp.chunk_rows, cpg) : 0;
    if (arr->lead_rows == 0 && lead_chunks == 0 && arr->groups > 1 && cp.chunk_rows <= piece_rows) lead_chunks = 1;
    return fasted_shared_chunks_init_plan(mem, bytes, 0, q_end, cp.chunk_rows, arr->groups > 1 ? arr->group_rows : 0,
                                          static_cast<int>(lead_chunks), chunks_out);
}

int fasted_join_stream_arriving(fasted_ctx* c, double eps, uint64_t capacity, unsigned flags, void* shared_mem,
                                const fasted_arrival* arrival, int32_t* pairs_host, uint64_t host_capacity,
                                fasted_join_stats* stats) {
    SharedChunks* t = static_cast<SharedChunks*>(shared_mem);
    if (!t || t->magic != kSharedMagic) return fail(FASTED_EINVAL, "not a shared chunk table");
    if (!arrival) return fail(FASTED_EINVAL, "no arrival description");
    return join_stream_core(c, eps, t->q_begin, t->q_end, capacity, flags, pairs_host, nullptr, host_capacity, nullptr,
                            nullptr, t, arrival, stats);
}

int fasted_tile_schedule(int64_t n, int64_t q_begin, int64_t q_end, int tile_m, int band_tiles, int symmetric,
                         int shard_rank, int shard_world, int grid, int cta, int32_t* tiles_out, int64_t max_tiles,
                         int64_t* count_out) {
    if (n <= 0 || q_begin < 0 || q_end < q_begin || q_end > n || grid <= 0 || cta < 0 || cta >= grid || !count_out ||
        (tile_m != fasted::kTileM && tile_m != fasted::kPairTileM) || band_tiles <= 0)
        return fail(FASTED_EINVAL, "bad argument");
    fasted::JoinParams p{};
    p.n = static_cast<int>(n);
    p.q_begin = static_cast<int>(q_begin);
    p.q_end = static_cast<int>(q_end);
    p.tile_m = tile_m;
    p.symmetric = symmetric ? 1 : 0;
    p.shard_rank = shard_rank;
    p.shard_world = shard_world;
    p.raw_dot = 0;
    p.key_shift = 32;
    p.key_qbase = 0;
    p.key32 = 0;
    if (shard_world > 1 && !symmetric) return fail(FASTED_EINVAL, "band snakes are for the symmetric schedule only");
    p.tiles_m = static_cast<int>((q_end - q_begin + tile_m - 1) / tile_m);
    p.tiles_n = static_cast<int>((n + fasted::kTileN - 1) / fasted::kTileN);
    p.band_tiles = std::max(1, std::min(band_tiles, std::max(p.tiles_m, 1)));
    fasted::TileIter ti;
    int64_t count = 0;
    for (ti.init(p, cta, grid); ti.valid; ti.advance(p)) {
        if (tiles_out && count < max_tiles) {
            tiles_out[2 * count] = ti.tm;
            tiles_out[2 * count + 1] = ti.tn;
        }
        ++count;
    }
    *count_out = count;
    return FASTED_OK;
}

int fasted_tile_schedule_stationary(int64_t n, int64_t q_begin, int64_t q_end, int rows_per_band, int symmetric, int grid,
                                    int cta, int32_t* tiles_out, int64_t max_tiles, int64_t* count_out) {
    if (n <= 0 || q_begin < 0 || q_end < q_begin || q_end > n || grid <= 0 || cta < 0 || cta >= grid || !count_out ||
        rows_per_band <= 0 || rows_per_band > grid)
        return fail(FASTED_EINVAL, "bad argument");
    fasted::JoinParams p{};
    p.n = static_cast<int>(n);
    p.q_begin = static_cast<int>(q_begin);
    p.q_end = static_cast<int>(q_end);
    p.tile_m = fasted::kTileM;
    p.symmetric = symmetric ? 1 : 0;
    p.tiles_m = static_cast<int>((q_end - q_begin + fasted::kTileM - 1) / fasted::kTileM);
    p.tiles_n = static_cast<int>((n + fasted::kTileN - 1) / fasted::kTileN);
    p.astat_rows = rows_per_band;
    fasted::AStatIter ti;
    int64_t count = 0;
    for (ti.init(p, cta, grid); ti.valid; ti.advance(p)) {
        if (tiles_out && count < max_tiles) {
            tiles_out[2 * count] = ti.tm;
            tiles_out[2 * count + 1] = ti.tn;
        }
        ++count;
    }
    *count_out = count;
    return FASTED_OK;
}

int fasted_selftest_wait_timeout(fasted_ctx* c, double limit_ms, unsigned long long* status_out, double* waited_ms_out) {
    if (!c || !status_out) return fail(FASTED_EINVAL, "null argument");
    if (!(limit_ms > 0) || limit_ms > 1000.0) return fail(FASTED_EINVAL, "limit must be in (0, 1000] ms");
    CU_TRY(cudaSetDevice(c->device));
    CU_TRY(cudaMemsetAsync(c->counters, 0, kCounterWords * sizeof(unsigned long long), c->stream));
    fasted::wait_timeout_selftest_kernel<<<1, 32, 0, c->stream>>>(static_cast<unsigned long long>(limit_ms * 1e6),
                                                                 c->counters + 2, c->counters + 3);
    CU_TRY(cudaGetLastError());
    unsigned long long h[2] = {0, 0};
    CU_TRY(cudaMemcpyAsync(h, c->counters + 2, sizeof(h), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    *status_out = h[0];
    if (waited_ms_out) *waited_ms_out = static_cast<double>(h[1]) / 1e6;
    return FASTED_OK;
}

int fasted_estimate_epsilon(fasted_ctx* c, double target_mean_neighbours, int64_t sample_rows, double rel_tol,
                            double* eps_out, double* achieved_out) {
    if (!c || !eps_out) return fail(FASTED_EINVAL, "null argument");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (!(target_mean_neighbours > 0) || target_mean_neighbours >= static_cast<double>(c->n))
        return fail(FASTED_EINVAL, "target must be in (0, n)");
    if (!(rel_tol > 0)) rel_tol = 0.01;
    const int64_t n = c->n;
    if (sample_rows <= 0) sample_rows = 4096;
    sample_rows = std::min<int64_t>(sample_rows, n);
    // Up to 8 bands of whole 128-row tiles spread evenly over the dataset.
    const int64_t nb = std::max<int64_t>(1, std::min<int64_t>(8, sample_rows / 128));
    const int64_t per = std::max<int64_t>(1, sample_rows / nb);
    int64_t begin[8], end[8], rows = 0;
    for (int64_t b = 0; b < nb; ++b) {
        int64_t a = (n / nb * b) / 128 * 128;
        begin[b] = std::min(a, n - std::min(per, n));
        end[b] = std::min(n, begin[b] + per);
        rows += end[b] - begin[b];
    }
    double ms = 0;
    int rc = fasted_row_norms(c, &ms);
    if (rc) return rc;
    // Upper bracket: d2 <= (|q| + |c|)^2 <= 4 * max norm.
    std::vector<float> norms(static_cast<size_t>(n));
    rc = fasted_get_norms(c, norms.data());
    if (rc) return rc;
    float mx = 0.f;
    for (float v : norms) mx = std::max(mx, v);
    double lo = 0.0, hi = std::sqrt(4.0 * static_cast<double>(mx)) * 1.0001 + 1e-30;
    double mid = hi, mean = 0;
    for (int it = 0; it < 60; ++it) {
        mid = 0.5 * (lo + hi);
        unsigned long long found = 0;
        for (int64_t b = 0; b < nb; ++b) {
            fasted_join_stats st{};
            rc = fasted_join(c, mid, begin[b], end[b], 1, FASTED_JOIN_NO_SORT | FASTED_JOIN_KEEP_NORMS, &st);
            if (rc) return rc;
            found += st.pairs_found;
        }
        mean = (static_cast<double>(found) - static_cast<double>(rows)) / static_cast<double>(rows);
        if (std::fabs(mean - target_mean_neighbours) <= rel_tol * target_mean_neighbours) break;
        if (mean > target_mean_neighbours)
            hi = mid;
        else
            lo = mid;
    }
    *eps_out = mid;
    if (achieved_out) *achieved_out = mean;
    return FASTED_OK;
}

// Records of a FASTED_JOIN_NO_SORT join are kept packed until they are asked for.
static int ensure_unpacked(fasted_ctx* c) {
    if (!c->unpack_pending) return FASTED_OK;
    CU_TRY(cudaSetDevice(c->device));
    if (c->stored > 0) {
        fasted::unpack_pairs_kernel<<<unpack_blocks(c, c->stored), 256, 0, c->stream>>>(
            c->keys, reinterpret_cast<int2*>(c->keys_alt), c->stored, 32, 0);
        CU_TRY(cudaGetLastError());
        CU_TRY(cudaStreamSynchronize(c->stream));
    }
    c->result_pairs = c->keys_alt;
    c->unpack_pending = false;
    return FASTED_OK;
}

int fasted_get_pairs(fasted_ctx* c, uint64_t first, uint64_t count, int32_t* pairs_out, float* dist2_out) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    {
        const int urc = ensure_unpacked(c);
        if (urc) return urc;
    }
    if (first + count > c->stored)
        return fail(FASTED_EINVAL, "range [%llu, %llu) exceeds the %llu stored pairs", (unsigned long long)first,
                    (unsigned long long)(first + count), (unsigned long long)c->stored);
    if (count == 0) return FASTED_OK;
    if (dist2_out && !c->result_dist) return fail(FASTED_ESTATE, "the last join did not record distances");
    CU_TRY(cudaSetDevice(c->device));
    if (pairs_out) CU_TRY(download_bytes(c, pairs_out, static_cast<const int2*>(c->result_pairs) + first, count * 8, c->stream));
    if (dist2_out) CU_TRY(download_bytes(c, dist2_out, c->result_dist + first, count * 4, c->stream));
    return FASTED_OK;
}

int fasted_pairs_device(fasted_ctx* c, void** pairs_dev, void** dist2_dev) {
    if (!c) return fail(FASTED_EINVAL, "ctx is null");
    {
        const int urc = ensure_unpacked(c);
        if (urc) return urc;
    }
    if (pairs_dev) *pairs_dev = c->result_pairs;
    if (dist2_dev) *dist2_dev = c->result_dist;
    return FASTED_OK;
}

int fasted_brute_force_f64_pairs(fasted_ctx* c, const int32_t* sample_rows, int n_samples, double eps,
                                 unsigned long long* counts_out, unsigned long long* keys_out, uint64_t capacity,
                                 unsigned long long* n_keys_out) {
    if (!c || !sample_rows || !counts_out || n_samples <= 0) return fail(FASTED_EINVAL, "bad argument");
    if (capacity > 0 && (!keys_out || !n_keys_out)) return fail(FASTED_EINVAL, "keys_out / n_keys_out is null");
    if (!c->points) return fail(FASTED_ESTATE, "no dataset is resident");
    if (c->d > 12000) return fail(FASTED_EINVAL, "brute-force check supports d <= 12000");
    for (int i = 0; i < n_samples; ++i)
        if (sample_rows[i] < 0 || sample_rows[i] >= c->n) return fail(FASTED_EINVAL, "sample row out of range");
    CU_TRY(cudaSetDevice(c->device));
    int* d_rows = nullptr;
    unsigned long long* d_counts = nullptr;  // n_samples counts followed by the key counter
    unsigned long long* d_keys = nullptr;
    cudaError_t e = cudaMalloc(&d_rows, n_samples * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&d_counts, (n_samples + 1) * 8);
    if (e == cudaSuccess && capacity > 0) e = cudaMalloc(&d_keys, capacity * 8);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_rows, sample_rows, n_samples * sizeof(int), cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_counts, 0, (n_samples + 1) * 8, c->stream);
    if (e == cudaSuccess) {
        const int threads = 256;
        const int bx = static_cast<int>(std::min<int64_t>((c->n + 7) / 8, 2048));
        dim3 grid(bx, n_samples);
        fasted::brute_f64_kernel<<<grid, threads, static_cast<size_t>(c->d) * 4, c->stream>>>(
            c->points, static_cast<int>(c->n), static_cast<int>(c->d), static_cast<int>(c->ld), d_rows, n_samples,
            eps * eps, d_counts, d_keys, capacity, d_counts + n_samples);
        e = cudaGetLastError();
    }
    unsigned long long nk = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(counts_out, d_counts, n_samples * 8, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&nk, d_counts + n_samples, 8, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e == cudaSuccess && capacity > 0) {
        const unsigned long long m = nk < capacity ? nk : capacity;
        if (m) e = cudaMemcpy(keys_out, d_keys, m * 8, cudaMemcpyDeviceToHost);
        *n_keys_out = nk;
    }
    if (d_rows) cudaFree(d_rows);
    if (d_counts) cudaFree(d_counts);
    if (d_keys) cudaFree(d_keys);
    if (e != cudaSuccess) return fail(FASTED_ECUDA, "brute-force check failed: %s", cudaGetErrorString(e));
    return FASTED_OK;
}

int fasted_brute_force_f64(fasted_ctx* c, const int32_t* sample_rows, int n_samples, double eps,
                           unsigned long long* counts_out) {
    return fasted_brute_force_f64_pairs(c, sample_rows, n_samples, eps, counts_out, nullptr, 0, nullptr);
}

// ---------------------------------------------------------------------------
// Join without any allocation
// ---------------------------------------------------------------------------
//
// Scratch for fasted_join_static_scratch: the row norms of up to
// kStaticMaxPoints points followed by the kernel's counter block.  It lives in
// the library image, so every GPU that loads this library keeps these 4 MiB +
// 256 bytes until the process exits, whether or not the entry point is used.
// In host code the symbol below is only a stand-in: the device address comes
// from cudaGetSymbolAddress, once per device.
namespace {
constexpr int64_t kStaticMaxPoints = 1 << 20;
constexpr size_t kStaticCounterBytes = 256;
constexpr size_t kStaticScratchBytes = static_cast<size_t>(kStaticMaxPoints) * sizeof(float) + kStaticCounterBytes;
}  // namespace
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// Set-up on the current device: resolve the scratch symbol and raise the kernels' dynamic shared
// memory limits.  Done on every call (both are table look-ups, neither allocates), so that nothing
// cached can go stale when the device's context is reset between calls.  The first fasted call of a
// process on a device makes the CUDA runtime load this library's module there (kernel images and
// the scratch array): that one-time load is the only moment device memory is taken.
int static_scratch_setup(int device, unsigned char** out) {
    int major = 0;
    CU_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10)
        return fail(FASTED_ENODEV, "device %d is sm_%dx; this library contains sm_100a code only", device, major);
    void* addr = nullptr;
    CU_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
    CU_TRY(cudaFuncSetAttribute(fasted::join_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                fasted::kJoinSmemBytes));
    CU_TRY(cudaFuncSetAttribute(fasted::row_norms_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                fasted::kNormSmemBytes));
    *out = static_cast<unsigned char*>(addr);
    return FASTED_OK;
}

int encode_map(CUtensorMap* map, const void* points, int64_t n, int64_t d, int64_t ld, int box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(FASTED_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(n)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(fasted::kTileK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(points), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FASTED_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FASTED_OK;
}
}  // namespace

int fasted_join_static_scratch(const void* points_dev, int64_t n, int64_t d, int64_t ld, double eps,
                               unsigned long long* keys_out_dev, uint64_t capacity, void* stream,
                               unsigned long long* pairs_found, unsigned long long* pairs_stored) {
    if (!points_dev || !pairs_found || !pairs_stored) return fail(FASTED_EINVAL, "null argument");
    if (capacity > 0 && !keys_out_dev) return fail(FASTED_EINVAL, "keys_out_dev is null but capacity is not 0");
    int rc = check_shape(n, d);
    if (rc) return rc;
    if (n > kStaticMaxPoints)
        return fail(FASTED_EINVAL,
                    "n = %lld exceeds the %lld points the built-in scratch area holds; use fasted_join, which allocates",
                    (long long)n, (long long)kStaticMaxPoints);
    if (ld < d || (ld % 8) != 0) return fail(FASTED_EINVAL, "ld (%lld) must be >= d and a multiple of 8", (long long)ld);
    if (reinterpret_cast<uintptr_t>(points_dev) % 16 != 0) return fail(FASTED_EINVAL, "points must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(keys_out_dev) % 8 != 0) return fail(FASTED_EINVAL, "keys_out_dev must be 8-byte aligned");
    if (eps != eps) return fail(FASTED_EINVAL, "epsilon is NaN");

    int device = -1;
    CU_TRY(cudaGetDevice(&device));
    unsigned char* scratch = nullptr;
    rc = static_scratch_setup(device, &scratch);
    if (rc) return rc;
    float* norms = reinterpret_cast<float*>(scratch);
    unsigned long long* counters =
        reinterpret_cast<unsigned long long*>(scratch + static_cast<size_t>(kStaticMaxPoints) * sizeof(float));
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    CUtensorMap map_a, map_b;
    rc = encode_map(&map_a, points_dev, n, d, ld, fasted::kTileM);
    if (rc) return rc;
    rc = encode_map(&map_b, points_dev, n, d, ld, fasted::kTileN);
    if (rc) return rc;

    int num_sms = 0;
    CU_TRY(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device));

    fasted::JoinParams p{};
    p.norms = norms;
    p.norms_vec4 = (reinterpret_cast<uintptr_t>(p.norms) & 15u) == 0 ? 1 : 0;
    p.counters = counters;
    p.keys = keys_out_dev;
    p.dist2 = nullptr;
    p.capacity = capacity;
    const double e2 = eps * eps;
    p.eps2 = e2 > FLT_MAX ? FLT_MAX : static_cast<float>(e2);
    p.n = static_cast<int>(n);
    p.q_begin = 0;
    p.q_end = static_cast<int>(n);
    p.k_steps = static_cast<int>((d + fasted::kTileK - 1) / fasted::kTileK);
    p.tiles_m = static_cast<int>((n + fasted::kTileM - 1) / fasted::kTileM);
    p.tiles_n = static_cast<int>((n + fasted::kTileN - 1) / fasted::kTileN);
    p.band_tiles = std::max(1, std::min(default_band_tiles(ld), p.tiles_m));
    p.total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    p.tile_m = fasted::kTileM;
    p.symmetric = 0;
    p.raw_dot = 0;
    p.shard_rank = 0;
    p.shard_world = 1;
    p.key_shift = 32;
    p.key_qbase = 0;
    p.key32 = 0;
    const int grid = static_cast<int>(std::min<long long>(p.total_tiles, num_sms));

    // The scratch area keeps whatever the previous call left: the counters must start at zero
    // (the norms are overwritten for rows [0, n) before the join reads them).
    CU_TRY(cudaMemsetAsync(counters, 0, kStaticCounterBytes, st));
    const int row_blocks = static_cast<int>((n + fasted::kNormRows - 1) / fasted::kNormRows);
    fasted::row_norms_kernel<0><<<std::min(row_blocks, num_sms * 3), fasted::kNormRows, fasted::kNormSmemBytes, st>>>(
        map_a, norms, static_cast<int>(n), p.k_steps, row_blocks, 0, counters + 2);
    CU_TRY(cudaGetLastError());
    fasted::join_kernel<<<grid, fasted::kJoinThreads, fasted::kJoinSmemBytes, st>>>(map_a, map_b, p);
    CU_TRY(cudaGetLastError());
    unsigned long long h[3] = {0, 0, 0};
    CU_TRY(cudaMemcpyAsync(h, counters, sizeof(h), cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    if (h[2]) return fail(FASTED_EKERNEL, "a device-side wait ran out (status 0x%llx)", h[2]);
    *pairs_found = h[0];
    *pairs_stored = h[0] < capacity ? h[0] : capacity;
    return FASTED_OK;
}

}  // extern "C"
