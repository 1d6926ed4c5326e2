// Drop-in for the reference's shared-library interface (layer 1 of
// include/fasted.h): runFromExponentialDataset, runFromFile, reRun,
// releaseResources, with the reference's stdout lines, Results struct,
// output-file format and error behaviour, on top of the context API.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iostream>
#include <memory>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include <omp.h>

#include "dataset.hpp"
#include "fasted.h"

namespace {

struct LegacyState {
    fasted_ctx* ctx = nullptr;           // GPU 0 of this process (FASTED_DEVICE)
    std::vector<fasted_ctx*> extra;      // further GPUs when FASTED_NUM_GPUS > 1
    int64_t n = 0, d = 0;
    bool have_points = false;
};
LegacyState g_state;

double now_s() {
    using clock = std::chrono::steady_clock;
    return std::chrono::duration<double>(clock::now().time_since_epoch()).count();
}

[[noreturn]] void die(const std::string& what) {
    // source/main.cu:244-247: message on stdout, then exit(EXIT_FAILURE).
    std::cout << "Error: Failed to run. " << what << std::endl;
    std::exit(EXIT_FAILURE);
}

void check(int rc) {
    if (rc != FASTED_OK) throw std::runtime_error(fasted_last_error());
}

fasted_ctx* context() {
    if (!g_state.ctx) {
        int dev = 0;
        if (const char* e = std::getenv("FASTED_DEVICE")) dev = std::atoi(e);
        check(fasted_create(dev, &g_state.ctx));
    }
    return g_state.ctx;
}

int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// All contexts of this process: GPU 0 first.  FASTED_NUM_GPUS (default 1, "all" = every device)
// counts devices upward from FASTED_DEVICE.
std::vector<fasted_ctx*> all_contexts() {
    std::vector<fasted_ctx*> v{context()};
    int want = 1;
    if (const char* e = std::getenv("FASTED_NUM_GPUS")) want = std::strcmp(e, "all") == 0 ? 1 << 20 : std::atoi(e);
    int first = 0;
    if (const char* e = std::getenv("FASTED_DEVICE")) first = std::atoi(e);
    while (static_cast<int>(g_state.extra.size()) + 1 < want) {
        fasted_ctx* c = nullptr;
        if (fasted_create(first + 1 + static_cast<int>(g_state.extra.size()), &c) != FASTED_OK) {
            if (want != (1 << 20)) throw std::runtime_error(fasted_last_error());
            break;  // "all": stop at the last device
        }
        g_state.extra.push_back(c);
    }
    for (fasted_ctx* c : g_state.extra) v.push_back(c);
    return v;
}

// Contiguous band of query rows of GPU g out of G (whole 128-row tiles), as in fasted_b200/dist.py.
void band_of(int64_t n, int g, int G, int64_t* begin, int64_t* end) {
    int64_t per = (n + G - 1) / G;
    per = round_up(per, 128);
    *begin = std::min<int64_t>(n, per * g);
    *end = std::min<int64_t>(n, *begin + per);
}

// Merge G lists of (query, candidate) records, each sorted row-major and pairwise disjoint, into one
// sorted list.  The query range is cut into one slice per thread; a slice's records are a contiguous
// run of every list (found by bisection), so the slices merge independently into known offsets.
void merge_sorted_lists(const std::vector<std::vector<int32_t>>& part, const std::vector<std::vector<float>>& part_d,
                        int64_t n, int32_t* out, float* out_d) {
    const int G = static_cast<int>(part.size());
    const int T = std::max(1, omp_get_max_threads());
    auto lower = [&](int g, int64_t q) {  // first record of list g whose query index is >= q
        const int32_t* p = part[g].data();
        size_t lo = 0, hi = part[g].size() / 2;
        while (lo < hi) {
            const size_t mid = (lo + hi) / 2;
            if (p[2 * mid] < q) lo = mid + 1; else hi = mid;
        }
        return lo;
    };
#pragma omp parallel for schedule(static, 1) num_threads(T)
    for (int t = 0; t < T; ++t) {
        const int64_t q0 = n * t / T, q1 = n * (t + 1) / T;
        std::vector<size_t> at(G), end(G);
        size_t o = 0;
        for (int g = 0; g < G; ++g) {
            at[g] = lower(g, q0);
            end[g] = lower(g, q1);
            o += at[g];
        }
        for (;;) {
            int best = -1;
            uint64_t best_key = 0;
            for (int g = 0; g < G; ++g) {
                if (at[g] == end[g]) continue;
                const int32_t* r = part[g].data() + 2 * at[g];
                const uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(r[0])) << 32) | static_cast<uint32_t>(r[1]);
                if (best < 0 || key < best_key) {
                    best = g;
                    best_key = key;
                }
            }
            if (best < 0) break;
            out[2 * o] = part[best][2 * at[best]];
            out[2 * o + 1] = part[best][2 * at[best] + 1];
            if (out_d) out_d[o] = part_d[best][at[best]];
            ++o;
            ++at[best];
        }
    }
}

inline char* put_uint(char* p, uint32_t v) {
    char tmp[10];
    int len = 0;
    do {
        tmp[len++] = static_cast<char>('0' + v % 10);
        v /= 10;
    } while (v);
    while (len) *p++ = tmp[--len];
    return p;
}

// Writes "q, c\n" per pair (source/pair.cuh:51-54), optionally "q, c, dist\n".  The reference streams
// one `os << pair << std::endl` (a flush) per pair; here every append is formatted by all host threads
// into slices of their own, which are then written in order.  Appends may come while the GPU is still
// joining later query rows (fasted_join_stream), so the text is produced behind the join as well.
class PairsWriter {
public:
    explicit PairsWriter(const std::string& path) : f_(std::fopen(path.c_str(), "wb")) {}
    // (the reference ignores a failed open: its std::ofstream is never checked)
    ~PairsWriter() {
        if (f_) std::fclose(f_);
    }
    void append(const int32_t* pairs, const float* dist2, size_t count) {
        if (!f_ || count == 0) return;
        const size_t slice = size_t(1) << 18;  // pairs per formatting task
        const size_t tasks = (count + slice - 1) / slice;
        const size_t wave = static_cast<size_t>(std::max(1, omp_get_max_threads()));
        if (bufs_.size() < wave) bufs_.resize(wave);
        for (size_t t0 = 0; t0 < tasks; t0 += wave) {
            const size_t nt = std::min(wave, tasks - t0);
#pragma omp parallel for schedule(static, 1)
            for (size_t k = 0; k < nt; ++k) {
                const size_t begin = (t0 + k) * slice, end = std::min(count, begin + slice);
                std::vector<char>& b = bufs_[k];
                b.resize((end - begin) * (dist2 ? 48 : 24));
                char* p = b.data();
                for (size_t i = begin; i < end; ++i) {
                    p = put_uint(p, static_cast<uint32_t>(pairs[2 * i]));
                    *p++ = ',';
                    *p++ = ' ';
                    p = put_uint(p, static_cast<uint32_t>(pairs[2 * i + 1]));
                    if (dist2) p += std::snprintf(p, 24, ", %.9g", std::sqrt(static_cast<double>(dist2[i])));
                    *p++ = '\n';
                }
                b.resize(static_cast<size_t>(p - b.data()));
            }
            for (size_t k = 0; k < nt; ++k) std::fwrite(bufs_[k].data(), 1, bufs_[k].size(), f_);
        }
    }

private:
    FILE* f_;
    std::vector<std::vector<char>> bufs_;
};

struct StreamSink {
    PairsWriter* writer;   // null: the records are brought to the host and dropped, as the reference
                           // does when savePairs is false (source/findPairs.cuh:703-714)
    uint64_t delivered;
};

int stream_sink(void* user, const int32_t* pairs, const float* dist2, uint64_t /*first*/, uint64_t count) {
    StreamSink* s = static_cast<StreamSink*>(user);
    if (s->writer) s->writer->append(pairs, dist2, static_cast<size_t>(count));
    s->delivered += count;
    return 0;
}

// The body of the reference's run() + FindPairs() (source/main.cu:198-248,
// source/findPairs.cuh:615-764) on the resident dataset.
Results join_resident(double epsilon, bool save_pairs, const std::string& dataset_name, double start_time,
                      bool keep_norms) {
    fasted_ctx* ctx = context();
    const int64_t n = g_state.n, d = g_state.d;
    const int64_t n_pad = round_up(n, 256), d_pad = round_up(d, 64);

    std::string out_dir = "/scratch/bc2497/pairsData/";
    if (const char* e = std::getenv("FASTED_OUTPUT_DIR")) {
        out_dir = e;
        if (!out_dir.empty() && out_dir.back() != '/') out_dir += '/';
    }
    const std::string output_path = out_dir + dataset_name + "_" + std::to_string(epsilon);
    const bool write_dist = save_pairs && std::getenv("FASTED_WRITE_DIST") &&
                            std::strcmp(std::getenv("FASTED_WRITE_DIST"), "1") == 0;

    std::cout << "Padded Search Dimensions:" << std::endl;
    std::cout << "M: " << n_pad << std::endl;
    std::cout << "N: " << n_pad << std::endl;
    std::cout << "K: " << d_pad << std::endl;
    std::cout << "Input Search Dimensions:" << std::endl;
    std::cout << "M: " << n << std::endl;
    std::cout << "N: " << n << std::endl;
    std::cout << "K: " << d << std::endl;

    // Default: all N x N entries are computed, like the reference, so that "Estimated TFLOPS" counts
    // executed work.  FASTED_SYMMETRIC=1: d2(i,j) == d2(j,i) bit for bit, so each unordered pair is
    // computed once and both orientations are emitted -- identical output in about half the time; the
    // TFLOPS line still divides 2*N*N*D by the time, and the schedule line says so.
    const char* sym_env = std::getenv("FASTED_SYMMETRIC");
    const bool symmetric = sym_env && std::strcmp(sym_env, "1") == 0;
    unsigned flags = write_dist ? FASTED_JOIN_DIST2 : 0u;
    if (symmetric) flags |= FASTED_JOIN_SYMMETRIC;
    if (keep_norms) flags |= FASTED_JOIN_KEEP_NORMS;  // reRun: the dataset, hence its norms, is unchanged
    std::cout << "Schedule: "
              << (symmetric ? "symmetric (each unordered pair computed once; executed flops are about half of 2*N*N*D)"
                            : "full (all N x N entries computed)")
              << std::endl;
    fasted_join_stats st{};
    std::vector<fasted_ctx*> gpus = all_contexts();
    // FASTED_EXACT_NORMS=1: correctly rounded row norms instead of the reference's round-toward-zero chain
    // (not the reference's numerics; closer to an FP64 join on this GPU, see fasted_set_option).
    const char* exact_env = std::getenv("FASTED_EXACT_NORMS");
    const bool exact_norms = exact_env && std::strcmp(exact_env, "1") == 0;
    for (fasted_ctx* g : gpus) check(fasted_set_option(g, "exact_norms", exact_norms ? 1 : 0));
    if (exact_norms) std::cout << "Row norms: correctly rounded (FASTED_EXACT_NORMS=1)" << std::endl;
    std::vector<fasted_join_stats> per_gpu(gpus.size());
    const std::string pairs_path = output_path + ".pairs";
    double sort_start = now_s();

    if (gpus.size() == 1 && !symmetric) {
        // One GPU, full schedule: sort, device-to-host copy and the text file all run behind the join,
        // chunk of query rows by chunk (fasted_join_stream); nothing of the list is kept on the host.
        std::unique_ptr<PairsWriter> writer;
        if (save_pairs) {
            std::cout << "Output file is: " << pairs_path << std::endl;
            writer.reset(new PairsWriter(pairs_path));
        }
        StreamSink sink{writer.get(), 0};
        check(fasted_join_stream(ctx, epsilon, 0, -1, 0, flags, nullptr, nullptr, 0, stream_sink, &sink, &st));
        writer.reset();
        std::printf("Number of pairs found %llu\n", st.pairs_found);
        std::printf("Number of pairs stored %llu\n", st.pairs_stored);
        sort_start = now_s() - st.tail_ms / 1e3;
    } else {
        if (gpus.size() == 1) {
            check(fasted_join(ctx, epsilon, 0, -1, 0, flags, &st));
            per_gpu[0] = st;
        } else {
            // One host thread per GPU (the join call blocks).  Symmetric: GPU g computes its snake of
            // upper-triangle bands and emits both orientations, so every GPU's sorted list spans all
            // query rows and the lists are merged on the host.  Full: GPU g joins the g-th contiguous band
            // of query rows; the lists are laid end to end.  No collective either way.
            const int G = static_cast<int>(gpus.size());
            std::vector<int> rc(gpus.size(), FASTED_OK);
            std::vector<std::string> err(gpus.size());
            std::vector<std::thread> workers;
            for (int g = 0; g < G; ++g)
                workers.emplace_back([&, g] {
                    if (symmetric) {
                        rc[g] = fasted_join_symmetric_shard(gpus[g], epsilon, g, G, 0, flags, &per_gpu[g]);
                    } else {
                        int64_t b, e;
                        band_of(n, g, G, &b, &e);
                        rc[g] = fasted_join(gpus[g], epsilon, b, e,
                                            static_cast<uint64_t>(std::max<int64_t>(e - b, 1)) * 256, flags, &per_gpu[g]);
                    }
                    if (rc[g] != FASTED_OK) err[g] = fasted_last_error();
                });
            for (auto& w : workers) w.join();
            for (int g = 0; g < G; ++g)
                if (rc[g] != FASTED_OK) throw std::runtime_error(err[g]);
            for (int g = 0; g < G; ++g) {  // the slowest GPU sets the time, the counts add up
                st.pairs_found += per_gpu[g].pairs_found;
                st.pairs_stored += per_gpu[g].pairs_stored;
                st.kernel_ms = std::max(st.kernel_ms, per_gpu[g].kernel_ms);
                st.norms_ms = std::max(st.norms_ms, per_gpu[g].norms_ms);
                st.join_ms = std::max(st.join_ms, per_gpu[g].join_ms);
                st.sort_ms = std::max(st.sort_ms, per_gpu[g].sort_ms);
            }
        }

        sort_start = now_s();
        std::printf("Number of pairs found %llu\n", st.pairs_found);
        std::printf("Number of pairs stored %llu\n", st.pairs_stored);
        // The reference copies every stored pair to the host even when it does not
        // save them (source/findPairs.cuh:703-714); so does this.
        std::vector<int32_t> pairs(static_cast<size_t>(st.pairs_stored) * 2);
        std::vector<float> dist2(write_dist ? static_cast<size_t>(st.pairs_stored) : 0);
        if (gpus.size() == 1 || !symmetric) {
            // Bands are contiguous in the query index: the band lists end to end are the global order.
            size_t at = 0;
            for (size_t g = 0; g < gpus.size(); ++g) {
                const uint64_t m = per_gpu[g].pairs_stored;
                check(fasted_get_pairs(gpus[g], 0, m, pairs.data() + 2 * at, write_dist ? dist2.data() + at : nullptr));
                at += static_cast<size_t>(m);
            }
        } else {
            std::vector<std::vector<int32_t>> part(gpus.size());
            std::vector<std::vector<float>> part_d(gpus.size());
            for (size_t g = 0; g < gpus.size(); ++g) {
                const uint64_t m = per_gpu[g].pairs_stored;
                part[g].resize(static_cast<size_t>(m) * 2);
                if (write_dist) part_d[g].resize(static_cast<size_t>(m));
                check(fasted_get_pairs(gpus[g], 0, m, part[g].data(), write_dist ? part_d[g].data() : nullptr));
            }
            merge_sorted_lists(part, part_d, n, pairs.data(), write_dist ? dist2.data() : nullptr);
        }
        if (save_pairs) {
            std::cout << "Output file is: " << pairs_path << std::endl;
            PairsWriter writer(pairs_path);
            writer.append(pairs.data(), write_dist ? dist2.data() : nullptr, pairs.size() / 2);
        }
    }
    const double end_time = now_s();

    const double total_time = end_time - start_time;
    const double kernel_s = st.kernel_ms / 1e3;
    std::printf("Total Elapsed time: %f seconds\n", total_time);
    std::printf("Total Kernel Elapsed time: %f seconds\n", kernel_s);
    std::printf("SumSquard Kernel Elapsed time: %f seconds\n", st.norms_ms / 1e3);
    std::printf("FindPairs Kernel Elapsed time: %f seconds\n", st.join_ms / 1e3);
    std::printf("Pairs sort Elapsed time: %f seconds\n", st.sort_ms / 1e3 + (end_time - sort_start));
    std::cout << "Pairs found: " << st.pairs_found << std::endl;
    const double tflops = 2.0 * static_cast<double>(n) * static_cast<double>(n) * static_cast<double>(d) / kernel_s / 1e12;
    std::printf("Estimated TFLOPS %.3f\n", tflops);
    std::fflush(stdout);

    Results r;
    r.totalTime = total_time;
    r.TFLOPS = tflops;
    r.pairsFound = st.pairs_found;
    r.pairsStored = st.pairs_stored;
    r.inputProblemShape = mmaShape{static_cast<int>(n), static_cast<int>(n), static_cast<int>(d)};
    r.paddedProblemShape = mmaShape{static_cast<int>(n_pad), static_cast<int>(n_pad), static_cast<int>(d_pad)};
    return r;
}

Results run_dataset(fasted::HostDataset (*make)(void*), void* arg, double epsilon, bool save_pairs) {
    try {
        const double start = now_s();
        // The CUDA context of every GPU this process drives is created while the host builds the
        // dataset (the reference pays for it inside its timed call, source/findPairs.cuh:616-622).
        std::exception_ptr warm_error;
        std::thread warm([&warm_error] {
            try {
                all_contexts();
            } catch (...) {
                warm_error = std::current_exception();
            }
        });
        struct Joiner {
            std::thread& t;
            ~Joiner() {
                if (t.joinable()) t.join();
            }
        } joiner{warm};
        std::cout << "Building point list" << std::endl;
        fasted::HostDataset ds = make(arg);
        std::cout << "Number of points is: " << ds.n << std::endl;
        std::cout << "Padding with " << round_up(ds.n, 256) - ds.n << " points" << std::endl;
        std::cout << "Dataset creation time: " << now_s() - start << " (sec)" << std::endl;
        warm.join();
        if (warm_error) std::rethrow_exception(warm_error);
        const double join_start = now_s();
        check(fasted_set_points_host_f16(context(), ds.values.data(), ds.n, ds.d, ds.d));
        {
            // Replication over the GPUs of this process: ONE NCCL broadcast from GPU 0.  Where NCCL is
            // not installed, every further GPU pulls its copy from GPU 0 instead (peer copies).
            std::vector<fasted_ctx*> gpus = all_contexts();
            if (gpus.size() > 1) {
                const double t0 = now_s();
                double ms = 0;
                if (fasted_broadcast_points(gpus.data(), static_cast<int>(gpus.size()), &ms) == FASTED_OK) {
                    std::printf("Replication over %zu GPUs (NCCL broadcast): %f seconds\n", gpus.size(), ms / 1e3);
                } else {
                    std::vector<int> rc(gpus.size(), FASTED_OK);
                    std::vector<std::string> err(gpus.size());
                    std::vector<std::thread> pulls;
                    for (size_t g = 1; g < gpus.size(); ++g)
                        pulls.emplace_back([&, g] {
                            rc[g] = fasted_copy_points_from(gpus[g], gpus[0]);
                            if (rc[g] != FASTED_OK) err[g] = fasted_last_error();
                        });
                    for (auto& t : pulls) t.join();
                    for (size_t g = 1; g < gpus.size(); ++g)
                        if (rc[g] != FASTED_OK) throw std::runtime_error(err[g]);
                    std::printf("Replication over %zu GPUs (peer copies): %f seconds\n", gpus.size(), now_s() - t0);
                }
            }
        }
        g_state.n = ds.n;
        g_state.d = ds.d;
        g_state.have_points = true;
        return join_resident(epsilon, save_pairs, ds.name, join_start, false);
    } catch (const std::exception& e) {
        die(e.what());
    }
}

struct ExpArgs {
    int n, d;
    double lambda, max_value;
};

}  // namespace

extern "C" {

Results runFromExponentialDataset(int size, int dimensionality, double lambda, double maxValue, double epsilon,
                                  bool savePairs) {
    std::cout << "Running from a generated exponential dataset" << std::endl;
    ExpArgs a{size, dimensionality, lambda, maxValue};
    return run_dataset(
        [](void* p) {
            const ExpArgs* a = static_cast<const ExpArgs*>(p);
            return fasted::make_exponential_dataset(a->n, a->d, a->lambda, a->max_value);
        },
        &a, epsilon, savePairs);
}

Results runFromFile(const char* filename, double epsilon, bool savePairs) {
    std::string name(filename ? filename : "");
    std::cout << "Running from file: " << name << std::endl;
    return run_dataset([](void* p) { return fasted::read_csv_dataset(*static_cast<std::string*>(p)); }, &name, epsilon,
                       savePairs);
}

Results reRun(double epsilon, bool savePairs) {
    try {
        if (!g_state.have_points) throw std::runtime_error("reRun called before runFromFile/runFromExponentialDataset");
        return join_resident(epsilon, savePairs, "", now_s(), true);
    } catch (const std::exception& e) {
        die(e.what());
    }
}

void releaseResources(void) {
    for (fasted_ctx* c : g_state.extra) fasted_destroy(c);
    if (g_state.ctx) fasted_destroy(g_state.ctx);
    g_state = LegacyState{};
}

}  // extern "C"
