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
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include <omp.h>

#include "dataset.hpp"
#include "fasted.h"

namespace {

struct LegacyState {
    fasted_ctx* ctx = nullptr;
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
// one `os << pair << std::endl` (a flush) per pair; here threads format disjoint slices into their own
// buffers, which are then written in order.
void write_pairs_file(const std::string& path, const std::vector<int32_t>& pairs, const std::vector<float>* dist2) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return;  // the reference ignores a failed open (std::ofstream never checked)
    const size_t count = pairs.size() / 2;
    const size_t slice = size_t(1) << 20;  // pairs per formatting task
    const size_t tasks = (count + slice - 1) / slice;
    const size_t wave = static_cast<size_t>(std::max(1, omp_get_max_threads()));
    std::vector<std::vector<char>> bufs(wave);
    for (size_t t0 = 0; t0 < tasks; t0 += wave) {
        const size_t nt = std::min(wave, tasks - t0);
#pragma omp parallel for schedule(static, 1)
        for (size_t k = 0; k < nt; ++k) {
            const size_t begin = (t0 + k) * slice, end = std::min(count, begin + slice);
            std::vector<char>& b = bufs[k];
            b.resize((end - begin) * (dist2 ? 48 : 24));
            char* p = b.data();
            for (size_t i = begin; i < end; ++i) {
                p = put_uint(p, static_cast<uint32_t>(pairs[2 * i]));
                *p++ = ',';
                *p++ = ' ';
                p = put_uint(p, static_cast<uint32_t>(pairs[2 * i + 1]));
                if (dist2) {
                    p += std::snprintf(p, 24, ", %.9g", std::sqrt(static_cast<double>((*dist2)[i])));
                }
                *p++ = '\n';
            }
            b.resize(static_cast<size_t>(p - b.data()));
        }
        for (size_t k = 0; k < nt; ++k) std::fwrite(bufs[k].data(), 1, bufs[k].size(), f);
    }
    std::fclose(f);
}

// The body of the reference's run() + FindPairs() (source/main.cu:198-248,
// source/findPairs.cuh:615-764) on the resident dataset.
Results join_resident(double epsilon, bool save_pairs, const std::string& dataset_name, double start_time) {
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

    // d2(i,j) == d2(j,i) bit for bit, so by default each unordered pair is computed once and both
    // orientations are emitted; FASTED_SYMMETRIC=0 computes all N x N entries like the reference.
    const char* sym_env = std::getenv("FASTED_SYMMETRIC");
    const bool symmetric = !(sym_env && std::strcmp(sym_env, "0") == 0);
    unsigned flags = write_dist ? FASTED_JOIN_DIST2 : 0u;
    if (symmetric) flags |= FASTED_JOIN_SYMMETRIC;
    fasted_join_stats st{};
    check(fasted_join(ctx, epsilon, 0, -1, 0, flags, &st));

    const double sort_start = now_s();
    std::printf("Number of pairs found %llu\n", st.pairs_found);
    std::printf("Number of pairs stored %llu\n", st.pairs_stored);
    // The reference copies every stored pair to the host even when it does not
    // save them (source/findPairs.cuh:703-714); so does this.
    std::vector<int32_t> pairs(static_cast<size_t>(st.pairs_stored) * 2);
    std::vector<float> dist2(write_dist ? static_cast<size_t>(st.pairs_stored) : 0);
    check(fasted_get_pairs(ctx, 0, st.pairs_stored, pairs.data(), write_dist ? dist2.data() : nullptr));
    if (save_pairs) {
        const std::string pairs_path = output_path + ".pairs";
        std::cout << "Output file is: " << pairs_path << std::endl;
        write_pairs_file(pairs_path, pairs, write_dist ? &dist2 : nullptr);
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
        std::cout << "Building point list" << std::endl;
        fasted::HostDataset ds = make(arg);
        std::cout << "Number of points is: " << ds.n << std::endl;
        std::cout << "Padding with " << round_up(ds.n, 256) - ds.n << " points" << std::endl;
        std::cout << "Dataset creation time: " << now_s() - start << " (sec)" << std::endl;
        const double join_start = now_s();
        check(fasted_set_points_host_f16(context(), ds.values.data(), ds.n, ds.d, ds.d));
        g_state.n = ds.n;
        g_state.d = ds.d;
        g_state.have_points = true;
        return join_resident(epsilon, save_pairs, ds.name, join_start);
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
        return join_resident(epsilon, savePairs, "", now_s());
    } catch (const std::exception& e) {
        die(e.what());
    }
}

void releaseResources(void) {
    if (g_state.ctx) fasted_destroy(g_state.ctx);
    g_state = LegacyState{};
}

}  // extern "C"
