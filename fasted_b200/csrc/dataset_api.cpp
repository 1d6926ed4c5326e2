// C entry points of the host-side dataset builders (include/fasted.h).
#include <cstring>
#include <exception>
#include <ios>
#include <stdexcept>

#include "dataset.hpp"

#include <sys/stat.h>

#include <mutex>
#include <string>
#include "error.hpp"
#include "fasted.h"

namespace {

int copy_out(const fasted::HostDataset& ds, uint16_t* out, int64_t n, int64_t d, int64_t ld_out) {
    if (ds.n != n || ds.d != d)
        return fasted::fail(FASTED_EINVAL, "dataset is %lld x %lld, caller expected %lld x %lld", (long long)ds.n,
                            (long long)ds.d, (long long)n, (long long)d);
    for (int64_t r = 0; r < n; ++r) {
        std::memcpy(out + r * ld_out, ds.values.data() + r * d, static_cast<size_t>(d) * 2);
        if (ld_out > d) std::memset(out + r * ld_out + d, 0, static_cast<size_t>(ld_out - d) * 2);
    }
    return FASTED_OK;
}

template <class F>
int guarded(F&& f) {
    try {
        return f();
    } catch (const std::ios_base::failure& e) {
        return fasted::fail(FASTED_EIO, "%s", e.what());
    } catch (const std::exception& e) {
        return fasted::fail(FASTED_EINVAL, "%s", e.what());
    }
}

}  // namespace

extern "C" {

int fasted_dataset_exponential_f16(int64_t n, int64_t d, double lambda, double max_value, uint16_t* out,
                                   int64_t ld_out) {
    if (!out || ld_out < d) return fasted::fail(FASTED_EINVAL, "bad output buffer");
    return guarded([&] {
        const fasted::HostDataset ds = fasted::make_exponential_dataset(n, d, lambda, max_value);
        return copy_out(ds, out, n, d, ld_out);
    });
}

// A caller asks for the shape, allocates, then asks for the values: the file parsed for the first call
// is kept for the second (one entry, dropped when it has been handed out or when another file is asked for).
namespace {
struct ParsedCsv {
    std::string path;
    long long size = -1, mtime_ns = -1;
    fasted::HostDataset ds;
    bool valid = false;
};
ParsedCsv g_parsed;
std::mutex g_parsed_mutex;

bool file_stamp(const char* path, long long* size, long long* mtime_ns) {
    struct stat st;
    if (::stat(path, &st) != 0) return false;
    *size = static_cast<long long>(st.st_size);
    *mtime_ns = static_cast<long long>(st.st_mtim.tv_sec) * 1000000000LL + st.st_mtim.tv_nsec;
    return true;
}
}  // namespace

int fasted_dataset_csv_shape(const char* path, int64_t* n, int64_t* d) {
    if (!path || !n || !d) return fasted::fail(FASTED_EINVAL, "null argument");
    return guarded([&] {
        fasted::HostDataset ds = fasted::read_csv_dataset(path);
        *n = ds.n;
        *d = ds.d;
        std::lock_guard<std::mutex> lock(g_parsed_mutex);
        g_parsed.valid = file_stamp(path, &g_parsed.size, &g_parsed.mtime_ns);
        g_parsed.path = path;
        g_parsed.ds = std::move(ds);
        return (int)FASTED_OK;
    });
}

int fasted_dataset_csv_f16(const char* path, uint16_t* out, int64_t n, int64_t d, int64_t ld_out) {
    if (!path || !out || ld_out < d) return fasted::fail(FASTED_EINVAL, "bad argument");
    return guarded([&] {
        {
            std::lock_guard<std::mutex> lock(g_parsed_mutex);
            long long size = -1, mtime_ns = -1;
            if (g_parsed.valid && g_parsed.path == path && file_stamp(path, &size, &mtime_ns) && size == g_parsed.size &&
                mtime_ns == g_parsed.mtime_ns) {
                const fasted::HostDataset ds = std::move(g_parsed.ds);
                g_parsed = ParsedCsv{};
                return copy_out(ds, out, n, d, ld_out);
            }
            g_parsed = ParsedCsv{};
        }
        const fasted::HostDataset ds = fasted::read_csv_dataset(path);
        return copy_out(ds, out, n, d, ld_out);
    });
}

}  // extern "C"
