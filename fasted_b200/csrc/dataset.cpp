#include "dataset.hpp"

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <charconv>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <ios>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include <omp.h>

namespace fasted {

uint16_t float_to_half_rn(float f) {
    uint32_t u;
    std::memcpy(&u, &f, sizeof(u));
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u) return static_cast<uint16_t>(sign | 0x7e00u);   // NaN
    if (abs >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);  // >= 65520 or inf
    if (abs < 0x38800000u) {
        // Below the smallest normal half (2^-14): result = nearest multiple of 2^-24.
        // Adding 0.5f puts that multiple's integer count into the low mantissa bits
        // of a float in [0.5, 1), with the FPU doing the round-to-nearest-even.
        float a;
        std::memcpy(&a, &abs, sizeof(a));
        volatile float t = a + 0.5f;  // ulp of t is 2^-24
        float tv = t;
        uint32_t tb;
        std::memcpy(&tb, &tv, sizeof(tb));
        return static_cast<uint16_t>(sign | (tb - 0x3f000000u));
    }
    // Normal half: drop 13 mantissa bits with round-to-nearest-even, rebias the exponent.
    const uint32_t lsb = (abs >> 13) & 1u;
    const uint32_t rounded = abs + 0xfffu + lsb;
    return static_cast<uint16_t>(sign | ((rounded - 0x38000000u) >> 13));
}

namespace {

// The MT19937 state (std::mt19937's parameters: n = 624, m = 397, r = 31, a = 0x9908b0df).
struct MtState {
    uint32_t x[624];
};

void mt_seed(MtState& s, uint32_t seed) {
    s.x[0] = seed;
    for (uint32_t i = 1; i < 624; ++i) s.x[i] = 1812433253u * (s.x[i - 1] ^ (s.x[i - 1] >> 30)) + i;
}

// One regeneration of the whole state.  Written as three loops whose carried dependences are 227
// or more elements long, so that the compiler vectorises them.
__attribute__((target_clones("avx2", "default"))) void mt_twist(MtState& s) {
    uint32_t* x = s.x;
    constexpr uint32_t kUpper = 0x80000000u, kLower = 0x7fffffffu, kA = 0x9908b0dfu;
#pragma omp simd safelen(64)
    for (int i = 0; i < 227; ++i) {
        const uint32_t y = (x[i] & kUpper) | (x[i + 1] & kLower);
        x[i] = x[i + 397] ^ (y >> 1) ^ ((y & 1u) ? kA : 0u);
    }
#pragma omp simd safelen(64)
    for (int i = 227; i < 623; ++i) {
        const uint32_t y = (x[i] & kUpper) | (x[i + 1] & kLower);
        x[i] = x[i - 227] ^ (y >> 1) ^ ((y & 1u) ? kA : 0u);
    }
    const uint32_t y = (x[623] & kUpper) | (x[0] & kLower);
    x[623] = x[396] ^ (y >> 1) ^ ((y & 1u) ? kA : 0u);
}

// std::mt19937 holding this state with all of its outputs consumed (the next draw twists first):
// the engine's own text format is the 624 words followed by the position.
std::mt19937 engine_from_state(const MtState& s) {
    std::string text;
    text.reserve(624 * 11 + 8);
    for (int i = 0; i < 624; ++i) {
        text += std::to_string(s.x[i]);
        text += ' ';
    }
    text += "624";
    std::istringstream in(text);
    std::mt19937 engine;
    in >> engine;
    if (in.fail()) throw std::runtime_error("could not load the generator state");
    return engine;
}

}  // namespace

HostDataset make_exponential_dataset(int64_t n, int64_t d, double lambda, double max_value) {
    if (n <= 0 || d <= 0) throw std::runtime_error("No points were generated.");
    HostDataset ds;
    ds.n = n;
    ds.d = d;
    ds.name = "Exponential_" + std::to_string(n) + "_" + std::to_string(d) + "_" + std::to_string(lambda);
    ds.values.resize(static_cast<size_t>(n) * static_cast<size_t>(d));
    uint16_t* out = ds.values.data();
    const size_t total = ds.values.size();
    constexpr uint32_t kSeed = 2137834274u;

    // The reference draws all N*D values from ONE sequential engine, which at 4e9 values takes
    // minutes.  libstdc++'s exponential_distribution<double> consumes exactly two 32-bit engine
    // outputs per draw, so value k starts at engine position 2k as long as no earlier draw was
    // rejected.  The engine's state is advanced by a vectorised restatement of the MT19937
    // recurrence (mt_twist, many times faster than drawing), which leaves a state snapshot at every
    // chunk boundary; the other threads load snapshots into std::mt19937 engines and draw the chunks
    // with the standard distribution.  If ANY draw anywhere is
    // rejected the positions after it shift and the whole dataset is redone sequentially.  The
    // stream is bit-identical either way.
    const int threads = omp_get_max_threads();
    bool parallel_ok = false;
    if (threads > 1 && total >= (size_t(1) << 20)) {
        constexpr size_t kChunk = 312 * 2048;  // draws per chunk: 2 * kChunk outputs = 2048 whole state blocks
        const size_t chunks = (total + kChunk - 1) / kChunk;
        // One thread walks the state (vectorised twists only) and hands every chunk to the team as a
        // task the moment its snapshot exists; the others draw the chunks with the standard engine and
        // distribution meanwhile.  Chunk c starts at output 2 * c * kChunk, a multiple of 624: its
        // snapshot is the state after that many outputs' worth of twists, about to be twisted once
        // more by the chunk's first draw.
        std::vector<MtState> snaps(chunks);
        std::atomic<long long> rejections{0};
#pragma omp parallel
#pragma omp single
        {
            MtState st;
            mt_seed(st, kSeed);
            for (size_t c = 0; c < chunks; ++c) {
                snaps[c] = st;
#pragma omp task firstprivate(c) shared(snaps, rejections)
                {
                    if (!rejections.load(std::memory_order_relaxed)) {
                        std::mt19937 engine = engine_from_state(snaps[c]);
                        std::exponential_distribution<double> dist(lambda);
                        const size_t begin = c * kChunk, end = std::min(total, begin + kChunk);
                        for (size_t i = begin; i < end; ++i) {
                            const double v = dist(engine);
                            if (v < 0.0 || v > max_value) {
                                rejections.fetch_add(1, std::memory_order_relaxed);
                                break;
                            }
                            out[i] = float_to_half_rn(static_cast<float>(v));
                        }
                    }
                }
                if (c + 1 < chunks)
                    for (size_t k = 0; k < 2 * kChunk / 624; ++k) mt_twist(st);
            }
        }
        parallel_ok = rejections.load() == 0;
    }
    if (!parallel_ok) {
        std::mt19937 engine(kSeed);
        std::exponential_distribution<double> dist(lambda);
        for (size_t i = 0; i < total; ++i) {
            double v = dist(engine);
            while (v < 0.0 || v > max_value) v = dist(engine);
            out[i] = float_to_half_rn(static_cast<float>(v));
        }
    }
    return ds;
}

std::string dataset_name_from_path(const std::string& path) {
    const size_t slash = path.find_last_of("/\\");
    std::string file = path.substr(slash + 1);  // npos + 1 == 0
    const size_t dot = file.find_last_of(".");
    return file.substr(0, dot);
}

namespace {

// Converts one token like std::stod: leading white space skipped, trailing
// characters ignored, no digits -> invalid_argument, overflow -> out_of_range.
double parse_token_strtod(const char* begin, const char* end) {
    char buf[64];
    const size_t len = static_cast<size_t>(end - begin);
    std::string big;
    const char* z;
    if (len < sizeof(buf)) {
        std::memcpy(buf, begin, len);
        buf[len] = 0;
        z = buf;
    } else {
        big.assign(begin, end);
        z = big.c_str();
    }
    char* stop = nullptr;
    errno = 0;
    const double v = std::strtod(z, &stop);
    if (stop == z) throw std::invalid_argument("stod");
    if (errno == ERANGE) throw std::out_of_range("stod");
    return v;
}

// The same result, several times faster for ordinary decimal tokens: std::from_chars (correctly
// rounded, like strtod).  Everything it treats differently from strtod -- a leading '+', hexadecimal
// floats, values that overflow or underflow (where strtod reports ERANGE), empty tokens -- goes to the
// strtod path above, so the outcome, errors included, is always std::stod's.
double parse_token(const char* begin, const char* end) {
    const char* p = begin;
    while (p < end && (*p == ' ' || (*p >= '\t' && *p <= '\r'))) ++p;
    if (p < end && *p != '+') {
        double v = 0.0;
        const std::from_chars_result r = std::from_chars(p, end, v, std::chars_format::general);
        const bool hex_prefix = r.ptr < end && (*r.ptr == 'x' || *r.ptr == 'X');
        if (r.ec == std::errc() && r.ptr != p && !hex_prefix) {
            const double a = v < 0 ? -v : v;
            if (a >= 2.2250738585072014e-308 || a == 0.0) {
                if (a != 0.0) return v;
                // a true zero, or an underflow that strtod would report: look for a non-zero digit
                bool nonzero = false;
                for (const char* q = p; q < r.ptr && *q != 'e' && *q != 'E'; ++q) nonzero |= (*q >= '1' && *q <= '9');
                if (!nonzero) return v;
            }
        }
    }
    return parse_token_strtod(begin, end);
}

// Number of ','-separated tokens std::getline would deliver for this line.
int64_t count_tokens(const char* b, const char* e) {
    if (b == e) return 0;
    int64_t c = 1;
    for (const char* p = b; p < e; ++p)
        if (*p == ',') ++c;
    if (e[-1] == ',') --c;  // getline yields no empty token after a trailing delimiter
    return c;
}

}  // namespace

HostDataset read_csv_dataset(const std::string& path) {
    if (path.empty()) throw std::invalid_argument("filepath must be set.");
    std::string text;
    {
        FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) throw std::ios_base::failure("Failed to open file: " + path);
        std::fseek(f, 0, SEEK_END);
        const long size = std::ftell(f);
        std::fseek(f, 0, SEEK_SET);
        if (size > 0) {
            text.resize(static_cast<size_t>(size));
            const size_t got = std::fread(&text[0], 1, text.size(), f);
            text.resize(got);
        } else {  // not seekable: read what comes
            char buf[1 << 16];
            size_t got;
            while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
        }
        std::fclose(f);
    }

    // Line table (a final line without '\n' counts; an empty tail after the last '\n' does not).
    std::vector<std::pair<size_t, size_t>> lines;
    size_t pos = 0;
    while (pos < text.size()) {
        const void* nl = std::memchr(text.data() + pos, '\n', text.size() - pos);
        const size_t end = nl ? static_cast<size_t>(static_cast<const char*>(nl) - text.data()) : text.size();
        lines.emplace_back(pos, end);
        pos = end + 1;
    }
    if (lines.empty()) throw std::runtime_error("No points were generated.");

    HostDataset ds;
    ds.name = dataset_name_from_path(path);
    ds.n = static_cast<int64_t>(lines.size());
    ds.d = count_tokens(text.data() + lines[0].first, text.data() + lines[0].second);
    if (ds.d == 0) throw std::runtime_error("No points were generated.");
    ds.values.assign(static_cast<size_t>(ds.n) * static_cast<size_t>(ds.d), 0);

    int64_t bad_line = -1;
    int bad_kind = 0;  // 1 ragged, 2 parse
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < ds.n; ++r) {
        const char* b = text.data() + lines[static_cast<size_t>(r)].first;
        const char* e = text.data() + lines[static_cast<size_t>(r)].second;
        int kind = 0;
        if (count_tokens(b, e) != ds.d) {
            kind = 1;
        } else {
            uint16_t* out = &ds.values[static_cast<size_t>(r) * static_cast<size_t>(ds.d)];
            const char* p = b;
            for (int64_t c = 0; c < ds.d && !kind; ++c) {
                const char* q = static_cast<const char*>(std::memchr(p, ',', static_cast<size_t>(e - p)));
                if (!q) q = e;
                try {
                    out[c] = float_to_half_rn(static_cast<float>(parse_token(p, q)));
                } catch (const std::exception&) {
                    kind = 2;
                }
                p = q + 1;
            }
        }
        if (kind) {
#pragma omp critical
            if (bad_line < 0 || r < bad_line) {
                bad_line = r;
                bad_kind = kind;
            }
        }
    }
    if (bad_line >= 0) {
        if (bad_kind == 1)
            throw std::runtime_error("Dimensions of subsequent points didn't match the first point (line " +
                                     std::to_string(bad_line) + ")");
        throw std::invalid_argument("Failed to parse a value from dataset at line " + std::to_string(bad_line));
    }
    return ds;
}

}  // namespace fasted
