// Harness around the reference's own GPU join (findPairs.cuh and everything it
// includes, compiled unmodified from the reference checkout for sm_100; see
// oracle/Makefile target `ref`).  TEST INFRASTRUCTURE: it produces the
// reference's pair list for a given binary16 matrix so that the product's
// output can be compared with it on the same inputs, and it reports the
// reference kernel's own timing on the same GPU.
//
//   ref_join <points.bin> <epsilon> <out_prefix>
//
// points.bin: two little-endian int64 (n, d) followed by n*d binary16 values.
// The values are handed to the reference's PointListBuilder through a
// PointGenerator (half -> double is exact, and the builder's
// double -> float -> half brings every value back unchanged); the builder pads
// exactly as the reference's run() asks (source/main.cu:205-209).
// Writes <out_prefix>.pairs ("q, c" lines, sorted) via the reference's own
// savePairs path and prints the reference's Results fields as one line
// "REF_RESULTS totalTime TFLOPS pairsFound pairsStored".
#include <cstdint>
#include <cstdio>
#include <optional>
#include <string>
#include <vector>

#include <cuda_fp16.h>

#include "DataLoader/PointGenerator.hpp"
#include "DataLoader/PointListBuilder.hpp"
#include "findPairs.cuh"

class BinaryHalfGenerator : public SimSearch::PointGenerator {
   public:
    explicit BinaryHalfGenerator(const char* path) {
        FILE* f = std::fopen(path, "rb");
        if (!f) throw std::runtime_error("cannot open input");
        int64_t hdr[2];
        if (std::fread(hdr, sizeof(int64_t), 2, f) != 2) throw std::runtime_error("short header");
        n_ = hdr[0];
        d_ = hdr[1];
        bits_.resize(static_cast<size_t>(n_ * d_));
        if (std::fread(bits_.data(), 2, bits_.size(), f) != bits_.size()) throw std::runtime_error("short body");
        std::fclose(f);
    }
    std::optional<std::vector<double>> next() override {
        if (row_ >= n_) return std::nullopt;
        std::vector<double> p(static_cast<size_t>(d_));
        for (int64_t k = 0; k < d_; ++k) {
            half_float::half h;
            std::memcpy(&h, &bits_[static_cast<size_t>(row_ * d_ + k)], 2);
            p[static_cast<size_t>(k)] = static_cast<double>(static_cast<float>(h));
        }
        ++row_;
        return p;
    }
    std::string getName() override { return "binary"; }

   private:
    int64_t n_ = 0, d_ = 0, row_ = 0;
    std::vector<uint16_t> bits_;
};

int main(int argc, char** argv) {
    if (argc != 4) {
        std::fprintf(stderr, "usage: ref_join <points.bin> <epsilon> <out_prefix>\n");
        return 1;
    }
    const double eps = std::stod(argv[2]);
    BinaryHalfGenerator gen(argv[1]);
    Points::PointListBuilder<half_float::half> builder(&gen);
    Mma::mmaShape bDims = SimSearch::GetBlockTileDims();
    auto pointList = builder.build(bDims.k, SimSearch::rasterizeSize * bDims.m);
    Mma::mmaShape padded{pointList.getNumPoints(), pointList.getNumPoints(), pointList.getDimensions()};
    Mma::mmaShape input{pointList.getActualNumPoints(), pointList.getActualNumPoints(),
                        pointList.getActualDimensions()};
    auto params = SimSearch::FindPairsParamsHost{eps, padded, input, pointList, true, false, std::string(argv[3])};
    SimSearch::Results r = SimSearch::FindPairs(params);
    SimSearch::releaseGlobalMemory();
    std::printf("REF_RESULTS %.6f %.6f %llu %llu\n", r.totalTime, r.TFLOPS, r.pairsFound, r.pairsStored);
    return 0;
}
