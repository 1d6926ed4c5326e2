// Harness around the reference's own host-side loader headers (compiled
// unmodified from the reference checkout; see oracle/Makefile target `ref`).
// TEST INFRASTRUCTURE: it exists to pin the CPU oracle's dataset functions
// against what the reference itself produces.
//
//   ref_datagen exp <N> <D> <lambda> <max> <dimFactor> <pointsFactor> <out.bin>
//   ref_datagen csv <file> <dimFactor> <pointsFactor> <out.bin>
//
// out.bin: four little-endian int64 (paddedN, N, paddedD, D) followed by
// paddedN*paddedD binary16 values, row-major.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "DataLoader/ExponentialPointGenerator.hpp"
#include "DataLoader/FilePointGenerator.hpp"
#include "DataLoader/PointListBuilder.hpp"

static int dump(Points::PointList<half_float::half>& pl, const char* path) {
    FILE* f = std::fopen(path, "wb");
    if (!f) return 2;
    int64_t hdr[4] = {pl.getNumPoints(), pl.getActualNumPoints(), pl.getDimensions(),
                      pl.getActualDimensions()};
    std::fwrite(hdr, sizeof(int64_t), 4, f);
    static_assert(sizeof(half_float::half) == 2, "half must be 2 bytes");
    std::fwrite(pl.values.data(), 2, pl.values.size(), f);
    std::fclose(f);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 2 && std::strcmp(argv[1], "exp") == 0 && argc == 9) {
        SimSearch::ExponentialPointGenerator gen(std::stoi(argv[2]), std::stoi(argv[3]),
                                                 std::stod(argv[4]), std::stod(argv[5]));
        Points::PointListBuilder<half_float::half> b(&gen);
        std::printf("name %s\n", b.getDatasetName().c_str());
        auto pl = b.build(std::stoi(argv[6]), std::stoi(argv[7]));
        return dump(pl, argv[8]);
    }
    if (argc >= 2 && std::strcmp(argv[1], "csv") == 0 && argc == 6) {
        SimSearch::FilePointGenerator gen(argv[2], ',');
        Points::PointListBuilder<half_float::half> b(&gen);
        std::printf("name %s\n", b.getDatasetName().c_str());
        auto pl = b.build(std::stoi(argv[3]), std::stoi(argv[4]));
        return dump(pl, argv[5]);
    }
    std::fprintf(stderr, "usage: see the header of ref_datagen.cpp\n");
    return 1;
}
