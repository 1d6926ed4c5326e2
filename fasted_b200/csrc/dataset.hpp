// Host-side dataset construction for the drop-in interface: the seeded
// Exponential generator and the CSV reader, both producing binary16 rows.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace fasted {

struct HostDataset {
    std::vector<uint16_t> values;  // n rows of d binary16 bit patterns, row-major, no padding
    int64_t n = 0;
    int64_t d = 0;
    std::string name;
};

// float -> binary16, round to nearest even.
uint16_t float_to_half_rn(float f);

// Same stream as the reference's ExponentialPointGenerator
// (source/DataLoader/ExponentialPointGenerator.hpp:11, 22-31, 42-52):
// std::mt19937 seeded with 2137834274, std::exponential_distribution<double>,
// values outside [0, max_value] redrawn, row-major order; then
// double -> float -> half (source/DataLoader/PointListBuilder.hpp:57-66).
// Name: "Exponential_<N>_<D>_<lambda>" (ExponentialPointGenerator.hpp:59-62).
HostDataset make_exponential_dataset(int64_t n, int64_t d, double lambda, double max_value);

// CSV with the reference's rules (source/DataLoader/FilePointGenerator.hpp:20-56,
// source/DataLoader/PointListBuilder.hpp:154-163): one point per line, ','
// separated, each token converted like std::stod, the first row fixes the
// dimension, any other length is an error.  Name = file stem
// (FilePointGenerator.hpp:58-68).  Throws std::runtime_error /
// std::ios_base::failure / std::invalid_argument like the reference.
HostDataset read_csv_dataset(const std::string& path);

// "<dir>/<stem>" -> "<stem>" without its extension.
std::string dataset_name_from_path(const std::string& path);

}  // namespace fasted
