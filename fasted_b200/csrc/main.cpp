// Command-line front end with the reference's argument handling
// (source/main.cu:143-186):
//   main -e <numPoints> <numDimensions> <epsilon>     seeded synthetic dataset (lambda 40, max 10.0)
//   main <filename> <epsilon>                         CSV dataset
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <string>

#include "fasted.h"

static double parse_double(const std::string& s) {
    try {
        return std::stod(s);
    } catch (const std::invalid_argument&) {
        throw std::invalid_argument("Invalid argument: unable to parse double");
    } catch (const std::out_of_range&) {
        throw std::out_of_range("Out of range: the number is too large or too small for a double");
    }
}

int main(int argc, char* argv[]) {
    bool synthetic = false;
    for (int i = 1; i < argc; ++i)
        if (std::strcmp(argv[i], "-e") == 0) {
            synthetic = true;
            break;
        }
    if (synthetic) {
        if (argc != 5) {
            std::cerr << "Usage: " << argv[0] << " -e <numPoints> <numDimensions> <epsilon>" << std::endl;
            return 1;
        }
        const int n = std::stoi(argv[2]);
        const int d = std::stoi(argv[3]);
        const double eps = parse_double(argv[4]);
        runFromExponentialDataset(n, d, 40, 10.0, eps, false);
    } else {
        if (argc != 3) {
            std::cerr << "Usage: " << argv[0] << " <filename> <epsilon>" << std::endl;
            return 1;
        }
        const double eps = parse_double(argv[2]);
        runFromFile(argv[1], eps, false);
    }
    releaseResources();
    return 0;
}
