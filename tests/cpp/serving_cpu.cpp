// CPU-side check of include/sllm_serving.hpp: it compiles, and balancedAssignment deals sequences as documented.
// Prints the assignment for the lengths given on the command line: argv[1] = world, argv[2..] = lengths.
#include <cstdlib>
#include <iostream>
#include "sllm_serving.hpp"
int main(int argc, char** argv) {
    if (argc < 3) return 2;
    std::vector<size_t> lens;
    for (int i = 2; i < argc; ++i) lens.push_back(std::strtoull(argv[i], nullptr, 10));
    for (const auto& part : balancedAssignment(lens, std::strtoull(argv[1], nullptr, 10))) {
        for (size_t g : part) std::cout << g << ' ';
        std::cout << '\n';
    }
    try { balancedAssignment(lens, 0); return 3; } catch (const std::invalid_argument&) {}
    return 0;
}
