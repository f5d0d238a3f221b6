// Writes ../data/points.bin and ../data/cpu_points.bin for <n> generators in the reference's layouts
// (what its test/ppgen.cu does for a fixed count): the 256-row affine table and the generators as
// Jacobian records.  Built against include/grape_veneer.hpp only.
#include <cstdlib>

#include "grape_veneer.hpp"

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  const uint n = (uint)atol(argv[1]);
  const char* dir = argc > 2 ? argv[2] : "../data";
  try {
    affine_t* points = (affine_t*)grape_veneer::dev_alloc((size_t)n * 256 * sizeof(affine_t));
    std::vector<bn128> cpu_points = precompute_generators(n, 256, points);
    savebin(std::string(dir) + "/points.bin", points, (size_t)n * 256 * sizeof(affine_t));
    savebin(std::string(dir) + "/cpu_points.bin", cpu_points.data(), cpu_points.size() * sizeof(bn128), false);
  } catch (const std::exception& e) {
    fprintf(stderr, "make_points: %s\n", e.what());
    return 1;
  }
  return 0;
}
