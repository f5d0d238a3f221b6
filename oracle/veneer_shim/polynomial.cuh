// Stand-in for the reference header of the same name: a reference driver (test/*.cu, compiled where it
// lies, unmodified) that includes it gets the reference's host API from include/grape_veneer.hpp, i.e.
// from libgrape_b200.so, instead of the reference's own CUDA.  TEST INFRASTRUCTURE ONLY.
#pragma once
#include "common.cuh"
