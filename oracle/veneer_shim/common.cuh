// Common part of the stand-in headers: the reference's host API through include/grape_veneer.hpp, plus
// the few things its drivers take from the CUDA side of its headers directly (the event-timer macros of
// include/ioutils.cuh:24-38 and the int_to_fr / uint_to_fr kernels of include/fr-tensor.cuh:17-18, which
// test/matmul.cu and test/eleWiseMul.cu launch themselves).  TEST INFRASTRUCTURE ONLY.
#pragma once
#include <cuda_runtime.h>

#include <cassert>
#include <cmath>

#include "grape_veneer.hpp"
#include "../../grape_b200/csrc/field.cuh"
using namespace std;

#ifndef CUDA_TIMER_START
#define CUDA_TIMER_START(timer_name)                 \
  cudaEvent_t timer_name##_start, timer_name##_stop; \
  cudaEventCreate(&timer_name##_start);              \
  cudaEventCreate(&timer_name##_stop);               \
  cudaEventRecord(timer_name##_start, 0);
#define CUDA_TIMER_STOP(timer_name)                                                      \
  cudaEventRecord(timer_name##_stop, 0);                                                 \
  cudaEventSynchronize(timer_name##_stop);                                               \
  float timer_name##_elapsed_ms = 0.0f;                                                  \
  cudaEventElapsedTime(&timer_name##_elapsed_ms, timer_name##_start, timer_name##_stop); \
  printf("%s elapsed: %f ms\n", #timer_name, timer_name##_elapsed_ms);                   \
  cudaEventDestroy(timer_name##_start);                                                  \
  cudaEventDestroy(timer_name##_stop);
#endif

#ifndef GRAPE_SHIM_KERNELS
#define GRAPE_SHIM_KERNELS
// launched by the drivers on the default stream; the library's stream is synchronised with the device
// by the CUDA_DEBUG that follows every such launch in those drivers
static __global__ void int_to_fr(int* input, fr_t* out, size_t N) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) grape::fe_from_i32<grape::FrParams>(input[i]).store(out + i);
}
static __global__ void uint_to_fr(uint* input, fr_t* out, size_t N) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) grape::fe_from_u32<grape::FrParams>(input[i]).store(out + i);
}
#endif
