// Host shim placed IN FRONT of the reference project's oracle kernel templates when they are compiled
// for the CPU (see oracle/Makefile).  TEST INFRASTRUCTURE ONLY.
//
// The reference's oracle kernels (src/cuda/cubic_reference.cuh:3-40,
// src/cuda/strassen_reference_l1.cuh:5-117 and :119-183) are plain per-element scalar loops that use
// nothing of CUDA except the thread-index built-ins and one cutlass converter.  This header supplies
// those names so the unmodified template text compiles with g++.
#pragma once
#include <cstddef>
#include <cstdint>

#define __global__
struct ref_dim3 { unsigned x = 0, y = 0, z = 0; };
static thread_local ref_dim3 threadIdx, blockIdx;
static thread_local ref_dim3 blockDim = {1, 1, 1};

namespace cutlass {
template <typename To, typename From>
struct NumericConverter {
  To operator()(From const &v) const { return static_cast<To>(v); }
};
}  // namespace cutlass
