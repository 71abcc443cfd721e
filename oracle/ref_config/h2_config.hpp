// TEST INFRASTRUCTURE ONLY.  Stand-in for the build-generated configuration
// header of the reference (its build system is not run): CPU-only, no GPU,
// no DaCe.  Only used by the recipe that compiles the reference's CPU path.
#pragma once
#define H2_VERSION_MAJOR 0
#define H2_VERSION_MINOR 0
#define H2_VERSION_PATCH 0
#define H2_VERSION "0.0.0"
#define H2_HAS_HALF 0
#define H2_HAS_OPENMP 0
#define H2_HAS_CUDA 0
#define H2_HAS_ROCM 0
#define H2_HAS_MPI 1
#define H2_HAS_DACE 0
#define H2_PRETTY_FUNCTION __PRETTY_FUNCTION__
#define H2_RESTRICT __restrict__
#define H2_NOEXCEPT noexcept
#define H2_CXX_STANDARD 17
#define H2_CONSTEXPR_FUNC
#define H2_NODISCARD
