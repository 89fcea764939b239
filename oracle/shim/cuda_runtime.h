/*
 * Host stand-in for <cuda_runtime.h>, used ONLY by oracle/build_ref.sh to compile the reference's
 * own kernel sources for the CPU (test infrastructure, never part of the product library).
 * It gives the CUDA keywords and the few device intrinsics those kernels use a single-threaded
 * meaning: a kernel becomes a plain function, and the driver in ref_cpu_driver.inc calls it once
 * per emulated thread after setting blockIdx / threadIdx.
 */
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cfloat>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __restrict__
#define __shared__ static
#define __launch_bounds__(...)

struct shim_dim3 { unsigned x, y, z; };
typedef shim_dim3 dim3;
typedef shim_dim3 uint3;
static thread_local shim_dim3 blockIdx = {0, 0, 0};
static thread_local shim_dim3 threadIdx = {0, 0, 0};
static thread_local shim_dim3 blockDim = {1, 1, 1};
static thread_local shim_dim3 gridDim = {1, 1, 1};

struct float4 { float x, y, z, w; };

typedef void* cudaStream_t;
typedef int cudaError_t;
static const cudaError_t cudaSuccess = 0;
static inline cudaError_t cudaGetLastError() { return cudaSuccess; }
static inline const char* cudaGetErrorString(cudaError_t) { return "shim"; }

static inline int max(int a, int b) { return a > b ? a : b; }
static inline int min(int a, int b) { return a < b ? a : b; }

/* Single emulated thread: atomics are plain read-modify-writes, a shuffle returns its input. */
static inline unsigned atomicAnd(unsigned* p, unsigned v) { unsigned o = *p; *p = o & v; return o; }
static inline unsigned atomicOr(unsigned* p, unsigned v) { unsigned o = *p; *p = o | v; return o; }
static inline int atomicMax(int* p, int v) { int o = *p; if (v > o) *p = v; return o; }
static inline float __shfl_down_sync(unsigned, float v, int) { return v; }
static inline void __syncthreads() {}
static inline void __syncwarp() {}
static inline int __float_as_int(float f) { int i; std::memcpy(&i, &f, 4); return i; }
using std::isfinite;
