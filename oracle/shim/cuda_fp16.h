/* Host stand-in for <cuda_fp16.h> (see shim/cuda_runtime.h): `half` is the compiler's IEEE
 * binary16 type; conversions round to nearest even, as the device intrinsics do. */
#pragma once
typedef _Float16 half;
static inline float __half2float(half h) { return (float)h; }
static inline half __float2half(float f) { return (half)f; }
