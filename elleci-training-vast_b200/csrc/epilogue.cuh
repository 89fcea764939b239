// The scaling epilogue shared by the integer GEMM kernels: out = out_dtype(float(acc) * sc), where
// sc = (absmax[row*stride] / 127) * alpha is formed once per row in float32.
#pragma once
#include "common.cuh"

namespace el {

struct EpiParams {
    void* out;              // [R, ldo] of out_dtype
    long long ldo;          // row pitch in elements
    int out_dtype;          // EL_F16 / EL_BF16 / EL_F32 / EL_I32 (raw sums)
    const float* absmax;    // per row (stride 1) or one value (stride 0); nullptr means scale = alpha
    int absmax_stride;
    float alpha;
};

__device__ __forceinline__ float epi_row_scale(const EpiParams& e, int row) {
    if (e.absmax == nullptr) return e.alpha;
    const float a = e.absmax[(size_t)row * e.absmax_stride];
    return __fmul_rn(__fdiv_rn(a, 127.0f), e.alpha);
}

__device__ __forceinline__ void epi_store_one(const EpiParams& e, int row, int col, int acc, float sc) {
    const size_t o = (size_t)row * e.ldo + col;
    const float v = __fmul_rn((float)acc, sc);
    switch (e.out_dtype) {
        case EL_BF16: static_cast<__nv_bfloat16*>(e.out)[o] = __float2bfloat16_rn(v); break;
        case EL_F16: static_cast<__half*>(e.out)[o] = __float2half_rn(v); break;
        case EL_F32: static_cast<float*>(e.out)[o] = v; break;
        default: static_cast<int*>(e.out)[o] = acc; break;
    }
}

// Stores 32 consecutive columns of one row held in registers (the unit a tensor-memory load returns).
// `vec_ok`: the row pitch and base keep 16-byte alignment for this chunk.
__device__ __forceinline__ void epi_store_chunk32(const EpiParams& e, int row, int col0, int C, const uint32_t (&acc)[32],
                                                  float sc, bool vec_ok) {
    const size_t o = (size_t)row * e.ldo + col0;
    if (vec_ok && col0 + 32 <= C) {
        if (e.out_dtype == EL_BF16 || e.out_dtype == EL_F16) {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float lo = __fmul_rn((float)(int)acc[2 * i], sc), hi = __fmul_rn((float)(int)acc[2 * i + 1], sc);
                w[i] = (e.out_dtype == EL_BF16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
            }
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(e.out) + o);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        } else {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint32_t*>(e.out) + o);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int a = (int)acc[4 * i + j];
                    w[j] = (e.out_dtype == EL_F32) ? __float_as_uint(__fmul_rn((float)a, sc)) : (uint32_t)a;
                }
                dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < C) epi_store_one(e, row, col0 + i, (int)acc[i], sc);
    }
}

}  // namespace el
