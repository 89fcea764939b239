// Row-wise helpers shared by the kernels that process one token row per CTA: 8-element vector I/O for the three
// activation types (float32, bfloat16, float16) and CTA-wide reductions.
#pragma once
#include "common.cuh"

namespace el {
namespace rowio {

template <typename T> struct Io;
template <> struct Io<float> {
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw load_raw(const float* p) {
        Raw r;
        r.a = *reinterpret_cast<const float4*>(p);
        r.b = *reinterpret_cast<const float4*>(p + 4);
        return r;
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float v[8]) {
        v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
    }
    static __device__ __forceinline__ Raw pack(const float v[8]) {
        Raw r;
        r.a = make_float4(v[0], v[1], v[2], v[3]);
        r.b = make_float4(v[4], v[5], v[6], v[7]);
        return r;
    }
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ void round8(float*) {}
    static __device__ __forceinline__ void load8(const float* p, float v[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store8(float* p, const float v[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Io<__nv_bfloat16> {
    struct Raw { uint4 a; };
    static __device__ __forceinline__ Raw load_raw(const __nv_bfloat16* p) { return Raw{*reinterpret_cast<const uint4*>(p)}; }
    static __device__ __forceinline__ void unpack(const Raw& r, float v[8]) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    // values that are already bfloat16-representable: packing is exact
    static __device__ __forceinline__ Raw pack(const float v[8]) {
        return Raw{make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]))};
    }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    // Eight values rounded to bfloat16 in place, two per packed conversion (the single-value conversion runs on the
    // slow conversion unit, the packed one does not).
    static __device__ __forceinline__ void round8(float v[8]) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const uint32_t p = pack_bf16x2(v[i], v[i + 1]);
            v[i] = __uint_as_float(p << 16);
            v[i + 1] = __uint_as_float(p & 0xFFFF0000u);
        }
    }
    static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float v[8]) { unpack(load_raw(p), v); }
    static __device__ __forceinline__ void store8(__nv_bfloat16* p, const float v[8]) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                                  pack_bf16x2(v[6], v[7]));
    }
};
template <> struct Io<__half> {
    struct Raw { uint4 a; };
    static __device__ __forceinline__ Raw load_raw(const __half* p) { return Raw{*reinterpret_cast<const uint4*>(p)}; }
    static __device__ __forceinline__ void unpack(const Raw& r, float v[8]) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ Raw pack(const float v[8]) {
        return Raw{make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]), pack_f16x2(v[6], v[7]))};
    }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ void round8(float v[8]) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const uint32_t p = pack_f16x2(v[i], v[i + 1]);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&p));
            v[i] = f.x;
            v[i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void load8(const __half* p, float v[8]) { unpack(load_raw(p), v); }
    static __device__ __forceinline__ void store8(__half* p, const float v[8]) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]),
                                                  pack_f16x2(v[6], v[7]));
    }
};

__device__ __forceinline__ void load8_w(const float* p, float v[8]) { Io<float>::load8(p, v); }

constexpr int RN_THREADS = 256;

// Sum over the CTA; every thread gets the result.  `red` holds one double per warp.
__device__ __forceinline__ double block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < RN_THREADS / 32; ++i) t += red[i];     // same order in every thread
    __syncthreads();
    return t;
}

__device__ __forceinline__ float block_max_f(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < RN_THREADS / 32; ++i) t = fmaxf(t, red[i]);
    __syncthreads();
    return t;
}

}  // namespace rowio
}  // namespace el
