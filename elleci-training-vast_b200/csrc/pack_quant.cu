// Memory-bound kernels of the INT2 linear path: ternary packing / unpacking, per-token and per-tensor
// absmax int8 quantisation, gradient quantisation for the integer weight gradient.
// All of them stream their operands once with 16-byte accesses where the shape allows it.
#include "common.cuh"
#include "epilogue.cuh"

namespace el {

// ---------------------------------------------------------------------------------------------------------
// pack / ternarise / unpack
// ---------------------------------------------------------------------------------------------------------

// One thread per packed byte (four weights).
template <bool FROM_FLOAT>
__global__ void pack_kernel(const void* __restrict__ src, float gamma, uint8_t* __restrict__ Wp, int N, int K,
                            int pK, int pad_code) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)N * pK) return;
    const int n = (int)(t / pK), b = (int)(t % pK);
    uint32_t byte = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int k = b * 4 + j;
        uint32_t code = (uint32_t)pad_code;
        if (k < K) {
            int q;
            if (FROM_FLOAT) {
                const float w = static_cast<const float*>(src)[(size_t)n * K + k];
                float r = rintf(__fdiv_rn(w, gamma));     // round half to even
                r = fminf(1.0f, fmaxf(-1.0f, r));
                q = (r != r) ? 0 : (int)r;
            } else {
                q = static_cast<const int8_t*>(src)[(size_t)n * K + k];
                q = max(-1, min(1, q));
            }
            code = (uint32_t)(q + 1);
        }
        byte |= code << (2 * j);
    }
    Wp[t] = (uint8_t)byte;
}

template <typename OutT>
__device__ __forceinline__ OutT from_int(int v);
template <> __device__ __forceinline__ float from_int<float>(int v) { return (float)v; }
template <> __device__ __forceinline__ __half from_int<__half>(int v) { return __float2half((float)v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_int<__nv_bfloat16>(int v) { return __float2bfloat16((float)v); }
template <> __device__ __forceinline__ int8_t from_int<int8_t>(int v) { return (int8_t)v; }

template <typename OutT>
__global__ void unpack_kernel(const uint8_t* __restrict__ Wp, OutT* __restrict__ out, int N, int K, int pK) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)N * pK) return;
    const int n = (int)(t / pK), b = (int)(t % pK);
    const uint32_t byte = Wp[t];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int k = b * 4 + j;
        if (k < K) out[(size_t)n * K + k] = from_int<OutT>(decode2(byte >> (2 * j)));
    }
}

// Vector forms for matrices whose rows are whole 16-weight words (K % 16 == 0) at 16-byte aligned addresses: a thread
// takes one 32-bit word of codes (16 weights), consecutive threads consecutive words, so a warp reads 128 and writes 512
// (int8) to 2048 (float32) contiguous bytes per step; four steps are in flight per thread.
template <typename OutT> __device__ __forceinline__ void store16_ternary(OutT* out, const uint32_t w[4]);
template <> __device__ __forceinline__ void store16_ternary<int8_t>(int8_t* out, const uint32_t w[4]) {
    *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float s8_of(uint32_t word, int i) { return (float)(int)(int8_t)(word >> (8 * i)); }
template <> __device__ __forceinline__ void store16_ternary<__nv_bfloat16>(__nv_bfloat16* out, const uint32_t w[4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
        reinterpret_cast<uint4*>(out)[h] =
            make_uint4(pack_bf16x2(s8_of(w[2 * h], 0), s8_of(w[2 * h], 1)), pack_bf16x2(s8_of(w[2 * h], 2), s8_of(w[2 * h], 3)),
                       pack_bf16x2(s8_of(w[2 * h + 1], 0), s8_of(w[2 * h + 1], 1)), pack_bf16x2(s8_of(w[2 * h + 1], 2), s8_of(w[2 * h + 1], 3)));
}
template <> __device__ __forceinline__ void store16_ternary<__half>(__half* out, const uint32_t w[4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
        reinterpret_cast<uint4*>(out)[h] =
            make_uint4(pack_f16x2(s8_of(w[2 * h], 0), s8_of(w[2 * h], 1)), pack_f16x2(s8_of(w[2 * h], 2), s8_of(w[2 * h], 3)),
                       pack_f16x2(s8_of(w[2 * h + 1], 0), s8_of(w[2 * h + 1], 1)), pack_f16x2(s8_of(w[2 * h + 1], 2), s8_of(w[2 * h + 1], 3)));
}
template <> __device__ __forceinline__ void store16_ternary<float>(float* out, const uint32_t w[4]) {
#pragma unroll
    for (int h = 0; h < 4; ++h)
        reinterpret_cast<float4*>(out)[h] = make_float4(s8_of(w[h], 0), s8_of(w[h], 1), s8_of(w[h], 2), s8_of(w[h], 3));
}

template <typename OutT>
__global__ void __launch_bounds__(256)
unpack_vec_kernel(const uint32_t* __restrict__ Wp, OutT* __restrict__ out, long long n_words) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += 4 * stride) {
        uint32_t code[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) code[j] = (i + j * stride < n_words) ? __ldg(Wp + i + j * stride) : 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (i + j * stride < n_words) {
                uint32_t w[4];
                decode16(code[j], w);
                store16_ternary<OutT>(out + (i + j * stride) * 16, w);
            }
        }
    }
}

// Ternarise + pack, vector form (K % 16 == 0, 16-byte aligned rows): a thread takes 16 consecutive weights as four
// 16-byte loads, interleaved over the warp so that every load instruction reads 512 contiguous bytes, and writes the
// four packed bytes it produced (byte j*32 + lane of the warp's 128-byte output run).
__global__ void __launch_bounds__(256)
ternarize_pack_vec_kernel(const float4* __restrict__ src, float gamma, uint8_t* __restrict__ Wp, long long n_bytes) {
    const int lane = threadIdx.x & 31;
    const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long b0 = warp_id * 128; b0 < n_bytes; b0 += n_warps * 128) {      // 128 packed bytes = 512 weights per warp and step
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long b = b0 + j * 32 + lane;
            v[j] = (b < n_bytes) ? __ldg(src + b) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long b = b0 + j * 32 + lane;
            if (b < n_bytes) {
                const float w4[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                uint32_t byte = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float r = rintf(__fdiv_rn(w4[i], gamma));     // round half to even
                    r = fminf(1.0f, fmaxf(-1.0f, r));
                    const int q = (r != r) ? 0 : (int)r;
                    byte |= (uint32_t)(q + 1) << (2 * i);
                }
                Wp[b] = (uint8_t)byte;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// per-token quantisation: one CTA per row
// ---------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) red[w] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    v = (l < nw) ? red[l] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    return v;
}


template <typename T>
__device__ __forceinline__ void load8(const T* p, float v[8]);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float v[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float v[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        const float2 f = __half22float2(h);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float v[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Eight consecutive elements as loaded (16 bytes of a 2-byte type, 32 bytes of float): rows are kept in registers in this
// form between the absmax pass and the quantisation pass.
template <typename T> struct Raw8 { uint4 a; };
template <> struct Raw8<float> { uint4 a, b; };
template <typename T> __device__ __forceinline__ Raw8<T> raw_load(const T* p) {
    Raw8<T> r;
    r.a = *reinterpret_cast<const uint4*>(p);
    return r;
}
template <> __device__ __forceinline__ Raw8<float> raw_load<float>(const float* p) {
    Raw8<float> r;
    r.a = *reinterpret_cast<const uint4*>(p);
    r.b = *reinterpret_cast<const uint4*>(p + 4);
    return r;
}
__device__ __forceinline__ void raw_unpack(const Raw8<__nv_bfloat16>& r, float v[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ void raw_unpack(const Raw8<__half>& r, float v[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void raw_unpack(const Raw8<float>& r, float v[8]) {
    v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
    v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y); v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
}

__device__ __forceinline__ int quant_half_even(float x, float s) {
    float r = rintf(__fmul_rn(x, s));
    r = fminf(127.0f, fmaxf(-128.0f, r));
    return (int)r;
}

// VEC: the row pitch and base allow 8-element vector loads and 8-byte stores.
// MODE 0: absmax + quantise; 1: raw absmax only; 2: quantise with the raw absmax found in row_absmax.
// ROW_CACHE: vectors of 8 elements a thread keeps in registers between the passes (2 for rows up to 4096 elements: fewer
// registers, more resident CTAs; 6 for rows up to 12288; longer rows re-read their tail).
template <typename T, bool VEC, int MODE, int ROW_CACHE>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const T* __restrict__ x, long long ldx, int8_t* __restrict__ q, float* __restrict__ row_absmax, int K,
                     float eps, const float* __restrict__ fold_absmax, float* __restrict__ fold_max) {
    __shared__ float red[8];
    const int m = blockIdx.x;
    const T* xr = x + (size_t)m * ldx;
    int8_t* qr = q + (size_t)m * K;
    float amax = 0.0f;
    bool row_finite = false;        // known to hold no infinity: the unchecked conversion is exact
    Raw8<T> cache[ROW_CACHE];
    if (MODE == 2) {
        amax = row_absmax[m];
        __syncthreads();            // every thread has read the raw value before thread 0 floors it in place
    } else {
        if (VEC) {
            // The row is read from memory once: up to ROW_CACHE vectors per thread stay in registers for the second pass.
            // fmaxf drops NaN operands and keeps infinities: only a row that holds an infinity needs the checked pass
#pragma unroll
            for (int c = 0; c < ROW_CACHE; ++c) {
                const int k = (threadIdx.x + c * 256) * 8;
                if (k < K) {
                    cache[c] = raw_load<T>(xr + k);
                    float v[8];
                    raw_unpack(cache[c], v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
                }
            }
            for (int k = (threadIdx.x + ROW_CACHE * 256) * 8; k < K; k += 256 * 8) {
                float v[8];
                load8<T>(xr + k, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            }
            amax = block_max(amax, red);
            if (!(amax <= 3.402823466e38f)) {          // same value in every thread of the CTA
                amax = 0.0f;
                for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
                    float v[8];
                    load8<T>(xr + k, v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(finite_or_zero(v[i])));
                }
            } else {
                row_finite = true;
            }
        } else {
            for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(finite_or_zero(to_float<T>(xr[k]))));
        }
        if (!row_finite) amax = block_max(amax, red);
    }
    if (MODE == 1) {
        if (threadIdx.x == 0) row_absmax[m] = amax;
        return;
    }
    const float a = fmaxf(amax, eps);
    const float s = __fdiv_rn(127.0f, a);
    if (threadIdx.x == 0) {
        row_absmax[m] = a;
        if (fold_max != nullptr) {
            const float g = __fmul_rn(amax, __fdiv_rn(fold_absmax[m], 127.0f));
            if (g > 0.0f) atomicMax(reinterpret_cast<int*>(fold_max), __float_as_int(g));
        }
    }
    if (VEC) {
        // second read of the row: served by L1/L2.  q8_sat rounds, clamps and turns NaN into 0.
        if (row_finite) {           // MODE 0 only: the cached vectors are valid
#pragma unroll
            for (int c = 0; c < ROW_CACHE; ++c) {
                const int k = (threadIdx.x + c * 256) * 8;
                if (k < K) {
                    float v[8];
                    raw_unpack(cache[c], v);
                    int qi[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) qi[i] = q8_sat(__fmul_rn(v[i], s));
                    *reinterpret_cast<uint2*>(qr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
                }
            }
            for (int k = (threadIdx.x + ROW_CACHE * 256) * 8; k < K; k += 256 * 8) {
                float v[8];
                load8<T>(xr + k, v);
                int qi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) qi[i] = q8_sat(__fmul_rn(v[i], s));
                *reinterpret_cast<uint2*>(qr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
            }
        } else {
            for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
                float v[8];
                load8<T>(xr + k, v);
                int qi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) qi[i] = q8_sat(__fmul_rn(finite_or_nan(v[i]), s));
                *reinterpret_cast<uint2*>(qr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
            }
        }
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x)
            qr[k] = (int8_t)quant_half_even(finite_or_zero(to_float<T>(xr[k])), s);
    }
}

// Per-token quantisation whose int8 output is permuted inside every group of 16 reduction indices (even indices
// first, then odd): the operand layout that matches decode16_deint.  One CTA per row; K % 16 == 0.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_perm_kernel(const T* __restrict__ x, long long ldx, int8_t* __restrict__ q, float* __restrict__ row_absmax,
                          int K, float eps) {
    __shared__ float red[8];
    // A kernel launched behind this one as a programmatic dependent may start its own preamble now (it waits for this
    // grid to complete before it reads q or row_absmax); without such a dependent this does nothing.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int m = blockIdx.x;
    const T* xr = x + (size_t)m * ldx;
    int8_t* qr = q + (size_t)m * K;
    float amax = 0.0f;
    for (int k = threadIdx.x * 16; k < K; k += blockDim.x * 16) {
        float v[16];
        load8<T>(xr + k, v);
        load8<T>(xr + k + 8, v + 8);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));       // drops NaN, keeps infinities
    }
    amax = block_max(amax, red);
    const bool row_finite = amax <= 3.402823466e38f;      // same value in every thread of the CTA
    if (!row_finite) {
        amax = 0.0f;
        for (int k = threadIdx.x * 16; k < K; k += blockDim.x * 16) {
            float v[16];
            load8<T>(xr + k, v);
            load8<T>(xr + k + 8, v + 8);
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(finite_or_zero(v[i])));
        }
        amax = block_max(amax, red);
    }
    const float a = fmaxf(amax, eps);
    const float s = __fdiv_rn(127.0f, a);
    if (threadIdx.x == 0) row_absmax[m] = a;
    for (int k = threadIdx.x * 16; k < K; k += blockDim.x * 16) {
        float v[16];
        load8<T>(xr + k, v);
        load8<T>(xr + k + 8, v + 8);
        int qi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) qi[i] = q8_sat(__fmul_rn(row_finite ? v[i] : finite_or_nan(v[i]), s));
        uint32_t w[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int s0 = (g < 2) ? 8 * g : 8 * (g - 2) + 1;      // output bytes 4g..4g+3 take sources s0, s0+2, s0+4, s0+6
            w[g] = pack4_s8(qi[s0], qi[s0 + 2], qi[s0 + 4], qi[s0 + 6]);
        }
        *reinterpret_cast<uint4*>(qr + k) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// ---------------------------------------------------------------------------------------------------------
// per-tensor quantisation (the reference CUDA path's rule)
// ---------------------------------------------------------------------------------------------------------

// The three per-tensor kernels take the tensor as 16-element vectors (two 16-byte loads of 16-bit data, one 16-byte
// store of int8) over the part that allows it (`n_vec` vectors: the whole tensor when its base is 16-byte aligned, less
// the tail) and element by element over the rest.
template <typename T>
__global__ void __launch_bounds__(256)
tensor_absmax_kernel(const T* __restrict__ x, float* __restrict__ absmax, long long size, long long n_vec) {
    __shared__ float red[8];
    float amax = 0.0f;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
#pragma unroll 4
    for (long long i = tid; i < n_vec; i += stride) {
        float v[16];
        load8<T>(x + i * 16, v);
        load8<T>(x + i * 16 + 8, v + 8);
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(finite_or_zero(v[j])));
    }
    for (long long i = n_vec * 16 + tid; i < size; i += stride) amax = fmaxf(amax, fabsf(finite_or_zero(to_float<T>(x[i]))));
    amax = block_max(amax, red);
    if (threadIdx.x == 0 && amax > 0.0f) atomicMax(reinterpret_cast<int*>(absmax), __float_as_int(amax));
}

__device__ __forceinline__ int tensor_q8(float v, float inv) {
    const float r = fmaxf(-127.0f, fminf(127.0f, roundf(__fmul_rn(finite_or_zero(v), inv))));   // half away from zero
    return (int)r;
}

template <typename T>
__global__ void __launch_bounds__(256)
tensor_quant_kernel(const T* __restrict__ x, int8_t* __restrict__ q, const float* __restrict__ absmax, long long size,
                    long long n_vec) {
    const float a = *absmax;
    const float inv = (a > 1e-8f) ? __fdiv_rn(127.0f, a) : 0.0f;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
#pragma unroll 4
    for (long long i = tid; i < n_vec; i += stride) {
        float v[16];
        load8<T>(x + i * 16, v);
        load8<T>(x + i * 16 + 8, v + 8);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            w[j] = pack4_s8(tensor_q8(v[4 * j], inv), tensor_q8(v[4 * j + 1], inv), tensor_q8(v[4 * j + 2], inv), tensor_q8(v[4 * j + 3], inv));
        reinterpret_cast<uint4*>(q)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (long long i = n_vec * 16 + tid; i < size; i += stride) q[i] = (int8_t)tensor_q8(to_float<T>(x[i]), inv);
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ void store8_scaled(T* out, uint32_t lo, uint32_t hi, float sc);
template <> __device__ __forceinline__ void store8_scaled<float>(float* out, uint32_t lo, uint32_t hi, float sc) {
    reinterpret_cast<float4*>(out)[0] = make_float4(__fmul_rn(s8_of(lo, 0), sc), __fmul_rn(s8_of(lo, 1), sc), __fmul_rn(s8_of(lo, 2), sc), __fmul_rn(s8_of(lo, 3), sc));
    reinterpret_cast<float4*>(out)[1] = make_float4(__fmul_rn(s8_of(hi, 0), sc), __fmul_rn(s8_of(hi, 1), sc), __fmul_rn(s8_of(hi, 2), sc), __fmul_rn(s8_of(hi, 3), sc));
}
template <> __device__ __forceinline__ void store8_scaled<__nv_bfloat16>(__nv_bfloat16* out, uint32_t lo, uint32_t hi, float sc) {
    *reinterpret_cast<uint4*>(out) = make_uint4(pack_bf16x2(__fmul_rn(s8_of(lo, 0), sc), __fmul_rn(s8_of(lo, 1), sc)),
                                                pack_bf16x2(__fmul_rn(s8_of(lo, 2), sc), __fmul_rn(s8_of(lo, 3), sc)),
                                                pack_bf16x2(__fmul_rn(s8_of(hi, 0), sc), __fmul_rn(s8_of(hi, 1), sc)),
                                                pack_bf16x2(__fmul_rn(s8_of(hi, 2), sc), __fmul_rn(s8_of(hi, 3), sc)));
}
template <> __device__ __forceinline__ void store8_scaled<__half>(__half* out, uint32_t lo, uint32_t hi, float sc) {
    *reinterpret_cast<uint4*>(out) = make_uint4(pack_f16x2(__fmul_rn(s8_of(lo, 0), sc), __fmul_rn(s8_of(lo, 1), sc)),
                                                pack_f16x2(__fmul_rn(s8_of(lo, 2), sc), __fmul_rn(s8_of(lo, 3), sc)),
                                                pack_f16x2(__fmul_rn(s8_of(hi, 0), sc), __fmul_rn(s8_of(hi, 1), sc)),
                                                pack_f16x2(__fmul_rn(s8_of(hi, 2), sc), __fmul_rn(s8_of(hi, 3), sc)));
}

template <typename T>
__global__ void __launch_bounds__(256)
tensor_dequant_kernel(const int8_t* __restrict__ q, const float* __restrict__ absmax, T* __restrict__ out, long long size,
                      long long n_vec) {
    const float sc = __fdiv_rn(*absmax, 127.0f);
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
#pragma unroll 4
    for (long long i = tid; i < n_vec; i += stride) {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(q) + i);
        store8_scaled<T>(out + i * 16, w.x, w.y, sc);
        store8_scaled<T>(out + i * 16 + 8, w.z, w.w, sc);
    }
    for (long long i = n_vec * 16 + tid; i < size; i += stride) out[i] = from_float<T>(__fmul_rn((float)q[i], sc));
}

// ---------------------------------------------------------------------------------------------------------
// gradient quantisation: Gq = clamp(rint((dY * x_absmax[m]/127) * inv), +-127)
// ---------------------------------------------------------------------------------------------------------

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
quantize_grad_kernel(const T* __restrict__ dY, long long ld, const float* __restrict__ x_absmax,
                     const float* __restrict__ g_absmax, int8_t* __restrict__ Gq, int N) {
    const int m = blockIdx.x;
    const float g = *g_absmax;
    const float inv = (g >= 1e-30f) ? __fdiv_rn(127.0f, g) : 0.0f;
    const float sx = __fdiv_rn(x_absmax[m], 127.0f);
    const T* yr = dY + (size_t)m * ld;
    int8_t* gr = Gq + (size_t)m * N;
    auto qz = [&](float v) -> int {
        const float f = __fmul_rn(finite_or_zero(v), sx);
        float r = rintf(__fmul_rn(f, inv));
        r = fminf(127.0f, fmaxf(-127.0f, r));
        return (int)r;
    };
    if (VEC) {
        for (int k = threadIdx.x * 8; k < N; k += blockDim.x * 8) {
            float v[8];
            load8<T>(yr + k, v);
            int qi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)      // non-finite -> NaN -> 0; the conversion rounds and clamps at 127, max() at -127
                qi[i] = max(-127, q8_sat(__fmul_rn(__fmul_rn(finite_or_nan(v[i]), sx), inv)));
            *reinterpret_cast<uint2*>(gr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
        }
    } else {
        for (int k = threadIdx.x; k < N; k += blockDim.x) gr[k] = (int8_t)qz(to_float<T>(yr[k]));
    }
}

// The same quantisation for a token-sharded layer: this rank holds the gradient rows of its own tokens, and the weight
// gradient of output features [d*win, (d+1)*win) is formed on rank d.  The row is quantised once and each column window
// is stored straight into its owner's receive buffer (own memory or a peer mapping: plain stores over NVLink) at row
// row_offset + m, so the all-to-all of the int8 gradient is this kernel's output.  The per-tensor maximum is the largest
// of the ranks' partial maxima in g_slots; block 0 also leaves it in g_out for the weight-gradient kernel.
struct ScatterDst {
    int8_t* p[8];
};

template <typename T>
__global__ void __launch_bounds__(256)
quantize_grad_scatter_kernel(const T* __restrict__ dY, long long ld, const float* __restrict__ x_absmax,
                             const float* __restrict__ g_slots, int n_slots, float* __restrict__ g_out, ScatterDst dst,
                             int win, long long row_offset, int N) {
    const int m = blockIdx.x;
    float g = 0.0f;
    for (int i = 0; i < n_slots; ++i) g = fmaxf(g, g_slots[i]);
    if (m == 0 && threadIdx.x == 0 && g_out != nullptr) *g_out = g;
    const float inv = (g >= 1e-30f) ? __fdiv_rn(127.0f, g) : 0.0f;
    const float sx = __fdiv_rn(x_absmax[m], 127.0f);
    const T* yr = dY + (size_t)m * ld;
    for (int k = threadIdx.x * 8; k < N; k += blockDim.x * 8) {
        float v[8];
        load8<T>(yr + k, v);
        int qi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            qi[i] = max(-127, q8_sat(__fmul_rn(__fmul_rn(finite_or_nan(v[i]), sx), inv)));
        const int d = k / win, c = k - d * win;                 // win % 8 == 0: the eight values share one window
        int8_t* out = dst.p[d] + (size_t)(row_offset + m) * win + c;
        *reinterpret_cast<uint2*>(out) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
    }
}

// Copy of a local block into the same offset of several buffers (peer mappings): the push half of an all-gather.
struct PutDst {
    char* p[8];
};

__global__ void __launch_bounds__(256)
peer_put_vec_kernel(const uint4* __restrict__ src, PutDst dst, int n_dst, size_t n_vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (i + j * stride < n_vec) v[j] = __ldg(src + i + j * stride);
        for (int d = 0; d < n_dst; ++d) {
            uint4* out = reinterpret_cast<uint4*>(dst.p[d]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + j * stride < n_vec) out[i + j * stride] = v[j];
        }
    }
}

__global__ void __launch_bounds__(256)
peer_put_word_kernel(const uint32_t* __restrict__ src, PutDst dst, int n_dst, size_t n_words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t v = src[i];
        for (int d = 0; d < n_dst; ++d) reinterpret_cast<uint32_t*>(dst.p[d])[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------

static inline int grid_for(long long work, int block, int cap = 0) {
    long long g = (work + block - 1) / block;
    if (cap > 0 && g > cap) g = cap;
    return (int)(g < 1 ? 1 : g);
}

int launch_pack(const void* src, bool from_float, float gamma, uint8_t* Wp, int N, int K, int pad_code, cudaStream_t st) {
    const int pK = (K + 3) / 4;
    const long long work = (long long)N * pK;
    if (work == 0) return EL_OK;
    if (from_float && K % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        int sms = 148;
        device_sm_count(&sms);
        ternarize_pack_vec_kernel<<<grid_for(work, 256 * 4, sms * 16), 256, 0, st>>>(static_cast<const float4*>(src), gamma, Wp, work);
        return check_launch();
    }
    if (from_float) pack_kernel<true><<<grid_for(work, 256), 256, 0, st>>>(src, gamma, Wp, N, K, pK, pad_code);
    else pack_kernel<false><<<grid_for(work, 256), 256, 0, st>>>(src, gamma, Wp, N, K, pK, pad_code);
    return check_launch();
}

int launch_unpack(const uint8_t* Wp, void* out, int out_dtype, int N, int K, cudaStream_t st) {
    const int pK = (K + 3) / 4;
    const long long work = (long long)N * pK;
    if (work == 0) return EL_OK;
    if (K % 16 == 0 && (reinterpret_cast<uintptr_t>(Wp) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        int sms = 148;
        device_sm_count(&sms);
        const long long n_words = work / 4;
        const int gv = grid_for(n_words, 256 * 4, sms * 16);
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(Wp);
        switch (out_dtype) {
            case EL_F16: unpack_vec_kernel<__half><<<gv, 256, 0, st>>>(wp, (__half*)out, n_words); break;
            case EL_BF16: unpack_vec_kernel<__nv_bfloat16><<<gv, 256, 0, st>>>(wp, (__nv_bfloat16*)out, n_words); break;
            case EL_F32: unpack_vec_kernel<float><<<gv, 256, 0, st>>>(wp, (float*)out, n_words); break;
            case EL_I32: unpack_vec_kernel<int8_t><<<gv, 256, 0, st>>>(wp, (int8_t*)out, n_words); break;
            default: return EL_ERR_INVALID_ARG;
        }
        return check_launch();
    }
    const int g = grid_for(work, 256);
    switch (out_dtype) {
        case EL_F16: unpack_kernel<__half><<<g, 256, 0, st>>>(Wp, (__half*)out, N, K, pK); break;
        case EL_BF16: unpack_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(Wp, (__nv_bfloat16*)out, N, K, pK); break;
        case EL_F32: unpack_kernel<float><<<g, 256, 0, st>>>(Wp, (float*)out, N, K, pK); break;
        case EL_I32: unpack_kernel<int8_t><<<g, 256, 0, st>>>(Wp, (int8_t*)out, N, K, pK); break;
        default: return EL_ERR_INVALID_ARG;
    }
    return check_launch();
}

template <typename T>
static int launch_quantize_rows_t(const T* x, long long ldx, int8_t* q, float* a, int M, int K, float eps, int mode,
                                  const float* fold_absmax, float* fold_max, cudaStream_t st) {
    const bool vec = (K % 8 == 0) && (ldx % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
#define EL_QR(V, MD) do { if (K <= 4096) quantize_rows_kernel<T, V, MD, 2><<<M, 256, 0, st>>>(x, ldx, q, a, K, eps, fold_absmax, fold_max); \
                         else quantize_rows_kernel<T, V, MD, 6><<<M, 256, 0, st>>>(x, ldx, q, a, K, eps, fold_absmax, fold_max); } while (0)
    if (mode == 0) { if (vec) EL_QR(true, 0); else EL_QR(false, 0); }
    else if (mode == 1) { if (vec) EL_QR(true, 1); else EL_QR(false, 1); }
    else { if (vec) EL_QR(true, 2); else EL_QR(false, 2); }
#undef EL_QR
    return check_launch();
}

int launch_quantize_rows(const void* x, int dt, long long ldx, int8_t* q, float* a, int M, int K, float eps, int mode,
                         const float* fold_absmax, float* fold_max, cudaStream_t st) {
    if (M == 0) return EL_OK;
    switch (dt) {
        case EL_F16: return launch_quantize_rows_t((const __half*)x, ldx, q, a, M, K, eps, mode, fold_absmax, fold_max, st);
        case EL_BF16: return launch_quantize_rows_t((const __nv_bfloat16*)x, ldx, q, a, M, K, eps, mode, fold_absmax, fold_max, st);
        case EL_F32: return launch_quantize_rows_t((const float*)x, ldx, q, a, M, K, eps, mode, fold_absmax, fold_max, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

int launch_quantize_rows_perm(const void* x, int dt, long long ldx, int8_t* q, float* a, int M, int K, float eps,
                              cudaStream_t st) {
    if (M == 0) return EL_OK;
    if (K % 16 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15))
        return EL_ERR_ALIGNMENT;
    switch (dt) {
        case EL_F16: quantize_rows_perm_kernel<__half><<<M, 256, 0, st>>>((const __half*)x, ldx, q, a, K, eps); break;
        case EL_BF16: quantize_rows_perm_kernel<__nv_bfloat16><<<M, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, q, a, K, eps); break;
        case EL_F32: quantize_rows_perm_kernel<float><<<M, 256, 0, st>>>((const float*)x, ldx, q, a, K, eps); break;
        default: return EL_ERR_INVALID_ARG;
    }
    return check_launch();
}

template <typename T>
static int launch_quantize_tensor_t(const T* x, int8_t* q, float* absmax, long long size, cudaStream_t st) {
    int sms = 148;
    device_sm_count(&sms);
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0;
    const long long n_vec = vec ? size / 16 : 0;
    const int g = grid_for(vec ? (size + 15) / 16 : size, 256, sms * 8);
    tensor_absmax_kernel<T><<<g, 256, 0, st>>>(x, absmax, size, n_vec);
    int rc = check_launch();
    if (rc != EL_OK) return rc;
    tensor_quant_kernel<T><<<g, 256, 0, st>>>(x, q, absmax, size, n_vec);
    return check_launch();
}

int launch_quantize_tensor(const void* x, int dt, int8_t* q, float* absmax, long long size, cudaStream_t st) {
    EL_CUDA_TRY(cudaMemsetAsync(absmax, 0, sizeof(float), st));
    if (size == 0) return EL_OK;
    switch (dt) {
        case EL_F16: return launch_quantize_tensor_t((const __half*)x, q, absmax, size, st);
        case EL_BF16: return launch_quantize_tensor_t((const __nv_bfloat16*)x, q, absmax, size, st);
        case EL_F32: return launch_quantize_tensor_t((const float*)x, q, absmax, size, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

int launch_dequantize_tensor(const int8_t* q, const float* absmax, void* out, int dt, long long size, cudaStream_t st) {
    if (size == 0) return EL_OK;
    int sms = 148;
    device_sm_count(&sms);
    const bool vec = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(q)) & 15) == 0;
    const long long n_vec = vec ? size / 16 : 0;
    const int g = grid_for(vec ? (size + 15) / 16 : size, 256, sms * 8);
    switch (dt) {
        case EL_F16: tensor_dequant_kernel<__half><<<g, 256, 0, st>>>(q, absmax, (__half*)out, size, n_vec); break;
        case EL_BF16: tensor_dequant_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(q, absmax, (__nv_bfloat16*)out, size, n_vec); break;
        case EL_F32: tensor_dequant_kernel<float><<<g, 256, 0, st>>>(q, absmax, (float*)out, size, n_vec); break;
        default: return EL_ERR_INVALID_ARG;
    }
    return check_launch();
}

template <typename T>
static int launch_quantize_grad_t(const T* dY, long long ld, const float* xa, const float* ga, int8_t* Gq, int M, int N,
                                  cudaStream_t st) {
    const bool vec = (N % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(dY) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(Gq) & 7) == 0);
    if (vec) quantize_grad_kernel<T, true><<<M, 256, 0, st>>>(dY, ld, xa, ga, Gq, N);
    else quantize_grad_kernel<T, false><<<M, 256, 0, st>>>(dY, ld, xa, ga, Gq, N);
    return check_launch();
}

int launch_quantize_grad(const void* dY, int dt, long long ld, const float* xa, const float* ga, int8_t* Gq, int M, int N,
                         cudaStream_t st) {
    if (M == 0 || N == 0) return EL_OK;
    switch (dt) {
        case EL_F16: return launch_quantize_grad_t((const __half*)dY, ld, xa, ga, Gq, M, N, st);
        case EL_BF16: return launch_quantize_grad_t((const __nv_bfloat16*)dY, ld, xa, ga, Gq, M, N, st);
        case EL_F32: return launch_quantize_grad_t((const float*)dY, ld, xa, ga, Gq, M, N, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

template <typename T>
static int launch_quantize_grad_scatter_t(const T* dY, long long ld, const float* xa, const float* g_slots, int n_slots,
                                          float* g_out, const ScatterDst& dst, int win, long long row_offset, int M, int N,
                                          cudaStream_t st) {
    quantize_grad_scatter_kernel<T><<<M, 256, 0, st>>>(dY, ld, xa, g_slots, n_slots, g_out, dst, win, row_offset, N);
    return check_launch();
}

int launch_quantize_grad_scatter(const void* dY, int dt, long long ld, const float* xa, const float* g_slots, int n_slots,
                                 float* g_out, void* const* Gq_all, int n_ranks, long long row_offset, int M, int N,
                                 cudaStream_t st) {
    if (n_ranks < 1 || n_ranks > 8 || n_slots < 1 || N % n_ranks != 0) return EL_ERR_INVALID_ARG;
    const int win = N / n_ranks;
    if (win % 8 != 0 || ld % 8 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (reinterpret_cast<uintptr_t>(dY) & 15) return EL_ERR_ALIGNMENT;
    ScatterDst dst{};
    for (int d = 0; d < n_ranks; ++d) {
        if (Gq_all[d] == nullptr) return EL_ERR_NULL_PTR;
        if (reinterpret_cast<uintptr_t>(Gq_all[d]) & 7) return EL_ERR_ALIGNMENT;
        dst.p[d] = static_cast<int8_t*>(Gq_all[d]);
    }
    if (M == 0 || N == 0) return EL_OK;
    switch (dt) {
        case EL_F16: return launch_quantize_grad_scatter_t((const __half*)dY, ld, xa, g_slots, n_slots, g_out, dst, win, row_offset, M, N, st);
        case EL_BF16: return launch_quantize_grad_scatter_t((const __nv_bfloat16*)dY, ld, xa, g_slots, n_slots, g_out, dst, win, row_offset, M, N, st);
        case EL_F32: return launch_quantize_grad_scatter_t((const float*)dY, ld, xa, g_slots, n_slots, g_out, dst, win, row_offset, M, N, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

int launch_peer_put(const void* src, void* const* dst_all, int n_dst, size_t dst_offset, size_t bytes, int max_ctas,
                    cudaStream_t st) {
    if (n_dst < 0 || n_dst > 8) return EL_ERR_INVALID_ARG;
    if (n_dst == 0 || bytes == 0) return EL_OK;
    if ((reinterpret_cast<uintptr_t>(src) & 3) || (dst_offset & 3) || (bytes & 3)) return EL_ERR_ALIGNMENT;
    PutDst dst{};
    bool vec = ((reinterpret_cast<uintptr_t>(src) | dst_offset | bytes) & 15) == 0;
    for (int d = 0; d < n_dst; ++d) {
        if (dst_all[d] == nullptr) return EL_ERR_NULL_PTR;
        if (reinterpret_cast<uintptr_t>(dst_all[d]) & 3) return EL_ERR_ALIGNMENT;
        vec = vec && (reinterpret_cast<uintptr_t>(dst_all[d]) & 15) == 0;
        dst.p[d] = static_cast<char*>(dst_all[d]) + dst_offset;
    }
    int sms = 148;
    device_sm_count(&sms);
    const int cap = max_ctas > 0 ? max_ctas : 4 * sms;
    if (vec) {
        const size_t n = bytes / 16;
        peer_put_vec_kernel<<<grid_for((long long)((n + 3) / 4), 256, cap), 256, 0, st>>>(static_cast<const uint4*>(src), dst, n_dst, n);
    } else {
        const size_t n = bytes / 4;
        peer_put_word_kernel<<<grid_for((long long)n, 256, cap), 256, 0, st>>>(static_cast<const uint32_t*>(src), dst, n_dst, n);
    }
    return check_launch();
}

// int32 sums -> scaled output, four columns per thread; VEC: C % 4 == 0 and 16-byte aligned sums and 8-byte (16-bit types)
// or 16-byte aligned output rows, so the four columns move as one load and one store
template <bool VEC>
__global__ void __launch_bounds__(256)
scale_rows_kernel(const int* __restrict__ acc, EpiParams epi, int M, int C) {
    const int cg = (C + 3) / 4;
    const long long work = (long long)M * cg, stride = (long long)gridDim.x * blockDim.x;
#pragma unroll 4
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < work; t += stride) {
        const int m = (int)(t / cg), c0 = (int)(t % cg) * 4;
        const float sc = epi_row_scale(epi, m);
        if (VEC) {
            const int4 a = __ldg(reinterpret_cast<const int4*>(acc + (size_t)m * C + c0));
            const size_t o = (size_t)m * epi.ldo + c0;
            const float f0 = __fmul_rn((float)a.x, sc), f1 = __fmul_rn((float)a.y, sc), f2 = __fmul_rn((float)a.z, sc), f3 = __fmul_rn((float)a.w, sc);
            switch (epi.out_dtype) {
                case EL_BF16: *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(epi.out) + o) = make_uint2(pack_bf16x2(f0, f1), pack_bf16x2(f2, f3)); break;
                case EL_F16: *reinterpret_cast<uint2*>(static_cast<__half*>(epi.out) + o) = make_uint2(pack_f16x2(f0, f1), pack_f16x2(f2, f3)); break;
                case EL_F32: *reinterpret_cast<float4*>(static_cast<float*>(epi.out) + o) = make_float4(f0, f1, f2, f3); break;
                default: *reinterpret_cast<int4*>(static_cast<int*>(epi.out) + o) = a; break;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j < C) epi_store_one(epi, m, c0 + j, acc[(size_t)m * C + c0 + j], sc);
        }
    }
}

int launch_scale_rows(const int* acc, const EpiParams& epi, int M, int C, cudaStream_t st) {
    const long long work = (long long)M * ((C + 3) / 4);
    if (work == 0) return EL_OK;
    const size_t out_elem = (epi.out_dtype == EL_BF16 || epi.out_dtype == EL_F16) ? 2 : 4;
    const bool vec = C % 4 == 0 && epi.ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(acc) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(epi.out) & (4 * out_elem - 1)) == 0;
    int sms = 148;
    device_sm_count(&sms);
    const int g = grid_for(work, 256 * 4, sms * 8);
    if (vec) scale_rows_kernel<true><<<g, 256, 0, st>>>(acc, epi, M, C);
    else scale_rows_kernel<false><<<g, 256, 0, st>>>(acc, epi, M, C);
    return check_launch();
}

// Cross-rank reduction, owner side: out rows = scale(sum over n_parts of parts[p][Mr, C]) written into the row window
// [row_offset, row_offset + Mr) of every rank's output matrix (own buffer and peer mappings: plain stores over NVLink).
struct GatherDst {
    void* p[8];
};

__global__ void __launch_bounds__(256)
reduce_scale_gather_kernel(const int* __restrict__ parts, int n_parts, GatherDst dst, int n_ranks, long long row_offset,
                           EpiParams epi, int Mr, int C) {
    // one thread per 8 columns: 32 bytes of every part in flight, one 16-byte (two-byte outputs) or two 16-byte stores
    // per destination, so that a warp's stores to a peer are 512 contiguous bytes
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int cg = C >> 3;
    if (t >= (long long)Mr * cg) return;
    const int m = (int)(t / cg), c0 = (int)(t % cg) * 8;
    const size_t part_stride = (size_t)Mr * C;
    const int4* src = reinterpret_cast<const int4*>(parts + (size_t)m * C + c0);
    int4 lo = src[0], hi = src[1];
    for (int p = 1; p < n_parts; ++p) {
        const int4* q = reinterpret_cast<const int4*>(parts + p * part_stride + (size_t)m * C + c0);
        const int4 a = q[0], b = q[1];
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
    }
    const float sc = epi_row_scale(epi, m);
    const float f[8] = {__fmul_rn((float)lo.x, sc), __fmul_rn((float)lo.y, sc), __fmul_rn((float)lo.z, sc), __fmul_rn((float)lo.w, sc),
                        __fmul_rn((float)hi.x, sc), __fmul_rn((float)hi.y, sc), __fmul_rn((float)hi.z, sc), __fmul_rn((float)hi.w, sc)};
    const size_t o = (size_t)(row_offset + m) * C + c0;
    if (epi.out_dtype == EL_F32) {
        for (int d = 0; d < n_ranks; ++d) {
            float4* out = reinterpret_cast<float4*>(static_cast<float*>(dst.p[d]) + o);
            out[0] = make_float4(f[0], f[1], f[2], f[3]);
            out[1] = make_float4(f[4], f[5], f[6], f[7]);
        }
    } else {
        uint4 v;
        if (epi.out_dtype == EL_BF16) v = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        else v = make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
        for (int d = 0; d < n_ranks; ++d) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(dst.p[d]) + o) = v;
    }
}

int launch_reduce_scale_gather(const int* parts, int n_parts, void* const* out_all, int n_ranks, long long row_offset,
                               long long rows_total, const EpiParams& epi, int Mr, int C, cudaStream_t st) {
    (void)rows_total;
    GatherDst dst{};
    for (int d = 0; d < n_ranks; ++d) {
        if (out_all[d] == nullptr) return EL_ERR_NULL_PTR;
        if (reinterpret_cast<uintptr_t>(out_all[d]) & 15) return EL_ERR_ALIGNMENT;
        dst.p[d] = out_all[d];
    }
    if (reinterpret_cast<uintptr_t>(parts) & 15) return EL_ERR_ALIGNMENT;
    if (C % 8 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    const long long work = (long long)Mr * (C >> 3);
    if (work == 0) return EL_OK;
    reduce_scale_gather_kernel<<<(int)((work + 255) / 256), 256, 0, st>>>(parts, n_parts, dst, n_ranks, row_offset, epi, Mr, C);
    return check_launch();
}

}  // namespace el
