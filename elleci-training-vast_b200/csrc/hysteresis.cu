// Stand-alone hysteresis update: float32 weight gradient in, packed ternary weights and packed int4
// counters rewritten in place.  HBM-bound: per weight it reads 4 B of gradient, 0.25 B of weight and
// 0.5 B of counter and writes 0.75 B back.  One thread owns the four weights of one packed weight byte
// (and the two counter bytes that go with it), so the repack needs no atomics.
#include "common.cuh"

namespace el {

template <bool VEC, bool FTZ>
__global__ void __launch_bounds__(256)
hysteresis_kernel(const float* __restrict__ dW, uint8_t* __restrict__ Wp, uint8_t* __restrict__ Hp, HystParams p,
                  int N, int K, int pK, int pH, uint32_t idx_base) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)N * pK) return;
    const int n = (int)(t / pK), b = (int)(t % pK);
    const int k0 = b * 4;
    const float* g = dW + (size_t)n * K + k0;
    float grad[4];
    uint32_t hbits;
    const size_t hoff = (size_t)n * pH + (size_t)(k0 >> 1);
    if (VEC) {   // K % 4 == 0 and dW 16-byte aligned: every group is whole
        const float4 v = *reinterpret_cast<const float4*>(g);
        grad[0] = v.x; grad[1] = v.y; grad[2] = v.z; grad[3] = v.w;
        hbits = *reinterpret_cast<const uint16_t*>(Hp + hoff);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) grad[j] = (k0 + j < K) ? g[j] : 0.0f;
        hbits = Hp[hoff];
        if (k0 + 2 < K) hbits |= (uint32_t)Hp[hoff + 1] << 8;
    }
    uint32_t wbits = Wp[t];
    const uint32_t idx0 = idx_base + (uint32_t)n * (uint32_t)K + (uint32_t)k0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (VEC || k0 + j < K) {
            int q = decode2(wbits >> (2 * j));
            int h = (int)((hbits >> (4 * j)) & 0xFu);
            h = (h & 8) ? h - 16 : h;
            hyst_update_one<FTZ>(grad[j], q, h, idx0 + j, p);
            wbits = (wbits & ~(3u << (2 * j))) | ((uint32_t)(q + 1) << (2 * j));
            hbits = (hbits & ~(0xFu << (4 * j))) | (((uint32_t)h & 0xFu) << (4 * j));
        }
    }
    Wp[t] = (uint8_t)wbits;
    if (VEC) {
        *reinterpret_cast<uint16_t*>(Hp + hoff) = (uint16_t)hbits;
    } else {
        Hp[hoff] = (uint8_t)hbits;
        if (k0 + 2 < K) Hp[hoff + 1] = (uint8_t)(hbits >> 8);
    }
}

// The same update with one thread per 32 consecutive weights (K % 32 == 0, so a chunk never crosses a row): 128 bytes
// of gradient, 8 bytes of packed weights and 16 bytes of packed counters per thread, and the trimmed 32-weight update
// of the fused epilogue (hyst_update_chunk32) - the per-weight instruction count, not HBM, bounds this kernel.
template <bool FTZ, bool ALIGNED>
__global__ void __launch_bounds__(256)
hysteresis_chunk_kernel(const float* __restrict__ dW, uint8_t* __restrict__ Wp, uint8_t* __restrict__ Hp, HystParams p,
                        long long chunks, uint32_t idx_base) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    const float4* g = reinterpret_cast<const float4*>(dW) + c * 8;
    uint32_t acc[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float4 v = g[j];
        acc[4 * j] = __float_as_uint(v.x); acc[4 * j + 1] = __float_as_uint(v.y);
        acc[4 * j + 2] = __float_as_uint(v.z); acc[4 * j + 3] = __float_as_uint(v.w);
    }
    uint2* wptr = reinterpret_cast<uint2*>(Wp) + c;
    uint4* hptr = reinterpret_cast<uint4*>(Hp) + c;
    const uint2 w2 = *wptr;
    const uint4 h4 = *hptr;
    uint32_t w[2] = {w2.x, w2.y};
    uint32_t h[4] = {h4.x, h4.y, h4.z, h4.w};
    hyst_update_chunk32<FTZ, ALIGNED, false>(acc, 0.0f, w, h, idx_base + (uint32_t)(c * 32), p);
    *wptr = make_uint2(w[0], w[1]);
    *hptr = make_uint4(h[0], h[1], h[2], h[3]);
}

int launch_hysteresis(const float* dW, uint8_t* Wp, uint8_t* Hp, const HystParams& p, int N, int K, uint32_t idx_base,
                      cudaStream_t st) {
    const int pK = (K + 3) / 4, pH = (K + 1) / 2;
    const long long work = (long long)N * pK;
    if (work == 0) return EL_OK;
    if (K % 32 == 0 && (reinterpret_cast<uintptr_t>(dW) & 15) == 0 && (reinterpret_cast<uintptr_t>(Wp) & 7) == 0 &&
        (reinterpret_cast<uintptr_t>(Hp) & 15) == 0) {
        const long long chunks = (long long)N * (K / 32);
        const int cgrid = (int)((chunks + 255) / 256);
        const bool aligned = (idx_base & 31u) == 0;
#define EL_HC(F, A) hysteresis_chunk_kernel<F, A><<<cgrid, 256, 0, st>>>(dW, Wp, Hp, p, chunks, idx_base)
        if (p.ftz) { if (aligned) EL_HC(true, true); else EL_HC(true, false); }
        else { if (aligned) EL_HC(false, true); else EL_HC(false, false); }
#undef EL_HC
        return check_launch();
    }
    const int grid = (int)((work + 255) / 256);
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(dW) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(Hp) & 1) == 0);
    if (vec && p.ftz) hysteresis_kernel<true, true><<<grid, 256, 0, st>>>(dW, Wp, Hp, p, N, K, pK, pH, idx_base);
    else if (vec) hysteresis_kernel<true, false><<<grid, 256, 0, st>>>(dW, Wp, Hp, p, N, K, pK, pH, idx_base);
    else if (p.ftz) hysteresis_kernel<false, true><<<grid, 256, 0, st>>>(dW, Wp, Hp, p, N, K, pK, pH, idx_base);
    else hysteresis_kernel<false, false><<<grid, 256, 0, st>>>(dW, Wp, Hp, p, N, K, pK, pH, idx_base);
    return check_launch();
}

}  // namespace el
