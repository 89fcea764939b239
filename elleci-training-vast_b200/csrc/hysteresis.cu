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

int launch_hysteresis(const float* dW, uint8_t* Wp, uint8_t* Hp, const HystParams& p, int N, int K, uint32_t idx_base,
                      cudaStream_t st) {
    const int pK = (K + 3) / 4, pH = (K + 1) / 2;
    const long long work = (long long)N * pK;
    if (work == 0) return EL_OK;
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
