// Shared device helpers of the INT2 linear library: field codes, the per-weight hysteresis update,
// number conversions and the host-side launch bookkeeping.  sm_100a only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/elleci_int2.h"

namespace el {

// ---- host-side error bookkeeping ---------------------------------------------------------------------
int record_cuda_error(cudaError_t e);   // stores e for el_last_cuda_error(), returns EL_ERR_CUDA
int check_launch();                      // cudaGetLastError() -> EL_OK / EL_ERR_CUDA
int device_sm_count(int* out);           // SM count of the current device (cached per device)
int require_sm100();                     // EL_OK when the current device is compute capability 10.x

// "Set up once per device" bookkeeping that host threads may race on.  The set-up calls guarded by it are idempotent
// (a function attribute, a queried constant), so two threads that both find the flag clear simply both run them; the
// flag itself is an atomic, published after the set-up returned.
// Decode calls of up to this many tokens use the warp-MMA kernel in its single-launch form (every CTA quantises the tokens
// itself); larger ones quantise once and run it on the quantised tokens.
constexpr int DECODE_MMA_SINGLE_MAX = 8;

struct DeviceOnce {
    std::atomic<int> done[64];
    bool is_done(int dev) const { return dev >= 0 && dev < 64 && done[dev].load(std::memory_order_acquire) != 0; }
    void mark(int dev) {
        if (dev >= 0 && dev < 64) done[dev].store(1, std::memory_order_release);
    }
};

#define EL_CUDA_TRY(call)                                          \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return ::el::record_cuda_error(e__); \
    } while (0)

// ---- 2-bit weight code: 0 -> -1, 1 -> 0, 2 -> +1, 3 -> 0 -------------------------------------------------
__device__ __forceinline__ int decode2(uint32_t c) {
    c &= 3u;
    return (c == 2u) - (c == 0u);
}

// Sixteen 2-bit codes (one 32-bit word, code j at bits 2j) -> sixteen int8 in natural order, as four words.
// A byte-permute with the table {0xFF,0x00,0x01,0x00} decodes four codes at once when each code sits in
// its own nibble; the even and odd codes are split into two nibble streams and interleaved again.
__device__ __forceinline__ void decode16(uint32_t x, uint32_t out[4]) {
    const uint32_t lut = 0x000100FFu;
    const uint32_t te = x & 0x33333333u;          // nibble i = code 2i
    const uint32_t to = (x >> 2) & 0x33333333u;   // nibble i = code 2i+1
    const uint32_t e0 = __byte_perm(lut, 0, te);        // codes 0,2,4,6
    const uint32_t e1 = __byte_perm(lut, 0, te >> 16);  // codes 8,10,12,14
    const uint32_t o0 = __byte_perm(lut, 0, to);        // codes 1,3,5,7
    const uint32_t o1 = __byte_perm(lut, 0, to >> 16);  // codes 9,11,13,15
    out[0] = __byte_perm(e0, o0, 0x5140);
    out[1] = __byte_perm(e0, o0, 0x7362);
    out[2] = __byte_perm(e1, o1, 0x5140);
    out[3] = __byte_perm(e1, o1, 0x7362);
}

// The same sixteen codes without the final interleave: out = codes {0,2,4,6}, {8,10,12,14}, {1,3,5,7}, {9,11,13,15}.
// Position p of a 16-group then holds weight KPERM16[p]; an operand whose reduction index is laid out with the
// same permutation (el_quantize_rows with kperm) gives the same integer sums for four fewer instructions per word.
__device__ __forceinline__ void decode16_deint(uint32_t x, uint32_t out[4]) {
    const uint32_t lut = 0x000100FFu;
    const uint32_t te = x & 0x33333333u;
    const uint32_t to = (x >> 2) & 0x33333333u;
    out[0] = __byte_perm(lut, 0, te);
    out[1] = __byte_perm(lut, 0, te >> 16);
    out[2] = __byte_perm(lut, 0, to);
    out[3] = __byte_perm(lut, 0, to >> 16);
}

// ---- float helpers ----------------------------------------------------------------------------------------
__device__ __forceinline__ float ftz32(float x) { return fabsf(x) < 1.17549435e-38f ? 0.0f : x; }
__host__ inline float ftz32_host(float x) {
    return (x < 1.17549435e-38f && x > -1.17549435e-38f) ? 0.0f : x;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float finite_or_zero(float v) { return (fabsf(v) <= 3.402823466e38f) ? v : 0.0f; }

// v for finite v, NaN for infinities and NaN (v - v is 0 only for finite v).  Followed by q8_sat, which turns NaN into
// 0, this counts non-finite inputs as zero with two additions instead of a compare and a select.
__device__ __forceinline__ float finite_or_nan(float v) { return __fadd_rn(v, __fsub_rn(v, v)); }

// round to nearest even and clamp to [-128, 127] in one conversion; NaN gives 0
__device__ __forceinline__ int q8_sat(float v) {
    int q;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(v));
    return q;
}

// the low bytes of four integers as one word (a in the lowest byte)
__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm((uint32_t)a, (uint32_t)b, 0x0040), __byte_perm((uint32_t)c, (uint32_t)d, 0x0040), 0x5410);
}

// ---- hysteresis: one weight ---------------------------------------------------------------------------------
struct HystParams {
    float lr_scaled;     // (lr*lr_scale)*thr, flushed like the reference's fast-math build when ftz
    uint32_t decay_u24;  // number of 24-bit random values u with u/2^24 < decay_rate (the decay test, as an integer)
    int thr;             // clamp(threshold, 1, 7)
    uint32_t s1, s2;     // step*2654435761, step*2246822519 (uint32 wrap-around)
    int ftz;
    const int32_t* step_ptr;   // when not null, the step is read from device memory by the kernel (hyst_resolve_step)
};

// The parameters with s1, s2 formed from the step in device memory, for kernels launched with a step pointer (a training
// step recorded once and replayed cannot carry the step number as a launch argument).
__device__ __forceinline__ HystParams hyst_resolve_step(const HystParams& p) {
    HystParams r = p;
    if (p.step_ptr != nullptr) {
        const uint32_t step = (uint32_t)*p.step_ptr;
        r.s1 = step * 2654435761u;
        r.s2 = step * 2246822519u;
    }
    return r;
}

__device__ __forceinline__ uint32_t mix2(uint32_t h) {
    h = ((h >> 16) ^ h) * 0x45d9f3bu;
    h = ((h >> 16) ^ h) * 0x45d9f3bu;
    return h;
}

// Updates (q, h) of weight `idx` from its gradient.  q in {-1,0,1}, h a signed counter.
// FTZ reproduces the reference build's flush of float32 denormals (inputs and result of the one multiply that can
// meet them) with the hardware's own .ftz multiply.
template <bool FTZ>
__device__ __forceinline__ void hyst_update_one(float grad, int& q, int& h, uint32_t idx, const HystParams& p) {
    const uint32_t u1 = mix2(idx ^ p.s1) & 0xFFFFFFu;
    const uint32_t u2 = mix2(idx ^ p.s2) & 0xFFFFFFu;
    float d_raw;
    if (FTZ) asm("mul.ftz.f32 %0, %1, %2;" : "=f"(d_raw) : "f"(-grad), "f"(p.lr_scaled));
    else d_raw = __fmul_rn(-grad, p.lr_scaled);
    const float a = fabsf(d_raw);
    const float fl = floorf(a);
    const float frac = __fsub_rn(a, fl);
    const float r1 = (float)u1 * (1.0f / 16777216.0f);
    float v = __fadd_rn(fl, (r1 < frac) ? 1.0f : 0.0f);
    v = (d_raw >= 0.0f) ? v : -v;
    int delta = __float2int_rz(v);   // saturating; NaN converts to 0
    delta = max(-31, min(31, delta));
    int hn = h + delta;
    if (q != 0 && u2 < p.decay_u24) hn -= q;
    const int thr = p.thr;
    // crossing +thr moves -1 -> 0 -> +1 and resets the counter; at +1 the counter saturates (clamp); same downwards
    const int mv = (hn >= thr && q < 1) ? 1 : ((hn <= -thr && q > -1) ? -1 : 0);
    q += mv;
    h = mv ? 0 : max(-thr, min(thr, hn));
}

// The same update for 32 consecutive weights of one row held as packed words (w: 2 words of 2-bit codes, h: 4 words of
// int4 counters), from their int32 gradient sums acc[32] scaled by sc.  Same results as 32 calls of hyst_update_one,
// with the per-weight work trimmed for the fused weight-gradient epilogue, which is bound by these instructions:
//  * stochastic rounding in integers: with T = ceil(|d|*2^24) (one saturating conversion, NaN -> 0),
//    floor(|d|) + [u1/2^24 < frac(|d|)] = ((T - 1 - u1) >> 24) + 1 exactly, for every |d| up to the clamp at 31;
//  * codes are sanitised (3 -> 1) once per word and stay biased (q+1), counters are read biased by 8 (word ^ 0x88888888);
//  * the new words are built from zero with one multiply-add per field instead of a masked read-modify-write;
//  * ALIGNED (idx0 a multiple of 32): idx0 + j = idx0 ^ j, so the counter xor seed is one operation per weight.
// FROM_ACC: acc holds int32 sums to be scaled by sc; otherwise acc holds the bits of float32 gradients (sc unused).
template <bool FTZ, bool ALIGNED, bool FROM_ACC = true>
__device__ __forceinline__ void hyst_update_chunk32(const uint32_t acc[32], float sc, uint32_t w[2], uint32_t h[4],
                                                    uint32_t idx0, const HystParams& p) {
    uint32_t ws[2], hb[4], wn[2] = {0u, 0u}, hn[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 2; ++i) ws[i] = w[i] ^ ((w[i] & (w[i] >> 1) & 0x55555555u) << 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) hb[i] = h[i] ^ 0x88888888u;
    const uint32_t b1 = idx0 ^ p.s1, b2 = idx0 ^ p.s2;
    const int thr = p.thr;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int wi = j >> 4, wsft = (j & 15) * 2, hi = j >> 3, hsft = (j & 7) * 4;
        const int qb = (int)((ws[wi] >> wsft) & 3u);             // q + 1
        const int nib = (int)((hb[hi] >> hsft) & 0xFu);          // h + 8
        const uint32_t u1 = mix2(ALIGNED ? (b1 ^ (uint32_t)j) : ((idx0 + j) ^ p.s1)) & 0xFFFFFFu;
        const uint32_t u2 = mix2(ALIGNED ? (b2 ^ (uint32_t)j) : ((idx0 + j) ^ p.s2)) & 0xFFFFFFu;
        const float grad = FROM_ACC ? __fmul_rn((float)(int)acc[j], sc) : __uint_as_float(acc[j]);
        float d_raw;
        if (FTZ) asm("mul.ftz.f32 %0, %1, %2;" : "=f"(d_raw) : "f"(-grad), "f"(p.lr_scaled));
        else d_raw = __fmul_rn(-grad, p.lr_scaled);
        const int T = __float2int_ru(__fmul_rn(fabsf(d_raw), 16777216.0f));      // saturates; NaN -> 0
        const int mag = min(((T - 1 - (int)u1) >> 24) + 1, 31);
        const int sgn = (__float_as_int(d_raw) >> 31) | 1;
        int hv = nib - 8 + sgn * mag;
        if (qb != 1 && u2 < p.decay_u24) hv -= qb - 1;
        const int up = (hv >= thr && qb < 2) ? 1 : 0;
        const int dn = (hv <= -thr && qb > 0) ? 1 : 0;
        const int mv = up - dn;
        const int hc = mv ? 0 : max(-thr, min(thr, hv));
        wn[wi] += (uint32_t)(qb + mv) << wsft;
        hn[hi] += (uint32_t)hc << hsft;                          // signed fields: the bias below turns them into nibbles
    }
    w[0] = wn[0];
    w[1] = wn[1];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = (hn[i] + 0x88888888u) ^ 0x88888888u;
}

// Host-side preparation of HystParams from the API arguments.
inline HystParams make_hyst_params(float lr, float lr_scale, int threshold, float decay, uint32_t step, int ftz) {
    HystParams p;
    p.thr = threshold < 1 ? 1 : (threshold > 7 ? 7 : threshold);
    if (ftz) { lr = ftz32_host(lr); lr_scale = ftz32_host(lr_scale); decay = ftz32_host(decay); }
    volatile float prod = lr * lr_scale;
    float pr = prod;
    if (ftz) pr = ftz32_host(pr);
    volatile float ls = pr * (float)p.thr;
    p.lr_scaled = ftz ? ftz32_host(ls) : (float)ls;
    // r2 = u/2^24 < decay  <=>  u < decay*2^24 (exact in double)  <=>  u < ceil(decay*2^24) for integer u
    const double t = (double)decay * 16777216.0;
    if (!(t > 0.0)) p.decay_u24 = 0;                    // also NaN: the comparison is then always false
    else if (t >= 16777216.0) p.decay_u24 = 16777216u;
    else {
        uint32_t c = (uint32_t)t;
        if ((double)c < t) ++c;
        p.decay_u24 = c;
    }
    p.s1 = step * 2654435761u;
    p.s2 = step * 2246822519u;
    p.ftz = ftz;
    p.step_ptr = nullptr;
    return p;
}

// ---- output conversion -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace el
