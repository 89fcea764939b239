/*
 * CPU restatement in C of the integer pieces of the BitNet INT2 linear hot path.
 * TEST INFRASTRUCTURE ONLY: this file is the checker (and the timed CPU baseline) for the CUDA
 * kernels.  Nothing in the product library links against it.
 *
 * Reference lines followed (paths relative to the reference project root):
 *   2-bit / 4-bit field codes ............ kernels/int2/int2_packed.cuh:13-86
 *   hysteresis update per weight ......... kernels/int2/int2_hysteresis_v2.cu:66-151
 *   per-token absmax int8 quantisation ... model/common/bitnet_legacy.py:71-78
 *   integer forward / dX sums ............ kernels/int2/int2_matmul_int8_tc_v2.cu:466-470,
 *                                          kernels/int2/int2_backward_int8_tc_v2.cu:436-440
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -shared -fPIC).  All functions are re-entrant.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static inline int decode2(unsigned c) { /* int2_packed.cuh:13-18 */
    c &= 3u;
    return c == 0u ? -1 : (c == 2u ? 1 : 0);
}

static inline float ftz32(float x) { return fabsf(x) < 1.17549435e-38f ? 0.0f : x; }

static inline uint32_t mix2(uint32_t h) { /* int2_hysteresis_v2.cu:89-91 */
    h = ((h >> 16) ^ h) * 0x45d9f3bu;
    h = ((h >> 16) ^ h) * 0x45d9f3bu;
    return h;
}

/* Number of worker threads the OpenMP loops will use. */
ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the number of worker threads of the OpenMP loops (a launcher may have exported OMP_NUM_THREADS=1). */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/*
 * Hysteresis update of an [N,K] weight matrix from a float32 gradient, in place.
 * idx_base offsets the random-number counter for a row shard of a larger matrix.
 * ftz != 0 models the reference build's flush-to-zero arithmetic.
 */
ORACLE_API void oracle_hysteresis_step(const float* dW, uint8_t* W_packed, uint8_t* H_packed,
                                       float lr, float lr_scale, int threshold, float decay_rate,
                                       uint32_t step, int N, int K, uint32_t idx_base, int ftz) {
    const int pK = (K + 3) / 4, pH = (K + 1) / 2;
    const int thr = threshold < 1 ? 1 : (threshold > 7 ? 7 : threshold);
    if (ftz) { lr = ftz32(lr); lr_scale = ftz32(lr_scale); decay_rate = ftz32(decay_rate); }
    float prod = lr * lr_scale;
    if (ftz) prod = ftz32(prod);
    float lr_scaled = prod * (float)thr;
    if (ftz) lr_scaled = ftz32(lr_scaled);
    const uint32_t s1 = step * 2654435761u, s2 = step * 2246822519u;

#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        uint8_t* wrow = W_packed + (size_t)n * pK;
        uint8_t* hrow = H_packed + (size_t)n * pH;
        const float* grow = dW + (size_t)n * K;
        for (int k = 0; k < K; ++k) {
            const uint32_t idx = idx_base + (uint32_t)n * (uint32_t)K + (uint32_t)k;
            const int wsh = (k & 3) * 2, hsh = (k & 1) * 4;
            const int q = decode2(wrow[k >> 2] >> wsh);
            int hb = (hrow[k >> 1] >> hsh) & 0xF;
            const int h = (hb & 8) ? hb - 16 : hb;

            const float r1 = (float)(mix2(idx ^ s1) & 0xFFFFFFu) / 16777216.0f;
            const float r2 = (float)(mix2(idx ^ s2) & 0xFFFFFFu) / 16777216.0f;

            float g = grow[k];
            if (ftz) g = ftz32(g);
            float d_raw = -g * lr_scaled;
            if (ftz) d_raw = ftz32(d_raw);
            const float sgn = (d_raw >= 0.0f) ? 1.0f : -1.0f;
            const float a = fabsf(d_raw);
            const float fl = floorf(a);
            const float frac = a - fl;
            const float v = sgn * (fl + (r1 < frac ? 1.0f : 0.0f));
            int delta;
            if (v != v) delta = 0;                 /* NaN converts to 0 on the GPU */
            else if (v >= 31.0f) delta = 31;       /* conversion saturates, then clamp +-31 */
            else if (v <= -31.0f) delta = -31;
            else delta = (int)v;

            int hn = h + delta;
            if (q != 0 && r2 < decay_rate) hn -= (q > 0) ? 1 : -1;

            int qn = q;
            if (hn >= thr) {
                if (q == -1) { qn = 0; hn = 0; }
                else if (q == 0) { qn = 1; hn = 0; }
                else hn = thr;
            } else if (hn <= -thr) {
                if (q == 1) { qn = 0; hn = 0; }
                else if (q == 0) { qn = -1; hn = 0; }
                else hn = -thr;
            }
            if (hn > thr) hn = thr;
            if (hn < -thr) hn = -thr;

            wrow[k >> 2] = (uint8_t)((wrow[k >> 2] & ~(3u << wsh)) | ((unsigned)(qn + 1) << wsh));
            hrow[k >> 1] = (uint8_t)((hrow[k >> 1] & ~(0xFu << hsh)) | (((unsigned)hn & 0xFu) << hsh));
        }
    }
}

/* Per-token absmax int8 quantisation of float32 rows (bitnet_legacy.py:71-78). */
ORACLE_API void oracle_quantize_rows(const float* x, int8_t* q, float* absmax, int M, int K, float eps) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float* xr = x + (size_t)m * K;
        float a = 0.0f;
        for (int k = 0; k < K; ++k) {
            float v = xr[k];
            if (!isfinite(v)) v = 0.0f;
            v = fabsf(v);
            if (v > a) a = v;
        }
        if (a < eps) a = eps;
        absmax[m] = a;
        const float s = 127.0f / a;
        for (int k = 0; k < K; ++k) {
            float v = xr[k];
            if (!isfinite(v)) v = 0.0f;
            float r = nearbyintf(v * s); /* half to even under the default rounding mode */
            if (r > 127.0f) r = 127.0f;
            if (r < -128.0f) r = -128.0f;
            q[(size_t)m * K + k] = (int8_t)r;
        }
    }
}

/* Unpack [N, ceil(K/4)] 2-bit rows into [N,K] int8. */
ORACLE_API void oracle_unpack_ternary(const uint8_t* W_packed, int8_t* out, int N, int K) {
    const int pK = (K + 3) / 4;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            out[(size_t)n * K + k] = (int8_t)decode2(W_packed[(size_t)n * pK + (k >> 2)] >> ((k & 3) * 2));
}

/* acc[m,n] = sum_k Xq[m,k]*Wq[n,k]   (Wq given unpacked, [N,K] int8). */
ORACLE_API void oracle_gemm_nt_i8(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const int8_t* a = A + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const int8_t* b = B + (size_t)n * K;
            int32_t s = 0;
            for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)b[k];
            C[(size_t)m * N + n] = s;
        }
    }
}

/* acc[i,j] = sum_r A[r,i]*B[r,j]   (both operands reduction-major: dX with B = Wq, dW with A = Gq). */
ORACLE_API void oracle_gemm_tn_i8(const int8_t* A, const int8_t* B, int32_t* C, int R, int I, int J) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < I; ++i) {
        int32_t* c = C + (size_t)i * J;
        memset(c, 0, sizeof(int32_t) * (size_t)J);
        for (int r = 0; r < R; ++r) {
            const int32_t a = A[(size_t)r * I + i];
            if (a == 0) continue;
            const int8_t* b = B + (size_t)r * J;
            for (int j = 0; j < J; ++j) c[j] += a * (int32_t)b[j];
        }
    }
}

/* ---- sigmoid of the SwiGLU gate --------------------------------------------------------------------------
 * The reference's feed-forward block uses torch's silu (model/model.py:107-108): x * sigmoid(x), computed in
 * float32 with the platform's exponential, which is not reproducible across platforms.  The restatement fixes
 * the exponential: t clamped to [-87, 87], n = round-half-even(t*log2(e)) taken by adding and subtracting
 * 1.5*2^23, r = t - n*ln2 in two fused steps, degree-7 Taylor polynomial in Horner form with fused
 * multiply-adds, times 2^n built in the exponent field; every step one correctly rounded float32 operation
 * (fmaf is exact-then-rounded by definition).  About 1 ulp.  NaN is clamped away by fmaxf. */
static inline float exp_fixed(float t) {
    t = fminf(fmaxf(t, -87.0f), 87.0f);
    const float magic = 12582912.0f;
    volatile float prod = t * 1.44269504088896341f;
    volatile float nm = prod + magic;
    const float nmv = nm;
    const float n = nmv - magic;
    float r = fmaf(n, -0.693145751953125f, t);
    r = fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    union { uint32_t u; float f; } bits, scale;
    bits.f = nmv;
    scale.u = (bits.u + 127u) << 23;
    return p * scale.f;
}

/* sig[i] = 1 / (1 + e^-g[i]) in float32. */
ORACLE_API void oracle_sigmoid_fixed(const float* g, float* sig, long long n) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const float d = 1.0f + exp_fixed(-g[i]);
        sig[i] = 1.0f / d;
    }
}
