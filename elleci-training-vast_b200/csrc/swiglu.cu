// SwiGLU gate fused with the pre-linear RMSNorm and the per-token int8 quantiser of the down projection, and the
// backward pass of the three.
//
// The reference's feed-forward block is  w3( silu(w1 x) * w2 x )  (model/model.py:86-108), and its INT2 linear layer
// normalises and quantises whatever it is given (core/bitnet/bitnet_int2_optimized.py:72-86,201-210).  Between the
// gate/up GEMMs and the down GEMM lie, as tensor operations: silu, the product, the float32 norm, two casts, the
// weight product and the quantiser - about thirteen bytes of memory traffic per hidden element.  Here one kernel reads
// the gate and up rows and writes the int8 row of the down projection (five bytes per element); the backward kernel
// reads the gradient of the normalised product and the gate and up rows and writes both gradients.
//
// Every float32 step is a single correctly rounded operation in a fixed order (the exponential is a fixed polynomial
// evaluated with fused multiply-adds, row sums are accumulated in float64), so the CPU oracle reproduces the kernels
// bit for bit.
#include "row_io.cuh"

namespace el {

int device_sm_count(int* out);
size_t rmsnorm_backward_workspace_bytes(int K);

namespace {

using namespace rowio;

// e^t in float32 for the sigmoid: t clamped to [-87, 87] (beyond it 1 + e^t no longer changes, or the sigmoid is below
// 2e-38), n = round-half-even(t*log2(e)) taken by adding and subtracting 1.5*2^23 (its low mantissa bits are n as an
// integer), r = t - n*ln2 in two fused steps, degree-7 Taylor polynomial in Horner form with fused multiply-adds, times
// 2^n built in the exponent field.  About 1 ulp.  A NaN argument is clamped away (fmaxf returns the other operand); the
// callers multiply by the argument afterwards, which brings the NaN back.
__device__ __forceinline__ float exp_fixed(float t) {
    t = fminf(fmaxf(t, -87.0f), 87.0f);
    const float magic = 12582912.0f;
    const float nm = __fadd_rn(__fmul_rn(t, 1.44269504088896341f), magic);
    const float n = __fsub_rn(nm, magic);
    float r = __fmaf_rn(n, -0.693145751953125f, t);
    r = __fmaf_rn(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    const float scale = __int_as_float((__float_as_int(nm) + 127) << 23);       // 2^n, n in [-126, 127]
    return __fmul_rn(p, scale);
}

// 1/d correctly rounded for a d whose reciprocal is a normal number (here d = 1 + e^t lies in [1, 2^126]): the hardware
// approximation and one Newton step in two fused multiply-adds - the general-purpose reciprocal is this sequence plus a
// check and a branch for the arguments that cannot occur here.
__device__ __forceinline__ float rcp_normal(float d) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    const float e = __fmaf_rn(-d, r, 1.0f);
    return __fmaf_rn(r, e, r);
}

// sigmoid(g) = 1 / (1 + e^-g)
__device__ __forceinline__ float sigmoid_fixed(float g) { return rcp_normal(__fadd_rn(1.0f, exp_fixed(-g))); }

// Eight elements of the gate: sig = sigmoid(g), s = io(g * sig), h = io(s * u) - silu rounded to the I/O type, then the
// product rounded to the I/O type, as the two tensor operations of the reference round them.
template <typename T>
__device__ __forceinline__ void gated8(const float g[8], const float u[8], float sig[8], float s[8], float h[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        sig[i] = sigmoid_fixed(g[i]);
        s[i] = __fmul_rn(g[i], sig[i]);
    }
    Io<T>::round8(s);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(s[i], u[i]);
    Io<T>::round8(h);
}

// One CTA per token.  H % 8 == 0, rows 16-byte aligned.  `weight` null: no normalisation (y = h, rstd is not written).
// ROW_CACHE as in the RMSNorm kernel: vectors of 8 hidden values a thread keeps in registers between the passes.
template <typename T, int ROW_CACHE>
__global__ void __launch_bounds__(RN_THREADS, ROW_CACHE == 2 ? 4 : (sizeof(T) == 4 ? 2 : 3))
swiglu_quantize_rows_kernel(const T* __restrict__ gate, const T* __restrict__ up, long long ld, const float* __restrict__ weight,
                            int8_t* __restrict__ q, float* __restrict__ row_absmax, float* __restrict__ rstd_out, int H,
                            float norm_eps, float quant_eps) {
    __shared__ double red_d[RN_THREADS / 32];
    __shared__ float red_f[RN_THREADS / 32];
    const int m = blockIdx.x;
    const T* gr = gate + (size_t)m * ld;
    const T* ur = up + (size_t)m * ld;
    int8_t* qr = q + (size_t)m * H;
    const bool has_norm = weight != nullptr;

    auto hidden = [&](int k, float h[8]) {
        float g[8], u[8], sig[8], s[8];
        Io<T>::load8(gr + k, g);
        Io<T>::load8(ur + k, u);
        gated8<T>(g, u, sig, s, h);
    };

    typename Io<T>::Raw cache[ROW_CACHE];
    const int k_tail = (threadIdx.x + ROW_CACHE * RN_THREADS) * 8;

    // ---- h, and its mean of squares -> rstd ------------------------------------------------------------------------------
    double ss = 0.0;
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < H) {
            float h[8];
            hidden(k, h);
            cache[c] = Io<T>::pack(h);
            if (has_norm) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(h[i], h[i]);
            }
        }
    }
    float r = 1.0f;
    if (has_norm) {
        for (int k = k_tail; k < H; k += RN_THREADS * 8) {
            float h[8];
            hidden(k, h);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(h[i], h[i]);
        }
        ss = block_sum(ss, red_d);
        const float ms = __fdiv_rn((float)ss, (float)H);
        r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, norm_eps)));
    }

    // y = io(io(h*r) * io(w)), or h itself
    auto normed = [&](const float h[8], int k, float y[8]) {
        if (has_norm) {
            float w[8];
            Io<float>::load8(weight + k, w);
            Io<T>::round8(w);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(h[i], r);
            Io<T>::round8(y);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(y[i], w[i]);
            Io<T>::round8(y);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = h[i];
        }
    };

    // ---- absmax of the row that is quantised ---------------------------------------------------------------------------
    // Taken on the bit patterns of |y| as integers: the order of the finite values is the same, and an infinity or a NaN
    // comes out on top, so one comparison at the end tells whether the row needs the checked passes.
    int amax_bits = 0;
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < H) {
            float h[8], y[8];
            Io<T>::unpack(cache[c], h);
            normed(h, k, y);
            cache[c] = Io<T>::pack(y);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_int(y[i]) & 0x7fffffff);
        }
    }
    for (int k = k_tail; k < H; k += RN_THREADS * 8) {
        float h[8], y[8];
        hidden(k, h);
        normed(h, k, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_int(y[i]) & 0x7fffffff);
    }
    const bool row_finite = !__syncthreads_or(amax_bits >= 0x7f800000);     // same answer in every thread of the CTA
    float amax = block_max_f(__int_as_float(amax_bits), red_f);              // used only when every thread's value is finite
    if (!row_finite) {        // the row holds an infinity or a NaN: the maximum over its finite values only
        amax = 0.0f;
        for (int k = threadIdx.x * 8; k < H; k += RN_THREADS * 8) {
            float h[8], y[8];
            hidden(k, h);
            normed(h, k, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(finite_or_zero(y[i])));
        }
        amax = block_max_f(amax, red_f);
    }
    const float a = fmaxf(amax, quant_eps);
    const float s = __fdiv_rn(127.0f, a);
    if (threadIdx.x == 0) {
        row_absmax[m] = a;
        if (has_norm) rstd_out[m] = r;
    }

    // ---- quantise --------------------------------------------------------------------------------------------------------
    auto quantise_y = [&](const float y[8], int k) {
        int qi[8];
        if (row_finite) {
            // |y*s| <= 127: adding 1.5*2^23 rounds to the nearest even integer and leaves it in the low mantissa bits
#pragma unroll
            for (int i = 0; i < 8; ++i) qi[i] = __float_as_int(__fadd_rn(__fmul_rn(y[i], s), 12582912.0f));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) qi[i] = q8_sat(__fmul_rn(finite_or_nan(y[i]), s));
        }
        *reinterpret_cast<uint2*>(qr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
    };
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < H) {
            float y[8];
            Io<T>::unpack(cache[c], y);
            quantise_y(y, k);
        }
    }
    for (int k = k_tail; k < H; k += RN_THREADS * 8) {
        float h[8], y[8];
        hidden(k, h);
        normed(h, k, y);
        quantise_y(y, k);
    }
}

// Backward.  Upstream gradient gy [M,H] with respect to the normalised product y (or to h itself when `weight` is
// null).  Follows autograd through the reference's tensor operations, each intermediate rounded where a tensor of the
// I/O type would hold it:
//   s = io(g*sig(g));  h = io(s*u)
//   with the norm:  gn = io(gy*io(w));  c = sum_k gn*h;  dh = io(gn*rstd - h*(rstd^3*c/H));  dweight[k] += gy*io(h*rstd)
//   ds = io(dh*u);  d_up = io(dh*s);  d_gate = io((ds*sig) * (1 + g*(1 - sig)))
// CTA b takes the tokens b, b + gridDim.x, ...; a thread owns the same columns in every token, so the per-column sums of
// dweight live in shared memory without any exchange, and the CTA writes its [H] partial sums to partial[b] at the end.
// SIG_CACHE (with the norm only): vectors of 8 sigmoids a thread keeps in registers from the first pass (the row sum c) to
// the second, so that the exponential is evaluated once per element for rows up to SIG_CACHE*2048 elements.
template <typename T, bool NORM, int SIG_CACHE>
__global__ void __launch_bounds__(RN_THREADS)
swiglu_backward_kernel(const T* __restrict__ gy, const T* __restrict__ gate, const T* __restrict__ up, long long ld,
                       const float* __restrict__ weight, const float* __restrict__ rstd, T* __restrict__ d_gate,
                       T* __restrict__ d_up, long long ld_d, double* __restrict__ partial, int M, int H) {
    extern __shared__ double col_sum[];          // [H] when NORM
    __shared__ double red_d[RN_THREADS / 32];
    if (NORM) {
        for (int k = threadIdx.x * 8; k < H; k += RN_THREADS * 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) col_sum[k + i] = 0.0;
        }
    }
    const int k_tail = (threadIdx.x + SIG_CACHE * RN_THREADS) * 8;
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        const T* yr = gy + (size_t)m * H;
        const T* gr = gate + (size_t)m * ld;
        const T* ur = up + (size_t)m * ld;
        T* dgr = d_gate + (size_t)m * ld_d;
        T* dur = d_up + (size_t)m * ld_d;
        float r = 1.0f, coef = 0.0f;
        float sig_c[SIG_CACHE > 0 ? SIG_CACHE : 1][8];

        // c += sum over the 8 elements at k of gn * h; hands back the sigmoids
        auto row_dot = [&](int k, float sig[8]) -> double {
            float yv[8], g[8], u[8], w[8];
            Io<T>::load8(yr + k, yv);
            Io<T>::load8(gr + k, g);
            Io<T>::load8(ur + k, u);
            Io<float>::load8(weight + k, w);
            float sv[8], h[8];
            gated8<T>(g, u, sig, sv, h);
            Io<T>::round8(w);
#pragma unroll
            for (int i = 0; i < 8; ++i) yv[i] = __fmul_rn(yv[i], w[i]);
            Io<T>::round8(yv);
            double c = 0.0;
#pragma unroll
            for (int i = 0; i < 8; ++i) c += (double)__fmul_rn(yv[i], h[i]);
            return c;
        };
        // the gradients of the 8 elements at k, given their sigmoids
        auto row_grad = [&](int k, const float sig[8]) {
            float yv[8], g[8], u[8], w[8], og[8], ou[8];
            Io<T>::load8(yr + k, yv);
            Io<T>::load8(gr + k, g);
            Io<T>::load8(ur + k, u);
            float sv[8], dh[8], ds[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sv[i] = __fmul_rn(g[i], sig[i]);
            Io<T>::round8(sv);
            if (NORM) {
                float h[8], gn[8], hn[8];
                Io<float>::load8(weight + k, w);
                Io<T>::round8(w);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    h[i] = __fmul_rn(sv[i], u[i]);
                    gn[i] = __fmul_rn(yv[i], w[i]);
                }
                Io<T>::round8(h);
                Io<T>::round8(gn);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dh[i] = __fsub_rn(__fmul_rn(gn[i], r), __fmul_rn(h[i], coef));
                    hn[i] = __fmul_rn(h[i], r);
                }
                Io<T>::round8(dh);
                Io<T>::round8(hn);
#pragma unroll
                for (int i = 0; i < 8; ++i) col_sum[k + i] += (double)__fmul_rn(yv[i], hn[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) dh[i] = yv[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ds[i] = __fmul_rn(dh[i], u[i]);
            Io<T>::round8(ds);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ou[i] = __fmul_rn(dh[i], sv[i]);
                og[i] = __fmul_rn(__fmul_rn(ds[i], sig[i]), __fadd_rn(1.0f, __fmul_rn(g[i], __fsub_rn(1.0f, sig[i]))));
            }
            Io<T>::store8(dgr + k, og);
            Io<T>::store8(dur + k, ou);
        };

        if (NORM) {
            r = rstd[m];
            double c = 0.0;
#pragma unroll
            for (int cv = 0; cv < SIG_CACHE; ++cv) {
                const int k = (threadIdx.x + cv * RN_THREADS) * 8;
                if (k < H) c += row_dot(k, sig_c[cv]);
            }
            for (int k = k_tail; k < H; k += RN_THREADS * 8) {
                float sig[8];
                c += row_dot(k, sig);
            }
            c = block_sum(c, red_d);
            const float r3 = __fmul_rn(__fmul_rn(r, r), r);
            coef = __fdiv_rn(__fmul_rn(r3, (float)c), (float)H);
#pragma unroll
            for (int cv = 0; cv < SIG_CACHE; ++cv) {
                const int k = (threadIdx.x + cv * RN_THREADS) * 8;
                if (k < H) row_grad(k, sig_c[cv]);
            }
        }
        for (int k = NORM ? k_tail : threadIdx.x * 8; k < H; k += RN_THREADS * 8) {
            float g[8], sig[8];
            Io<T>::load8(gr + k, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) sig[i] = sigmoid_fixed(g[i]);
            row_grad(k, sig);
        }
    }
    if (NORM) {
        double* out = partial + (size_t)blockIdx.x * H;
        for (int k = threadIdx.x * 8; k < H; k += RN_THREADS * 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) out[k + i] = col_sum[k + i];
        }
    }
}

// dweight[k] = float(sum of the CTAs' partial sums), in a fixed order of additions for any grid (32 columns per CTA, the
// eight warps each add every eighth partial in order, warp 0 adds the eight results in order).
__global__ void __launch_bounds__(256)
swiglu_dweight_kernel(const double* __restrict__ partial, int n_parts, float* __restrict__ dweight, int H) {
    __shared__ double part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k = blockIdx.x * 32 + lane;
    double s = 0.0;
    if (k < H) {
#pragma unroll 4
        for (int p = warp; p < n_parts; p += 8) s += partial[(size_t)p * H + k];
    }
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && k < H) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += part[w][lane];
        dweight[k] = (float)t;
    }
}

int backward_grid(int M, int H, bool norm) {
    int sms = 148;
    device_sm_count(&sms);
    int per_sm = 4;
    if (norm) {
        const size_t smem = (size_t)H * sizeof(double);
        per_sm = (int)((200u * 1024u) / (smem ? smem : 1));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 4) per_sm = 4;
    }
    const int grid = sms * per_sm;
    return M < grid ? (M < 1 ? 1 : M) : grid;
}

// The layer's input as the fused training kernels form it, written out in the I/O type instead of being quantised: for
// the small-M decode call, whose kernels quantise their few tokens themselves.  x is the layer input, or the gate when
// `up` is given (h = io(io(x*sig(x))*up)); with `weight` the row is normalised (y = io(io(h*rstd)*io(w))).  One CTA per
// token, same order of operations as swiglu_quantize_rows_kernel / rmsnorm_quantize_rows_kernel, so quantising y gives the
// int8 row those kernels give.
template <typename T>
__global__ void __launch_bounds__(RN_THREADS)
prelinear_rows_kernel(const T* __restrict__ x, const T* __restrict__ up, long long ld, const float* __restrict__ weight,
                      T* __restrict__ y, int K, float norm_eps) {
    __shared__ double red_d[RN_THREADS / 32];
    const int m = blockIdx.x;
    const T* xr = x + (size_t)m * ld;
    const T* ur = up ? up + (size_t)m * ld : nullptr;
    T* yr = y + (size_t)m * K;
    auto hidden = [&](int k, float h[8]) {
        Io<T>::load8(xr + k, h);
        if (ur) {
            float g[8], u[8], sig[8], s[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] = h[i];
            Io<T>::load8(ur + k, u);
            gated8<T>(g, u, sig, s, h);
        }
    };
    float r = 1.0f;
    if (weight) {
        double ss = 0.0;
        for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
            float h[8];
            hidden(k, h);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(h[i], h[i]);
        }
        ss = block_sum(ss, red_d);
        const float ms = __fdiv_rn((float)ss, (float)K);
        r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, norm_eps)));
    }
    for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
        float h[8];
        hidden(k, h);
        if (weight) {
            float w[8];
            Io<float>::load8(weight + k, w);
            Io<T>::round8(w);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(h[i], r);
            Io<T>::round8(h);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(h[i], w[i]);
            Io<T>::round8(h);
        }
        Io<T>::store8(yr + k, h);
    }
}

// sig[i] = sigmoid(g[i]) as the fused kernels compute it (a check of the fixed arithmetic against a CPU restatement).
__global__ void __launch_bounds__(256) sigmoid_fixed_kernel(const float* __restrict__ g, float* __restrict__ sig, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        sig[i] = sigmoid_fixed(g[i]);
}

}  // namespace

size_t swiglu_backward_workspace_bytes(int H) { return rmsnorm_backward_workspace_bytes(H); }

int launch_prelinear_rows(const void* x, const void* up, int dt, long long ld, const float* weight, float norm_eps, void* y, int M,
                          int K, cudaStream_t st) {
    if (M == 0) return EL_OK;
    if (K <= 0 || K % 8 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    const size_t esz = (dt == EL_F32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(up) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) ||
        ((size_t)ld * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15))
        return EL_ERR_ALIGNMENT;
    switch (dt) {
        case EL_BF16:
            prelinear_rows_kernel<__nv_bfloat16><<<M, RN_THREADS, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)up, ld, weight,
                                                                           (__nv_bfloat16*)y, K, norm_eps);
            break;
        case EL_F16:
            prelinear_rows_kernel<__half><<<M, RN_THREADS, 0, st>>>((const __half*)x, (const __half*)up, ld, weight, (__half*)y, K, norm_eps);
            break;
        case EL_F32:
            prelinear_rows_kernel<float><<<M, RN_THREADS, 0, st>>>((const float*)x, (const float*)up, ld, weight, (float*)y, K, norm_eps);
            break;
        default: return EL_ERR_INVALID_ARG;
    }
    return check_launch();
}

int launch_sigmoid_fixed(const float* g, float* sig, long long n, cudaStream_t st) {
    if (n == 0) return EL_OK;
    int sms = 148;
    device_sm_count(&sms);
    sigmoid_fixed_kernel<<<sms * 8, 256, 0, st>>>(g, sig, n);
    return check_launch();
}

int launch_swiglu_quantize_rows(const void* gate, const void* up, int dt, long long ld, const float* weight, float norm_eps,
                                int8_t* q, float* row_absmax, float* rstd, int M, int H, float quant_eps, cudaStream_t st) {
    if (M == 0) return EL_OK;
    if (H <= 0 || H % 8 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    const size_t esz = (dt == EL_F32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(gate) & 15) || (reinterpret_cast<uintptr_t>(up) & 15) || ((size_t)ld * esz) % 16 != 0 ||
        (reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
        return EL_ERR_ALIGNMENT;
#define EL_SGQ(T, NC) swiglu_quantize_rows_kernel<T, NC><<<M, RN_THREADS, 0, st>>>((const T*)gate, (const T*)up, ld, weight, q, row_absmax, rstd, H, norm_eps, quant_eps)
    switch (dt) {
        case EL_BF16: if (H <= 4096) EL_SGQ(__nv_bfloat16, 2); else EL_SGQ(__nv_bfloat16, 6); break;
        case EL_F16: if (H <= 4096) EL_SGQ(__half, 2); else EL_SGQ(__half, 6); break;
        case EL_F32: if (H <= 4096) EL_SGQ(float, 2); else EL_SGQ(float, 6); break;
        default: return EL_ERR_INVALID_ARG;
    }
#undef EL_SGQ
    return check_launch();
}

template <typename T, int SIG_CACHE>
static int launch_swiglu_backward_norm(const T* gy, const T* gate, const T* up, long long ld, const float* weight, const float* rstd,
                                       T* d_gate, T* d_up, long long ld_d, float* dweight, double* partial, int M, int H,
                                       cudaStream_t st) {
    const int grid = backward_grid(M, H, true);
    const size_t smem = (size_t)H * sizeof(double);
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(swiglu_backward_kernel<T, true, SIG_CACHE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024));
        attr_once.mark(dev);
    }
    swiglu_backward_kernel<T, true, SIG_CACHE><<<grid, RN_THREADS, smem, st>>>(gy, gate, up, ld, weight, rstd, d_gate, d_up, ld_d,
                                                                               partial, M, H);
    int rc = check_launch();
    if (rc != EL_OK) return rc;
    swiglu_dweight_kernel<<<(H + 31) / 32, 256, 0, st>>>(partial, grid, dweight, H);
    return check_launch();
}

template <typename T>
static int launch_swiglu_backward_t(const T* gy, const T* gate, const T* up, long long ld, const float* weight, const float* rstd,
                                    T* d_gate, T* d_up, long long ld_d, float* dweight, double* partial, int M, int H,
                                    cudaStream_t st) {
    if (!weight) {
        const int grid = backward_grid(M, H, false);
        swiglu_backward_kernel<T, false, 0><<<grid, RN_THREADS, 0, st>>>(gy, gate, up, ld, nullptr, nullptr, d_gate, d_up, ld_d,
                                                                         nullptr, M, H);
        return check_launch();
    }
    // registers per thread that cost no occupancy: rows up to 4096 elements run four CTAs per SM, longer rows two or one
    if (H <= 4096) return launch_swiglu_backward_norm<T, 2>(gy, gate, up, ld, weight, rstd, d_gate, d_up, ld_d, dweight, partial, M, H, st);
    return launch_swiglu_backward_norm<T, 6>(gy, gate, up, ld, weight, rstd, d_gate, d_up, ld_d, dweight, partial, M, H, st);
}

int launch_swiglu_backward(const void* gy, const void* gate, const void* up, int dt, long long ld, const float* weight,
                           const float* rstd, void* d_gate, void* d_up, long long ld_d, float* dweight, void* workspace,
                           size_t workspace_bytes, int M, int H, cudaStream_t st) {
    if (H <= 0 || H % 8 != 0 || (weight && (size_t)H * sizeof(double) > 200u * 1024u)) return EL_ERR_UNSUPPORTED_SHAPE;
    if (weight && workspace_bytes < swiglu_backward_workspace_bytes(H)) return EL_ERR_INVALID_ARG;
    const size_t esz = (dt == EL_F32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(gy) & 15) || (reinterpret_cast<uintptr_t>(gate) & 15) || (reinterpret_cast<uintptr_t>(up) & 15) ||
        (reinterpret_cast<uintptr_t>(d_gate) & 15) || (reinterpret_cast<uintptr_t>(d_up) & 15) || ((size_t)ld * esz) % 16 != 0 ||
        ((size_t)ld_d * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return EL_ERR_ALIGNMENT;
    if (M == 0) {
        if (weight) EL_CUDA_TRY(cudaMemsetAsync(dweight, 0, (size_t)H * sizeof(float), st));
        return EL_OK;
    }
    double* partial = static_cast<double*>(workspace);
    switch (dt) {
        case EL_BF16:
            return launch_swiglu_backward_t((const __nv_bfloat16*)gy, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, ld, weight,
                                            rstd, (__nv_bfloat16*)d_gate, (__nv_bfloat16*)d_up, ld_d, dweight, partial, M, H, st);
        case EL_F16:
            return launch_swiglu_backward_t((const __half*)gy, (const __half*)gate, (const __half*)up, ld, weight, rstd,
                                            (__half*)d_gate, (__half*)d_up, ld_d, dweight, partial, M, H, st);
        case EL_F32:
            return launch_swiglu_backward_t((const float*)gy, (const float*)gate, (const float*)up, ld, weight, rstd, (float*)d_gate,
                                            (float*)d_up, ld_d, dweight, partial, M, H, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

}  // namespace el
