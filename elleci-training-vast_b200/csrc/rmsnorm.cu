// Pre-linear RMSNorm fused with the per-token int8 quantiser, and its backward pass.
//
// The reference normalises the activations right before every INT2 linear call
// (core/bitnet/bitnet_int2_optimized.py:72-86, model/common/bitnet_legacy.py:10-25):
//     norm = x_f32 * rsqrt(mean(x_f32^2) + eps);  y = norm.type_as(x) * weight.type_as(x)
// and then quantises y per token.  Done as separate tensor operations this reads and writes the [M, K] activation
// about eight times; here one kernel reads the row and writes the int8 row, its absmax and its rstd.
//
// Row sums (of squares, and in the backward pass) are accumulated in float64, so that their float32 value does not
// depend on the order of the additions: the result is the one the CPU oracle defines, bit for bit.
#include "row_io.cuh"

namespace el {

int device_sm_count(int* out);

namespace {

using namespace rowio;

// One CTA per token.  K % 8 == 0; x rows, weight and q rows 16-byte (q: 8-byte) aligned.  ROW_CACHE: vectors of 8
// elements a thread keeps in registers between the passes (2 for rows up to 4096 elements: fewer registers, more CTAs
// per SM, more bytes in flight; 6 for rows up to 12288).
template <typename T, int ROW_CACHE>
__global__ void __launch_bounds__(RN_THREADS, ROW_CACHE == 2 ? 6 : 3)
rmsnorm_quantize_rows_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ weight, int8_t* __restrict__ q,
                             float* __restrict__ row_absmax, float* __restrict__ rstd_out, int K, float norm_eps,
                             float quant_eps) {
    __shared__ double red_d[RN_THREADS / 32];
    __shared__ float red_f[RN_THREADS / 32];
    const int m = blockIdx.x;
    const T* xr = x + (size_t)m * ldx;
    int8_t* qr = q + (size_t)m * K;

    // The row is read from memory once: up to ROW_CACHE vectors of 8 elements per thread stay in registers for the two
    // later passes; longer rows re-read their tail.
    typename Io<T>::Raw cache[ROW_CACHE];
    const int k_tail = (threadIdx.x + ROW_CACHE * RN_THREADS) * 8;

    // ---- mean of squares -> rstd -------------------------------------------------------------------------------------
    double ss = 0.0;
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < K) {
            cache[c] = Io<T>::load_raw(xr + k);
            float v[8];
            Io<T>::unpack(cache[c], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(v[i], v[i]);
        }
    }
    for (int k = k_tail; k < K; k += RN_THREADS * 8) {
        float v[8];
        Io<T>::load8(xr + k, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(v[i], v[i]);
    }
    ss = block_sum(ss, red_d);
    const float ms = __fdiv_rn((float)ss, (float)K);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, norm_eps)));

    // y = io(io(x*r) * io(w))
    auto normed = [&](const float v[8], const float w[8], float y[8]) {
        float wr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            y[i] = __fmul_rn(v[i], r);
            wr[i] = w[i];
        }
        Io<T>::round8(y);
        Io<T>::round8(wr);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(y[i], wr[i]);
        Io<T>::round8(y);
    };

    // ---- absmax of the normalised row ----------------------------------------------------------------------------------
    // fmaxf drops NaN and keeps infinities: the checked pass runs only for a row that needs it
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < K) {
            float v[8], w[8], y[8];
            Io<T>::unpack(cache[c], v);
            load8_w(weight + k, w);
            normed(v, w, y);
            cache[c] = Io<T>::pack(y);          // from here on the cache holds the normalised row (exact: y is of type T)
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
        }
    }
    for (int k = k_tail; k < K; k += RN_THREADS * 8) {
        float v[8], w[8], y[8];
        Io<T>::load8(xr + k, v);
        load8_w(weight + k, w);
        normed(v, w, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(y[i]));
    }
    amax = block_max_f(amax, red_f);
    const bool row_finite = amax <= 3.402823466e38f;
    if (!row_finite) {
        amax = 0.0f;
        for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
            float v[8], w[8], y[8];
            Io<T>::load8(xr + k, v);
            load8_w(weight + k, w);
            normed(v, w, y);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(finite_or_zero(y[i])));
        }
        amax = block_max_f(amax, red_f);
    }
    const float a = fmaxf(amax, quant_eps);
    const float s = __fdiv_rn(127.0f, a);
    if (threadIdx.x == 0) {
        row_absmax[m] = a;
        rstd_out[m] = r;
    }

    // ---- quantise --------------------------------------------------------------------------------------------------------
    auto quantise_y = [&](const float y[8], int k) {
        int qi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) qi[i] = q8_sat(__fmul_rn(row_finite ? y[i] : finite_or_nan(y[i]), s));
        *reinterpret_cast<uint2*>(qr + k) = make_uint2(pack4_s8(qi[0], qi[1], qi[2], qi[3]), pack4_s8(qi[4], qi[5], qi[6], qi[7]));
    };
#pragma unroll
    for (int c = 0; c < ROW_CACHE; ++c) {
        const int k = (threadIdx.x + c * RN_THREADS) * 8;
        if (k < K) {
            float y[8];
            Io<T>::unpack(cache[c], y);
            quantise_y(y, k);
        }
    }
    for (int k = k_tail; k < K; k += RN_THREADS * 8) {
        float v[8], w[8], y[8];
        Io<T>::load8(xr + k, v);
        load8_w(weight + k, w);
        normed(v, w, y);
        quantise_y(y, k);
    }
}

// Backward.  CTA b takes the tokens b, b + gridDim.x, ...; thread t owns the same columns in every token, so the
// per-column sums of dweight live in shared memory (one double per column) without any exchange between threads.
// At the end the CTA writes its [K] partial sums to `partial[b]`.
template <typename T>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_backward_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ weight,
                        const float* __restrict__ rstd, T* __restrict__ dx, double* __restrict__ partial, int M, int K) {
    extern __shared__ double col_sum[];          // [K]
    __shared__ double red_d[RN_THREADS / 32];
    for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) col_sum[k + i] = 0.0;
    }
    for (int m = blockIdx.x; m < M; m += gridDim.x) {
        const T* gr = g + (size_t)m * K;
        const T* xr = x + (size_t)m * K;
        T* dr = dx + (size_t)m * K;
        const float r = rstd[m];
        // c = sum_k io(g*io(w)) * x
        double c = 0.0;
        for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
            float gv[8], xv[8], w[8];
            Io<T>::load8(gr + k, gv);
            Io<T>::load8(xr + k, xv);
            load8_w(weight + k, w);
            Io<T>::round8(w);
#pragma unroll
            for (int i = 0; i < 8; ++i) gv[i] = __fmul_rn(gv[i], w[i]);
            Io<T>::round8(gv);
#pragma unroll
            for (int i = 0; i < 8; ++i) c += (double)__fmul_rn(gv[i], xv[i]);
        }
        c = block_sum(c, red_d);
        const float r3 = __fmul_rn(__fmul_rn(r, r), r);
        const float coef = __fdiv_rn(__fmul_rn(r3, (float)c), (float)K);
        for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
            float gv[8], xv[8], w[8], o[8], gn[8], xn[8];
            Io<T>::load8(gr + k, gv);
            Io<T>::load8(xr + k, xv);
            load8_w(weight + k, w);
            Io<T>::round8(w);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                gn[i] = __fmul_rn(gv[i], w[i]);
                xn[i] = __fmul_rn(xv[i], r);
            }
            Io<T>::round8(gn);
            Io<T>::round8(xn);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                o[i] = __fsub_rn(__fmul_rn(gn[i], r), __fmul_rn(xv[i], coef));
                col_sum[k + i] += (double)__fmul_rn(gv[i], xn[i]);
            }
            Io<T>::store8(dr + k, o);
        }
    }
    double* out = partial + (size_t)blockIdx.x * K;
    for (int k = threadIdx.x * 8; k < K; k += RN_THREADS * 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[k + i] = col_sum[k + i];
    }
}

// dweight[k] = float(sum of the CTAs' partial sums).  A CTA covers 32 columns (one per lane); its eight warps each add
// every eighth partial in order, and warp 0 adds the eight results in order: a fixed order of additions for any grid.
__global__ void __launch_bounds__(256)
rmsnorm_dweight_kernel(const double* __restrict__ partial, int n_parts, float* __restrict__ dweight, int K) {
    __shared__ double part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k = blockIdx.x * 32 + lane;
    double s = 0.0;
    if (k < K) {
#pragma unroll 4
        for (int p = warp; p < n_parts; p += 8) s += partial[(size_t)p * K + k];
    }
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && k < K) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += part[w][lane];
        dweight[k] = (float)t;
    }
}

int backward_grid(int M, int K) {
    int sms = 148;
    device_sm_count(&sms);
    const size_t smem = (size_t)K * sizeof(double);
    int per_sm = (int)((200u * 1024u) / (smem ? smem : 1));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const int grid = sms * per_sm;
    return M < grid ? (M < 1 ? 1 : M) : grid;
}

}  // namespace

// Largest number of CTAs the backward kernel may use (sizes the workspace independently of M).
size_t rmsnorm_backward_workspace_bytes(int K) {
    if (K <= 0) return 0;
    int sms = 148;
    device_sm_count(&sms);
    return (size_t)sms * 4 * (size_t)K * sizeof(double);
}

int launch_rmsnorm_quantize_rows(const void* x, int dt, long long ldx, const float* weight, float norm_eps, int8_t* q,
                                 float* row_absmax, float* rstd, int M, int K, float quant_eps, cudaStream_t st) {
    if (M == 0) return EL_OK;
    if (K <= 0 || K % 8 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    const size_t esz = (dt == EL_F32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || ((size_t)ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) ||
        (reinterpret_cast<uintptr_t>(q) & 7))
        return EL_ERR_ALIGNMENT;
#define EL_RNQ(T, NC) rmsnorm_quantize_rows_kernel<T, NC><<<M, RN_THREADS, 0, st>>>((const T*)x, ldx, weight, q, row_absmax, rstd, K, norm_eps, quant_eps)
    switch (dt) {
        case EL_BF16: if (K <= 4096) EL_RNQ(__nv_bfloat16, 2); else EL_RNQ(__nv_bfloat16, 6); break;
        case EL_F16: if (K <= 4096) EL_RNQ(__half, 2); else EL_RNQ(__half, 6); break;
        case EL_F32: if (K <= 4096) EL_RNQ(float, 2); else EL_RNQ(float, 6); break;
        default: return EL_ERR_INVALID_ARG;
    }
#undef EL_RNQ
    return check_launch();
}

template <typename T>
static int launch_rmsnorm_backward_t(const T* g, const T* x, const float* weight, const float* rstd, T* dx, float* dweight,
                                     double* partial, int M, int K, cudaStream_t st) {
    const int grid = backward_grid(M, K);
    const size_t smem = (size_t)K * sizeof(double);
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(rmsnorm_backward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_once.mark(dev);
    }
    rmsnorm_backward_kernel<T><<<grid, RN_THREADS, smem, st>>>(g, x, weight, rstd, dx, partial, M, K);
    int rc = check_launch();
    if (rc != EL_OK) return rc;
    rmsnorm_dweight_kernel<<<(K + 31) / 32, 256, 0, st>>>(partial, grid, dweight, K);
    return check_launch();
}

int launch_rmsnorm_backward(const void* g, const void* x, int dt, const float* weight, const float* rstd, void* dx,
                            float* dweight, void* workspace, size_t workspace_bytes, int M, int K, cudaStream_t st) {
    if (K <= 0 || K % 8 != 0 || (size_t)K * sizeof(double) > 200u * 1024u) return EL_ERR_UNSUPPORTED_SHAPE;
    if (workspace_bytes < rmsnorm_backward_workspace_bytes(K)) return EL_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(g) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dx) & 15) ||
        (reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return EL_ERR_ALIGNMENT;
    if (M == 0) {
        EL_CUDA_TRY(cudaMemsetAsync(dweight, 0, (size_t)K * sizeof(float), st));
        return EL_OK;
    }
    double* partial = static_cast<double*>(workspace);
    switch (dt) {
        case EL_BF16:
            return launch_rmsnorm_backward_t((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, weight, rstd, (__nv_bfloat16*)dx,
                                             dweight, partial, M, K, st);
        case EL_F16:
            return launch_rmsnorm_backward_t((const __half*)g, (const __half*)x, weight, rstd, (__half*)dx, dweight, partial, M, K, st);
        case EL_F32:
            return launch_rmsnorm_backward_t((const float*)g, (const float*)x, weight, rstd, (float*)dx, dweight, partial, M, K, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

}  // namespace el
