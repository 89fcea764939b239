// Decode GEMV for a handful of tokens (M <= 8) on the CUDA cores, one launch: Y[m,n] = (sum_k Q(x)[m,k]*Wq[n,k]) *
// (absmax[m]/127) * gamma.  At these sizes the call is bound by streaming W_packed once and by fixed latencies, so
// the kernel avoids every extra launch and every cross-CTA exchange:
//   phase 1  each CTA quantises the M token rows itself (absmax, then int8) into shared memory; the int8 values are
//            laid out for the lanes that will read them (conflict-free 16-byte loads) and permuted inside groups of
//            16 to match the cheap de-interleaved weight decode;
//   phase 2  warps stride over weight rows; a lane loads 16 bytes of packed weights (64 weights) at a time, expands
//            them with byte permutes and accumulates dp4a against the tokens; a shuffle reduction finishes the row.
// The integers and the rounding are those of el_quantize_rows + el_gemm_fwd.
#include "common.cuh"
#include "epilogue.cuh"

namespace el {

template <typename T> __device__ __forceinline__ void gv_load16(const T* p, float v[16]);
template <> __device__ __forceinline__ void gv_load16<__nv_bfloat16>(const __nv_bfloat16* p, float v[16]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 r = reinterpret_cast<const uint4*>(p)[h];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[8 * h + 2 * i] = __uint_as_float(w[i] << 16);
            v[8 * h + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
}
template <> __device__ __forceinline__ void gv_load16<__half>(const __half* p, float v[16]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 r = reinterpret_cast<const uint4*>(p)[h];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[8 * h + 2 * i] = f.x;
            v[8 * h + 2 * i + 1] = f.y;
        }
    }
}
template <> __device__ __forceinline__ void gv_load16<float>(const float* p, float v[16]) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const float4 a = reinterpret_cast<const float4*>(p)[h];
        v[4 * h] = a.x; v[4 * h + 1] = a.y; v[4 * h + 2] = a.z; v[4 * h + 3] = a.w;
    }
}

// Quantises 16 consecutive values of one token and stores them in the lane order of phase 2.  CHECKED: non-finite
// values count as zero (the slow path, taken only when a token holds an infinity).
template <typename T, bool CHECKED>
__device__ __forceinline__ uint4 gv_quant16(const T* src, float s) {
    float v[16];
    gv_load16<T>(src, v);
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = q8_sat(__fmul_rn(CHECKED ? finite_or_zero(v[i]) : v[i], s));
    uint32_t w[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        // bytes 4g..4g+3 of the output take the sources p<8 ? 2p : 2(p-8)+1
        const int p0 = 4 * g;
        const int s0 = (p0 < 8) ? 2 * p0 : 2 * (p0 - 8) + 1;           // sources s0, s0+2, s0+4, s0+6
        w[g] = pack4_s8(q[s0], q[s0 + 2], q[s0 + 4], q[s0 + 6]);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Shared memory: float amax[MT]; then per token ceil(K/2048)*128 uint4 (chunk i of 64 weights -> four uint4 at
// ((i/32)*4 + j)*32 + i%32, so that consecutive lanes read consecutive 16-byte words).
// One CTA of THREADS threads per SM: the token quantisation of phase 1 is repeated by every CTA, so few large CTAs
// keep its share of the instruction count small.
template <typename T, int MT, int RB, int THREADS>
__global__ void __launch_bounds__(THREADS, 1)
gemv_small_kernel(const T* __restrict__ x, const uint8_t* __restrict__ Wp, EpiParams epi, int M, int N, int K, float eps) {
    extern __shared__ uint4 gv_smem[];
    float* s_amax = reinterpret_cast<float*>(gv_smem);
    uint4* xs = gv_smem + 2;                      // 32 bytes reserved for the absmax values
    const int chunks = K >> 6;                    // 64 weights per chunk
    const int xs_per_m = ((chunks + 31) >> 5) * 128;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int WARPS = THREADS / 32;

    // ---- phase 0: the first batch of packed weights is requested before anything else ------------------------------------
    // A warp works on RB rows at once and on two 64-weight chunks per lane and row, so that 2*RB 16-byte loads per
    // lane are in flight: a row of 1024 packed bytes alone would leave the warp waiting on one memory latency per row.
    // Warp w of CTA b is warp number w*gridDim.x + b of the grid and takes the rows congruent to that number: rows that
    // do not divide evenly among the warps are spread over all CTAs.  The host picks RB so that a warp's rows are one
    // batch.  The loads do not depend on the tokens, so their DRAM latency runs under the quantisation of phase 1;
    // when the launch is a programmatic dependent launch they also run under the tail of the previous kernel.
    const int pK = K >> 2;
    const int warps_total = gridDim.x * WARPS;
    const int nb_first = warp * gridDim.x + blockIdx.x;
    uint4 pk[2][RB];
    auto load_batch = [&](int nb, int i0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = i0 + 32 * u;
#pragma unroll
            for (int r = 0; r < RB; ++r) {
                const int n = nb + r * warps_total;
                pk[u][r] = (i < chunks && n < N) ? __ldg(reinterpret_cast<const uint4*>(Wp + (size_t)n * pK) + i)
                                                 : make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);   // zeros
            }
        }
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    load_batch(nb_first, lane);
    // everything below reads the tokens or writes the output: wait for the work queued before this launch
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool prefetched = true;

    // ---- phase 1: per-token absmax, then int8 into shared memory -----------------------------------------------------
    // fmaxf drops NaN operands and keeps infinities: a finite maximum means that the token holds no infinity, and NaN
    // quantises to 0 by the conversion itself, which is what counting non-finite values as zero gives.
    __shared__ float red[MT][WARPS];
    __shared__ int s_checked;
    float amax[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) amax[m] = 0.0f;
    for (int g = tid; g < (K >> 4); g += THREADS) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                float v[16];
                gv_load16<T>(x + (size_t)m * K + g * 16, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) amax[m] = fmaxf(amax[m], fabsf(v[i]));
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float v = amax[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (lane == 0) red[m][warp] = v;
    }
    __syncthreads();
    if (tid == 0) {
        bool inf_seen = false;
        for (int m = 0; m < MT; ++m) {
            float v = 0.0f;
            for (int w = 0; w < WARPS; ++w) v = fmaxf(v, red[m][w]);
            inf_seen = inf_seen || !(v <= 3.402823466e38f);
            s_amax[m] = fmaxf(v, eps);
        }
        s_checked = inf_seen ? 1 : 0;
    }
    __syncthreads();
    if (s_checked) {
        // some token holds an infinity: redo the maxima with non-finite values counted as zero
        __syncthreads();
#pragma unroll
        for (int m = 0; m < MT; ++m) amax[m] = 0.0f;
        for (int g = tid; g < (K >> 4); g += THREADS) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < M) {
                    float v[16];
                    gv_load16<T>(x + (size_t)m * K + g * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) amax[m] = fmaxf(amax[m], fabsf(finite_or_zero(v[i])));
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = amax[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red[m][warp] = v;
        }
        __syncthreads();
        if (tid < MT) {
            float v = 0.0f;
            for (int w = 0; w < WARPS; ++w) v = fmaxf(v, red[tid][w]);
            s_amax[tid] = fmaxf(v, eps);
        }
        __syncthreads();
    }
    const bool checked = s_checked != 0;
    for (int g = tid; g < (K >> 4); g += THREADS) {
        const int i = g >> 2, j = g & 3;
        const int slot = ((i >> 5) * 4 + j) * 32 + (i & 31);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float s = __fdiv_rn(127.0f, s_amax[m]);
                const T* src = x + (size_t)m * K + g * 16;
                xs[m * xs_per_m + slot] = checked ? gv_quant16<T, true>(src, s) : gv_quant16<T, false>(src, s);
            }
        }
    }
    __syncthreads();

    // ---- phase 2: stream the weight rows ---------------------------------------------------------------------------------
    for (int nb = nb_first; nb < N; nb += warps_total * RB) {
        int acc[RB][MT];
#pragma unroll
        for (int r = 0; r < RB; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0;
        for (int i0 = lane; i0 < chunks; i0 += 64) {
            if (!prefetched) load_batch(nb, i0);
            prefetched = false;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = i0 + 32 * u;
                if (i >= chunks) continue;
                const int base = (i >> 5) * 128 + (i & 31);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 xv[MT];
#pragma unroll
                    for (int m = 0; m < MT; ++m) xv[m] = (m < M) ? xs[m * xs_per_m + base + j * 32] : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int r = 0; r < RB; ++r) {
                        if (r > 0 && nb + r * warps_total >= N) continue;      // same for the whole warp
                        const uint32_t word = (j == 0) ? pk[u][r].x : (j == 1) ? pk[u][r].y : (j == 2) ? pk[u][r].z : pk[u][r].w;
                        uint32_t wv[4];
                        decode16_deint(word, wv);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            acc[r][m] = __dp4a((int)wv[0], (int)xv[m].x, acc[r][m]);
                            acc[r][m] = __dp4a((int)wv[1], (int)xv[m].y, acc[r][m]);
                            acc[r][m] = __dp4a((int)wv[2], (int)xv[m].z, acc[r][m]);
                            acc[r][m] = __dp4a((int)wv[3], (int)xv[m].w, acc[r][m]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
            const int n = nb + r * warps_total;
            if (n >= N) continue;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], o);
            }
            if (lane == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < M) {
                        const float sc = __fmul_rn(__fdiv_rn(s_amax[m], 127.0f), epi.alpha);
                        epi_store_one(epi, m, n, acc[r][m], sc);
                    }
                }
            }
        }
    }
}

template <typename T, int MT, int RB, int THREADS>
static int launch_gemv_rb(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, size_t smem, int grid,
                          cudaStream_t st, bool overlap) {
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(gemv_small_kernel<T, MT, RB, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_once.mark(dev);
    }
    // overlap: programmatic dependent launch.  The kernel may start while earlier work of the stream still runs; it only
    // loads packed weights until its griddepcontrol.wait, which returns once that earlier work has completed.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    EL_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_small_kernel<T, MT, RB, THREADS>, x, Wp, epi, M, N, K, 1e-5f));
    return check_launch();
}

template <typename T, int MT>
static int launch_gemv_t(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap) {
    constexpr int THREADS = (MT <= 2) ? 768 : (MT <= 4) ? 512 : 384;       // by registers: one CTA per SM each time
    constexpr int WARPS = THREADS / 32;
    const int chunks = K >> 6;
    const size_t smem = 32 + (size_t)MT * (((chunks + 31) >> 5) * 128) * sizeof(uint4);
    if (smem > 200 * 1024) return EL_ERR_UNSUPPORTED_SHAPE;
    int sms = 0;
    const int rc = device_sm_count(&sms);
    if (rc != EL_OK) return rc;
    int grid = (N + WARPS - 1) / WARPS;
    if (grid > sms) grid = sms;
    // smallest batch (1, 2 or 4 rows per warp) that covers a warp's rows in one pass; 4 if even that needs several
    const int per_warp = (N + grid * WARPS - 1) / (grid * WARPS);
    if (per_warp <= 1) return launch_gemv_rb<T, MT, 1, THREADS>(x, Wp, epi, M, N, K, smem, grid, st, overlap);
    if (per_warp <= 2) return launch_gemv_rb<T, MT, 2, THREADS>(x, Wp, epi, M, N, K, smem, grid, st, overlap);
    return launch_gemv_rb<T, MT, 4, THREADS>(x, Wp, epi, M, N, K, smem, grid, st, overlap);
}

template <typename T>
static int launch_gemv_m(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap) {
    if (M <= 1) return launch_gemv_t<T, 1>(x, Wp, epi, M, N, K, st, overlap);
    if (M <= 2) return launch_gemv_t<T, 2>(x, Wp, epi, M, N, K, st, overlap);
    if (M <= 4) return launch_gemv_t<T, 4>(x, Wp, epi, M, N, K, st, overlap);
    return launch_gemv_t<T, 8>(x, Wp, epi, M, N, K, st, overlap);
}

// x [M,K] float (16-byte aligned rows), 1 <= M <= 8, K % 64 == 0.  epi.absmax is not read: the scales are computed here.
int launch_gemv_small(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap) {
    if (M < 1 || M > 8 || K % 64 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(Wp) & 15)) return EL_ERR_ALIGNMENT;
    switch (x_dtype) {
        case EL_BF16: return launch_gemv_m((const __nv_bfloat16*)x, Wp, epi, M, N, K, st, overlap);
        case EL_F16: return launch_gemv_m((const __half*)x, Wp, epi, M, N, K, st, overlap);
        case EL_F32: return launch_gemv_m((const float*)x, Wp, epi, M, N, K, st, overlap);
        default: return EL_ERR_INVALID_ARG;
    }
}

}  // namespace el
