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

constexpr int GV_THREADS = 256;

// Shared memory: float amax[MT]; then per token ceil(K/2048)*128 uint4 (chunk i of 64 weights -> four uint4 at
// ((i/32)*4 + j)*32 + i%32, so that consecutive lanes read consecutive 16-byte words).
template <typename T, int MT, int RB>
__global__ void __launch_bounds__(GV_THREADS, (MT <= 4) ? 3 : 2)
gemv_small_kernel(const T* __restrict__ x, const uint8_t* __restrict__ Wp, EpiParams epi, int M, int N, int K, float eps) {
    extern __shared__ uint4 gv_smem[];
    float* s_amax = reinterpret_cast<float*>(gv_smem);
    uint4* xs = gv_smem + 2;                      // 32 bytes reserved for the absmax values
    const int chunks = K >> 6;                    // 64 weights per chunk
    const int xs_per_m = ((chunks + 31) >> 5) * 128;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- phase 0: the first batch of packed weights is requested before anything else ------------------------------------
    // A warp works on RB rows at once and on two 64-weight chunks per lane and row, so that 2*RB 16-byte loads per
    // lane are in flight: a row of 1024 packed bytes alone would leave the warp waiting on one memory latency per row.
    // The host picks RB so that the grid is a single wave in which every warp has exactly one batch of RB rows.  The
    // loads do not depend on the tokens, so their DRAM latency runs under the quantisation of phase 1; when the launch
    // is a programmatic dependent launch they also run under the tail of the previous kernel of the stream.
    const int pK = K >> 2;
    const int warps_total = gridDim.x * (GV_THREADS / 32);
    const int nb_first = blockIdx.x * (GV_THREADS / 32) + warp;
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
    float amax[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) amax[m] = 0.0f;
    for (int g = tid; g < (K >> 4); g += GV_THREADS) {
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
    __shared__ float red[MT][GV_THREADS / 32];
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
#pragma unroll
        for (int w = 0; w < GV_THREADS / 32; ++w) v = fmaxf(v, red[tid][w]);
        s_amax[tid] = fmaxf(v, eps);
    }
    __syncthreads();
    for (int g = tid; g < (K >> 4); g += GV_THREADS) {
        const int i = g >> 2, j = g & 3;
        const int slot = ((i >> 5) * 4 + j) * 32 + (i & 31);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                float v[16];
                gv_load16<T>(x + (size_t)m * K + g * 16, v);
                const float s = __fdiv_rn(127.0f, s_amax[m]);
                uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
                for (int p = 0; p < 16; ++p) {
                    const int src = (p < 8) ? 2 * p : 2 * (p - 8) + 1;
                    float r = rintf(__fmul_rn(finite_or_zero(v[src]), s));
                    r = fminf(127.0f, fmaxf(-128.0f, r));
                    w[p >> 2] |= (uint32_t)((int)r & 0xFF) << (8 * (p & 3));
                }
                xs[m * xs_per_m + slot] = make_uint4(w[0], w[1], w[2], w[3]);
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
#pragma unroll
            for (int m = 0; m < MT; ++m) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], o);
            }
            const int n = nb + r * warps_total;
            if (lane == 0 && n < N) {
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

template <typename T, int MT, int RB>
static int launch_gemv_rb(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, size_t smem, int grid,
                          cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        EL_CUDA_TRY(cudaFuncSetAttribute(gemv_small_kernel<T, MT, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    gemv_small_kernel<T, MT, RB><<<grid, GV_THREADS, smem, st>>>(x, Wp, epi, M, N, K, 1e-5f);
    return check_launch();
}

template <typename T, int MT>
static int launch_gemv_t(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st) {
    const int chunks = K >> 6;
    const size_t smem = 32 + (size_t)MT * (((chunks + 31) >> 5) * 128) * sizeof(uint4);
    if (smem > 200 * 1024) return EL_ERR_UNSUPPORTED_SHAPE;
    int sms = 0;
    const int rc = device_sm_count(&sms);
    if (rc != EL_OK) return rc;
    // resident CTAs per SM: three by registers for up to four tokens, two otherwise; fewer when shared memory binds
    int per_sm = (MT <= 4) ? 3 : 2;
    while (per_sm > 1 && smem * per_sm > 200 * 1024) --per_sm;
    const int slots = sms * per_sm;
    const int rows_per_cta1 = GV_THREADS / 32;
    // smallest batch (1, 2 or 4 rows per warp) whose grid fits in one wave; 4 if even that needs more than one
    int rb = 1;
    while (rb < 4 && (N + rows_per_cta1 * rb - 1) / (rows_per_cta1 * rb) > slots) rb *= 2;
    const int grid = (N + rows_per_cta1 * rb - 1) / (rows_per_cta1 * rb);
    if (rb == 1) return launch_gemv_rb<T, MT, 1>(x, Wp, epi, M, N, K, smem, grid, st);
    if (rb == 2) return launch_gemv_rb<T, MT, 2>(x, Wp, epi, M, N, K, smem, grid < slots ? grid : slots, st);
    return launch_gemv_rb<T, MT, 4>(x, Wp, epi, M, N, K, smem, grid < slots ? grid : slots, st);
}

template <typename T>
static int launch_gemv_m(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st) {
    if (M <= 1) return launch_gemv_t<T, 1>(x, Wp, epi, M, N, K, st);
    if (M <= 2) return launch_gemv_t<T, 2>(x, Wp, epi, M, N, K, st);
    if (M <= 4) return launch_gemv_t<T, 4>(x, Wp, epi, M, N, K, st);
    return launch_gemv_t<T, 8>(x, Wp, epi, M, N, K, st);
}

// x [M,K] float (16-byte aligned rows), 1 <= M <= 8, K % 64 == 0.  epi.absmax is not read: the scales are computed here.
int launch_gemv_small(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st) {
    if (M < 1 || M > 8 || K % 64 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(Wp) & 15)) return EL_ERR_ALIGNMENT;
    switch (x_dtype) {
        case EL_BF16: return launch_gemv_m((const __nv_bfloat16*)x, Wp, epi, M, N, K, st);
        case EL_F16: return launch_gemv_m((const __half*)x, Wp, epi, M, N, K, st);
        case EL_F32: return launch_gemv_m((const float*)x, Wp, epi, M, N, K, st);
        default: return EL_ERR_INVALID_ARG;
    }
}

}  // namespace el
