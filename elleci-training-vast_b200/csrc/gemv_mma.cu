// Decode GEMV for a few to 32 tokens, one launch: Y[m,n] = (sum_k Q(x)[m,k]*Wq[n,k]) * (absmax[m]/127) * gamma.
//
// The call is bound by streaming W_packed once and by the 2-bit -> int8 expansion of the weights; the products themselves
// are few.  With more than a handful of tokens the dp4a of the CUDA-core GEMV (one per token and 4 weights) outgrow the
// expansion, so this kernel feeds the expanded weights to the warp-level int8 MMA (m16n8k32: 16 weight rows x 8 tokens x
// 32 reduction indices per instruction), which makes the multiply cost per weight independent of the token count.  The
// deep tcgen05 pipeline of the large GEMMs is the wrong tool here: its fill latency alone exceeds this call's budget.
//
//   phase 0  every warp requests its first weight fragment (no dependence on the tokens);
//   phase 1  the CTA quantises the tokens (absmax, then int8) into shared memory, laid out as MMA B fragments and
//            permuted inside groups of 16 to match the cheap de-interleaved weight decode;
//   phase 2  CTA b owns the 16-row groups b, b + gridDim.x, ...; its 16 warps split the reduction in blocks of 256
//            indices.  A lane loads 16 bytes (64 weights) of rows r and r+8, expands them and issues 8 MMAs per token
//            group; the warps' partial sums meet in shared memory (red.shared.add) and the CTA scales and stores them.
// The reduction index may be permuted freely as long as weights and tokens use the same permutation: lane (r, s) owns
// the 64 consecutive indices 64*s.. of the block for both operands, so no data moves between lanes.
// The integers and the rounding are those of el_quantize_rows + el_gemm_fwd.
#include "common.cuh"
#include "epilogue.cuh"

namespace el {

int device_sm_count(int* out);

namespace {

constexpr int GM_THREADS = 512;
constexpr int GM_WARPS = GM_THREADS / 32;

template <typename T> __device__ __forceinline__ void gm_load16(const T* p, float v[16]);
template <> __device__ __forceinline__ void gm_load16<__nv_bfloat16>(const __nv_bfloat16* p, float v[16]) {
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
template <> __device__ __forceinline__ void gm_load16<__half>(const __half* p, float v[16]) {
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
template <> __device__ __forceinline__ void gm_load16<float>(const float* p, float v[16]) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const float4 a = reinterpret_cast<const float4*>(p)[h];
        v[4 * h] = a.x; v[4 * h + 1] = a.y; v[4 * h + 2] = a.z; v[4 * h + 3] = a.w;
    }
}

// 16 consecutive values -> int8 in the order {0,2,4,6, 8,10,12,14, 1,3,5,7, 9,11,13,15}
template <typename T, bool CHECKED>
__device__ __forceinline__ uint4 gm_quant16(const T* src, float s) {
    float v[16];
    gm_load16<T>(src, v);
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = q8_sat(__fmul_rn(CHECKED ? finite_or_zero(v[i]) : v[i], s));
    return make_uint4(pack4_s8(q[0], q[2], q[4], q[6]), pack4_s8(q[8], q[10], q[12], q[14]), pack4_s8(q[1], q[3], q[5], q[7]),
                      pack4_s8(q[9], q[11], q[13], q[15]));
}

__device__ __forceinline__ void mma_s8(int d[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT token groups of 8.  Shared memory: [0,256) absmax floats; then the tokens as B fragments, uint4 index
// ((kb*4 + w)*MT + m)*4 + s for the 16 indices 256*kb + 64*s + 16*w .. of token m (a quarter-warp then reads eight
// consecutive uint4: no bank conflicts); then two [16][MT] int32 accumulators for the cross-warp sums.
// PREQ: the tokens arrive quantised (xq int8 [M,K] in the permuted order, amax_in [M], written by the launch before this
// one) and are only copied into shared memory; otherwise every CTA quantises x itself.
template <typename T, int NT, bool PREQ>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemv_mma_kernel(const T* __restrict__ x, const int8_t* xq, const float* amax_in, const uint8_t* __restrict__ Wp, EpiParams epi,
                int M, int N, int K, float eps) {
    constexpr int MT = NT * 8;
    extern __shared__ uint4 gm_smem[];
    float* s_amax = reinterpret_cast<float*>(gm_smem);
    uint4* xs = gm_smem + 16;
    const int kblocks = (K + 255) >> 8;
    int* acc_sm = reinterpret_cast<int*>(xs + (size_t)kblocks * 16 * MT);
    __shared__ int s_checked;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r8 = lane >> 2, seg = lane & 3;
    const int pK = K >> 2;
    const int row_groups = (N + 15) >> 4;

    // ---- phase 0: first weight fragment -----------------------------------------------------------------------------------
    // Work items of a warp: (row group g, reduction block kb) with g = blockIdx.x + i*gridDim.x, kb = warp + j*GM_WARPS.
    const uint4 zeros = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
    auto load_frag = [&](int g, int kb, uint4& lo, uint4& hi) {
        const int k0 = kb * 256 + seg * 64;
        const int n0 = g * 16 + r8;
        const bool k_ok = k0 < K;
        lo = (k_ok && n0 < N) ? __ldg(reinterpret_cast<const uint4*>(Wp + (size_t)n0 * pK + (k0 >> 2))) : zeros;
        hi = (k_ok && n0 + 8 < N) ? __ldg(reinterpret_cast<const uint4*>(Wp + (size_t)(n0 + 8) * pK + (k0 >> 2))) : zeros;
    };
    // A warp's work items in order: row groups outermost, its blocks warp, warp + 16, ... inside.  The fragments of the
    // next DEPTH items are always in flight (a warp has only a handful of items, each worth a fraction of a memory latency
    // of work), the first ones from before the token quantisation.
    const bool has_work = warp < kblocks;          // a warp whose first block lies beyond the reduction never has work
    const int nk = has_work ? (kblocks - warp + GM_WARPS - 1) / GM_WARPS : 1;      // blocks per row group for this warp
    constexpr int DEPTH = 2;
    uint4 qlo[DEPTH], qhi[DEPTH];
    int fetch_g = blockIdx.x, fetch_j = 0;         // next item to request
    auto fetch = [&](uint4& lo, uint4& hi) {
        if (has_work && fetch_g < row_groups) load_frag(fetch_g, warp + fetch_j * GM_WARPS, lo, hi);
        else { lo = zeros; hi = zeros; }
        if (++fetch_j == nk) { fetch_j = 0; fetch_g += gridDim.x; }
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) fetch(qlo[i], qhi[i]);
    // everything below reads the tokens or writes the output: wait for the work queued before this launch
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- phase 1: per-token absmax, then int8 B fragments into shared memory ------------------------------------------------
    // Warp w takes the tokens w, w + 16, ...: a token's maximum then needs no exchange between warps, and the tokens
    // are read by all warps at once instead of one after the other.
    const int groups = K >> 4;
    for (int i = tid; i < 2 * 16 * MT; i += GM_THREADS) acc_sm[i] = 0;
    if (tid == 0) s_checked = 0;
    if (PREQ) {
        if (tid < MT) s_amax[tid] = tid < M ? __ldcg(amax_in + tid) : 1.0f;
    } else {
        __syncthreads();
        for (int m = warp; m < M; m += GM_WARPS) {
            float amax = 0.0f;
            for (int g = lane; g < groups; g += 32) {
                float v[16];
                gm_load16<T>(x + (size_t)m * K + g * 16, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));        // drops NaN, keeps infinities
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (!(amax <= 3.402823466e38f)) {
                // the token holds an infinity: redo its maximum with non-finite values counted as zero
                amax = 0.0f;
                for (int g = lane; g < groups; g += 32) {
                    float v[16];
                    gm_load16<T>(x + (size_t)m * K + g * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(finite_or_zero(v[i])));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (lane == 0) s_checked = 1;
            }
            if (lane == 0) s_amax[m] = fmaxf(amax, eps);
        }
    }
    __syncthreads();
    const bool checked = s_checked != 0;
    // A warp fills, per step, the 16 groups of one 256-block for a pair of tokens: two 256-byte runs of global memory,
    // and shared-memory addresses that fall four to each 16-byte bank group (the uint4 index is ... + m*4 + s).
    const int work = kblocks * (MT / 2) * 32;
    for (int i = tid; i < work; i += GM_THREADS) {
        const int l = i & 31, chunk = i >> 5;
        const int kb = chunk / (MT / 2), m = (chunk - kb * (MT / 2)) * 2 + (l >> 4);
        const int g = kb * 16 + (l & 15);
        const int sg = (g >> 2) & 3, w = g & 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);                  // padding tokens and indices beyond K multiply by zero
        if (m < M && g < groups) {
            if (PREQ) {
                v = __ldcg(reinterpret_cast<const uint4*>(xq + (size_t)m * K) + g);
            } else {
                const float s = __fdiv_rn(127.0f, s_amax[m]);
                const T* src = x + (size_t)m * K + g * 16;
                v = checked ? gm_quant16<T, true>(src, s) : gm_quant16<T, false>(src, s);
            }
        }
        xs[((kb * 4 + w) * MT + m) * 4 + sg] = v;
    }
    __syncthreads();

    // ---- phase 2 ------------------------------------------------------------------------------------------------------------------
    int gi = 0;                                   // row groups done by this CTA (selects the accumulator buffer)
    for (int g = blockIdx.x; g < row_groups; g += gridDim.x, ++gi) {
        int d[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) d[t][0] = d[t][1] = d[t][2] = d[t][3] = 0;
        if (has_work) {
            for (int kb = warp; kb < kblocks; kb += GM_WARPS) {
                const uint4 lo = qlo[0], hi = qhi[0];
#pragma unroll
                for (int i = 0; i + 1 < DEPTH; ++i) { qlo[i] = qlo[i + 1]; qhi[i] = qhi[i + 1]; }
                fetch(qlo[DEPTH - 1], qhi[DEPTH - 1]);
                const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t dl[4], dh[4];
                    decode16_deint(wl[w], dl);
                    decode16_deint(wh[w], dh);
                    const uint32_t a_even[4] = {dl[0], dh[0], dl[1], dh[1]};     // indices {0,2,4,6 | 8,10,12,14} of the group
                    const uint32_t a_odd[4] = {dl[2], dh[2], dl[3], dh[3]};      // indices {1,3,5,7 | 9,11,13,15}
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const uint4 xv = xs[((kb * 4 + w) * MT + t * 8 + r8) * 4 + seg];
                        mma_s8(d[t], a_even, xv.x, xv.y);
                        mma_s8(d[t], a_odd, xv.z, xv.w);
                    }
                }
            }
            // partial sums of this warp's blocks -> the CTA's accumulator for this row group
            int* acc = acc_sm + (gi & 1) * 16 * MT;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int col = t * 8 + seg * 2;
                atomicAdd(&acc[r8 * MT + col], d[t][0]);
                atomicAdd(&acc[r8 * MT + col + 1], d[t][1]);
                atomicAdd(&acc[(r8 + 8) * MT + col], d[t][2]);
                atomicAdd(&acc[(r8 + 8) * MT + col + 1], d[t][3]);
            }
        }
        __syncthreads();
        // scale, store, and clear the buffer for the row group after next (a barrier lies in between)
        int* acc = acc_sm + (gi & 1) * 16 * MT;
        for (int i = tid; i < 16 * MT; i += GM_THREADS) {
            const int m = i >> 4, row = i & 15;
            const int n = g * 16 + row;
            const int v = acc[row * MT + m];
            acc[row * MT + m] = 0;
            if (m < M && n < N) {
                const float sc = __fmul_rn(__fdiv_rn(s_amax[m], 127.0f), epi.alpha);
                epi_store_one(epi, m, n, v, sc);
            }
        }
    }
}

template <typename T, int NT, bool PREQ>
int launch_gemv_mma_t(const T* x, const int8_t* xq, const float* amax, const uint8_t* Wp, const EpiParams& epi, int M, int N,
                      int K, cudaStream_t st, bool overlap) {
    constexpr int MT = NT * 8;
    const int kblocks = (K + 255) >> 8;
    const size_t smem = 256 + (size_t)kblocks * 16 * MT * sizeof(uint4) + 2 * 16 * MT * sizeof(int);
    if (smem > 200 * 1024) return EL_ERR_UNSUPPORTED_SHAPE;
    int sms = 0;
    const int rc = device_sm_count(&sms);
    if (rc != EL_OK) return rc;
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(gemv_mma_kernel<T, NT, PREQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_once.mark(dev);
    }
    const int row_groups = (N + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(row_groups < sms ? row_groups : sms));
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    EL_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_mma_kernel<T, NT, PREQ>, x, xq, amax, Wp, epi, M, N, K, 1e-5f));
    return check_launch();
}

template <typename T>
int launch_gemv_mma_m(const T* x, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap) {
    if (M <= 8) return launch_gemv_mma_t<T, 1, false>(x, nullptr, nullptr, Wp, epi, M, N, K, st, overlap);
    if (M <= 16) return launch_gemv_mma_t<T, 2, false>(x, nullptr, nullptr, Wp, epi, M, N, K, st, overlap);
    return launch_gemv_mma_t<T, 4, false>(x, nullptr, nullptr, Wp, epi, M, N, K, st, overlap);
}

}  // namespace

// Whether launch_gemv_mma takes the problem: up to 32 tokens whose int8 image fits in shared memory.
bool gemv_mma_fits(int M, int K) {
    if (M < 1 || M > 32 || K <= 0 || K % 64 != 0) return false;
    const int mt = M <= 8 ? 8 : (M <= 16 ? 16 : 32);
    const size_t kblocks = (size_t)(K + 255) >> 8;
    return 256 + kblocks * 16 * mt * sizeof(uint4) + 2 * 16 * mt * sizeof(int) <= 200 * 1024;
}

// x [M,K] float (16-byte aligned rows), K % 64 == 0.  epi.absmax is not read: the scales are computed here.
int launch_gemv_mma(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st,
                    bool overlap) {
    if (!gemv_mma_fits(M, K)) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(Wp) & 15)) return EL_ERR_ALIGNMENT;
    switch (x_dtype) {
        case EL_BF16: return launch_gemv_mma_m((const __nv_bfloat16*)x, Wp, epi, M, N, K, st, overlap);
        case EL_F16: return launch_gemv_mma_m((const __half*)x, Wp, epi, M, N, K, st, overlap);
        case EL_F32: return launch_gemv_mma_m((const float*)x, Wp, epi, M, N, K, st, overlap);
        default: return EL_ERR_INVALID_ARG;
    }
}

// The same kernel on tokens that launch_quantize_rows_perm has already quantised on this stream (xq int8 [M,K], amax [M]):
// no CTA repeats the quantisation, which is what the single-launch form spends most of its time on from about 16 tokens
// up (148 CTAs each converting all M*K values).  The launch is a programmatic dependent of the quantiser: its CTAs
// request their first weight fragments while the quantiser still runs and read the tokens after it has completed.  That
// is safe whatever else the stream holds, because the quantiser itself started after all earlier work had finished.
// Any number of tokens: they are taken 32 (or 16, or 8) at a time, one launch each; the weights of the later launches
// come from L2.
bool gemv_mma_preq_fits(int M, int K) {
    if (M < 1 || K <= 0 || K % 64 != 0) return false;
    return gemv_mma_fits(M < 32 ? M : 32, K);
}

int launch_gemv_mma_preq(const int8_t* xq, const float* amax, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K,
                         cudaStream_t st) {
    if (!gemv_mma_preq_fits(M, K)) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(Wp) & 15)) return EL_ERR_ALIGNMENT;
    const size_t out_bytes = (epi.out_dtype == EL_F16 || epi.out_dtype == EL_BF16) ? 2 : 4;
    for (int m0 = 0; m0 < M; m0 += 32) {
        const int mc = (M - m0) < 32 ? (M - m0) : 32;
        EpiParams e = epi;
        e.out = static_cast<unsigned char*>(epi.out) + (size_t)m0 * epi.ldo * out_bytes;
        const int8_t* q = xq + (size_t)m0 * K;
        const float* a = amax + m0;
        const __nv_bfloat16* none = nullptr;
        int rc;
        if (mc <= 8) rc = launch_gemv_mma_t<__nv_bfloat16, 1, true>(none, q, a, Wp, e, mc, N, K, st, true);
        else if (mc <= 16) rc = launch_gemv_mma_t<__nv_bfloat16, 2, true>(none, q, a, Wp, e, mc, N, K, st, true);
        else rc = launch_gemv_mma_t<__nv_bfloat16, 4, true>(none, q, a, Wp, e, mc, N, K, st, true);
        if (rc != EL_OK) return rc;
    }
    return EL_OK;
}

}  // namespace el
