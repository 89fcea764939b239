// Small-M ("decode") linear layer for sm_100a: Y[m, n] = (sum_k Xq[m,k] * Wq[n,k]) * (absmax[m]/127) * gamma for
// M <= 64 tokens.  The work is streaming the packed 2-bit weights from HBM once, so the kernel is organised around
// that stream:
//   * operands swapped: the weights are the 128-row MMA operand (A, expanded in shared memory), the few tokens
//     are the narrow N operand (B, 16/32/64 rows, zero-filled by TMA beyond M), so no tensor-core rows are wasted;
//   * one CTA per SM, and the (128-row weight tile, 128-deep reduction block) units are dealt out as one contiguous
//     range per CTA (stream-K), so every SM pulls the same number of bytes whatever N/128 is;
//   * eight packed-tile slots and eight expanded-tile slots, one of each per transform warp: warp w expands the units
//     w, w+8, ... of its CTA on its own, so eight units are in flight and a unit's latencies overlap with the others';
//   * the expansion uses the de-interleaved decode; the tokens were quantised with the matching permutation of the
//     reduction index (launch_quantize_rows_perm), which leaves the integer sums unchanged;
//   * partial sums of a tile that spans several CTAs are added into an int32 workspace with red.global.add (exact,
//     order-free); the CTA that contributes the tile's last reduction block scales it, writes Y and zeroes the
//     workspace again, so the workspace only has to be zero before its first use.
// Every mbarrier wait is bounded (see tc_ptx.cuh).
#include "common.cuh"
#include "epilogue.cuh"
#include "tc_ptx.cuh"

namespace el {
namespace dec {

using namespace tc;

constexpr int TILE_N = 128;      // weight rows per tile (UMMA M)
constexpr int BK = 128;          // reduction depth per unit
constexpr int DP = 8;            // packed-tile slots: one per transform warp
constexpr int DA = 8;            // expanded-tile slots: one per transform warp
constexpr int A_BYTES = TILE_N * BK;        // 16 KB
constexpr int P_BYTES = TILE_N * BK / 4;    // 4 KB
constexpr int WARP_TMA = 0, WARP_MMA = 1, NUM_EPI_WARPS = 4, WARP_XF0 = 6, NUM_XF_WARPS = 8;
constexpr int NUM_THREADS = (WARP_XF0 + NUM_XF_WARPS) * 32;

template <int NU> struct Cfg {
    static constexpr int B_BYTES = NU * BK;                       // token tile
    static constexpr int SLOT = B_BYTES + P_BYTES;                // one slot of the deep ring: [B][P]
    static constexpr int SMEM_BYTES = DA * A_BYTES + DP * SLOT + 1024 + 512;
};

struct Params {
    int M, N, K;
    int tiles, k_blocks;          // N/128 rounded up, K/128 rounded up
    long long units;              // tiles * k_blocks
    EpiParams epi;                // Y, pitch N, dtype, absmax (stride 1), gamma
    int* acc_ws;                  // [64, N] int32, zero on entry, left zero
    int* tile_count;              // [tiles * 4] int32 (one per 32-row quarter), zero on entry, left zero
    int32_t* status;
};

template <int NU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
    using C = Cfg<NU>;
    constexpr uint32_t TMEM_COLS = (2 * NU < 32) ? 32 : 2 * NU;
    constexpr uint32_t TX_BYTES = C::SLOT;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t ring_a = smem_base;                          // DA x 16 KB
    const uint32_t ring_p = smem_base + DA * A_BYTES;           // DP x SLOT
    const uint32_t bars = ring_p + DP * C::SLOT;
    uint8_t* bars_gen = smem_gen + DA * A_BYTES + DP * C::SLOT;
    auto bar_pfull = [&](int s) { return bars + 8u * s; };
    auto bar_pempty = [&](int s) { return bars + 8u * (DP + s); };
    auto bar_ready = [&](int s) { return bars + 8u * (2 * DP + s); };
    auto bar_aempty = [&](int s) { return bars + 8u * (2 * DP + DA + s); };
    auto bar_tfull = [&](int a) { return bars + 8u * (2 * DP + 2 * DA + a); };
    auto bar_tempty = [&](int a) { return bars + 8u * (2 * DP + 2 * DA + 2 + a); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * DP + 2 * DA + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long u_lo = p.units * blockIdx.x / gridDim.x, u_hi = p.units * (blockIdx.x + 1) / gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < DP; ++s) {
            mbar_init(bar_pfull(s), 1);
            mbar_init(bar_pempty(s), 2);          // the transform warp that read P, and the MMAs that read B
        }
        for (int s = 0; s < DA; ++s) {
            mbar_init(bar_ready(s), 1);
            mbar_init(bar_aempty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull(a), 1);
            mbar_init(bar_tempty(a), NUM_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_holder)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    bool failed = false;

    if (warp == WARP_TMA) {
        // ================= producer: packed weight tile + token tile of every unit =================
        // The ring holds eight units (32 KB of packed weights) per SM, too few bytes in flight to keep HBM busy; so all
        // of this CTA's weight tiles are first requested into L2 (the whole matrix is a fraction of it), and the ring's
        // loads then find them there.
        for (long long u = u_lo + lane; u < u_hi; u += 32)
            tma_prefetch_2d(&tmW, (int)(u % p.k_blocks) * (BK / 4), (int)(u / p.k_blocks) * TILE_N);
        __syncwarp();
        if (lane == 0) {
            int sp = 0;
            uint32_t php = 0;
            for (long long u = u_lo; u < u_hi; ++u) {
                const int t = (int)(u / p.k_blocks), kb = (int)(u % p.k_blocks);
                if (!mbar_wait(bar_pempty(sp), php ^ 1u, p.status, 11)) { failed = true; break; }
                const uint32_t slot = ring_p + sp * C::SLOT;
                mbar_expect_tx(bar_pfull(sp), TX_BYTES);
                tma_load_2d(slot, &tmX, bar_pfull(sp), kb * BK, 0);                            // Xq [NU rows x 128 B]
                tma_load_2d(slot + C::B_BYTES, &tmW, bar_pfull(sp), kb * (BK / 4), t * TILE_N);   // W  [128 rows x 32 B]
                if (++sp == DP) { sp = 0; php ^= 1u; }
            }
        }
    } else if (warp == WARP_MMA) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(0, 0, NU);
            int sp = 0, sa = 0, it = 0;
            uint32_t php = 0, pha = 0;
            for (long long u = u_lo; u < u_hi && !failed; ++it) {
                const int kb0 = (int)(u % p.k_blocks);
                const long long rest = u_hi - u;
                const int cnt = (int)((p.k_blocks - kb0) < rest ? (p.k_blocks - kb0) : rest);
                const int acc = it & 1;
                const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(bar_tempty(acc), acc_ph ^ 1u, p.status, 12)) { failed = true; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * NU);
                for (int i = 0; i < cnt; ++i) {
                    if (!mbar_wait(bar_pfull(sp), php, p.status, 13)) { failed = true; break; }
                    if (!mbar_wait(bar_ready(sa), pha, p.status, 14)) { failed = true; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = ring_a + sa * A_BYTES, b_addr = ring_p + sp * C::SLOT;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        umma_i8(d_tmem, make_desc(a_addr + k * 32, 16), make_desc(b_addr + k * 32, 16), idesc, (i | k) != 0);
                    umma_commit(bar_aempty(sa));
                    umma_commit(bar_pempty(sp));
                    if (++sp == DP) { sp = 0; php ^= 1u; }
                    if (++sa == DA) { sa = 0; pha ^= 1u; }
                }
                if (!failed) umma_commit(bar_tfull(acc));
                u += cnt;
            }
        }
    } else if (warp < WARP_XF0) {
        // ================= epilogue: partial sums -> workspace; last contributor of a tile finishes it =========
        const int quarter = warp & 3;
        const int n_in_tile = quarter * 32 + lane;
        // The tokens' scales, two per lane (tokens `lane` and `lane + 32`), handed out by shuffle.  Loading a scale inside
        // the store loops would put a global load and a division behind every store (the compiler must assume the two
        // alias), one trip to L2 per token: that chain was a sixth of the call at 64 tokens.
        const float sc_lo = (lane < p.M) ? epi_row_scale(p.epi, lane) : 0.0f;
        const float sc_hi = (lane + 32 < p.M) ? epi_row_scale(p.epi, lane + 32) : 0.0f;
        auto scale_of = [&](int m) { return __shfl_sync(0xffffffffu, m < 32 ? sc_lo : sc_hi, m & 31); };
        int it = 0;
        for (long long u = u_lo; u < u_hi && !failed; ++it) {
            const int t = (int)(u / p.k_blocks), kb0 = (int)(u % p.k_blocks);
            const long long rest = u_hi - u;
            const int cnt = (int)((p.k_blocks - kb0) < rest ? (p.k_blocks - kb0) : rest);
            const int acc = it & 1;
            const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
            if (!mbar_wait_warp(bar_tfull(acc), acc_ph, p.status, 15)) { failed = true; break; }
            tcgen05_fence_after();
            const int n = t * TILE_N + n_in_tile;
            const bool n_ok = n < p.N;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * NU);
            const bool whole = (cnt == p.k_blocks);      // this CTA holds the complete sums of the tile
            uint32_t v[NU];                               // the whole accumulator row: every load in flight, one wait
#pragma unroll
            for (int c = 0; c < NU / 16; ++c) tmem_ld16(taddr + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&v[c * 16]));
            tmem_ld_wait();
            tcgen05_fence_before();                       // the sums are in registers: hand the accumulator back first
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty(acc));
#pragma unroll
            for (int m = 0; m < NU; ++m) {
                if (m < p.M) {
                    if (whole) {
                        const float sc = scale_of(m);
                        if (n_ok) epi_store_one(p.epi, m, n, (int)v[m], sc);
                    } else if (n_ok) {
                        atomicAdd(p.acc_ws + (size_t)m * p.N + n, (int)v[m]);
                    }
                }
            }
            if (!whole) {
                // Publish this warp's partial sums, then count the segment's reduction blocks towards this quarter
                // of the tile.  Each quarter (32 weight rows) has its own counter, so no warp waits for another:
                // the warp that brings a quarter's count to k_blocks holds the last contribution and finishes it.
                __threadfence();
                __syncwarp();
                int before = 0;
                int* counter = p.tile_count + t * 4 + quarter;
                if (lane == 0) before = atomicAdd(counter, cnt);
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before + cnt == p.k_blocks) {
                    __threadfence();
                    for (int m0 = 0; m0 < p.M; m0 += 32) {      // 32 independent loads in flight per lane
                        int sum[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[j] = (n_ok && m0 + j < p.M) ? __ldcg(p.acc_ws + (size_t)(m0 + j) * p.N + n) : 0;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (m0 + j < p.M) {
                                const float sc = scale_of(m0 + j);
                                if (n_ok) {
                                    __stcg(p.acc_ws + (size_t)(m0 + j) * p.N + n, 0);
                                    epi_store_one(p.epi, m0 + j, n, sum[j], sc);
                                }
                            }
                        }
                    }
                    if (lane == 0) *counter = 0;
                }
            }
            u += cnt;
        }
    } else {
        // ================= transform: packed rows -> swizzled int8 A tile (de-interleaved decode) =================
        // Warp w owns packed slot w and expanded slot w and takes the units j = w, w+8, ... of this CTA; lane l takes
        // the 16-byte segments l, l+32, ... (row = segment/2) of the 128 x 32-byte packed tile.
        static_assert(DP == NUM_XF_WARPS && DA == NUM_XF_WARPS, "one slot of each ring per transform warp");
        const int xw = warp - WARP_XF0;
        const long long n_units = u_hi - u_lo;
        for (long long j = xw; j < n_units; j += NUM_XF_WARPS) {
            const uint32_t phs = (uint32_t)(j / NUM_XF_WARPS) & 1u;
            if (!mbar_wait_warp(bar_pfull(xw), phs, p.status, 16)) { failed = true; break; }
            const uint8_t* sp_gen = smem_gen + DA * A_BYTES + xw * C::SLOT + C::B_BYTES;
            uint4 pk[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) pk[q] = *reinterpret_cast<const uint4*>(sp_gen + (lane + 32 * q) * 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pempty(xw));
            if (!mbar_wait_warp(bar_aempty(xw), phs ^ 1u, p.status, 17)) { failed = true; break; }
            uint8_t* dst = smem_gen + xw * A_BYTES;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int item = lane + 32 * q, row = item >> 1, seg = item & 1;
                const uint32_t px[4] = {pk[q].x, pk[q].y, pk[q].z, pk[q].w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t o[4];
                    decode16_deint(px[w], o);
                    const int chunk = seg * 4 + w;
                    *reinterpret_cast<uint4*>(dst + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ready(xw));
        }
    }

    // ---- teardown ------------------------------------------------------------------------------------------------
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int NU>
static int launch_t(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, cudaStream_t st) {
    constexpr int smem = Cfg<NU>::SMEM_BYTES;
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(decode_tc_kernel<NU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_once.mark(dev);
    }
    int sms = 0;
    const int rc = device_sm_count(&sms);
    if (rc != EL_OK) return rc;
    const int grid = (int)(p.units < sms ? p.units : sms);
    decode_tc_kernel<NU><<<grid, NUM_THREADS, smem, st>>>(tmW, tmX, p);
    return check_launch();
}

}  // namespace dec

namespace tc {
int make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols,
             uint32_t box_rows, bool swizzle128);
}

size_t decode_workspace_bytes(int N) {
    const size_t tiles = (size_t)(N + dec::TILE_N - 1) / dec::TILE_N;
    return ((size_t)64 * (size_t)N + 4 * tiles) * sizeof(int);
}

// Xq: int8 [M,K] quantised with the 16-group permutation; absmax [M]; workspace zero (see the file comment).
int launch_decode_tc(const int8_t* Xq, const uint8_t* Wp, const EpiParams& epi, void* workspace, int M, int N, int K,
                     int32_t* status, cudaStream_t st) {
    if (M < 1 || M > 64 || N < 1 || K < 1) return EL_ERR_UNSUPPORTED_SHAPE;
    if (K % 64 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return EL_ERR_ALIGNMENT;
    int rc = require_sm100();
    if (rc != EL_OK) return rc;
    dec::Params p{};
    p.M = M; p.N = N; p.K = K;
    p.tiles = (N + dec::TILE_N - 1) / dec::TILE_N;
    p.k_blocks = (K + dec::BK - 1) / dec::BK;
    p.units = (long long)p.tiles * p.k_blocks;
    p.epi = epi;
    p.acc_ws = static_cast<int*>(workspace);
    p.tile_count = p.acc_ws + (size_t)64 * N;
    p.status = status;
    const int nu = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap tmW, tmX;
    if ((rc = tc::make_map(&tmW, Wp, K / 4, N, K / 4, 32, dec::TILE_N, false)) != EL_OK) return rc;
    if ((rc = tc::make_map(&tmX, Xq, K, M, K, 128, nu, true)) != EL_OK) return rc;
    switch (nu) {
        case 16: return dec::launch_t<16>(tmW, tmX, p, st);
        case 32: return dec::launch_t<32>(tmW, tmX, p, st);
        default: return dec::launch_t<64>(tmW, tmX, p, st);
    }
}

// ---- decode call that allocates nothing ------------------------------------------------------------------------------
//
// Some hosts of this library cannot hand it device memory: an inference server whose plug-ins are forbidden to call
// cudaMalloc once serving has started, a runtime that owns the whole memory pool, a process already at its memory
// budget.  el_linear_decode needs three scratch buffers from its caller; this variant keeps them in one array that
// is part of the loaded library image, so the caller passes only the input, the weights and the output.

constexpr int STATIC_MAX_TOKENS = 64;
constexpr int STATIC_MAX_N = 16384;       // largest out_features
constexpr int STATIC_MAX_K = 16384;       // largest in_features
constexpr size_t STATIC_WS_BYTES = ((size_t)64 * STATIC_MAX_N + 4 * (size_t)(STATIC_MAX_N / dec::TILE_N)) * sizeof(int);
constexpr size_t STATIC_XQ_OFFSET = (STATIC_WS_BYTES + 255) & ~(size_t)255;
constexpr size_t STATIC_XQ_BYTES = (size_t)STATIC_MAX_TOKENS * STATIC_MAX_K;
constexpr size_t STATIC_ABSMAX_OFFSET = STATIC_XQ_OFFSET + STATIC_XQ_BYTES;
constexpr size_t STATIC_TOTAL_BYTES = STATIC_ABSMAX_OFFSET + 256;          // about 5.3 MB per device

// Lives in every GPU that loads the library, until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_decode_scratch[STATIC_TOTAL_BYTES];

static std::atomic<void*> g_decode_scratch_ptr[64];    // device address of the array, per device ordinal (filled at set-up)

// Set-up for the current device: resolves the array's device address once.  Not an allocation.  Host threads that
// race through the first call each resolve the same address and store the same value.
static int decode_static_setup(unsigned char** out) {
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return EL_ERR_DEVICE;
    void* ptr = g_decode_scratch_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        EL_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_decode_scratch));
        if (ptr == nullptr) return EL_ERR_DEVICE;
        g_decode_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = static_cast<unsigned char*>(ptr);
    return EL_OK;
}

int launch_quantize_rows_perm(const void* x, int dt, long long ldx, int8_t* q, float* a, int M, int K, float eps,
                              cudaStream_t st);
int launch_gemv_small(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap);
int launch_gemv_mma(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st,
                    bool overlap);
bool gemv_mma_fits(int M, int K);
bool gemv_mma_preq_fits(int M, int K);
int launch_gemv_mma_preq(const int8_t* xq, const float* amax, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K,
                         cudaStream_t st);
bool decode_overlap();
int decode_gemv_max_tokens();
int decode_mma_max_tokens();

}  // namespace el

extern "C" EL_API int el_linear_decode_static(const void* x, int x_dtype, const uint8_t* W_packed, void* Y, int out_dtype,
                                              float gamma, int M, int N, int K, int32_t* dev_status, el_stream_t stream) {
    using namespace el;
    auto is_float = [](int dt) { return dt == EL_F16 || dt == EL_BF16 || dt == EL_F32; };
    if (M < 0 || N < 0 || K < 0 || !is_float(x_dtype) || !is_float(out_dtype)) return EL_ERR_INVALID_ARG;
    if (M > STATIC_MAX_TOKENS || N > STATIC_MAX_N || K > STATIC_MAX_K) return EL_ERR_TOO_LARGE;
    if (M == 0 || N == 0) return EL_OK;
    if (K == 0 || K % 64 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (!x || !W_packed || !Y) return EL_ERR_NULL_PTR;
    cudaStream_t st = (cudaStream_t)stream;
    // Set-up comes first, whichever kernel this call ends up on: the first call on a device resolves the array's
    // address even when it is a one-token warm-up, so no later call has to do it (inside a stream capture, say).
    unsigned char* base = nullptr;
    int rc = decode_static_setup(&base);
    if (rc != EL_OK) return rc;
    if (M <= decode_gemv_max_tokens()) {      // the few-token kernel needs no scratch at all
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_small(x, x_dtype, W_packed, gepi, M, N, K, st, decode_overlap());
    }
    if (M <= DECODE_MMA_SINGLE_MAX && M <= decode_mma_max_tokens() && gemv_mma_fits(M, K)) {      // neither does the warp-MMA kernel
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_mma(x, x_dtype, W_packed, gepi, M, N, K, st, decode_overlap());
    }
    int8_t* xq = reinterpret_cast<int8_t*>(base + STATIC_XQ_OFFSET);
    float* absmax = reinterpret_cast<float*>(base + STATIC_ABSMAX_OFFSET);
    if (M <= decode_mma_max_tokens() && gemv_mma_preq_fits(M, K)) {      // the warp-MMA kernel on tokens quantised once
        rc = launch_quantize_rows_perm(x, x_dtype, K, xq, absmax, M, K, 1e-5f, st);
        if (rc != EL_OK) return rc;
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_mma_preq(xq, absmax, W_packed, gepi, M, N, K, st);
    }
    // The array keeps whatever the previous call left.  The partial-sum rows and the tile counters this call will use
    // must start at zero, so they are cleared here on the caller's stream (the rest of the array is overwritten
    // before it is read).
    const size_t tiles = (size_t)(N + dec::TILE_N - 1) / dec::TILE_N;
    EL_CUDA_TRY(cudaMemsetAsync(base, 0, (size_t)M * N * sizeof(int), st));
    EL_CUDA_TRY(cudaMemsetAsync(base + (size_t)64 * N * sizeof(int), 0, 4 * tiles * sizeof(int), st));
    rc = launch_quantize_rows_perm(x, x_dtype, K, xq, absmax, M, K, 1e-5f, st);
    if (rc != EL_OK) return rc;
    const EpiParams epi{Y, (long long)N, out_dtype, absmax, 1, gamma};
    return launch_decode_tc(xq, W_packed, epi, base, M, N, K, dev_status, st);
}
