// Single-CTA tensor-core integer GEMMs of the INT2 linear path for sm_100a: tcgen05.mma kind::i8 with the int32
// accumulators in tensor memory, operands staged by TMA, and the scaling (or hysteresis) epilogue reading the
// accumulators back with tcgen05.ld.  This file carries the weight-gradient GEMM (plain and fused with the hysteresis
// update) and single-CTA forward / dX modes; the default forward / dX kernels run on CTA pairs (gemm_tc2.cu).
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0      TMA producer: activations (and, for the weight-gradient GEMM, both operands) plus the packed
//               2-bit weight tile of every 128-deep reduction block, through a ring of shared-memory stages
//   warp 1      allocates tensor memory; one lane issues the MMAs and commits them to the ring's barriers
//   warps 2-5   epilogue: tcgen05.ld of one of two accumulators while the MMAs fill the other
//   warps 6-13  FWD / DX: expand the packed weight tile into the 128-byte-swizzled int8 operand tile;
//               DW: no tile to expand, so they join the epilogue (twelve epilogue warps, three per lane quarter;
//               sixteen, four per quarter, in the fused dW + hysteresis kernel)
//
// The three GEMMs differ only in where the reduction index lies in memory:
//   FWD  Y [M,N] = Xq [M,K] . Wq[N,K]^T   A K-major (TMA),  B K-major  (expanded from W_packed rows)
//   DX   dX[M,K] = dYq[M,N] . Wq[N,K]     A K-major (TMA),  B MN-major (the same expanded rows, read transposed)
//   DW   dW[N,K] = Gq [M,N]^T . Xq[M,K]   A MN-major (TMA), B MN-major (TMA)
// so the expanded weight tile has one shared-memory image (row r at r*128 bytes, 16-byte chunk c at
// (c ^ (r & 7)) * 16) and only the matrix descriptors change.
//
// Every wait on an mbarrier is bounded: when it gives up, the kernel records a code in *status, lets its
// outstanding copies land, frees tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "tc_ptx.cuh"

namespace el {

enum { MODE_FWD = 0, MODE_DX = 1, MODE_DW = 2 };
enum { EPI_SCALE = 0, EPI_HYST = 1 };

namespace tc {

constexpr int BM = 128;            // rows of an output tile (UMMA M)
constexpr int BK = 128;            // reduction depth per stage (bytes of int8)
constexpr int UMMA_K = 32;         // reduction depth of one kind::i8 instruction
constexpr int WARP_TMA = 0, WARP_MMA = 1, NUM_EPI_WARPS = 4, WARP_XF0 = 6, NUM_XF_WARPS = 8;   // warps 2..5: epilogue
constexpr int NUM_THREADS = (WARP_XF0 + NUM_XF_WARPS) * 32;   // 448
// The fused weight-gradient kernel has no weight tile to expand and is bound by its epilogue: it runs sixteen epilogue
// warps (four per quarter of the tensor-memory lanes, two 32-column chunks each) instead of twelve.
constexpr int DW_EXTRA_WARPS = 4;
__host__ __device__ constexpr int num_threads(int mode, int epi) {
    return NUM_THREADS + ((mode == MODE_DW && epi == EPI_HYST) ? DW_EXTRA_WARPS * 32 : 0);
}

constexpr int A_BYTES = BM * BK;                       // 16 KB
template <int BN> struct Cfg {
    static constexpr int B_BYTES = BN * BK;            // expanded / int8 B tile
    static constexpr int P_BYTES = BN * BK / 4;        // packed weight tile
    __host__ __device__ static constexpr int STAGES(int mode) { return mode == MODE_DW ? (BN == 256 ? 4 : 6) : (BN == 256 ? 3 : 5); }
    __host__ __device__ static constexpr int STAGE_BYTES(int mode) { return A_BYTES + B_BYTES + (mode == MODE_DW ? 0 : P_BYTES); }
    __host__ __device__ static constexpr int SMEM_BYTES(int mode) { return STAGES(mode) * STAGE_BYTES(mode) + 1024 /*align*/ + 256 /*barriers*/; }
};

struct Params {
    int R, C, D;                    // output rows, output columns, reduction depth
    int tiles_r, tiles_c, k_blocks;
    EpiParams epi;
    int vec_ok;                     // output rows keep 16-byte alignment
    int32_t* status;
    // hysteresis epilogue (DW only)
    uint8_t* Wp;
    uint8_t* Hp;
    int pK, pH;
    HystParams hp;
    uint32_t idx_base;
};

// ---- the kernel ----------------------------------------------------------------------------------------------

template <int MODE, int BN, int EPI>
__global__ void __launch_bounds__(num_threads(MODE, EPI), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
    using C = Cfg<BN>;
    constexpr int STAGES = C::STAGES(MODE);
    constexpr int STAGE_BYTES = C::STAGE_BYTES(MODE);
    constexpr bool XFORM = (MODE != MODE_DW);
    constexpr uint32_t TMEM_COLS = 2 * BN;     // two accumulators of BN int32 columns (256 or 512: powers of two)
    constexpr uint32_t TX_BYTES = A_BYTES + (XFORM ? C::P_BYTES : C::B_BYTES);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // stage s: [A 16K][B BN*128][P BN*32]
    const uint32_t bars = smem_base + STAGES * STAGE_BYTES;
    uint8_t* bars_gen = smem_gen + STAGES * STAGE_BYTES;
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_ready = [&](int s) { return bars + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    auto bar_tfull = [&](int a) { return bars + 8u * (3 * STAGES + a); };
    auto bar_tempty = [&](int a) { return bars + 8u * (3 * STAGES + 2 + a); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (3 * STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_r * p.tiles_c;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_ready(s), NUM_XF_WARPS);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull(a), 1);
            mbar_init(bar_tempty(a), num_threads(MODE, EPI) / 32 - 2 - (XFORM ? NUM_XF_WARPS : 0));
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
        // ================= producer =================
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
                const int r0 = (t % p.tiles_r) * BM, c0 = (t / p.tiles_r) * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(bar_empty(s), ph ^ 1u, p.status, 1)) { failed = true; break; }
                    const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES, sp = sb + C::B_BYTES;
                    const int d0 = kb * BK;
                    mbar_expect_tx(bar_full(s), TX_BYTES);
                    if (MODE == MODE_FWD) {
                        tma_load_2d(sa, &tmA, bar_full(s), d0, r0);            // Xq  [128 rows x 128 B]
                        tma_load_2d(sp, &tmB, bar_full(s), d0 >> 2, c0);       // W   [BN rows x 32 B]
                    } else if (MODE == MODE_DX) {
                        tma_load_2d(sa, &tmA, bar_full(s), d0, r0);            // dYq [128 rows x 128 B]
                        tma_load_2d(sp, &tmB, bar_full(s), c0 >> 2, d0);       // W   [128 rows x BN/4 B]
                    } else {
                        tma_load_2d(sa, &tmA, bar_full(s), r0, d0);            // Gq  [128 m-rows x 128 n]
#pragma unroll
                        for (int b = 0; b < BN / 128; ++b)
                            tma_load_2d(sb + b * 16384, &tmB, bar_full(s), c0 + b * 128, d0);   // Xq [128 m-rows x 128 k]
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(MODE == MODE_DW, MODE != MODE_FWD, BN);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(bar_tempty(acc), acc_ph ^ 1u, p.status, 2)) { failed = true; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(bar_full(s), ph, p.status, 3)) { failed = true; break; }
                    if (XFORM && !mbar_wait(bar_ready(s), ph, p.status, 4)) { failed = true; break; }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: step 32 bytes along the row; MN-major: step 32 reduction rows of 128 bytes
                        const uint64_t da = (MODE == MODE_DW) ? make_desc(sa + k * 4096, 16384) : make_desc(sa + k * 32, 16);
                        const uint64_t db = (MODE == MODE_FWD) ? make_desc(sb + k * 32, 16) : make_desc(sb + k * 4096, 16384);
                        umma_i8(d_tmem, da, db, idesc, (kb | k) != 0);
                    }
                    umma_commit(bar_empty(s));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (!failed) umma_commit(bar_tfull(acc));
            }
        }
    } else if (warp < WARP_XF0 || !XFORM) {
        // ================= epilogue =================
        // Without a weight tile to expand (DW) the transform warps join in: three warps (four in the fused kernel)
        // share each quarter of the tensor-memory lanes and take the 32-column chunks round-robin.
        constexpr int EPI_SPLIT = XFORM ? 1 : (num_threads(MODE, EPI) / 32 - 2) / 4;      // 3, or 4 in the fused kernel
        const int quarter = warp & 3;                 // the tensor-memory lanes this warp may read
        const int sub = (warp - 2) >> 2;              // 0 for warps 2-5, 1 for 6-9, 2 for 10-13, 3 for 14-17
        const int row_in_tile = quarter * 32 + lane;
        HystParams hp;                                // with the step taken from device memory when the launch says so
        if (EPI == EPI_HYST) hp = hyst_resolve_step(p.hp);
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x, ++it) {
            const int r0 = (t % p.tiles_r) * BM, c0 = (t / p.tiles_r) * BN;
            const int acc = it & 1;
            const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
            const int row = r0 + row_in_tile;
            const bool row_ok = row < p.R;
            // Fused update: the packed weights and counters of this warp's chunks do not depend on the accumulator, so they
            // are requested before the wait for it and arrive while the tile's MMAs still run.
            constexpr int HYST_CHUNKS = (BN / 32 + EPI_SPLIT - 1) / EPI_SPLIT;
            uint2 w_pre[HYST_CHUNKS];
            uint4 h_pre[HYST_CHUNKS];
            if (EPI == EPI_HYST) {
#pragma unroll
                for (int i = 0; i < HYST_CHUNKS; ++i) {
                    const int c = (XFORM ? 0 : sub) + i * EPI_SPLIT;
                    const int col0 = c0 + c * 32;
                    if (c < BN / 32 && row_ok && col0 < p.C) {     // K % 32 == 0: a chunk is inside or outside as a whole
                        w_pre[i] = *reinterpret_cast<const uint2*>(p.Wp + (size_t)row * p.pK + (col0 >> 2));
                        h_pre[i] = *reinterpret_cast<const uint4*>(p.Hp + (size_t)row * p.pH + (col0 >> 1));
                    }
                }
            }
            if (!mbar_wait_warp(bar_tfull(acc), acc_ph, p.status, 5)) { failed = true; break; }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            if (EPI == EPI_SCALE) {
                const float sc = row_ok ? epi_row_scale(p.epi, row) : 0.0f;
#pragma unroll 1
                for (int c = (XFORM ? 0 : sub); c < BN / 32; c += EPI_SPLIT) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    const int col0 = c0 + c * 32;
                    if (row_ok && col0 < p.C) epi_store_chunk32(p.epi, row, col0, p.C, v, sc, p.vec_ok != 0);
                }
            } else {
                // weight-gradient tile -> hysteresis update of 32 weights of row `row` per chunk
                const float sc = epi_row_scale(p.epi, 0);   // g_absmax/127 (one scale for the tensor)
#pragma unroll
                for (int i = 0; i < HYST_CHUNKS; ++i) {
                    const int c = (XFORM ? 0 : sub) + i * EPI_SPLIT;
                    if (c >= BN / 32) break;
                    uint32_t v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    const int col0 = c0 + c * 32;
                    if (row_ok && col0 < p.C) {
                        uint32_t w[2] = {w_pre[i].x, w_pre[i].y};
                        uint32_t h[4] = {h_pre[i].x, h_pre[i].y, h_pre[i].z, h_pre[i].w};
                        const uint32_t idx0 = p.idx_base + (uint32_t)row * (uint32_t)p.C + (uint32_t)col0;
                        if ((p.idx_base & 31u) == 0) hyst_update_chunk32<true, true>(v, sc, w, h, idx0, hp);     // C % 32 == 0
                        else hyst_update_chunk32<true, false>(v, sc, w, h, idx0, hp);
                        *reinterpret_cast<uint2*>(p.Wp + (size_t)row * p.pK + (col0 >> 2)) = make_uint2(w[0], w[1]);
                        *reinterpret_cast<uint4*>(p.Hp + (size_t)row * p.pH + (col0 >> 1)) = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty(acc));
        }
    } else if (XFORM) {
        // ================= transform: packed 2-bit rows -> swizzled int8 operand tile =================
        const int xt = threadIdx.x - WARP_XF0 * 32;       // 0..255
        constexpr int PROW = (MODE == MODE_FWD) ? 32 : BN / 4;     // packed bytes per tile row
        constexpr int SEGS = PROW / 16;                              // 16-byte segments (64 weights) per row
        constexpr int ROWS = (MODE == MODE_FWD) ? BN : 128;
        constexpr int ITEMS = ROWS * SEGS;
        int s = 0;
        uint32_t ph = 0;
        for (int t = blockIdx.x; t < num_tiles && !failed; t += gridDim.x) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!mbar_wait_warp(bar_full(s), ph, p.status, 6)) { failed = true; break; }
                uint8_t* sb = smem_gen + s * STAGE_BYTES + A_BYTES;
                const uint8_t* sp = sb + C::B_BYTES;
#pragma unroll
                for (int i = xt; i < ITEMS; i += NUM_XF_WARPS * 32) {
                    const int row = i / SEGS, seg = i % SEGS;
                    const uint4 pk = *reinterpret_cast<const uint4*>(sp + row * PROW + seg * 16);
                    const uint32_t px[4] = {pk.x, pk.y, pk.z, pk.w};
                    uint8_t* dst_row = sb + (seg >> 1) * 16384 + row * 128;
                    // lanes of one quarter-warp that write different 128-column blocks (DX) would meet in the same
                    // banks; the second block takes its four words in the order 2,3,0,1 instead
                    const bool rot = (seg >> 1) != 0;
#pragma unroll
                    for (int w0 = 0; w0 < 4; ++w0) {
                        const uint32_t src = rot ? px[w0 ^ 2] : px[w0];
                        const int w = rot ? (w0 ^ 2) : w0;
                        uint32_t o[4];
                        decode16(src, o);
                        const int chunk = (seg & 1) * 4 + w;
                        *reinterpret_cast<uint4*>(dst_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ready(s));
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
    }

    // ---- teardown ------------------------------------------------------------------------------------------------
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
        // a wait gave up somewhere: give copies and MMAs still in flight time to land before the CTA's
        // shared and tensor memory are released
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

// ---- host side -------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    // resolved once; a function-local static is initialised under the language's own lock
    static const EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(ptr);
        return nullptr;
    }();
    return fn;
}

// 2-D byte tensor [rows, cols] with row pitch `pitch`; box [box_rows, box_cols]; out-of-range reads give zero.
int make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols,
                    uint32_t box_rows, bool swizzle128) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return EL_ERR_DRIVER;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch & 15) != 0) return EL_ERR_ALIGNMENT;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? EL_OK : EL_ERR_DRIVER;
}

// Output tensor [rows, cols] of 2- or 4-byte elements for the epilogue's TMA stores: boxes of `box_cols` columns x 32
// rows whose rows are 64 or 128 bytes (swizzled by that width); the store clips at the edges.
int make_map_out(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes, int esz, int box_cols) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return EL_ERR_DRIVER;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0) return EL_ERR_ALIGNMENT;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    if (box_cols * esz != 64 && box_cols * esz != 128) return EL_ERR_INVALID_ARG;
    cuuint32_t box[2] = {(cuuint32_t)box_cols, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_cols * esz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? EL_OK : EL_ERR_DRIVER;
}

template <int MODE, int BN, int EPI>
static int launch_t(const CUtensorMap& tmA, const CUtensorMap& tmB, Params& p, cudaStream_t st) {
    constexpr int smem = Cfg<BN>::SMEM_BYTES(MODE);
    static DeviceOnce attr_once;
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_once.is_done(dev)) {
        EL_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<MODE, BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_once.mark(dev);
    }
    int sms = 0;
    int rc = device_sm_count(&sms);
    if (rc != EL_OK) return rc;
    p.tiles_r = (p.R + BM - 1) / BM;
    p.tiles_c = (p.C + BN - 1) / BN;
    p.k_blocks = (p.D + BK - 1) / BK;
    const long long tiles = (long long)p.tiles_r * p.tiles_c;
    if (tiles == 0) return EL_OK;
    if (p.k_blocks == 0) return EL_ERR_UNSUPPORTED_SHAPE;
    const int grid = (int)(tiles < sms ? tiles : sms);
    gemm_tc_kernel<MODE, BN, EPI><<<grid, num_threads(MODE, EPI), smem, st>>>(tmA, tmB, p);
    return check_launch();
}

}  // namespace tc

// Whether the tensor-core kernel can take this problem (TMA needs 16-byte aligned bases and pitches).
int gemm_tc_eligible(int mode, const void* A, const void* B, int R, int C, int D) {
    if (R <= 0 || C <= 0 || D <= 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return EL_ERR_ALIGNMENT;
    switch (mode) {
        case MODE_FWD: return (D % 64 == 0) ? EL_OK : EL_ERR_UNSUPPORTED_SHAPE;                    // Xq pitch D, W pitch D/4
        case MODE_DX: return (D % 16 == 0 && C % 64 == 0) ? EL_OK : EL_ERR_UNSUPPORTED_SHAPE;     // dYq pitch D(=N), W pitch C/4
        case MODE_DW: return (R % 16 == 0 && C % 16 == 0) ? EL_OK : EL_ERR_UNSUPPORTED_SHAPE;     // Gq pitch R(=N), Xq pitch C
        default: return EL_ERR_INVALID_ARG;
    }
}

int launch_gemm_tc(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, int32_t* status,
                   cudaStream_t st) {
    int rc = gemm_tc_eligible(mode, A, B, R, C, D);
    if (rc != EL_OK) return rc;
    rc = require_sm100();
    if (rc != EL_OK) return rc;
    tc::Params p{};
    p.R = R; p.C = C; p.D = D;
    p.epi = epi;
    p.status = status;
    const int esz = (epi.out_dtype == EL_BF16 || epi.out_dtype == EL_F16) ? 2 : 4;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(epi.out) & 15) == 0) && ((epi.ldo * esz) % 16 == 0);
    CUtensorMap tmA, tmB;
    constexpr int BN = 256;
    if (mode == MODE_FWD) {
        if ((rc = tc::make_map(&tmA, A, D, R, D, 128, 128, true)) != EL_OK) return rc;
        if ((rc = tc::make_map(&tmB, B, D / 4, C, D / 4, 32, BN, false)) != EL_OK) return rc;
        return tc::launch_t<MODE_FWD, BN, EPI_SCALE>(tmA, tmB, p, st);
    } else if (mode == MODE_DX) {
        if ((rc = tc::make_map(&tmA, A, D, R, D, 128, 128, true)) != EL_OK) return rc;
        if ((rc = tc::make_map(&tmB, B, C / 4, D, C / 4, BN / 4, 128, false)) != EL_OK) return rc;
        return tc::launch_t<MODE_DX, BN, EPI_SCALE>(tmA, tmB, p, st);
    } else {
        if ((rc = tc::make_map(&tmA, A, R, D, R, 128, 128, true)) != EL_OK) return rc;
        if ((rc = tc::make_map(&tmB, B, C, D, C, 128, 128, true)) != EL_OK) return rc;
        return tc::launch_t<MODE_DW, BN, EPI_SCALE>(tmA, tmB, p, st);
    }
}

int launch_dw_hysteresis_tc(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* Wp, uint8_t* Hp,
                            const HystParams& hp, uint32_t idx_base, int M, int N, int K, int32_t* status, cudaStream_t st) {
    int rc = gemm_tc_eligible(MODE_DW, Gq, Xq, N, K, M);
    if (rc != EL_OK) return rc;
    if (K % 32 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(Wp) & 7) || (reinterpret_cast<uintptr_t>(Hp) & 15)) return EL_ERR_ALIGNMENT;
    rc = require_sm100();
    if (rc != EL_OK) return rc;
    tc::Params p{};
    p.R = N; p.C = K; p.D = M;
    p.epi = EpiParams{nullptr, 0, EL_F32, g_absmax, 0, 1.0f};
    p.status = status;
    p.Wp = Wp; p.Hp = Hp; p.pK = K / 4; p.pH = K / 2;
    p.hp = hp; p.idx_base = idx_base;
    CUtensorMap tmA, tmB;
    if ((rc = tc::make_map(&tmA, Gq, N, M, N, 128, 128, true)) != EL_OK) return rc;
    if ((rc = tc::make_map(&tmB, Xq, K, M, K, 128, 128, true)) != EL_OK) return rc;
    return tc::launch_t<MODE_DW, 256, EPI_HYST>(tmA, tmB, p, st);
}

}  // namespace el
