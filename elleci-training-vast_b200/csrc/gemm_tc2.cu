// Forward and dX GEMMs on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Expanding the 2-bit weights to int8 costs ALU-pipe time per expanded byte, and the single-CTA kernel
// (gemm_tc.cu) pays it for a 256-row weight tile per 128 x 256 output tile.  Here two CTAs of a cluster share one
// 256 x 256 output tile: each loads its own 128 activation rows, expands only HALF of the weight tile (128 rows of
// 128 bytes per reduction block) and one thread of the leader CTA issues 256-row MMAs that read both halves, so the
// expansion work per MMA cycle is halved.  Per CTA and 128-deep reduction block:
//   A   16 KB  activations, TMA, 128-byte swizzle, K-major           (bytes counted on the leader's "full" barrier)
//   P    4 KB  packed weights, plain 16-byte global loads into the transform warp's registers, one block ahead
//   B   16 KB  expanded weights                                         (one arrival per CTA on the leader's "full")
// Two rings: A and B, 6 deep each.  Each reduction block is expanded by ONE transform warp per CTA into that warp's own
// B slot (six blocks are in flight on six warps), so a block's barrier, fence and signalling latency overlaps with
// the other blocks' work.
// The packed tile does not come through TMA and shared memory: a transform warp reads its block's 4 KB straight into
// registers.  That removes a third ring with its two barrier types and its producer warp and frees 24 KB for a sixth
// activation stage; on its own it changed the speed by nothing, but it lets a stage have one "full" and one "empty"
// barrier (see the kernel), which did (+8 % forward).
// FWD reads B K-major (rows = output features n); DX reads the same image MN-major (rows = reduction index n,
// 128 output columns k per CTA).  DX expands without the final byte interleave (decode16_deint), which permutes the
// output columns inside groups of 16; the epilogue undoes that while the sums are in registers.
// The leader commits each stage to the "empty" barriers of both CTAs and each tile to both "tmem_full" barriers; no
// cluster-multicast load or commit is used.  Every mbarrier wait is bounded (tc_ptx.cuh).
#include "common.cuh"
#include "epilogue.cuh"
#include "tc_ptx.cuh"

namespace el {

enum { MODE_FWD = 0, MODE_DX = 1 };

namespace tc2 {

using namespace tc;

constexpr int BM = 128;            // rows per CTA (the pair covers 256)
constexpr int BN = 256;            // output columns per pair tile (128 expanded per CTA)
constexpr int BK = 128;
constexpr int DA = 6;              // depth of the activation ring
constexpr int DB = 6;              // depth of the expanded-weight ring: one slot per transform warp
constexpr int A_BYTES = BM * BK, B_BYTES = 128 * BK;
constexpr int E_BYTES = 4 * 4096;   // epilogue staging for TMA stores: 4 KB per epilogue warp
constexpr int SMEM_BYTES = DA * A_BYTES + DB * B_BYTES + E_BYTES + 1024 + 512;
constexpr int WARP_TMA = 0, WARP_MMA = 1, NUM_EPI_WARPS = 4, WARP_XF0 = 6, NUM_XF_WARPS = 6;   // warps 2-5: epilogue
constexpr int NUM_THREADS = (WARP_XF0 + NUM_XF_WARPS) * 32;     // 384
constexpr uint32_t TMEM_COLS = 2 * BN;

constexpr int MAX_DST = 8;         // output destinations of one launch (the ranks of an N-sharded layer)
struct OutMaps {
    CUtensorMap m[MAX_DST];
};

struct Params {
    int R, C, D;
    int tiles_r, tiles_c, k_blocks;     // tiles_r counts 256-row pair tiles
    int k_split, kbp;                   // reduction split: k_split work items of kbp blocks per output tile (1, k_blocks = none)
    int group_rows;                     // row tiles per band of the tile order (see tile_coords)
    EpiParams epi;
    int vec_ok;
    int tma_store;                      // the output takes TMA stores (16-byte aligned base and pitch)
    int n_dst;                          // destinations that receive every output block (1 unless gathered over ranks)
    int rows_per_dst;                   // > 0: scatter instead - rows [d*rows_per_dst, (d+1)*rows_per_dst) go to destination d only
    int row_rotate;                     // scatter: row tiles are taken starting from this one (see tile_coords)
    const uint8_t* Wp;                  // packed weights, row pitch ldw bytes: rows are output features (FWD) or the
    long long ldw;                      // reduction index (DX); a row holds 4 weights per byte along the other index
    int32_t* status;
};

// Tile order: bands of `group_rows` row tiles; inside a band the column tiles follow one another and the band's row tiles
// run fastest.  The pairs of one wave then share a few weight tiles while the band's activation rows (sized by the host
// to stay in L2) are read from HBM once instead of once per column tile.  group_rows = tiles_r is the plain row-fastest
// order.
__device__ __forceinline__ void tile_coords(int t, const Params& p, int& tr, int& tc) {
    const int per_band = p.group_rows * p.tiles_c;
    const int band = t / per_band, in = t - band * per_band;
    const int first = band * p.group_rows;
    const int rows_here = min(p.group_rows, p.tiles_r - first);
    tc = in / rows_here;
    tr = first + (in - tc * rows_here);
    // Scatter over ranks: every rank walks the row tiles in the same cyclic order but starts at its own rows, so that at any
    // time the ranks store into different owners (one sender per receiving link) instead of all into the same one.
    tr += p.row_rotate;
    if (tr >= p.tiles_r) tr -= p.tiles_r;
}

// Work item w -> output tile and the first reduction block of its part.  With a split reduction the parts of one tile
// are num_tiles items apart, so they run on different pairs at the same time; part q writes its int32 partial sums
// to output q, and a second pass adds the parts and scales.
__device__ __forceinline__ void item_coords(int w, int num_tiles, const Params& p, int& tr, int& tc, int& part, int& kb0) {
    part = w / num_tiles;
    tile_coords(w - part * num_tiles, p, tr, tc);
    kb0 = part * p.kbp;
}

// LEAN = false: the transform warps hold two register images of a packed block (the loads run a whole block ahead),
// 160 registers per thread: the CTA fills the SM's register file.  LEAN = true: one image, the next block's loads issued
// right after the current one has been expanded, at most 128 registers: a quarter of the register file stays free and a
// kernel that needs no shared memory (the peer pushes of a multi-GPU step, on a side stream) can run beside this
// persistent one.  The lean form is about 9 % slower on its own (2140 against 2350 TOP/s at 4096 -> 11008).
template <int MODE, bool LEAN>
__global__ void __maxnreg__(LEAN ? 128 : 168)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ OutMaps outs, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t ring_b = smem_base + DA * A_BYTES;
    const uint32_t ring_e = ring_b + DB * B_BYTES;
    const uint32_t bars = ring_e + E_BYTES;
    uint8_t* bars_gen = smem_gen + DA * A_BYTES + DB * B_BYTES + E_BYTES;
    // Stage s of the two rings is one unit: its A tile and its expanded B tile are filled, consumed and released together.
    //   full   (leader's copy is used) one phase = both CTAs' A tiles landed (transaction bytes) + both halves expanded
    //          (one arrival per CTA's transform warp) + the leader producer's expect-arrival
    //   empty  (local) the MMAs that read stage s have completed
    // With every data movement and every MMA removed, the handshakes of this kernel alone took more than half of its time
    // when the MMA-issuing thread waited on two barriers and made four commits per block; it now waits on ONE barrier and
    // makes TWO commits per block (one per CTA).  Passing the peer's release through the leader's producer instead of a
    // second commit was tried and lost a third of the throughput: the handshake chain is latency-bound, and the relay
    // added a hop to it.
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_empty = [&](int s) { return bars + 8u * (DA + s); };
    static_assert(DA == DB, "the A and B rings advance in lockstep");
    auto bar_tfull = [&](int a) { return bars + 8u * (2 * DA + a); };        // local: accumulator complete
    auto bar_tempty = [&](int a) { return bars + 8u * (2 * DA + 2 + a); };   // leader: both epilogues done
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars_gen + 8 * (2 * DA + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_r * p.tiles_c;
    const int num_items = num_tiles * p.k_split;

    if (threadIdx.x == 0) {
        for (int s = 0; s < DA; ++s) {
            mbar_init(bar_full(s), 3);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull(a), 1);
            mbar_init(bar_tempty(a), 2 * NUM_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == WARP_MMA) {     // both CTAs of the pair take part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_holder)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers are initialised before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    bool failed = false;

    if (warp == WARP_TMA) {
        // ================= activation producer: this CTA's 128 rows of every reduction block =================
        // The whole warp waits (a warp whose lanes all wait on the barrier is woken sooner than a single waiting lane);
        // lane 0 issues the copy.
        {
            int s = 0;
            uint32_t ph = 0;
            for (int w = pair; w < num_items && !failed; w += num_pairs) {
                int trow, tcol, part, kb0;
                item_coords(w, num_tiles, p, trow, tcol, part, kb0);
                const int r0 = trow * (2 * BM) + (int)rank * BM;
                for (int kb = kb0; kb < kb0 + p.kbp; ++kb) {
                    if (!mbar_wait_cluster_warp(bar_empty(s), ph ^ 1u, p.status, 21)) { failed = true; break; }
                    if (lane == 0) {
                        if (rank == 0) mbar_expect_tx(bar_full(s), 2 * A_BYTES);
                        tma_load_2d_pair(smem_base + s * A_BYTES, &tmA, mapa_u32(bar_full(s), 0), kb * BK, r0);
                    }
                    __syncwarp();
                    if (++s == DA) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ================= MMA issuer (leader CTA only): the whole warp waits, lane 0 issues =================
        if (rank == 0) {
            constexpr uint32_t idesc = make_idesc(0, MODE == MODE_DX, BN, 2 * BM);
            int s = 0, it = 0;
            uint32_t ph = 0;
            for (int w = pair; w < num_items && !failed; w += num_pairs, ++it) {
                const int acc = it & 1;
                const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait_cluster_warp(bar_tempty(acc), acc_ph ^ 1u, p.status, 22)) { failed = true; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < p.kbp; ++kb) {          // the item's own blocks: the first one starts the sums
                    if (!mbar_wait_cluster_warp(bar_full(s), ph, p.status, 23)) { failed = true; break; }
                    tcgen05_fence_after();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_base + s * A_BYTES, b_addr = ring_b + s * B_BYTES;
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k) {
                            const uint64_t da = make_desc(a_addr + k * 32, 16);
                            const uint64_t db = (MODE == MODE_FWD) ? make_desc(b_addr + k * 32, 16) : make_desc(b_addr + k * 4096, 16384);
                            umma_i8_pair(d_tmem, da, db, idesc, (kb | k) != 0);
                        }
                        umma_commit_pair(mapa_u32(bar_empty(s), 0));
                        umma_commit_pair(mapa_u32(bar_empty(s), 1));
                    }
                    __syncwarp();
                    if (++s == DA) { s = 0; ph ^= 1u; }
                }
                if (!failed && lane == 0) {
                    umma_commit_pair(mapa_u32(bar_tfull(acc), 0));
                    umma_commit_pair(mapa_u32(bar_tfull(acc), 1));
                }
                __syncwarp();
            }
        }
    } else if (warp < WARP_XF0) {
        // ================= epilogue (each CTA stores its own 128 rows x 256 columns) =================
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        int it = 0;
        for (int w = pair; w < num_items && !failed; w += num_pairs, ++it) {
            int trow, tcol, part, kb0;
            item_coords(w, num_tiles, p, trow, tcol, part, kb0);
            const int r0 = trow * (2 * BM) + (int)rank * BM, c0 = tcol * BN;
            const int acc = it & 1;
            const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
            if (!mbar_wait_warp(bar_tfull(acc), acc_ph, p.status, 25)) { failed = true; break; }
            tcgen05_fence_after();
            const int row = r0 + row_in_tile;
            const bool row_ok = row < p.R;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            const float sc = row_ok ? epi_row_scale(p.epi, row) : 0.0f;
            const bool two_byte = (p.epi.out_dtype == EL_BF16 || p.epi.out_dtype == EL_F16);
            const uint32_t stage = ring_e + quarter * 4096;        // this warp's staging area
            uint8_t* stage_gen = smem_gen + DA * A_BYTES + DB * B_BYTES + quarter * 4096;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(taddr + c * 32, v);
                tmem_ld_wait();
                const int col0 = c0 + c * 32;
                // DX: column 16g+p of the tile holds output column 16g + KPERM16[p] (de-interleaved expansion), so output column
                // i of the chunk is read from register SRC(i); with the loops below unrolled this is a renaming, not a copy.
#define EL_SRC(i) ((MODE == MODE_DX) ? (((i) & ~15) + ((((i) & 15) & 1) ? 8 + (((i) & 15) >> 1) : (((i) & 15) >> 1))) : (i))
                if (p.tma_store) {
                    if (col0 >= p.C) continue;
                    // The warp's 32 rows go to shared memory in the tensor map's 128-byte swizzle (32 columns of four-byte
                    // or 64 columns of two-byte elements), then out with one TMA store, clipped at the matrix edges.
                    // Before the buffer is rewritten the store that last read it must have finished reading.
                    if (two_byte) {
                        // two 32-column chunks share one 4 KB buffer (32 rows x 128 bytes) and leave as one store
                        const int h = c & 1;
                        if (h == 0) {
                            if (lane == 0) bulk_wait_read<0>();
                            __syncwarp();
                        }
                        uint8_t* buf = stage_gen + lane * 128;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float lo = __fmul_rn((float)(int)v[EL_SRC(8 * j + 2 * i)], sc),
                                            hi = __fmul_rn((float)(int)v[EL_SRC(8 * j + 2 * i + 1)], sc);
                                o[i] = (p.epi.out_dtype == EL_BF16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
                            }
                            *reinterpret_cast<uint4*>(buf + (((4 * h + j) ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                        if (h == 0 && col0 + 32 < p.C) continue;      // the second half of the box follows
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int rb = r0 + quarter * 32, cb = col0 - 32 * h;
                            if (p.rows_per_dst > 0) {              // scatter: this 32-row block belongs to one owner
                                const int d = rb / p.rows_per_dst;
                                if (d < p.n_dst) tma_store_2d(&outs.m[d], stage, cb, rb - d * p.rows_per_dst);
                            } else {
                                for (int d = 0; d < p.n_dst; ++d)  // own buffer and, when gathering, every peer's
                                    tma_store_2d(&outs.m[d], stage, cb, rb);
                            }
                            bulk_commit();
                        }
                    } else {
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                        uint8_t* buf = stage_gen + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int a = (int)v[EL_SRC(4 * j + i)];
                                o[i] = (p.epi.out_dtype == EL_F32) ? __float_as_uint(__fmul_rn((float)a, sc)) : (uint32_t)a;
                            }
                            *reinterpret_cast<uint4*>(buf + ((j ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int rb = r0 + quarter * 32;
                            if (p.k_split > 1) {                   // split reduction: part q's sums go to partial output q
                                tma_store_2d(&outs.m[part], stage, col0, rb);
                            } else if (p.rows_per_dst > 0) {
                                const int d = rb / p.rows_per_dst;
                                if (d < p.n_dst) tma_store_2d(&outs.m[d], stage, col0, rb - d * p.rows_per_dst);
                            } else {
                                for (int d = 0; d < p.n_dst; ++d) tma_store_2d(&outs.m[d], stage, col0, rb);
                            }
                            bulk_commit();
                        }
                    }
                } else if (row_ok && col0 < p.C) {        // unaligned output: plain stores (rare)
                    uint32_t w[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = v[EL_SRC(i)];
                    epi_store_chunk32(p.epi, row, col0, p.C, w, sc, false);
                }
#undef EL_SRC
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(bar_tempty(acc), 0));
        }
        if (lane == 0) bulk_wait_all();      // this warp's TMA stores have left shared memory and reached global memory
    } else {
        // ================= transform: 128 packed rows of 32 bytes -> 128 rows of 128 int8, swizzled =================
        // Warp w expands the reduction blocks g = w, w+6, ... of this CTA's sequence (tile after tile, block after block)
        // on its own; lane l takes the 16-byte segments l, l+32, ... (row = segment/2) of the packed tile, straight from
        // global memory.  The loads of the warp's next block are issued before the current one is expanded, so their
        // latency runs under five other blocks' worth of work.
        const int xw = warp - WARP_XF0;
        static_assert(DB == NUM_XF_WARPS, "one B slot per transform warp");
        const int my_items = (num_items > pair) ? (num_items - pair + num_pairs - 1) / num_pairs : 0;
        const long long total = (long long)my_items * p.kbp;
        const uint4 zero_codes = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);     // sixteen weights 0 per word
        auto load_block = [&](long long g, uint4 (&pk)[8]) {
            const int i = (int)(g / p.kbp);
            int trow, tcol, part, kb0;
            item_coords(pair + i * num_pairs, num_tiles, p, trow, tcol, part, kb0);
            const int kb = kb0 + (int)(g - (long long)i * p.kbp);
            const int c0 = tcol * BN + (int)rank * 128;             // this CTA's 128 output columns
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int item = lane + 32 * j, row = item >> 1, seg = item & 1;
                const uint8_t* src;
                bool ok;
                if (MODE == MODE_FWD) {         // rows = output features c0 + row, bytes = reduction indices kb*128 + seg*64 ..
                    ok = (c0 + row < p.C) && (kb * BK + seg * 64 < p.D);
                    src = p.Wp + (long long)(c0 + row) * p.ldw + kb * (BK / 4) + seg * 16;
                } else {                        // rows = reduction indices kb*128 + row, bytes = output columns c0 + seg*64 ..
                    ok = (kb * BK + row < p.D) && (c0 + seg * 64 < p.C);
                    src = p.Wp + (long long)(kb * BK + row) * p.ldw + (c0 >> 2) + seg * 16;
                }
                pk[j] = ok ? __ldg(reinterpret_cast<const uint4*>(src)) : zero_codes;
            }
        };
        uint4 cur[8], nxt[8];
        if (xw < total) load_block(xw, cur);
        for (long long g = xw; g < total && !failed; g += NUM_XF_WARPS) {
            // Block g uses this warp's own B slot (g % 6 == xw).  A barrier only tells the parity of its phase, so a
            // waiter must never be two phases away from it: with one slot per warp the previous use of the slot was this
            // warp's previous block (g-6).
            const bool more = g + NUM_XF_WARPS < total;
            if (!LEAN && more) load_block(g + NUM_XF_WARPS, nxt);        // a whole block ahead, into the second image
            const int sb_i = xw;
            const uint32_t phb = (uint32_t)(g / DB) & 1u;
            if (!mbar_wait_warp(bar_empty(sb_i), phb ^ 1u, p.status, 28)) { failed = true; break; }
            uint8_t* sb = smem_gen + DA * A_BYTES + sb_i * B_BYTES;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int item = lane + 32 * j, row = item >> 1, seg = item & 1;
                const uint32_t px[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
                uint8_t* dst_row = sb + row * 128;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t o[4];
                    if (MODE == MODE_DX) decode16_deint(px[w], o);
                    else decode16(px[w], o);
                    const int chunk = seg * 4 + w;
                    *reinterpret_cast<uint4*>(dst_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
            if (LEAN) {
                asm volatile("" ::: "memory");  // keeps the compiler from starting the next loads while `cur` is still needed
                if (more) load_block(g + NUM_XF_WARPS, cur);        // into the one image, as soon as it is free
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(bar_full(sb_i), 0));
            if (!LEAN && more) {
#pragma unroll
                for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
            }
        }
    }

    // ---- teardown: both CTAs are done with each other's shared and tensor memory before either frees anything ------
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == WARP_MMA) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int MODE, bool LEAN>
static int launch_t(const CUtensorMap& tmA, const OutMaps& outs, Params& p, cudaStream_t st) {
    static std::atomic<int> max_pairs[64];      // co-resident CTA pairs per device; 0 = not yet queried
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return EL_ERR_DEVICE;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int dev_pairs = max_pairs[dev].load(std::memory_order_acquire);
    if (dev_pairs == 0) {       // host threads may race here: both then query and store the same number
        EL_CUDA_TRY(cudaFuncSetAttribute(gemm_tc2_kernel<MODE, LEAN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        int sms = 0;
        const int rc = device_sm_count(&sms);
        if (rc != EL_OK) return rc;
        cfg.gridDim = dim3((unsigned)(sms & ~1), 1, 1);
        int clusters = 0;
        EL_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, gemm_tc2_kernel<MODE, LEAN>, &cfg));
        if (clusters < 1) return EL_ERR_DEVICE;
        dev_pairs = clusters < sms / 2 ? clusters : sms / 2;
        max_pairs[dev].store(dev_pairs, std::memory_order_release);
    }
    p.tiles_r = (p.R + 2 * BM - 1) / (2 * BM);
    p.tiles_c = (p.C + BN - 1) / BN;
    p.k_blocks = (p.D + BK - 1) / BK;
    // a band's activation rows (256 rows x D bytes per row tile) should fit in a third of the 126 MB L2
    const long long row_tile_bytes = 2LL * BM * (long long)p.k_blocks * BK;
    long long group = (40LL << 20) / (row_tile_bytes > 0 ? row_tile_bytes : 1);
    p.group_rows = (int)(group < 1 ? 1 : (group > p.tiles_r ? p.tiles_r : group));
    if (p.group_rows < 1) p.group_rows = 1;
    const long long tiles = (long long)p.tiles_r * p.tiles_c;
    if (tiles == 0) return EL_OK;
    if (p.k_blocks == 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (p.k_split < 1 || p.k_blocks % p.k_split != 0) p.k_split = 1;
    p.kbp = p.k_blocks / p.k_split;
    const long long items = tiles * p.k_split;
    const int pairs = (int)(items < dev_pairs ? items : dev_pairs);
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    EL_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE, LEAN>, tmA, outs, p));
    return check_launch();
}

}  // namespace tc2

namespace tc {
int make_map(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols,
             uint32_t box_rows, bool swizzle128);
int make_map_out(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes, int esz, int box_cols);
}
int gemm_tc_eligible(int mode, const void* A, const void* B, int R, int C, int D);
int launch_reduce_scale_gather(const int* parts, int n_parts, void* const* out_all, int n_ranks, long long row_offset,
                               long long rows_total, const EpiParams& epi, int Mr, int C, cudaStream_t st);

// A problem with few output tiles leaves most CTA pairs idle (4096 -> 512 at 4096 tokens is 32 tiles for 74 pairs).  Its
// reduction is then cut into q parts that run on different pairs at the same time; each part stores its int32 partial
// sums and a second pass adds them (exact) and applies the epilogue.  Returns q (1 = no split): the largest q <= 8 that
// keeps all parts in one wave, divides the number of reduction blocks and leaves at least 16 blocks per part, for
// reductions of at least 48 blocks.  (Shorter reductions gain nothing: at 4096 -> 512 and 32 blocks the second pass and
// its int32 round trip cost what the shorter main loop saves, measured.)
int gemm_tc2_k_split(int R, int C, int D) {
    int sms = 0;
    if (device_sm_count(&sms) != EL_OK || sms < 2) return 1;
    const long long pairs = sms / 2;
    const long long tiles = (long long)((R + 2 * tc2::BM - 1) / (2 * tc2::BM)) * ((C + tc2::BN - 1) / tc2::BN);
    const int k_blocks = (D + tc2::BK - 1) / tc2::BK;
    int best = 1;
    for (int q = 2; q <= 8; ++q)
        if (tiles * q <= pairs && k_blocks >= 48 && k_blocks % q == 0 && k_blocks / q >= 16) best = q;
    return best;
}

// Forward (mode 0) and dX (mode 1) on CTA pairs; same eligibility as the single-CTA kernel.
// `dst` (optional): n_dst base pointers of [R, ld_total] output matrices that all receive this launch's [R, C] result
// at column `col_offset` (the own buffer and the peers' buffers of an N-sharded layer: the all-gather of the output
// happens as TMA stores from the epilogue).  With dst == nullptr the result goes to epi.out alone.
// `rows_per_dst` > 0 selects the scatter form instead: dst[d] is a dense [rows_per_dst, C] matrix that receives the
// rows [d*rows_per_dst, (d+1)*rows_per_dst) of the result (the reduce-scatter half of a cross-rank reduction of dX).
int launch_gemm_tc2(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, int32_t* status,
                    cudaStream_t st, void* const* dst, int n_dst, long long ld_total, long long col_offset,
                    int rows_per_dst, int first_dst, void* workspace, size_t workspace_bytes, bool lean) {
    if (mode != MODE_FWD && mode != MODE_DX) return EL_ERR_INVALID_ARG;
    int rc = gemm_tc_eligible(mode, A, B, R, C, D);
    if (rc != EL_OK) return rc;
    rc = require_sm100();
    if (rc != EL_OK) return rc;
    tc2::Params p{};
    p.R = R; p.C = C; p.D = D;
    p.epi = epi;
    p.status = status;
    p.k_split = 1;
    const int esz = (epi.out_dtype == EL_BF16 || epi.out_dtype == EL_F16) ? 2 : 4;
    tc2::OutMaps outs{};
    CUtensorMap tmA;
    if (dst != nullptr && rows_per_dst > 0) {
        if (n_dst < 1 || n_dst > tc2::MAX_DST || rows_per_dst % 32 != 0 || (long long)rows_per_dst * n_dst < R) return EL_ERR_INVALID_ARG;
        for (int d = 0; d < n_dst; ++d) {
            if (dst[d] == nullptr) return EL_ERR_NULL_PTR;
            if ((rc = tc::make_map_out(&outs.m[d], dst[d], C, rows_per_dst, (uint64_t)C * esz, esz, 128 / esz)) != EL_OK) return rc;
        }
        p.n_dst = n_dst;
        p.rows_per_dst = rows_per_dst;
        if (first_dst < 0 || first_dst >= n_dst) return EL_ERR_INVALID_ARG;
        const int row_tiles = (R + 2 * tc2::BM - 1) / (2 * tc2::BM);
        p.row_rotate = (int)(((long long)first_dst * rows_per_dst / (2 * tc2::BM)) % row_tiles);
        p.tma_store = 1;
        p.vec_ok = 1;
    } else if (dst != nullptr) {
        if (n_dst < 1 || n_dst > tc2::MAX_DST || ld_total < col_offset + C || col_offset < 0) return EL_ERR_INVALID_ARG;
        if (C % 32 != 0) return EL_ERR_UNSUPPORTED_SHAPE;      // 32-column store boxes must not reach into a neighbour's window
        for (int d = 0; d < n_dst; ++d) {
            if (dst[d] == nullptr) return EL_ERR_NULL_PTR;
            const char* base = static_cast<const char*>(dst[d]) + col_offset * esz;
            if ((rc = tc::make_map_out(&outs.m[d], base, C, R, (uint64_t)ld_total * esz, esz, 128 / esz)) != EL_OK) return rc;
        }
        p.n_dst = n_dst;
        p.tma_store = 1;
        p.vec_ok = 1;
    } else {
        p.vec_ok = ((reinterpret_cast<uintptr_t>(epi.out) & 15) == 0) && ((epi.ldo * esz) % 16 == 0);
        p.tma_store = p.vec_ok;
        p.n_dst = 1;
        // split reduction: needs the caller's workspace, a dense scaled output and 8-column vectors in the second pass
        const int q = (workspace != nullptr && epi.out_dtype != EL_I32 && p.vec_ok && epi.ldo == C && C % 8 == 0 &&
                       (reinterpret_cast<uintptr_t>(workspace) & 15) == 0) ? gemm_tc2_k_split(R, C, D) : 1;
        if (q > 1 && (size_t)q * R * C * sizeof(int) <= workspace_bytes) {
            p.k_split = q;
            p.epi.out_dtype = EL_I32;                   // the parts are raw int32 sums; the second pass scales
            p.epi.absmax = nullptr;
            for (int part = 0; part < q; ++part) {
                char* base = static_cast<char*>(workspace) + (size_t)part * R * C * sizeof(int);
                if ((rc = tc::make_map_out(&outs.m[part], base, C, R, (uint64_t)C * 4, 4, 32)) != EL_OK) return rc;
            }
        } else if (p.tma_store && (rc = tc::make_map_out(&outs.m[0], epi.out, C, R, (uint64_t)epi.ldo * esz, esz, 128 / esz)) != EL_OK) {
            return rc;
        }
    }
    if ((rc = tc::make_map(&tmA, A, D, R, D, 128, 128, true)) != EL_OK) return rc;
    p.Wp = static_cast<const uint8_t*>(B);
    if (mode == MODE_FWD) {
        p.ldw = D / 4;              // [C output features, D/4 bytes]
        rc = lean ? tc2::launch_t<MODE_FWD, true>(tmA, outs, p, st) : tc2::launch_t<MODE_FWD, false>(tmA, outs, p, st);
    } else {
        p.ldw = C / 4;              // [D reduction rows, C/4 bytes]
        rc = lean ? tc2::launch_t<MODE_DX, true>(tmA, outs, p, st) : tc2::launch_t<MODE_DX, false>(tmA, outs, p, st);
    }
    if (rc != EL_OK || p.k_split == 1) return rc;
    void* out_one[1] = {epi.out};
    return launch_reduce_scale_gather(static_cast<const int*>(workspace), p.k_split, out_one, 1, 0, R, epi, R, C, st);
}

}  // namespace el
