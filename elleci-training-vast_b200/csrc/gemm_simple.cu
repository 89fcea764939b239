// CUDA-core integer GEMMs for shapes the tensor-core kernel cannot take (pitches that break the TMA
// alignment rules, tiny layers such as K = 16 or N = 48): C[i,j] = sum_r A(i,r) * B(j,r) with dp4a,
// 64x64 output tile per CTA, operands staged through shared memory with bounds-checked byte loads.
// Correct for every shape; it is not the fast path.
#include "common.cuh"
#include "epilogue.cuh"

namespace el {

enum { MODE_FWD = 0, MODE_DX = 1, MODE_DW = 2 };

struct SimpleParams {
    const int8_t* A;      // FWD: Xq [R,D]   DX: dYq [R,D]   DW: Gq [D,R]
    const void* B;        // FWD: W_packed [C, ceil(D/4)]   DX: W_packed [D, ceil(C/4)]   DW: Xq [D,C]
    int R, C, D;
    EpiParams epi;
};

template <int MODE>
__device__ __forceinline__ int a_elem(const SimpleParams& p, int i, int r) {
    if (i >= p.R || r >= p.D) return 0;
    if (MODE == MODE_DW) return p.A[(size_t)r * p.R + i];
    return p.A[(size_t)i * p.D + r];
}

template <int MODE>
__device__ __forceinline__ int b_elem(const SimpleParams& p, int j, int r) {
    if (j >= p.C || r >= p.D) return 0;
    if (MODE == MODE_FWD) {
        const uint8_t* W = static_cast<const uint8_t*>(p.B);
        const int pK = (p.D + 3) >> 2;
        return decode2(W[(size_t)j * pK + (r >> 2)] >> ((r & 3) * 2));
    } else if (MODE == MODE_DX) {
        const uint8_t* W = static_cast<const uint8_t*>(p.B);
        const int pK = (p.C + 3) >> 2;
        return decode2(W[(size_t)r * pK + (j >> 2)] >> ((j & 3) * 2));
    } else {
        return static_cast<const int8_t*>(p.B)[(size_t)r * p.C + j];
    }
}

template <int MODE>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const SimpleParams p) {
    __shared__ int8_t As[64][68];
    __shared__ int8_t Bs[64][68];
    const int tid = threadIdx.x;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    const int ty = tid >> 4, tx = tid & 15;
    int acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0;

    for (int r0 = 0; r0 < p.D; r0 += 64) {
#pragma unroll 4
        for (int e = tid; e < 64 * 64; e += 256) {
            const int fast = e & 63, slow = e >> 6;
            // A: reduction index contiguous in memory except in DW mode (row index contiguous)
            if (MODE == MODE_DW) As[fast][slow] = (int8_t)a_elem<MODE>(p, i0 + fast, r0 + slow);
            else As[slow][fast] = (int8_t)a_elem<MODE>(p, i0 + slow, r0 + fast);
            // B: reduction index contiguous only in FWD mode
            if (MODE == MODE_FWD) Bs[slow][fast] = (int8_t)b_elem<MODE>(p, j0 + slow, r0 + fast);
            else Bs[fast][slow] = (int8_t)b_elem<MODE>(p, j0 + fast, r0 + slow);
        }
        __syncthreads();
#pragma unroll 4
        for (int w = 0; w < 16; ++w) {
            int a[4], b[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                a[x] = *reinterpret_cast<const int*>(&As[ty * 4 + x][w * 4]);
                b[x] = *reinterpret_cast<const int*>(&Bs[tx * 4 + x][w * 4]);
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = __dp4a(a[x], b[y], acc[x][y]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const int i = i0 + ty * 4 + x;
        if (i >= p.R) continue;
        const float sc = epi_row_scale(p.epi, i);
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int j = j0 + tx * 4 + y;
            if (j < p.C) epi_store_one(p.epi, i, j, acc[x][y], sc);
        }
    }
}

int launch_gemm_simple(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi,
                       cudaStream_t st) {
    if (R == 0 || C == 0) return EL_OK;
    SimpleParams p{A, B, R, C, D, epi};
    dim3 grid((C + 63) / 64, (R + 63) / 64);
    if (grid.y > 65535) return EL_ERR_UNSUPPORTED_SHAPE;
    switch (mode) {
        case MODE_FWD: gemm_simple_kernel<MODE_FWD><<<grid, 256, 0, st>>>(p); break;
        case MODE_DX: gemm_simple_kernel<MODE_DX><<<grid, 256, 0, st>>>(p); break;
        case MODE_DW: gemm_simple_kernel<MODE_DW><<<grid, 256, 0, st>>>(p); break;
        default: return EL_ERR_INVALID_ARG;
    }
    return check_launch();
}

}  // namespace el
