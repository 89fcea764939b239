// C ABI of libelleci_int2.so: argument validation and dispatch.  No entry point allocates, synchronises or
// prints; every one returns an EL_* status.
#include "common.cuh"
#include "epilogue.cuh"

namespace el {

enum { MODE_FWD = 0, MODE_DX = 1, MODE_DW = 2 };

// kernels in the other translation units
int launch_pack(const void* src, bool from_float, float gamma, uint8_t* Wp, int N, int K, int pad_code, cudaStream_t st);
int launch_unpack(const uint8_t* Wp, void* out, int out_dtype, int N, int K, cudaStream_t st);
int launch_quantize_rows(const void* x, int dt, long long ldx, int8_t* q, float* a, int M, int K, float eps, int mode,
                         const float* fold_absmax, float* fold_max, cudaStream_t st);
int launch_scale_rows(const int* acc, const EpiParams& epi, int M, int C, cudaStream_t st);
int launch_quantize_tensor(const void* x, int dt, int8_t* q, float* absmax, long long size, cudaStream_t st);
int launch_dequantize_tensor(const int8_t* q, const float* absmax, void* out, int dt, long long size, cudaStream_t st);
int launch_quantize_grad(const void* dY, int dt, long long ld, const float* xa, const float* ga, int8_t* Gq, int M, int N,
                         cudaStream_t st);
int launch_hysteresis(const float* dW, uint8_t* Wp, uint8_t* Hp, const HystParams& p, int N, int K, uint32_t idx_base,
                      cudaStream_t st);
int launch_gemm_simple(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, cudaStream_t st);
int gemm_tc_eligible(int mode, const void* A, const void* B, int R, int C, int D);
int launch_gemm_tc(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, int32_t* status,
                   cudaStream_t st);
int launch_gemm_tc2(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, int32_t* status,
                    cudaStream_t st, void* const* dst, int n_dst, long long ld_total, long long col_offset, int rows_per_dst,
                    int first_dst, void* workspace, size_t workspace_bytes, bool lean);
int gemm_tc2_k_split(int R, int C, int D);
int launch_reduce_scale_gather(const int* parts, int n_parts, void* const* out_all, int n_ranks, long long row_offset,
                               long long rows_total, const EpiParams& epi, int Mr, int C, cudaStream_t st);
int launch_dw_hysteresis_tc(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* Wp, uint8_t* Hp,
                            const HystParams& hp, uint32_t idx_base, int M, int N, int K, int32_t* status, cudaStream_t st);

int launch_quantize_rows_perm(const void* x, int dt, long long ldx, int8_t* q, float* a, int M, int K, float eps,
                              cudaStream_t st);
size_t decode_workspace_bytes(int N);
int launch_decode_tc(const int8_t* Xq, const uint8_t* Wp, const EpiParams& epi, void* workspace, int M, int N, int K,
                     int32_t* status, cudaStream_t st);

int launch_rmsnorm_quantize_rows(const void* x, int dt, long long ldx, const float* weight, float norm_eps, int8_t* q,
                                 float* row_absmax, float* rstd, int M, int K, float quant_eps, cudaStream_t st);
size_t rmsnorm_backward_workspace_bytes(int K);
int launch_rmsnorm_backward(const void* g, const void* x, int dt, const float* weight, const float* rstd, void* dx,
                            float* dweight, void* workspace, size_t workspace_bytes, int M, int K, cudaStream_t st);
size_t swiglu_backward_workspace_bytes(int H);
int launch_sigmoid_fixed(const float* g, float* sig, long long n, cudaStream_t st);
int launch_prelinear_rows(const void* x, const void* up, int dt, long long ld, const float* weight, float norm_eps, void* y, int M,
                          int K, cudaStream_t st);
int launch_swiglu_quantize_rows(const void* gate, const void* up, int dt, long long ld, const float* weight, float norm_eps,
                                int8_t* q, float* row_absmax, float* rstd, int M, int H, float quant_eps, cudaStream_t st);
int launch_swiglu_backward(const void* gy, const void* gate, const void* up, int dt, long long ld, const float* weight,
                           const float* rstd, void* d_gate, void* d_up, long long ld_d, float* dweight, void* workspace,
                           size_t workspace_bytes, int M, int H, cudaStream_t st);
int launch_peer_barrier(unsigned int* const* flags_all, int n_ranks, int rank, unsigned int epoch, bool next_epoch,
                        int32_t* status, cudaStream_t st, const void* put_src, void* const* put_dst_all, size_t put_offset);
int launch_counter_add(int32_t* counter, int delta, cudaStream_t st);
int set_peer_barrier_limit_us(long long us);
int launch_quantize_grad_scatter(const void* dY, int dt, long long ld, const float* xa, const float* g_slots, int n_slots,
                                 float* g_out, void* const* Gq_all, int n_ranks, long long row_offset, int M, int N,
                                 cudaStream_t st);
int launch_peer_put(const void* src, void* const* dst_all, int n_dst, size_t dst_offset, size_t bytes, int max_ctas,
                    cudaStream_t st);
int launch_gemv_mma(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st,
                    bool overlap);
bool gemv_mma_fits(int M, int K);
int launch_gemv_small(const void* x, int x_dtype, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K, cudaStream_t st, bool overlap);
int decode_gemv_max_tokens();
bool gemv_mma_preq_fits(int M, int K);
int launch_gemv_mma_preq(const int8_t* xq, const float* amax, const uint8_t* Wp, const EpiParams& epi, int M, int N, int K,
                         cudaStream_t st);

static thread_local int g_last_cuda_error = 0;

int record_cuda_error(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return EL_ERR_CUDA;
}

int check_launch() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? EL_OK : record_cuda_error(e);
}

static std::atomic<int> g_dev_info[64];      // (compute capability major << 16) | SM count; 0 = not yet queried

static int device_info(int* sms, int* major) {
    int dev = 0;
    EL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        int a = 0, b = 0;
        EL_CUDA_TRY(cudaDeviceGetAttribute(&a, cudaDevAttrMultiProcessorCount, dev));
        EL_CUDA_TRY(cudaDeviceGetAttribute(&b, cudaDevAttrComputeCapabilityMajor, dev));
        if (sms) *sms = a;
        if (major) *major = b;
        return EL_OK;
    }
    int info = g_dev_info[dev].load(std::memory_order_acquire);
    if (info == 0) {   // threads that race here query and store the same word
        int a = 0, b = 0;
        EL_CUDA_TRY(cudaDeviceGetAttribute(&a, cudaDevAttrMultiProcessorCount, dev));
        EL_CUDA_TRY(cudaDeviceGetAttribute(&b, cudaDevAttrComputeCapabilityMajor, dev));
        info = (b << 16) | (a & 0xFFFF);
        g_dev_info[dev].store(info, std::memory_order_release);
    }
    if (sms) *sms = info & 0xFFFF;
    if (major) *major = info >> 16;
    return EL_OK;
}

int device_sm_count(int* out) { return device_info(out, nullptr); }

// Token count up to which the decode call uses the CUDA-core GEMV (el_set_decode_gemv_max_tokens).
// The tuning knobs are process-wide atomics: a call reads each one once, so a setter that runs on another host thread
// takes effect from some later call on, never halfway through one.
static std::atomic<int> g_gemv_max_tokens{2};
int decode_gemv_max_tokens() { return g_gemv_max_tokens.load(std::memory_order_relaxed); }
static std::atomic<int> g_mma_max_tokens{64};
int decode_mma_max_tokens() { return g_mma_max_tokens.load(std::memory_order_relaxed); }
static std::atomic<int> g_decode_overlap{0};
bool decode_overlap() { return g_decode_overlap.load(std::memory_order_relaxed) != 0; }

int require_sm100() {
    int major = 0;
    const int rc = device_info(nullptr, &major);
    if (rc != EL_OK) return rc;
    return major == 10 ? EL_OK : EL_ERR_DEVICE;
}

static inline bool float_dtype(int dt) { return dt == EL_F16 || dt == EL_BF16 || dt == EL_F32; }
static inline bool out_dtype_ok(int dt) { return dt == EL_F16 || dt == EL_BF16 || dt == EL_F32 || dt == EL_I32; }

// Tensor-core launch: forward and dX run on CTA pairs unless the single-CTA kernel is asked for; dW has one kernel.
static int launch_tc(int mode, bool single_cta, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi,
                     int32_t* status, cudaStream_t st, void* ws = nullptr, size_t ws_bytes = 0, bool lean = false) {
    // The weight-gradient GEMM has one kernel: a CTA-pair version of it (half of the Xq columns per CTA) was built and
    // measured 8-10 % slower than the single-CTA kernel at every size, and dropped.
    if (single_cta || mode == MODE_DW) return launch_gemm_tc(mode, A, B, R, C, D, epi, status, st);
    return launch_gemm_tc2(mode, A, B, R, C, D, epi, status, st, nullptr, 0, 0, 0, 0, 0, ws, ws_bytes, lean);
}

static int gemm_dispatch(int mode, const int8_t* A, const void* B, int R, int C, int D, const EpiParams& epi, int flags,
                         int32_t* status, cudaStream_t st, void* ws = nullptr, size_t ws_bytes = 0) {
    const bool lean = (flags & EL_FLAG_LEAN) != 0;
    flags &= ~EL_FLAG_LEAN;
    if (flags < EL_PATH_AUTO || flags > EL_PATH_TC_SINGLE) return EL_ERR_INVALID_ARG;
    if (R == 0 || C == 0) return EL_OK;
    if (flags == EL_PATH_SIMPLE) return launch_gemm_simple(mode, A, B, R, C, D, epi, st);
    const int elig = (D > 0) ? gemm_tc_eligible(mode, A, B, R, C, D) : EL_ERR_UNSUPPORTED_SHAPE;
    if (flags == EL_PATH_TC || flags == EL_PATH_TC_SINGLE)
        return elig != EL_OK ? elig : launch_tc(mode, flags == EL_PATH_TC_SINGLE, A, B, R, C, D, epi, status, st, ws, ws_bytes, lean);
    // auto: the tensor-core tiles are 128 rows deep; very small problems go to the CUDA-core kernel.  A few rows against a
    // large weight matrix still belong on the tensor-core kernel: the call is then the time to stream the packed weights
    // once, which the CUDA-core kernel takes twenty times longer for.
    if (elig == EL_OK && (R >= 32 || (long long)C * D >= (1ll << 18)))
        return launch_tc(mode, R <= 128, A, B, R, C, D, epi, status, st, ws, ws_bytes, lean);
    return launch_gemm_simple(mode, A, B, R, C, D, epi, st);
}

}  // namespace el

using namespace el;

extern "C" {

int el_version(void) { return 100; }

const char* el_status_string(int s) {
    switch (s) {
        case EL_OK: return "ok";
        case EL_ERR_INVALID_ARG: return "invalid argument";
        case EL_ERR_NULL_PTR: return "null pointer";
        case EL_ERR_ALIGNMENT: return "pointer or pitch alignment";
        case EL_ERR_UNSUPPORTED_SHAPE: return "shape not supported by the requested path";
        case EL_ERR_CUDA: return "CUDA runtime error";
        case EL_ERR_DEVICE: return "device is not sm_100";
        case EL_ERR_DRIVER: return "tensor-map descriptor rejected by the driver";
        case EL_ERR_TOO_LARGE: return "size exceeds the fixed capacity of this entry point (static scratch: M<=64, N<=16384, K<=16384)";
        default: return "unknown status";
    }
}

int el_last_cuda_error(void) { return g_last_cuda_error; }

int el_pack_ternary(const int8_t* w, uint8_t* W_packed, int N, int K, int pad_code, el_stream_t stream) {
    if (N < 0 || K < 0 || pad_code < 0 || pad_code > 3) return EL_ERR_INVALID_ARG;
    if (N == 0 || K == 0) return EL_OK;
    if (!w || !W_packed) return EL_ERR_NULL_PTR;
    return launch_pack(w, false, 1.0f, W_packed, N, K, pad_code, (cudaStream_t)stream);
}

int el_ternarize_pack(const float* W, float gamma, uint8_t* W_packed, int N, int K, el_stream_t stream) {
    if (N < 0 || K < 0 || !(gamma > 0.0f)) return EL_ERR_INVALID_ARG;
    if (N == 0 || K == 0) return EL_OK;
    if (!W || !W_packed) return EL_ERR_NULL_PTR;
    return launch_pack(W, true, gamma, W_packed, N, K, 0, (cudaStream_t)stream);
}

int el_unpack_ternary(const uint8_t* W_packed, void* out, int out_dtype, int N, int K, el_stream_t stream) {
    if (N < 0 || K < 0 || !out_dtype_ok(out_dtype)) return EL_ERR_INVALID_ARG;
    if (N == 0 || K == 0) return EL_OK;
    if (!W_packed || !out) return EL_ERR_NULL_PTR;
    return launch_unpack(W_packed, out, out_dtype, N, K, (cudaStream_t)stream);
}

int el_quantize_rows(const void* x, int x_dtype, long long ldx, int8_t* q, float* row_absmax, int M, int K, float eps,
                     int mode, const float* fold_absmax, float* fold_max, el_stream_t stream) {
    if (M < 0 || K < 0 || ldx < K || !float_dtype(x_dtype) || !(eps > 0.0f) || mode < 0 || mode > 2) return EL_ERR_INVALID_ARG;
    if ((fold_absmax == nullptr) != (fold_max == nullptr)) return EL_ERR_INVALID_ARG;
    if (mode == EL_QUANT_ABSMAX_ONLY && fold_max != nullptr) return EL_ERR_INVALID_ARG;
    if (M == 0) return EL_OK;
    if (!row_absmax || (K > 0 && (!x || (!q && mode != EL_QUANT_ABSMAX_ONLY)))) return EL_ERR_NULL_PTR;
    return launch_quantize_rows(x, x_dtype, ldx, q, row_absmax, M, K, eps, mode, fold_absmax, fold_max, (cudaStream_t)stream);
}

int el_quantize_tensor(const void* x, int x_dtype, int8_t* q, float* absmax, long long size, el_stream_t stream) {
    if (size < 0 || !float_dtype(x_dtype)) return EL_ERR_INVALID_ARG;
    if (!absmax || (size > 0 && (!x || !q))) return EL_ERR_NULL_PTR;
    return launch_quantize_tensor(x, x_dtype, q, absmax, size, (cudaStream_t)stream);
}

int el_dequantize_tensor(const int8_t* q, const float* absmax, void* out, int out_dtype, long long size, el_stream_t stream) {
    if (size < 0 || !float_dtype(out_dtype)) return EL_ERR_INVALID_ARG;
    if (size == 0) return EL_OK;
    if (!q || !absmax || !out) return EL_ERR_NULL_PTR;
    return launch_dequantize_tensor(q, absmax, out, out_dtype, size, (cudaStream_t)stream);
}

int el_quantize_grad(const void* dY, int dy_dtype, long long ld_dy, const float* x_absmax, const float* g_absmax, int8_t* Gq,
                     int M, int N, el_stream_t stream) {
    if (M < 0 || N < 0 || ld_dy < N || !float_dtype(dy_dtype)) return EL_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return EL_OK;
    if (!dY || !x_absmax || !g_absmax || !Gq) return EL_ERR_NULL_PTR;
    return launch_quantize_grad(dY, dy_dtype, ld_dy, x_absmax, g_absmax, Gq, M, N, (cudaStream_t)stream);
}

int el_scale_rows(const int32_t* acc, void* out, int out_dtype, const float* absmax, int absmax_stride, float gamma, int M,
                  int C, el_stream_t stream) {
    if (M < 0 || C < 0 || !out_dtype_ok(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || C == 0) return EL_OK;
    if (!acc || !out || !absmax) return EL_ERR_NULL_PTR;
    const EpiParams epi{out, (long long)C, out_dtype, absmax, absmax_stride, gamma};
    return launch_scale_rows(acc, epi, M, C, (cudaStream_t)stream);
}

int el_rmsnorm_quantize_rows(const void* x, int x_dtype, long long ldx, const float* weight, float norm_eps, int8_t* q,
                             float* row_absmax, float* rstd, int M, int K, float quant_eps, el_stream_t stream) {
    if (M < 0 || K < 0 || !float_dtype(x_dtype) || ldx < K) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (M == 0) return EL_OK;
    if (!x || !weight || !q || !row_absmax || !rstd) return EL_ERR_NULL_PTR;
    return launch_rmsnorm_quantize_rows(x, x_dtype, ldx, weight, norm_eps, q, row_absmax, rstd, M, K, quant_eps,
                                        (cudaStream_t)stream);
}

size_t el_rmsnorm_backward_workspace_bytes(int K) { return rmsnorm_backward_workspace_bytes(K); }

int el_rmsnorm_backward(const void* g, const void* x, int dtype, const float* weight, const float* rstd, void* dx,
                        float* dweight, void* workspace, size_t workspace_bytes, int M, int K, el_stream_t stream) {
    if (M < 0 || K < 0 || !float_dtype(dtype)) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (K == 0) return EL_OK;
    if (!weight || !dweight || !workspace || (M > 0 && (!g || !x || !rstd || !dx))) return EL_ERR_NULL_PTR;
    return launch_rmsnorm_backward(g, x, dtype, weight, rstd, dx, dweight, workspace, workspace_bytes, M, K,
                                   (cudaStream_t)stream);
}

int el_swiglu_quantize_rows(const void* gate, const void* up, int dtype, long long ld, const float* norm_weight, float norm_eps,
                            int8_t* q, float* row_absmax, float* rstd, int M, int H, float quant_eps, el_stream_t stream) {
    if (M < 0 || H < 0 || !float_dtype(dtype) || ld < H) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (M == 0) return EL_OK;
    if (!gate || !up || !q || !row_absmax || (norm_weight && !rstd)) return EL_ERR_NULL_PTR;
    return launch_swiglu_quantize_rows(gate, up, dtype, ld, norm_weight, norm_eps, q, row_absmax, rstd, M, H, quant_eps,
                                       (cudaStream_t)stream);
}

int el_prelinear_rows(const void* x, const void* up, int dtype, long long ld, const float* norm_weight, float norm_eps, void* y,
                      int M, int K, el_stream_t stream) {
    if (M < 0 || K < 0 || !float_dtype(dtype) || ld < K) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (M == 0) return EL_OK;
    if (!x || !y) return EL_ERR_NULL_PTR;
    return launch_prelinear_rows(x, up, dtype, ld, norm_weight, norm_eps, y, M, K, (cudaStream_t)stream);
}

int el_sigmoid_fixed(const float* g, float* sig, long long n, el_stream_t stream) {
    if (n < 0) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (n == 0) return EL_OK;
    if (!g || !sig) return EL_ERR_NULL_PTR;
    return launch_sigmoid_fixed(g, sig, n, (cudaStream_t)stream);
}

size_t el_swiglu_backward_workspace_bytes(int H) { return swiglu_backward_workspace_bytes(H); }

int el_swiglu_backward(const void* gy, const void* gate, const void* up, int dtype, long long ld, const float* norm_weight,
                       const float* rstd, void* d_gate, void* d_up, long long ld_d, float* d_norm_weight, void* workspace,
                       size_t workspace_bytes, int M, int H, el_stream_t stream) {
    if (M < 0 || H < 0 || !float_dtype(dtype) || ld < H || ld_d < H) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    if (H == 0) return EL_OK;
    if ((norm_weight && (!d_norm_weight || !workspace || (M > 0 && !rstd))) || (M > 0 && (!gy || !gate || !up || !d_gate || !d_up)))
        return EL_ERR_NULL_PTR;
    return launch_swiglu_backward(gy, gate, up, dtype, ld, norm_weight, rstd, d_gate, d_up, ld_d, d_norm_weight, workspace,
                                  workspace_bytes, M, H, (cudaStream_t)stream);
}

int el_gemm_fwd(const int8_t* Xq, const uint8_t* W_packed, void* Y, int out_dtype, const float* absmax, int absmax_stride,
                float gamma, int M, int N, int K, int flags, int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !out_dtype_ok(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return EL_OK;
    if (!Y || !absmax || (K > 0 && (!Xq || !W_packed))) return EL_ERR_NULL_PTR;
    const EpiParams epi{Y, (long long)N, out_dtype, absmax, absmax_stride, gamma};
    return gemm_dispatch(MODE_FWD, Xq, W_packed, M, N, K, epi, flags, dev_status, (cudaStream_t)stream);
}

size_t el_gemm_workspace_bytes(int mode, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (mode != 0 && mode != 1)) return 0;
    const int R = M, C = (mode == 0) ? N : K, D = (mode == 0) ? K : N;
    const int q = gemm_tc2_k_split(R, C, D);
    return q > 1 ? (size_t)q * R * C * sizeof(int) : 0;
}

int el_gemm_fwd_ws(const int8_t* Xq, const uint8_t* W_packed, void* Y, int out_dtype, const float* absmax, int absmax_stride,
                   float gamma, int M, int N, int K, int flags, void* workspace, size_t workspace_bytes, int32_t* dev_status,
                   el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !out_dtype_ok(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return EL_OK;
    if (!Y || !absmax || (K > 0 && (!Xq || !W_packed))) return EL_ERR_NULL_PTR;
    const EpiParams epi{Y, (long long)N, out_dtype, absmax, absmax_stride, gamma};
    return gemm_dispatch(MODE_FWD, Xq, W_packed, M, N, K, epi, flags, dev_status, (cudaStream_t)stream, workspace, workspace_bytes);
}

int el_gemm_dx_ws(const int8_t* dYq, const uint8_t* W_packed, void* dX, int out_dtype, const float* absmax, int absmax_stride,
                  float gamma, int M, int N, int K, int flags, void* workspace, size_t workspace_bytes, int32_t* dev_status,
                  el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !out_dtype_ok(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || K == 0) return EL_OK;
    if (!dX || !absmax || (N > 0 && (!dYq || !W_packed))) return EL_ERR_NULL_PTR;
    const EpiParams epi{dX, (long long)K, out_dtype, absmax, absmax_stride, gamma};
    return gemm_dispatch(MODE_DX, dYq, W_packed, M, K, N, epi, flags, dev_status, (cudaStream_t)stream, workspace, workspace_bytes);
}

int el_gemm_fwd_gather(const int8_t* Xq, const uint8_t* W_packed, void* const* Y_all, int n_ranks, long long ld_total,
                       long long col_offset, int out_dtype, const float* absmax, int absmax_stride, float gamma, int M, int N,
                       int K, int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !float_dtype(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return EL_OK;
    if (!Y_all || !absmax || !Xq || !W_packed) return EL_ERR_NULL_PTR;
    const EpiParams epi{nullptr, ld_total, out_dtype, absmax, absmax_stride, gamma};
    return launch_gemm_tc2(MODE_FWD, Xq, W_packed, M, N, K, epi, dev_status, (cudaStream_t)stream, Y_all, n_ranks, ld_total,
                           col_offset, 0, 0, nullptr, 0, false);
}

int el_gemm_dx_scatter(const int8_t* dYq, const uint8_t* W_packed, void* const* parts_all, int n_ranks, int rank, int M, int N,
                       int K, int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks) return EL_ERR_INVALID_ARG;
    if (M == 0 || K == 0) return EL_OK;
    if (M % (32 * n_ranks) != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (!dYq || !W_packed || !parts_all) return EL_ERR_NULL_PTR;
    const int Mr = M / n_ranks;
    void* dst[8];
    for (int d = 0; d < n_ranks; ++d) {
        if (!parts_all[d]) return EL_ERR_NULL_PTR;
        dst[d] = static_cast<char*>(parts_all[d]) + (size_t)rank * Mr * K * sizeof(int);     // slot `rank` of owner d
    }
    const EpiParams epi{nullptr, (long long)K, EL_I32, nullptr, 0, 1.0f};
    return launch_gemm_tc2(MODE_DX, dYq, W_packed, M, K, N, epi, dev_status, (cudaStream_t)stream, dst, n_ranks, 0, 0, Mr, rank,
                           nullptr, 0, false);
}

int el_reduce_scale_gather(const int32_t* parts, void* const* dX_all, int n_ranks, int rank, int out_dtype, const float* absmax,
                           float gamma, int M, int K, el_stream_t stream) {
    if (M < 0 || K < 0 || n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks || !float_dtype(out_dtype)) return EL_ERR_INVALID_ARG;
    if (M == 0 || K == 0) return EL_OK;
    if (M % n_ranks != 0 || K % 4 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (!parts || !dX_all || !absmax) return EL_ERR_NULL_PTR;
    const int Mr = M / n_ranks;
    const EpiParams epi{nullptr, (long long)K, out_dtype, absmax + (size_t)rank * Mr, 1, gamma};
    return launch_reduce_scale_gather(parts, n_ranks, dX_all, n_ranks, (long long)rank * Mr, M, epi, Mr, K, (cudaStream_t)stream);
}

int el_gemm_dx(const int8_t* dYq, const uint8_t* W_packed, void* dX, int out_dtype, const float* absmax, int absmax_stride,
               float gamma, int M, int N, int K, int flags, int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !out_dtype_ok(out_dtype) || (absmax_stride != 0 && absmax_stride != 1)) return EL_ERR_INVALID_ARG;
    if (M == 0 || K == 0) return EL_OK;
    if (!dX || !absmax || (N > 0 && (!dYq || !W_packed))) return EL_ERR_NULL_PTR;
    const EpiParams epi{dX, (long long)K, out_dtype, absmax, absmax_stride, gamma};
    return gemm_dispatch(MODE_DX, dYq, W_packed, M, K, N, epi, flags, dev_status, (cudaStream_t)stream);
}

int el_peer_barrier(uint32_t* const* flags_all, int n_ranks, int rank, uint32_t epoch, int32_t* dev_status, el_stream_t stream) {
    if (!flags_all) return EL_ERR_NULL_PTR;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    return launch_peer_barrier(reinterpret_cast<unsigned int* const*>(flags_all), n_ranks, rank, epoch, false, dev_status,
                               (cudaStream_t)stream, nullptr, nullptr, 0);
}

int el_peer_barrier_next(uint32_t* const* flags_all, int n_ranks, int rank, int32_t* dev_status, const void* word,
                         void* const* dst_all, size_t dst_offset, el_stream_t stream) {
    if (!flags_all) return EL_ERR_NULL_PTR;
    if ((word != nullptr) != (dst_all != nullptr)) return EL_ERR_INVALID_ARG;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    return launch_peer_barrier(reinterpret_cast<unsigned int* const*>(flags_all), n_ranks, rank, 0, true, dev_status,
                               (cudaStream_t)stream, word, dst_all, dst_offset);
}

int el_counter_add(int32_t* counter, int delta, el_stream_t stream) {
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    return launch_counter_add(counter, delta, (cudaStream_t)stream);
}

int el_peer_barrier_put(uint32_t* const* flags_all, int n_ranks, int rank, uint32_t epoch, int32_t* dev_status, const void* word,
                        void* const* dst_all, size_t dst_offset, el_stream_t stream) {
    if (!flags_all || !word || !dst_all) return EL_ERR_NULL_PTR;
    const int rc = require_sm100();
    if (rc != EL_OK) return rc;
    return launch_peer_barrier(reinterpret_cast<unsigned int* const*>(flags_all), n_ranks, rank, epoch, false, dev_status,
                               (cudaStream_t)stream, word, dst_all, dst_offset);
}

int el_quantize_grad_scatter(const void* dY, int dy_dtype, long long ld_dy, const float* x_absmax, const float* g_slots,
                             int n_slots, float* g_absmax_out, void* const* Gq_all, int n_ranks, long long row_offset, int M,
                             int N, el_stream_t stream) {
    if (M < 0 || N < 0 || ld_dy < N || row_offset < 0 || !float_dtype(dy_dtype)) return EL_ERR_INVALID_ARG;
    if (!Gq_all || !g_slots || (M > 0 && N > 0 && (!dY || !x_absmax))) return EL_ERR_NULL_PTR;
    return launch_quantize_grad_scatter(dY, dy_dtype, ld_dy, x_absmax, g_slots, n_slots, g_absmax_out, Gq_all, n_ranks,
                                        row_offset, M, N, (cudaStream_t)stream);
}

int el_peer_put(const void* src, void* const* dst, int n_dst, size_t dst_offset, size_t bytes, int max_ctas, el_stream_t stream) {
    if (bytes > 0 && n_dst > 0 && (!src || !dst)) return EL_ERR_NULL_PTR;
    if (max_ctas < 0) return EL_ERR_INVALID_ARG;
    return launch_peer_put(src, dst, n_dst, dst_offset, bytes, max_ctas, (cudaStream_t)stream);
}

int el_peer_put_dma(const void* src, void* const* dst, int n_dst, size_t dst_offset, size_t bytes, el_stream_t stream) {
    if (n_dst < 0 || n_dst > 8) return EL_ERR_INVALID_ARG;
    if (bytes == 0 || n_dst == 0) return EL_OK;
    if (!src || !dst) return EL_ERR_NULL_PTR;
    for (int d = 0; d < n_dst; ++d)
        if (dst[d] == nullptr) return EL_ERR_NULL_PTR;
    // one copy per destination, in the caller's order, each through a copy engine: no SM is involved
    for (int d = 0; d < n_dst; ++d)
        EL_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(dst[d]) + dst_offset, src, bytes, cudaMemcpyDeviceToDevice,
                                    (cudaStream_t)stream));
    return EL_OK;
}

int el_set_peer_barrier_limit_us(long long microseconds) { return set_peer_barrier_limit_us(microseconds); }

int el_gemm_dw(const int8_t* Gq, const int8_t* Xq, void* dW, int out_dtype, const float* g_absmax, int M, int N, int K,
               int flags, int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || (out_dtype != EL_F32 && out_dtype != EL_I32)) return EL_ERR_INVALID_ARG;
    if (N == 0 || K == 0) return EL_OK;
    if (!dW || !g_absmax || (M > 0 && (!Gq || !Xq))) return EL_ERR_NULL_PTR;
    const EpiParams epi{dW, (long long)K, out_dtype, g_absmax, 0, 1.0f};
    return gemm_dispatch(MODE_DW, Gq, Xq, N, K, M, epi, flags, dev_status, (cudaStream_t)stream);
}

int el_hysteresis_from_dw(const float* dW, uint8_t* W_packed, uint8_t* H_packed, float lr, float lr_scale, int threshold,
                          float decay_rate, int step, int N, int K, uint32_t idx_base, int ftz, el_stream_t stream) {
    if (N < 0 || K < 0) return EL_ERR_INVALID_ARG;
    if ((long long)N * K > 0x7FFFFFFFLL) return EL_ERR_UNSUPPORTED_SHAPE;   // the weight index is a 32-bit counter
    if (N == 0 || K == 0) return EL_OK;
    if (!dW || !W_packed || !H_packed) return EL_ERR_NULL_PTR;
    const HystParams hp = make_hyst_params(lr, lr_scale, threshold, decay_rate, (uint32_t)step, ftz != 0);
    return launch_hysteresis(dW, W_packed, H_packed, hp, N, K, idx_base, (cudaStream_t)stream);
}

int el_dw_hysteresis(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* W_packed, uint8_t* H_packed,
                     float lr, float lr_scale, int threshold, float decay_rate, int step, uint32_t idx_base, int M, int N,
                     int K, int32_t* dev_status, el_stream_t stream) {
    if (M <= 0 || N < 0 || K < 0) return EL_ERR_INVALID_ARG;
    if ((long long)N * K > 0x7FFFFFFFLL) return EL_ERR_UNSUPPORTED_SHAPE;
    if (N == 0 || K == 0) return EL_OK;
    if (!Gq || !Xq || !g_absmax || !W_packed || !H_packed) return EL_ERR_NULL_PTR;
    const HystParams hp = make_hyst_params(lr, lr_scale, threshold, decay_rate, (uint32_t)step, 1);
    return launch_dw_hysteresis_tc(Gq, Xq, g_absmax, W_packed, H_packed, hp, idx_base, M, N, K, dev_status,
                                   (cudaStream_t)stream);
}

int el_dw_hysteresis_step_ptr(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* W_packed, uint8_t* H_packed,
                              float lr, float lr_scale, int threshold, float decay_rate, const int32_t* step, uint32_t idx_base,
                              int M, int N, int K, int32_t* dev_status, el_stream_t stream) {
    if (M <= 0 || N < 0 || K < 0) return EL_ERR_INVALID_ARG;
    if ((long long)N * K > 0x7FFFFFFFLL) return EL_ERR_UNSUPPORTED_SHAPE;
    if (!step) return EL_ERR_NULL_PTR;
    if (reinterpret_cast<uintptr_t>(step) & 3) return EL_ERR_ALIGNMENT;
    if (N == 0 || K == 0) return EL_OK;
    if (!Gq || !Xq || !g_absmax || !W_packed || !H_packed) return EL_ERR_NULL_PTR;
    HystParams hp = make_hyst_params(lr, lr_scale, threshold, decay_rate, 0u, 1);
    hp.step_ptr = step;
    return launch_dw_hysteresis_tc(Gq, Xq, g_absmax, W_packed, H_packed, hp, idx_base, M, N, K, dev_status,
                                   (cudaStream_t)stream);
}

int el_set_decode_gemv_max_tokens(int max_tokens) {
    if (max_tokens < 0 || max_tokens > 8) return EL_ERR_INVALID_ARG;
    g_gemv_max_tokens.store(max_tokens, std::memory_order_relaxed);
    return EL_OK;
}

int el_set_decode_mma_max_tokens(int max_tokens) {
    if (max_tokens < 0 || max_tokens > 64) return EL_ERR_INVALID_ARG;
    g_mma_max_tokens.store(max_tokens, std::memory_order_relaxed);
    return EL_OK;
}

int el_set_decode_overlap(int enable) {
    g_decode_overlap.store(enable ? 1 : 0, std::memory_order_relaxed);
    return EL_OK;
}

size_t el_decode_workspace_bytes(int N) { return N > 0 ? decode_workspace_bytes(N) : 0; }

int el_linear_decode(const void* x, int x_dtype, const uint8_t* W_packed, void* Y, int out_dtype, float gamma,
                     int8_t* xq_scratch, float* absmax, void* workspace, size_t workspace_bytes, int M, int N, int K,
                     int32_t* dev_status, el_stream_t stream) {
    if (M < 0 || N < 0 || K < 0 || !float_dtype(x_dtype) || !float_dtype(out_dtype)) return EL_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return EL_OK;
    if (M > 64 || K == 0 || K % 64 != 0) return EL_ERR_UNSUPPORTED_SHAPE;
    if (!x || !W_packed || !Y || !xq_scratch || !absmax || !workspace) return EL_ERR_NULL_PTR;
    if (workspace_bytes < decode_workspace_bytes(N)) return EL_ERR_INVALID_ARG;
    if (M <= decode_gemv_max_tokens()) {      // a handful of tokens: one CUDA-core launch, no scratch touched
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_small(x, x_dtype, W_packed, gepi, M, N, K, (cudaStream_t)stream, decode_overlap());
    }
    if (M <= DECODE_MMA_SINGLE_MAX && M <= decode_mma_max_tokens() && gemv_mma_fits(M, K)) {
        // up to 8 tokens that fit in shared memory: one warp-MMA launch that quantises the tokens itself
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_mma(x, x_dtype, W_packed, gepi, M, N, K, (cudaStream_t)stream, decode_overlap());
    }
    if (M <= decode_mma_max_tokens() && gemv_mma_preq_fits(M, K)) {
        // more tokens: quantise them once, then the warp-MMA kernel on the quantised tokens, 32 at a time
        int rc = launch_quantize_rows_perm(x, x_dtype, K, xq_scratch, absmax, M, K, 1e-5f, (cudaStream_t)stream);
        if (rc != EL_OK) return rc;
        const EpiParams gepi{Y, (long long)N, out_dtype, nullptr, 0, gamma};
        return launch_gemv_mma_preq(xq_scratch, absmax, W_packed, gepi, M, N, K, (cudaStream_t)stream);
    }
    int rc = launch_quantize_rows_perm(x, x_dtype, K, xq_scratch, absmax, M, K, 1e-5f, (cudaStream_t)stream);
    if (rc != EL_OK) return rc;
    const EpiParams epi{Y, (long long)N, out_dtype, absmax, 1, gamma};
    return launch_decode_tc(xq_scratch, W_packed, epi, workspace, M, N, K, dev_status, (cudaStream_t)stream);
}

}  // extern "C"
