// Barrier between the ranks of an N-sharded layer (one process and one GPU per rank), as one tiny launch per rank.
//
// Every rank owns an array of n_ranks 32-bit flags in peer-mapped memory.  In barrier number `epoch` (1, 2, ... in the
// same order on every rank) rank r stores `epoch` into slot r of every rank's array (st.release.sys: its earlier work on
// the stream, including stores into peer memory, is visible before the flag) and then waits until all slots of its OWN
// array have reached `epoch`.  The wait only reads this GPU's memory, is bounded (about four seconds of cycles unless
// el_set_peer_barrier_limit_us says otherwise) and reports a rank that never arrives through the caller's status word
// instead of hanging.
// The epilogue-store collectives of the sharded layer (el_gemm_fwd_gather, el_gemm_dx_scatter,
// el_reduce_scale_gather) need exactly this: "all stores into my buffers have landed".  No counterpart in the reference.
#include "common.cuh"

namespace el {

namespace {

constexpr int PEER_MAX = 8;
constexpr long long PEER_WAIT_CYCLES = 1LL << 33;
std::atomic<long long> g_wait_limit_us{0};       // 0 = the default above

struct PeerFlags {
    unsigned int* p[PEER_MAX];
    unsigned int* put_dst[PEER_MAX];     // optional payload: one 32-bit word delivered to every rank ahead of the flag
};

// next_epoch: the barrier's number is not given but taken from memory: one more than the number this rank published last,
// which sits in its own slot of its own array.  A launch recorded once (a CUDA graph) can then be replayed, each replay
// being the next barrier; the explicit form may be mixed in, since it leaves its number in the same slot.
__global__ void __launch_bounds__(32)
peer_barrier_kernel(PeerFlags flags, int n_ranks, int rank, unsigned int epoch, int next_epoch, long long limit_cycles,
                    int32_t* status, const unsigned int* put_src) {
    const int i = threadIdx.x;
    if (next_epoch) {
        epoch = *reinterpret_cast<volatile unsigned int*>(flags.p[rank] + rank) + 1u;
        __syncwarp();                    // every lane has read the old number before lane `rank` overwrites it
    }
    if (i >= n_ranks) return;
    if (put_src != nullptr) *flags.put_dst[i] = *put_src;      // ordered before the flag by the fence and the release below
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[i] + rank), "r"(epoch) : "memory");
    const unsigned int* mine = flags.p[rank] + i;
    const long long t0 = clock64();
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int)(v - epoch) >= 0) break;            // wrap-safe "v >= epoch"
        if (clock64() - t0 > limit_cycles) {
            if (status != nullptr) atomicCAS(status, 0, 40 + i);      // rank i did not arrive
            break;
        }
    }
}

// A step counter kept in device memory (the hysteresis step of a recorded training step): one thread adds `delta`.
__global__ void counter_add_kernel(int32_t* counter, int delta) { *counter += delta; }

}  // namespace

int set_peer_barrier_limit_us(long long us) {
    if (us < 0) return EL_ERR_INVALID_ARG;
    g_wait_limit_us.store(us, std::memory_order_relaxed);
    return EL_OK;
}

int launch_counter_add(int32_t* counter, int delta, cudaStream_t st) {
    if (counter == nullptr) return EL_ERR_NULL_PTR;
    if (reinterpret_cast<uintptr_t>(counter) & 3) return EL_ERR_ALIGNMENT;
    counter_add_kernel<<<1, 1, 0, st>>>(counter, delta);
    return check_launch();
}

int launch_peer_barrier(unsigned int* const* flags_all, int n_ranks, int rank, unsigned int epoch, bool next_epoch,
                        int32_t* status, cudaStream_t st, const void* put_src, void* const* put_dst_all, size_t put_offset) {
    if (n_ranks < 1 || n_ranks > PEER_MAX || rank < 0 || rank >= n_ranks) return EL_ERR_INVALID_ARG;
    if ((put_src != nullptr) != (put_dst_all != nullptr)) return EL_ERR_INVALID_ARG;
    if (put_src != nullptr && ((reinterpret_cast<uintptr_t>(put_src) | put_offset) & 3)) return EL_ERR_ALIGNMENT;
    PeerFlags f{};
    for (int i = 0; i < n_ranks; ++i) {
        if (flags_all[i] == nullptr) return EL_ERR_NULL_PTR;
        if (reinterpret_cast<uintptr_t>(flags_all[i]) & 3) return EL_ERR_ALIGNMENT;
        f.p[i] = flags_all[i];
        if (put_src != nullptr) {
            if (put_dst_all[i] == nullptr) return EL_ERR_NULL_PTR;
            if (reinterpret_cast<uintptr_t>(put_dst_all[i]) & 3) return EL_ERR_ALIGNMENT;
            f.put_dst[i] = reinterpret_cast<unsigned int*>(static_cast<char*>(put_dst_all[i]) + put_offset);
        }
    }
    long long limit = PEER_WAIT_CYCLES;
    const long long us = g_wait_limit_us.load(std::memory_order_relaxed);
    if (us > 0) {
        int dev = 0, khz = 0;
        EL_CUDA_TRY(cudaGetDevice(&dev));
        EL_CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));     // the SM clock's maximum, kHz
        limit = us * (long long)(khz > 0 ? khz : 2000000) / 1000;
    }
    peer_barrier_kernel<<<1, 32, 0, st>>>(f, n_ranks, rank, epoch, next_epoch ? 1 : 0, limit, status,
                                          static_cast<const unsigned int*>(put_src));
    return check_launch();
}

}  // namespace el
