// ktc_p2p.cuh -- the device side of the peer-memory all-reduce, shared by its own kernel (ktc_p2p.cu) and by the
// second pass of the fused expression kernels (ktc_expr.cu), whose last block performs the exchange itself.
#pragma once

#include "ktc_internal.hpp"

namespace ktc {

constexpr int kP2pMaxWorld = KTC_P2P_MAX_RANKS;
constexpr int kP2pMaxFloats = KTC_P2P_MAX_FLOATS;
constexpr int kP2pMaxBufs = KTC_P2P_MAX_TENSORS;

struct Mailbox {
    unsigned int flags[2][kP2pMaxWorld];     // flags[set][r]: the last call for which rank r's values are complete
    unsigned int status;                     // 1: a wait ran out (sticky until read by the host)
    unsigned int pad[31];
    float slots[2][kP2pMaxWorld][kP2pMaxFloats];
};

struct P2pArgs {
    Mailbox* mine;
    Mailbox* peer[kP2pMaxWorld];
    int world, rank;
    unsigned int epoch;
    int n_bufs;
    float* buf[kP2pMaxBufs];
    int count[kP2pMaxBufs];
    long long limit_ns;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The whole exchange, run by ONE block of at least kP2pMaxWorld threads (every thread of the block must call it):
//   1. publish: the rank's values go straight from the source tensors into its slot of every peer's mailbox
//      (ordinary peer stores), a fence, then its flag in each mailbox;
//   2. wait: until every rank's flag for this call is in this rank's mailbox -- BOUNDED by a time limit and an
//      iteration limit; when it runs out the mailbox's status word is set and the tensors are left alone;
//   3. combine: the slots of the own mailbox are added in rank order and written back into the tensors, so every rank
//      performs the same float additions in the same order.
// `timed_out` is a shared-memory word of the calling block.
__device__ __forceinline__ void p2p_exchange_block(const P2pArgs& a, int* timed_out) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int set = a.epoch & 1;
    if (tid == 0) *timed_out = 0;
    int off = 0;
    for (int b = 0; b < a.n_bufs; ++b) {
        for (int j = tid; j < a.count[b]; j += nt) {
            const float v = __ldcg(&a.buf[b][j]);      // from L2: another block of the calling kernel may have written it
            for (int p = 0; p < a.world; ++p) a.peer[p]->slots[set][a.rank][off + j] = v;
        }
        off += a.count[b];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < a.world) st_release_sys(&a.peer[tid]->flags[set][a.rank], a.epoch);
    if (tid < a.world) {
        unsigned long long t0, t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        bool ok = false;
        for (int iter = 0; iter < (1 << 26); ++iter) {
            if (ld_acquire_sys(&a.mine->flags[set][tid]) == a.epoch) { ok = true; break; }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if ((long long)(t - t0) > a.limit_ns) break;
            __nanosleep(64);
        }
        if (!ok) *timed_out = 1;
    }
    __syncthreads();
    if (*timed_out) {
        if (tid == 0) a.mine->status = 1;
        return;
    }
    off = 0;
    for (int b = 0; b < a.n_bufs; ++b) {
        for (int j = tid; j < a.count[b]; j += nt) {
            float s = __ldcg(&a.mine->slots[set][0][off + j]);
            for (int r = 1; r < a.world; ++r) s = __fadd_rn(s, __ldcg(&a.mine->slots[set][r][off + j]));
            a.buf[b][j] = s;
        }
        off += a.count[b];
    }
}

// Host side (ktc_p2p.cu): checks the communicator and the tensors, takes the next call number and fills `out` for a
// kernel launched on the returned device's stream.
int p2p_prepare(ktc_p2p p, const ktc_buf* bufs, const int64_t* counts, int n_bufs, P2pArgs* out, Device** dev);

}  // namespace ktc
