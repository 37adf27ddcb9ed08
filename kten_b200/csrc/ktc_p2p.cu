// ktc_p2p.cu -- all-reduce of small tensors through peer memory, in one kernel.
//
// The only exchange on the sharded path is a sum of a few kilobytes (the loss partial and the
// broadcast-gradient results).  Through a collective library that is: pack the tensors, one
// all-reduce, unpack -- seven launches whose cost is pure latency.  Here one kernel per rank does
// all of it over NVLink / NVSwitch peer memory:
//   1. publish: every rank stores its values straight from the source tensors into its slot of
//      every peer's mailbox (ordinary peer stores), fences, and raises its flag in each mailbox;
//   2. wait: it waits until all ranks have raised their flag in its own mailbox -- a BOUNDED
//      wait: after a time limit or an iteration limit the kernel records a time-out and returns,
//      nothing is trapped and the context stays usable;
//   3. combine: it adds the slots of its own mailbox in rank order and writes the sums back into
//      the tensors: every rank performs the same float additions in the same order, so the result
//      is identical on all ranks and from run to run.
// Mailboxes are plain cudaMalloc memory shared between the one-process-per-GPU ranks with CUDA IPC
// handles (the caller carries the 64-byte handles between processes).  Two slot sets alternate by
// call so that a rank that runs ahead cannot overwrite values a slower rank is still reading: a
// rank can only be one call ahead, because finishing a call needs every peer's flag for it.
// Only ordinary loads and stores on mapped peer memory are used; no collective library is involved.
#include "ktc_p2p.cuh"

#include <cstring>

using namespace ktc;

namespace {

constexpr int kMaxWorld = kP2pMaxWorld;
constexpr int kMaxBufs = kP2pMaxBufs;
constexpr int kMaxFloats = kP2pMaxFloats;

__global__ void __launch_bounds__(1024) k_p2p_allreduce(const __grid_constant__ P2pArgs a) {
    __shared__ int timed_out;
    p2p_exchange_block(a, &timed_out);
}

struct P2pRec {
    int dev = -1, world = 0, rank = 0;
    Mailbox* mine = nullptr;
    Mailbox* peer[kMaxWorld] = {nullptr};
    bool opened[kMaxWorld] = {false};
    bool connected = false, live = false;
    unsigned int epoch = 0;
};
std::mutex g_p2p_mu;
std::vector<P2pRec> g_p2p;

int lookup(ktc_p2p h, P2pRec* out, const char* who) {
    std::lock_guard<std::mutex> lk(g_p2p_mu);
    if (h == 0 || h > g_p2p.size() || !g_p2p[h - 1].live) return fail(KTC_ESTATE, "%s: invalid peer-memory communicator", who);
    *out = g_p2p[h - 1];
    return KTC_OK;
}

}  // namespace

namespace ktc {

int p2p_prepare(ktc_p2p p, const ktc_buf* bufs, const int64_t* counts, int n_bufs, P2pArgs* out, Device** dev) {
    if (!bufs || !counts || n_bufs < 1 || n_bufs > kMaxBufs) return fail(KTC_EINVAL, "ktc_p2p_allreduce_sum: 1..%d tensors per call", kMaxBufs);
    P2pRec r; KTC_TRY(lookup(p, &r, "ktc_p2p_allreduce_sum"));
    if (!r.connected) return fail(KTC_ESTATE, "ktc_p2p_allreduce_sum: not connected");
    Device* d = device(r.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    P2pArgs a{};
    int64_t total = 0;
    for (int i = 0; i < n_bufs; ++i) {
        Buf b; KTC_TRY(resolve(bufs[i], &b));
        if (b.dev != r.dev) return fail(KTC_EINVAL, "ktc_p2p_allreduce_sum: tensor %d on device %d, communicator on %d", i, b.dev, r.dev);
        if (counts[i] < 0 || counts[i] > b.n) return fail(KTC_EINVAL, "ktc_p2p_allreduce_sum: tensor %d holds %lld floats, %lld given", i, (long long)b.n, (long long)counts[i]);
        a.buf[i] = b.ptr; a.count[i] = (int)counts[i];
        total += counts[i];
    }
    if (total > kMaxFloats) return fail(KTC_EINVAL, "ktc_p2p_allreduce_sum: %lld floats per call (at most %d)", (long long)total, kMaxFloats);
    unsigned int epoch;
    {
        std::lock_guard<std::mutex> lk(g_p2p_mu);
        epoch = ++g_p2p[p - 1].epoch;
    }
    a.mine = r.mine;
    for (int q = 0; q < r.world; ++q) a.peer[q] = r.peer[q];
    a.world = r.world; a.rank = r.rank; a.epoch = epoch; a.n_bufs = n_bufs;
    a.limit_ns = (long long)tune("p2p_wait_ms", 10000) * 1000000LL;
    *out = a; *dev = d;
    return KTC_OK;
}

}  // namespace ktc

extern "C" {

int ktc_p2p_create(int dev, int n_ranks, int rank, ktc_p2p* out, unsigned char handle_out[KTC_P2P_HANDLE_BYTES]) {
    if (!out || !handle_out) return fail(KTC_EINVAL, "ktc_p2p_create: null argument");
    if (n_ranks < 1 || n_ranks > kMaxWorld || rank < 0 || rank >= n_ranks)
        return fail(KTC_EINVAL, "ktc_p2p_create: rank %d of %d (at most %d ranks)", rank, n_ranks, kMaxWorld);
    static_assert(sizeof(cudaIpcMemHandle_t) == KTC_P2P_HANDLE_BYTES, "IPC handle size");
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    P2pRec r; r.dev = dev; r.world = n_ranks; r.rank = rank;
    KTC_CUDA(cudaMalloc(&r.mine, sizeof(Mailbox)));
    KTC_CUDA(cudaMemset(r.mine, 0, sizeof(Mailbox)));
    KTC_CUDA(cudaDeviceSynchronize());                     // the zeroed flags are in memory before any peer can see the handle
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, r.mine);
    if (e != cudaSuccess) { cudaGetLastError(); cudaFree(r.mine); return fail(KTC_ECOMM, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e)); }
    memcpy(handle_out, &h, KTC_P2P_HANDLE_BYTES);
    r.peer[rank] = r.mine;
    r.live = true;
    std::lock_guard<std::mutex> lk(g_p2p_mu);
    g_p2p.push_back(r);
    *out = (ktc_p2p)g_p2p.size();
    return KTC_OK;
}

int ktc_p2p_connect(ktc_p2p p, const unsigned char* all_handles) {
    if (!all_handles) return fail(KTC_EINVAL, "ktc_p2p_connect: handles are null");
    P2pRec r; KTC_TRY(lookup(p, &r, "ktc_p2p_connect"));
    if (r.connected) return fail(KTC_ESTATE, "ktc_p2p_connect: already connected");
    Device* d = device(r.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    for (int q = 0; q < r.world; ++q) {
        if (q == r.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, all_handles + (size_t)q * KTC_P2P_HANDLE_BYTES, KTC_P2P_HANDLE_BYTES);
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int k = 0; k < q; ++k) if (r.opened[k]) cudaIpcCloseMemHandle(r.peer[k]);
            return fail(KTC_ECOMM, "cudaIpcOpenMemHandle for rank %d failed: %s", q, cudaGetErrorString(e));
        }
        r.peer[q] = static_cast<Mailbox*>(ptr); r.opened[q] = true;
    }
    r.connected = true;
    std::lock_guard<std::mutex> lk(g_p2p_mu);
    g_p2p[p - 1] = r;
    return KTC_OK;
}

int ktc_test_p2p_connect_self(ktc_p2p p) {
    P2pRec r; KTC_TRY(lookup(p, &r, "ktc_test_p2p_connect_self"));
    if (r.connected) return fail(KTC_ESTATE, "ktc_test_p2p_connect_self: already connected");
    for (int q = 0; q < r.world; ++q) r.peer[q] = r.mine;       // the other ranks never publish: their flags stay 0
    r.connected = true;
    std::lock_guard<std::mutex> lk(g_p2p_mu);
    g_p2p[p - 1] = r;
    return KTC_OK;
}

int ktc_p2p_allreduce_sum(ktc_p2p p, const ktc_buf* bufs, const int64_t* counts, int n_bufs) {
    P2pArgs a{};
    Device* d = nullptr;
    KTC_TRY(p2p_prepare(p, bufs, counts, n_bufs, &a, &d));
    k_p2p_allreduce<<<1, 1024, 0, d->stream>>>(a);
    count_launch(1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "launch of the peer-memory all-reduce failed: %s", cudaGetErrorString(e));
    return KTC_OK;
}

int ktc_p2p_status(ktc_p2p p, int* status) {
    if (!status) return fail(KTC_EINVAL, "ktc_p2p_status: null status");
    P2pRec r; KTC_TRY(lookup(p, &r, "ktc_p2p_status"));
    Device* d = device(r.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    unsigned int s = 0;
    KTC_CUDA(cudaMemcpyAsync(&s, &r.mine->status, sizeof(s), cudaMemcpyDeviceToHost, d->stream));
    KTC_CUDA(cudaMemsetAsync(&r.mine->status, 0, sizeof(s), d->stream));
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    *status = s ? KTC_ETIMEOUT : KTC_OK;
    return KTC_OK;
}

int ktc_p2p_destroy(ktc_p2p p) {
    P2pRec r; KTC_TRY(lookup(p, &r, "ktc_p2p_destroy"));
    {
        std::lock_guard<std::mutex> lk(g_p2p_mu);
        g_p2p[p - 1].live = false;
    }
    Device* d = device(r.dev);
    if (d && use_device(d) == KTC_OK) cudaStreamSynchronize(d->stream);
    for (int q = 0; q < r.world; ++q) if (r.opened[q]) cudaIpcCloseMemHandle(r.peer[q]);
    cudaFree(r.mine);
    return KTC_OK;
}

}  // extern "C"
