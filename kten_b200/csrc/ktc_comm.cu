// ktc_comm.cu -- cross-GPU sum of partial reductions and weight gradients.
//
// The reference is single-device (a tensor lives on exactly one platform,
// kten-api/.../tensor/Tensor.kt:143); sharding batch-leading work over the
// GPUs of one box is new here.  One process drives one GPU; the only exchange
// on the path is an in-place all-reduce (sum, float32) of small packed buffers
// -- loss partials and broadcast-gradient (sum-to-shape) results -- enqueued on
// the device's compute stream so it is ordered after the kernels that produce
// the partials.
//
// NCCL is bound at run time with dlopen (no link-time dependency): whichever
// libnccl.so.2 the process already carries is used, otherwise the system one.
// Payloads here are kilobytes, so the collective is latency-bound; NVLink 5 /
// NVSwitch gives every peer the same distance and NCCL picks its low-latency
// protocol for that size.
#include "ktc_internal.hpp"

#include <dlfcn.h>

using namespace ktc;

namespace {

struct NcclId { char internal[128]; };
typedef int (*fn_get_id)(NcclId*);
typedef int (*fn_init_rank)(void** comm, int n, NcclId id, int rank);
typedef int (*fn_allreduce)(const void*, void*, size_t, int dtype, int op, void* comm, cudaStream_t);
typedef int (*fn_destroy)(void* comm);
typedef const char* (*fn_errstr)(int);

struct Nccl {
    void* handle = nullptr;
    fn_get_id get_id = nullptr; fn_init_rank init_rank = nullptr; fn_allreduce allreduce = nullptr;
    fn_destroy destroy = nullptr; fn_errstr errstr = nullptr;
};
Nccl g_nccl;
std::mutex g_comm_mu;
struct CommRec { void* comm = nullptr; int dev = -1; int n_ranks = 0; int rank = 0; bool live = false; };
std::vector<CommRec> g_comms;
std::atomic<int> g_inject_errors{0};

int load_nccl() {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (g_nccl.handle) return KTC_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) return fail(KTC_ECOMM, "cannot load libnccl: %s", dlerror());
    g_nccl.get_id = (fn_get_id)dlsym(h, "ncclGetUniqueId");
    g_nccl.init_rank = (fn_init_rank)dlsym(h, "ncclCommInitRank");
    g_nccl.allreduce = (fn_allreduce)dlsym(h, "ncclAllReduce");
    g_nccl.destroy = (fn_destroy)dlsym(h, "ncclCommDestroy");
    g_nccl.errstr = (fn_errstr)dlsym(h, "ncclGetErrorString");
    if (!g_nccl.get_id || !g_nccl.init_rank || !g_nccl.allreduce || !g_nccl.destroy)
        return fail(KTC_ECOMM, "libnccl lacks a required symbol");
    g_nccl.handle = h;
    return KTC_OK;
}

int nccl_fail(int rc, const char* what) {
    return fail(KTC_ECOMM, "%s failed: %s (%d)", what, g_nccl.errstr ? g_nccl.errstr(rc) : "nccl error", rc);
}

}  // namespace

extern "C" {

int ktc_comm_unique_id(unsigned char id[KTC_COMM_ID_BYTES]) {
    if (!id) return fail(KTC_EINVAL, "ktc_comm_unique_id: id is null");
    KTC_TRY(load_nccl());
    NcclId nid;
    int rc = g_nccl.get_id(&nid);
    if (rc != 0) return nccl_fail(rc, "ncclGetUniqueId");
    memcpy(id, nid.internal, KTC_COMM_ID_BYTES);
    return KTC_OK;
}

int ktc_comm_init_rank(int dev, int n_ranks, int rank, const unsigned char id[KTC_COMM_ID_BYTES], ktc_comm* out) {
    if (!id || !out) return fail(KTC_EINVAL, "ktc_comm_init_rank: null argument");
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(KTC_EINVAL, "ktc_comm_init_rank: rank %d of %d", rank, n_ranks);
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    KTC_TRY(load_nccl());
    NcclId nid; memcpy(nid.internal, id, KTC_COMM_ID_BYTES);
    void* comm = nullptr;
    int rc = g_nccl.init_rank(&comm, n_ranks, nid, rank);
    if (rc != 0) return nccl_fail(rc, "ncclCommInitRank");
    std::lock_guard<std::mutex> lk(g_comm_mu);
    CommRec r; r.comm = comm; r.dev = dev; r.n_ranks = n_ranks; r.rank = rank; r.live = true;
    g_comms.push_back(r);
    *out = (ktc_comm)g_comms.size();
    return KTC_OK;
}

int ktc_allreduce_sum(ktc_comm comm, ktc_buf buf, int64_t off, int64_t n) {
    CommRec r;
    {
        std::lock_guard<std::mutex> lk(g_comm_mu);
        if (comm == 0 || comm > g_comms.size() || !g_comms[comm - 1].live)
            return fail(KTC_ESTATE, "ktc_allreduce_sum: invalid communicator");
        r = g_comms[comm - 1];
    }
    Buf b; KTC_TRY(resolve(buf, &b));
    if (b.dev != r.dev) return fail(KTC_EINVAL, "ktc_allreduce_sum: buffer on device %d, communicator on %d", b.dev, r.dev);
    if (off < 0 || n < 0 || off + n > b.n) return fail(KTC_EINVAL, "ktc_allreduce_sum: range outside the buffer");
    if (g_inject_errors.load() > 0) { g_inject_errors.fetch_sub(1); return fail(KTC_ECOMM, "injected collective failure (test hook)"); }
    if (n == 0) return KTC_OK;
    Device* d = device(r.dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    int rc = g_nccl.allreduce(b.ptr + off, b.ptr + off, (size_t)n, /*ncclFloat32*/ 7, /*ncclSum*/ 0, r.comm, d->stream);
    if (rc != 0) return nccl_fail(rc, "ncclAllReduce");
    return KTC_OK;
}

int ktc_comm_destroy(ktc_comm comm) {
    CommRec r;
    {
        std::lock_guard<std::mutex> lk(g_comm_mu);
        if (comm == 0 || comm > g_comms.size() || !g_comms[comm - 1].live)
            return fail(KTC_ESTATE, "ktc_comm_destroy: invalid communicator");
        r = g_comms[comm - 1];
        g_comms[comm - 1].live = false;
    }
    Device* d = device(r.dev);
    if (d && use_device(d) == KTC_OK) cudaStreamSynchronize(d->stream);
    int rc = g_nccl.destroy(r.comm);
    if (rc != 0) return nccl_fail(rc, "ncclCommDestroy");
    return KTC_OK;
}

int ktc_test_inject_comm_error(int n_calls) {
    g_inject_errors.store(n_calls > 0 ? n_calls : 0);
    return KTC_OK;
}

}  // extern "C"
