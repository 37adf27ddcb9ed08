// ktc_runtime.cu -- devices, the buffer pool, handle table, transfers, timing.
//
// Design notes
//  * One compute stream per device; every kernel, copy and fill goes there, so
//    a block returned to the pool can be handed out again immediately: any
//    later use is ordered after the earlier work on the same stream.
//  * The pool keeps exact (512-byte rounded) sizes like the OpenCL backend's
//    reuse pool (OCLEnvironment.kt:98-107); tensors on this path recur in a
//    handful of sizes per graph, so exact-size bins hit almost always and
//    cudaMalloc/cudaFree (which synchronise the device) stay off the hot path.
#include "ktc_internal.hpp"

#include <cstdlib>
#include <cstring>

namespace ktc {

static thread_local std::string g_last_error;
static std::mutex g_mu;                       // guards g_devices, g_bufs, g_free_slots
static std::vector<Device*> g_devices;
static bool g_inited = false;
static std::vector<BufRec> g_bufs;
static std::vector<uint32_t> g_free_slots;
static std::atomic<int64_t> g_launches{0};
static std::mutex g_tune_mu;
static std::unordered_map<std::string, int> g_tune;

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
    g_last_error = buf;
}

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
    g_last_error = buf;
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return KTC_OK;
    return fail(KTC_ECUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Tunables are read on every launch.  Keys are string literals, so a small table keyed by the literal's address
// answers without a lock or a string; it is rebuilt after ktc_tune_set (a version number says so).
namespace {
struct TuneSlot { std::atomic<const char*> key{nullptr}; std::atomic<int> value{0}; std::atomic<uint32_t> version{0}; };
TuneSlot g_tune_fast[64];
std::atomic<uint32_t> g_tune_version{1};
}

int tune(const char* key, int dflt) {
    const uint32_t ver = g_tune_version.load(std::memory_order_acquire);
    const size_t h = (reinterpret_cast<uintptr_t>(key) >> 3) & 63;
    TuneSlot& slot = g_tune_fast[h];
    if (slot.version.load(std::memory_order_acquire) == ver) {                   // read, then make sure nobody rewrote the slot meanwhile
        const char* k = slot.key.load(std::memory_order_acquire);
        const int v = slot.value.load(std::memory_order_acquire);
        if (k == key && slot.version.load(std::memory_order_acquire) == ver) return v;
    }
    int val;
    {
        std::lock_guard<std::mutex> lk(g_tune_mu);
        auto it = g_tune.find(key);
        if (it != g_tune.end()) {
            val = it->second;
        } else {
            std::string env = std::string("KTC_") + key;
            for (auto& c : env) c = (char)toupper((unsigned char)c);
            const char* v = getenv(env.c_str());
            val = v ? atoi(v) : dflt;
            g_tune[key] = val;
        }
        slot.version.store(0, std::memory_order_release);      // readers skip the slot while it changes
        slot.value.store(val, std::memory_order_relaxed);
        slot.key.store(key, std::memory_order_release);
        slot.version.store(ver, std::memory_order_release);
    }
    return val;
}

// The index checks of gather / scatter / index-select / index-add kernels (they record an invalid index in a device
// word and skip the access) are read where the host waits for the stream anyway: ktc_sync and blocking copies.  With the
// tunable `index_check_sync` = 1 every such call waits and reports at once, as the reference throws at the call
// (JVMRawTensor.kt:334-353).
int take_index_error(Device* d, const char* what, int64_t axis_len, int axis) {
    snprintf(d->idx_what, sizeof(d->idx_what), "%s got invalid index, index value is out of bounds 0 and %lld at axis: %d", what, (long long)axis_len, axis);
    d->idx_pending = true;
    if (!tune("index_check_sync", 0)) return KTC_OK;
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    return check_deferred_index_error(d);
}

int check_deferred_index_error(Device* d) {
    if (!d->idx_pending) return KTC_OK;
    d->idx_pending = false;
    int h = 0;
    KTC_CUDA(cudaMemcpy(&h, d->idx_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (h == 0) return KTC_OK;
    KTC_CUDA(cudaMemset(d->idx_err, 0, sizeof(int)));
    return fail(KTC_EINVAL, "%s (the access was skipped; unless index_check_sync is set, the call that reports this is the first one that "
                            "waits for the device after the faulty call)", d->idx_what);
}

Device* device(int dev) {
    if (!g_inited) { set_error("ktc_init has not been called"); return nullptr; }
    if (dev < 0 || dev >= (int)g_devices.size()) { set_error("device %d out of range (have %d)", dev, (int)g_devices.size()); return nullptr; }
    return g_devices[dev];
}

int use_device(Device* d) {
    KTC_CUDA(cudaSetDevice(d->id));
    if (!d->ready) {
        std::lock_guard<std::mutex> lk(d->pool_mu);
        if (!d->ready) {
            KTC_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
            KTC_CUDA(cudaStreamCreateWithFlags(&d->stream_up, cudaStreamNonBlocking));
            KTC_CUDA(cudaStreamCreateWithFlags(&d->stream_down, cudaStreamNonBlocking));
            for (int i = 0; i < Device::kEventRing; ++i) KTC_CUDA(cudaEventCreateWithFlags(&d->ring[i], cudaEventDisableTiming));
            KTC_CUDA(cudaEventCreate(&d->ev_start));
            KTC_CUDA(cudaEventCreate(&d->ev_stop));
            KTC_CUDA(cudaMalloc(&d->err_flag, 3 * sizeof(int)));
            KTC_CUDA(cudaMemset(d->err_flag, 0, 3 * sizeof(int)));
            d->wait_flag = d->err_flag + 1;
            d->idx_err = d->err_flag + 2;
            d->ready = true;
        }
    }
    return KTC_OK;
}

static inline size_t round_bytes(int64_t n_floats) {
    size_t b = (size_t)n_floats * sizeof(float);
    if (b < 512) b = 512;
    return (b + 511) & ~(size_t)511;
}

static void trim_locked(Device* d) {
    for (auto& kv : d->free_lists) {
        for (void* p : kv.second) { cudaFree(p); d->cached_bytes -= (int64_t)kv.first; }
        kv.second.clear();
    }
    d->free_lists.clear();
}

int pool_alloc(Device* d, int64_t n_floats, float** ptr, size_t* rounded) {
    if (n_floats < 0) return fail(KTC_EINVAL, "negative allocation size %lld", (long long)n_floats);
    const size_t bytes = round_bytes(n_floats);
    std::lock_guard<std::mutex> lk(d->pool_mu);
    d->n_alloc_calls++;
    if (d->limit_bytes > 0 && d->live_bytes + (int64_t)bytes > d->limit_bytes)
        return fail(KTC_ENOMEM, "pool limit: %lld live + %zu requested > %lld allowed",
                    (long long)d->live_bytes, bytes, (long long)d->limit_bytes);
    auto it = d->free_lists.find(bytes);
    if (it != d->free_lists.end() && !it->second.empty()) {
        *ptr = (float*)it->second.back(); it->second.pop_back();
        d->cached_bytes -= (int64_t)bytes; d->live_bytes += (int64_t)bytes; d->n_pool_hits++;
        *rounded = bytes;
        return KTC_OK;
    }
    if (d->limit_bytes > 0 && d->live_bytes + d->cached_bytes + (int64_t)bytes > d->limit_bytes) trim_locked(d);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {           // give cached blocks back to the driver and retry once
        cudaGetLastError();
        trim_locked(d);
        e = cudaMalloc(&p, bytes);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(KTC_ENOMEM, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    d->live_bytes += (int64_t)bytes;
    *ptr = (float*)p; *rounded = bytes;
    return KTC_OK;
}

void pool_free(Device* d, void* ptr, size_t rounded) {
    std::lock_guard<std::mutex> lk(d->pool_mu);
    d->free_lists[rounded].push_back(ptr);
    d->live_bytes -= (int64_t)rounded; d->cached_bytes += (int64_t)rounded;
}

int resolve(ktc_buf h, Buf* out) {
    const uint32_t slot = (uint32_t)(h & 0xffffffffu), gen = (uint32_t)(h >> 32);
    std::lock_guard<std::mutex> lk(g_mu);
    if (slot == 0 || slot > g_bufs.size()) return fail(KTC_ESTATE, "invalid buffer handle 0x%llx", (unsigned long long)h);
    const BufRec& r = g_bufs[slot - 1];
    if (r.gen != gen || r.refcount <= 0) return fail(KTC_ESTATE, "buffer handle 0x%llx was already released", (unsigned long long)h);
    out->dev = r.dev; out->ptr = r.ptr; out->n = r.n;
    return KTC_OK;
}

static ktc_buf new_handle(int dev, float* ptr, int64_t n, size_t bytes, bool owned, ktc_buf parent = 0) {
    std::lock_guard<std::mutex> lk(g_mu);
    uint32_t slot;
    if (!g_free_slots.empty()) { slot = g_free_slots.back(); g_free_slots.pop_back(); }
    else { g_bufs.emplace_back(); slot = (uint32_t)g_bufs.size(); }
    BufRec& r = g_bufs[slot - 1];
    r.dev = dev; r.ptr = ptr; r.n = n; r.bytes = bytes; r.owned = owned; r.refcount = 1; r.parent = parent;
    r.gen += 1; if (r.gen == 0) r.gen = 1;
    return ((uint64_t)r.gen << 32) | slot;
}

}  // namespace ktc

using namespace ktc;

extern "C" {

const char* ktc_last_error(void) { return g_last_error.c_str(); }
const char* ktc_version(void) { return "kten-cuda 0.1 (sm_100a)"; }

int ktc_init(int* n_devices) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_inited) {
        int n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return fail(KTC_ECUDA, "no usable CUDA device (%s); this backend has no CPU path",
                        e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
        }
        for (int i = 0; i < n; ++i) {
            cudaDeviceProp p;
            KTC_CUDA(cudaGetDeviceProperties(&p, i));
            Device* d = new Device();
            d->id = i; d->sm_count = p.multiProcessorCount; d->total_mem = p.totalGlobalMem; d->name = p.name;
            g_devices.push_back(d);
        }
        g_inited = true;
    }
    if (n_devices) *n_devices = (int)g_devices.size();
    return KTC_OK;
}

int ktc_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_inited) return KTC_OK;
    for (Device* d : g_devices) {
        if (d->ready) {
            cudaSetDevice(d->id);
            cudaStreamSynchronize(d->stream);
            for (auto& r : g_bufs) if (r.refcount > 0 && r.owned && r.dev == d->id) { cudaFree(r.ptr); }
            { std::lock_guard<std::mutex> pl(d->pool_mu); for (auto& kv : d->free_lists) for (void* p : kv.second) cudaFree(p); d->free_lists.clear(); }
            if (d->l2_flush) cudaFree(d->l2_flush);
            cudaFree(d->err_flag);
            cudaEventDestroy(d->ev_start); cudaEventDestroy(d->ev_stop);
            for (int i = 0; i < Device::kEventRing; ++i) cudaEventDestroy(d->ring[i]);
            cudaStreamDestroy(d->stream_up); cudaStreamDestroy(d->stream_down);
            cudaStreamDestroy(d->stream);
        }
        delete d;
    }
    g_devices.clear(); g_bufs.clear(); g_free_slots.clear();
    g_inited = false;
    return KTC_OK;
}

int ktc_device_info(int dev, char* name, size_t name_len, int64_t* total_mem_bytes, int* sm_count) {
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    if (name && name_len) { strncpy(name, d->name.c_str(), name_len - 1); name[name_len - 1] = 0; }
    if (total_mem_bytes) *total_mem_bytes = (int64_t)d->total_mem;
    if (sm_count) *sm_count = d->sm_count;
    return KTC_OK;
}

int ktc_alloc(int dev, int64_t n_floats, ktc_buf* out) {
    if (!out) return fail(KTC_EINVAL, "ktc_alloc: out is null");
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    float* p; size_t rounded;
    KTC_TRY(pool_alloc(d, n_floats, &p, &rounded));
    *out = new_handle(dev, p, n_floats, rounded, true);
    return KTC_OK;
}

int ktc_wrap(int dev, void* device_ptr, int64_t n_floats, ktc_buf* out) {
    if (!out || !device_ptr || n_floats < 0) return fail(KTC_EINVAL, "ktc_wrap: bad argument");
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    *out = new_handle(dev, (float*)device_ptr, n_floats, 0, false);
    return KTC_OK;
}

int ktc_retain(ktc_buf h) {
    const uint32_t slot = (uint32_t)(h & 0xffffffffu), gen = (uint32_t)(h >> 32);
    std::lock_guard<std::mutex> lk(g_mu);
    if (slot == 0 || slot > g_bufs.size() || g_bufs[slot - 1].gen != gen || g_bufs[slot - 1].refcount <= 0)
        return fail(KTC_ESTATE, "ktc_retain: buffer handle 0x%llx was already released", (unsigned long long)h);
    g_bufs[slot - 1].refcount++;
    return KTC_OK;
}

int ktc_release(ktc_buf h) {
    const uint32_t slot = (uint32_t)(h & 0xffffffffu), gen = (uint32_t)(h >> 32);
    BufRec dead; bool free_it = false;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (slot == 0 || slot > g_bufs.size() || g_bufs[slot - 1].gen != gen || g_bufs[slot - 1].refcount <= 0)
            return fail(KTC_ESTATE, "ktc_release: buffer handle 0x%llx was already released", (unsigned long long)h);
        BufRec& r = g_bufs[slot - 1];
        if (--r.refcount == 0) { dead = r; free_it = true; r.ptr = nullptr; g_free_slots.push_back(slot); }
    }
    if (free_it && dead.owned) pool_free(g_devices[dead.dev], dead.ptr, dead.bytes);
    if (free_it && dead.parent) return ktc_release(dead.parent);
    return KTC_OK;
}

int ktc_view(ktc_buf buf, int64_t off, int64_t n, ktc_buf* out) {
    if (!out) return fail(KTC_EINVAL, "ktc_view: out is null");
    Buf b; KTC_TRY(resolve(buf, &b));
    if (off < 0 || n < 0 || off + n > b.n)
        return fail(KTC_EINVAL, "ktc_view: range [%lld, %lld) outside a buffer of %lld floats", (long long)off, (long long)(off + n), (long long)b.n);
    KTC_TRY(ktc_retain(buf));
    *out = new_handle(b.dev, b.ptr + off, n, 0, false, buf);
    return KTC_OK;
}

int ktc_refcount(ktc_buf h, int* count) {
    const uint32_t slot = (uint32_t)(h & 0xffffffffu), gen = (uint32_t)(h >> 32);
    std::lock_guard<std::mutex> lk(g_mu);
    if (slot == 0 || slot > g_bufs.size()) return fail(KTC_ESTATE, "invalid buffer handle");
    const BufRec& r = g_bufs[slot - 1];
    if (count) *count = (r.gen == gen) ? r.refcount : 0;
    return KTC_OK;
}

int ktc_buf_info(ktc_buf h, int* dev, int64_t* n_floats, void** device_ptr) {
    Buf b; KTC_TRY(resolve(h, &b));
    if (dev) *dev = b.dev;
    if (n_floats) *n_floats = b.n;
    if (device_ptr) *device_ptr = b.ptr;
    return KTC_OK;
}

int ktc_pool_stats(int dev, int64_t* live, int64_t* cached, int64_t* n_alloc, int64_t* n_hits) {
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    std::lock_guard<std::mutex> lk(d->pool_mu);
    if (live) *live = d->live_bytes;
    if (cached) *cached = d->cached_bytes;
    if (n_alloc) *n_alloc = d->n_alloc_calls;
    if (n_hits) *n_hits = d->n_pool_hits;
    return KTC_OK;
}

int ktc_pool_trim(int dev) {
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    KTC_TRY(use_device(d));
    KTC_CUDA(cudaStreamSynchronize(d->stream));   // cached blocks may still be read by queued work ...
    KTC_CUDA(cudaStreamSynchronize(d->stream_up));     // ... and by overlapped copies on the two copy streams
    KTC_CUDA(cudaStreamSynchronize(d->stream_down));
    std::lock_guard<std::mutex> lk(d->pool_mu);
    trim_locked(d);
    return KTC_OK;
}

int ktc_pool_limit(int dev, int64_t max_bytes) {
    Device* d = device(dev); if (!d) return KTC_ESTATE;
    std::lock_guard<std::mutex> lk(d->pool_mu);
    d->limit_bytes = max_bytes > 0 ? max_bytes : 0;
    return KTC_OK;
}

int ktc_host_alloc(int64_t n_floats, float** out) {
    if (!out || n_floats < 0) return fail(KTC_EINVAL, "ktc_host_alloc: bad argument");
    if (!g_inited) return fail(KTC_ESTATE, "ktc_init has not been called");
    void* p = nullptr;
    size_t bytes = (size_t)n_floats * sizeof(float); if (bytes == 0) bytes = 4;
    KTC_CUDA(cudaHostAlloc(&p, bytes, cudaHostAllocPortable));
    *out = (float*)p;
    return KTC_OK;
}

int ktc_host_free(float* p) {
    if (!p) return KTC_OK;
    KTC_CUDA(cudaFreeHost(p));
    return KTC_OK;
}

static int check_range(const Buf& b, int64_t off, int64_t n, const char* who) {
    if (off < 0 || n < 0 || off + n > b.n)
        return fail(KTC_EINVAL, "%s: range [%lld, %lld) outside a buffer of %lld floats", who,
                    (long long)off, (long long)(off + n), (long long)b.n);
    return KTC_OK;
}

// Overlapped copies run on their own streams so that uploads, kernels and downloads of a
// chunked pipeline proceed at the same time (the copy engines are full duplex).  Ordering is
// conservative: an upload starts after all compute work queued so far (which may still read the
// destination) and later compute work waits for it; a download starts after all compute work
// queued so far (which produces the source) and later compute work, which may overwrite the
// source, waits for it.
static cudaEvent_t next_event(Device* d) {
    std::lock_guard<std::mutex> lk(d->pool_mu);
    cudaEvent_t e = d->ring[d->ring_next];
    d->ring_next = (d->ring_next + 1) % Device::kEventRing;
    return e;
}

static int overlapped_copy(Device* d, cudaStream_t side, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, bool fenced) {
    if (fenced) {
        cudaEvent_t before = next_event(d);
        KTC_CUDA(cudaEventRecord(before, d->stream));
        KTC_CUDA(cudaStreamWaitEvent(side, before, 0));
    } else if (kind == cudaMemcpyDeviceToHost) {
        // a download always follows the compute work that produces its source
        cudaEvent_t before = next_event(d);
        KTC_CUDA(cudaEventRecord(before, d->stream));
        KTC_CUDA(cudaStreamWaitEvent(side, before, 0));
    }
    KTC_CUDA(cudaMemcpyAsync(dst, src, bytes, kind, side));
    if (fenced || kind == cudaMemcpyHostToDevice) {
        // compute work queued from now on sees the uploaded data / may overwrite the downloaded source
        cudaEvent_t after = next_event(d);
        KTC_CUDA(cudaEventRecord(after, side));
        KTC_CUDA(cudaStreamWaitEvent(d->stream, after, 0));
    }
    return KTC_OK;
}

int ktc_h2d(ktc_buf dst, int64_t dst_off, const float* src, int64_t n, int mode) {
    Buf b; KTC_TRY(resolve(dst, &b)); KTC_TRY(check_range(b, dst_off, n, "ktc_h2d"));
    if (n == 0) return KTC_OK;
    if (!src) return fail(KTC_EINVAL, "ktc_h2d: src is null");
    if (mode < 0 || mode > KTC_COPY_OVERLAP_UNFENCED) return fail(KTC_EINVAL, "ktc_h2d: unknown copy mode %d", mode);
    Device* d = device(b.dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    if (mode >= KTC_COPY_OVERLAP) return overlapped_copy(d, d->stream_up, b.ptr + dst_off, src, (size_t)n * 4, cudaMemcpyHostToDevice, mode == KTC_COPY_OVERLAP);
    KTC_CUDA(cudaMemcpyAsync(b.ptr + dst_off, src, (size_t)n * 4, cudaMemcpyHostToDevice, d->stream));
    if (mode == KTC_COPY_SYNC) KTC_CUDA(cudaStreamSynchronize(d->stream));
    return KTC_OK;
}

int ktc_d2h(float* dst, ktc_buf src, int64_t src_off, int64_t n, int mode) {
    Buf b; KTC_TRY(resolve(src, &b)); KTC_TRY(check_range(b, src_off, n, "ktc_d2h"));
    if (n == 0) return KTC_OK;
    if (!dst) return fail(KTC_EINVAL, "ktc_d2h: dst is null");
    if (mode < 0 || mode > KTC_COPY_OVERLAP_UNFENCED) return fail(KTC_EINVAL, "ktc_d2h: unknown copy mode %d", mode);
    Device* d = device(b.dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    if (mode >= KTC_COPY_OVERLAP) return overlapped_copy(d, d->stream_down, dst, b.ptr + src_off, (size_t)n * 4, cudaMemcpyDeviceToHost, mode == KTC_COPY_OVERLAP);
    KTC_CUDA(cudaMemcpyAsync(dst, b.ptr + src_off, (size_t)n * 4, cudaMemcpyDeviceToHost, d->stream));
    if (mode == KTC_COPY_SYNC) { KTC_CUDA(cudaStreamSynchronize(d->stream)); return check_deferred_index_error(d); }
    return KTC_OK;
}

int ktc_d2d(ktc_buf dst, int64_t dst_off, ktc_buf src, int64_t src_off, int64_t n) {
    Buf bd, bs; KTC_TRY(resolve(dst, &bd)); KTC_TRY(resolve(src, &bs));
    KTC_TRY(check_range(bd, dst_off, n, "ktc_d2d(dst)")); KTC_TRY(check_range(bs, src_off, n, "ktc_d2d(src)"));
    if (bd.dev != bs.dev) return fail(KTC_EINVAL, "ktc_d2d: buffers live on devices %d and %d", bd.dev, bs.dev);
    if (n == 0) return KTC_OK;
    Device* d = device(bd.dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    KTC_CUDA(cudaMemcpyAsync(bd.ptr + dst_off, bs.ptr + src_off, (size_t)n * 4, cudaMemcpyDeviceToDevice, d->stream));
    return KTC_OK;
}

int ktc_fill(ktc_buf buf, int64_t off, int64_t n, float value) {
    Buf b; KTC_TRY(resolve(buf, &b)); KTC_TRY(check_range(b, off, n, "ktc_fill"));
    if (n == 0) return KTC_OK;
    Device* d = device(b.dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    return launch_fill(d, b.ptr + off, n, value);
}

int ktc_sync(int dev) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    KTC_CUDA(cudaStreamSynchronize(d->stream));
    KTC_CUDA(cudaStreamSynchronize(d->stream_up));
    KTC_CUDA(cudaStreamSynchronize(d->stream_down));
    return check_deferred_index_error(d);
}

int ktc_copy_fence(int dev) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    cudaEvent_t up = next_event(d), down = next_event(d);
    KTC_CUDA(cudaEventRecord(up, d->stream_up));
    KTC_CUDA(cudaEventRecord(down, d->stream_down));
    KTC_CUDA(cudaStreamWaitEvent(d->stream, up, 0));
    KTC_CUDA(cudaStreamWaitEvent(d->stream, down, 0));
    // ... and copies issued after the fence start after the compute work issued before it (an unfenced
    // upload may then overwrite what earlier kernels read)
    cudaEvent_t done = next_event(d);
    KTC_CUDA(cudaEventRecord(done, d->stream));
    KTC_CUDA(cudaStreamWaitEvent(d->stream_up, done, 0));
    KTC_CUDA(cudaStreamWaitEvent(d->stream_down, done, 0));
    return KTC_OK;
}

int ktc_timer_start(int dev) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    KTC_CUDA(cudaEventRecord(d->ev_start, d->stream));
    return KTC_OK;
}

int ktc_timer_stop(int dev, float* elapsed_ms) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    KTC_CUDA(cudaEventRecord(d->ev_stop, d->stream));
    KTC_CUDA(cudaEventSynchronize(d->ev_stop));
    float ms = 0.f;
    KTC_CUDA(cudaEventElapsedTime(&ms, d->ev_start, d->ev_stop));
    if (elapsed_ms) *elapsed_ms = ms;
    return KTC_OK;
}

int64_t ktc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ktc_flush_l2(int dev) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    if (!d->l2_flush) {
        d->l2_flush_bytes = (size_t)256 << 20;       // twice the 126 MB L2
        KTC_CUDA(cudaMalloc(&d->l2_flush, d->l2_flush_bytes));
    }
    return launch_fill(d, (float*)d->l2_flush, (int64_t)(d->l2_flush_bytes / 4), 0.0f);
}

int ktc_tune_set(const char* key, int value) {
    if (!key) return fail(KTC_EINVAL, "ktc_tune_set: key is null");
    std::lock_guard<std::mutex> lk(g_tune_mu);
    g_tune[key] = value;
    g_tune_version.fetch_add(1, std::memory_order_acq_rel);        // the per-literal table is stale now
    return KTC_OK;
}

int ktc_test_bounded_wait(int dev, int64_t limit_ns, int* status) {
    Device* d = device(dev); if (!d) return KTC_ESTATE; KTC_TRY(use_device(d));
    if (limit_ns <= 0 || limit_ns > 2000000000LL) return fail(KTC_EINVAL, "ktc_test_bounded_wait: limit must be in (0, 2 s]");
    return launch_bounded_wait(d, limit_ns, status);
}

}  // extern "C"
