// ktc_internal.hpp -- shared state of libkten_cuda.so (not part of the C ABI).
//
// One Device record per visible GPU: a single in-order compute stream (the
// role of the one in-order command queue in the OpenCL backend,
// backend/kten-opencl/.../platform/OCLEnvironment.kt:291-299), an exact-size
// buffer reuse pool (OCLEnvironment.kt:98-107, 191-200) and the timing events.
// Buffers are rows of a handle table guarded by one mutex; a handle carries a
// generation so that a released handle is detected instead of reused silently
// (OCLMemoryObject.kt:167-170 throws on use after release).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/kten_cuda.h"

namespace ktc {

struct Device {
    int id = -1;
    bool ready = false;
    cudaStream_t stream = nullptr;
    cudaStream_t stream_up = nullptr, stream_down = nullptr;   // overlapped host<->device copies (mode KTC_COPY_OVERLAP)
    static constexpr int kEventRing = 256;
    cudaEvent_t ring[kEventRing] = {nullptr};                  // ordering events, reused round-robin
    int ring_next = 0;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    int sm_count = 0;
    size_t total_mem = 0;
    std::string name;
    // pool
    std::mutex pool_mu;
    std::unordered_map<size_t, std::vector<void*>> free_lists;   // rounded bytes -> idle blocks
    int64_t live_bytes = 0, cached_bytes = 0, limit_bytes = 0;
    int64_t n_alloc_calls = 0, n_pool_hits = 0;
    // misc device-side scratch owned by the runtime
    void* l2_flush = nullptr; size_t l2_flush_bytes = 0;
    int* err_flag = nullptr;          // device int: status slot of kernels that report at once (NaN search, bounded wait)
    int* wait_flag = nullptr;         // device int nothing ever sets (bounded-wait test hook)
    int* idx_err = nullptr;           // device int, set by kernels that meet an invalid index (gather / scatter / index ops)
    bool idx_pending = false;         // an index check is outstanding: read at the next call that waits for the stream
    char idx_what[160] = {0};         // the message of the last call that may have set it
};

struct BufRec {
    int dev = -1;
    float* ptr = nullptr;
    int64_t n = 0;          // floats
    size_t bytes = 0;       // pooled (rounded) size, 0 for wrapped memory
    int refcount = 0;
    bool owned = false;
    uint32_t gen = 0;
    ktc_buf parent = 0;     // views hold one reference on the buffer they alias
};

// resolved view of a handle, valid while the caller holds a reference
struct Buf {
    int dev; float* ptr; int64_t n;
};

void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

Device* device(int dev);                 // nullptr + error if not initialised / out of range
int use_device(Device* d);               // cudaSetDevice, KTC_ECUDA on failure
int resolve(ktc_buf h, Buf* out);        // KTC_ESTATE for stale handles
int pool_alloc(Device* d, int64_t n_floats, float** ptr, size_t* rounded);
void pool_free(Device* d, void* ptr, size_t rounded);
int check_cuda(cudaError_t e, const char* what);
void count_launch(int n = 1);
int tune(const char* key, int dflt);     // integer tunables (env KTC_<KEY> or ktc_tune_set); `key` must be a string literal
int take_index_error(Device* d, const char* what, int64_t axis_len, int axis);   // after a kernel that validates indices
int check_deferred_index_error(Device* d);                                       // after the stream has been waited for

#define KTC_CUDA(call) do { int _s = ::ktc::check_cuda((call), #call); if (_s != KTC_OK) return _s; } while (0)
#define KTC_TRY(call) do { int _s = (call); if (_s != KTC_OK) return _s; } while (0)

// temp device buffer drawn from the pool; returned on scope exit (stream
// ordered reuse on the single compute stream makes that safe).
struct Scratch {
    Device* d = nullptr; float* ptr = nullptr; size_t rounded = 0;
    int get(Device* dev, int64_t n_floats) { d = dev; return pool_alloc(dev, n_floats, &ptr, &rounded); }
    ~Scratch() { if (ptr) pool_free(d, ptr, rounded); }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// launchers implemented in the kernel translation units
int launch_map1(Device* d, int kind, int op, float* out, const float* a, int64_t n, float p0, float p1);
int launch_map2(Device* d, int op, float* out, const float* a, const float* b, int64_t n);
int launch_fill(Device* d, float* out, int64_t n, float v);
int launch_bcast(Device* d, int op, float* out, const int64_t* oshape, int ndim,
                 const float* a, const int64_t* astride, const float* b, const int64_t* bstride, float param = 0.f);
constexpr int kBcastSelectB = -1, kBcastMaskedFill = 100;      // internal op codes of launch_bcast
int launch_map1_more(Device* d, int op, float* out, const float* a, int64_t n);
int launch_eq_scalar(Device* d, int op, float* out, const float* a, int64_t n, float value, float eps);
int launch_compare_tensor(Device* d, int op, float* out, const float* a, const float* b, int64_t n, float eps);
int launch_contains_nan(Device* d, const float* a, int64_t n, int* result);
int launch_reduce_axis(Device* d, int op, float* out, float* out_idx, const float* in,
                       int64_t outer, int64_t A, int64_t inner);
int launch_scatter_axis(Device* d, float* target, const float* index, const float* src,
                        int64_t outer, int64_t A, int64_t inner);
int launch_bounded_wait(Device* d, int64_t limit_ns, int* status);

// map1 kinds
enum { M1_UNARY = 0, M1_SCALAR_R = 1, M1_SCALAR_L = 2, M1_CLAMP = 3, M1_COMPARE = 4 };

}  // namespace ktc
