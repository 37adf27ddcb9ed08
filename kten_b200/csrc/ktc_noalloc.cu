// ktc_noalloc.cu -- a full sum / mean that allocates nothing.
//
// Who this is for.  ktc_reduce_all splits a long reduction over many CTAs and
// draws the buffer for their partial results from the library's pool, which on
// a miss calls cudaMalloc.  Some callers cannot afford that inside their hot
// section: a training loop that has handed all free device memory to its own
// allocator, a latency-bound service that must not hit the device-wide
// synchronisation cudaMalloc implies, or code running while another component
// holds the allocator.  For them ktc_reduce_all_noalloc does the same
// reduction with its partials in a fixed array that is part of the library
// image: KTC_NOALLOC_SCRATCH_BYTES (16 KiB) of device memory, present on every
// GPU that loads the library for as long as the process lives.
//
// The caller passes the input and output buffers as usual (handles created
// earlier, at a time when set-up work was acceptable).  Nothing in this call --
// host or device side -- obtains memory: no cudaMalloc / cudaFree, no pool
// access, no allocating library routine.
//
// Limits and rules
//  * n <= KTC_NOALLOC_MAX_ELEMS (2^30); larger requests are refused with
//    KTC_EINVAL and a message naming the limit.
//  * The scratch array is shared by every call on a device and keeps whatever
//    the previous call left there.  Each call overwrites exactly the slots it
//    later reads, so nothing has to be cleared -- but two calls that overlap on
//    the same GPU would race on it.  A call is two launches on the device's
//    one compute stream; a per-device lock is held across the pair, so calls
//    from several host threads cannot interleave their launches (partial A,
//    partial B, final A would add B's partials).  Work that reaches the GPU
//    by other routes -- another process, another library's stream -- is not
//    covered: such callers serialise their calls themselves.
//  * The first call on a device looks up the device address of the array
//    (cudaGetSymbolAddress).  Make that first call before starting any stream
//    capture.
#include "ktc_internal.hpp"

namespace ktc {

constexpr int kNoallocMaxPartials = KTC_NOALLOC_SCRATCH_BYTES / (int)sizeof(double);   // 2048
constexpr int kNoallocThreads = 256;

// The array itself.  In host code this name is only a stand-in for the symbol;
// the address a kernel can use comes from cudaGetSymbolAddress (see below).
static __device__ __align__(256) double g_noalloc_partials[kNoallocMaxPartials];

// float run of at most 32 values, folded into a double: the accumulation scheme
// of the pooled reduction, so both entry points agree to the last bit on data
// whose sums are exact and to ~1 ulp of the float result otherwise.
struct RunSum {
    float run = 0.f; int cnt = 0; double acc = 0.0;
    __device__ __forceinline__ void add(float v) {
        run = __fadd_rn(run, v);
        if (++cnt == 32) { acc += (double)run; run = 0.f; cnt = 0; }
    }
    __device__ __forceinline__ double total() { return acc + (double)run; }
};

__device__ __forceinline__ double block_sum(double v, double* sm) {
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = (lane < (int)(blockDim.x >> 5)) ? sm[lane] : 0.0;
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    return v;
}

// pass 1: CTA b sums elements [b*seg, min(n, (b+1)*seg)) and stores one double
__global__ void __launch_bounds__(kNoallocThreads) k_noalloc_partial(const float* __restrict__ in, int64_t n, int64_t seg,
                                                                     double* __restrict__ partials, int vec_ok) {
    __shared__ double sm[32];
    const int64_t j0 = (int64_t)blockIdx.x * seg;
    const int64_t j1 = min(n, j0 + seg);
    RunSum s;
    if (vec_ok) {                                  // seg is a multiple of 4 and `in` is 16-byte aligned
        const float4* p4 = reinterpret_cast<const float4*>(in);
        const int64_t q0 = j0 >> 2, q1 = j1 >> 2;
        constexpr int U = 4;
        for (int64_t q = q0 + threadIdx.x; q < q1; q += (int64_t)blockDim.x * U) {
            float4 v[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) { const int64_t k = q + (int64_t)u * blockDim.x; if (k < q1) v[u] = __ldcs(p4 + k); }
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t k = q + (int64_t)u * blockDim.x;
                if (k < q1) { s.add(v[u].x); s.add(v[u].y); s.add(v[u].z); s.add(v[u].w); }
            }
        }
        for (int64_t j = (q1 << 2) + threadIdx.x; j < j1; j += blockDim.x) s.add(in[j]);   // < 4 trailing floats of the last CTA
    } else {
        for (int64_t j = j0 + threadIdx.x; j < j1; j += blockDim.x) s.add(in[j]);
    }
    const double total = block_sum(s.total(), sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = total;
}

// pass 2: one CTA adds the partials in slot order and writes the float result
__global__ void __launch_bounds__(kNoallocThreads) k_noalloc_final(const double* __restrict__ partials, int n_partials,
                                                                   float* __restrict__ out, int is_mean, double count) {
    __shared__ double sm[32];
    double v = 0.0;
    for (int i = threadIdx.x; i < n_partials; i += blockDim.x) v += partials[i];
    v = block_sum(v, sm);
    if (threadIdx.x == 0) out[0] = (float)(is_mean ? v / count : v);      // mean of nothing is NaN, as in ktc_reduce_all
}

// device address of the scratch array, looked up once per device
static std::mutex g_sym_mu;
static std::mutex g_call_mu[64];           // held across the two launches of a call
static double* g_sym_ptr[64] = {nullptr};

static int scratch_for(Device* d, double** out) {
    if (d->id < 0 || d->id >= 64) return fail(KTC_ENOTSUP, "ktc_reduce_all_noalloc: device index %d is beyond the 64 supported", d->id);
    std::lock_guard<std::mutex> lk(g_sym_mu);
    if (!g_sym_ptr[d->id]) {
        double* p = nullptr;
        KTC_CUDA(cudaSetDevice(d->id));                                    // the lookup is per device
        KTC_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_partials));
        if (!p) return fail(KTC_ECUDA, "ktc_reduce_all_noalloc: no device address for the scratch array");
        g_sym_ptr[d->id] = p;
    }
    *out = g_sym_ptr[d->id];
    return KTC_OK;
}

}  // namespace ktc

using namespace ktc;

extern "C" int ktc_reduce_all_noalloc(int op, ktc_buf out, ktc_buf in, int64_t n) {
    if (op != KTC_SUM && op != KTC_MEAN) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: op must be KTC_SUM or KTC_MEAN");
    if (n < 0) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: negative element count");
    if (n > KTC_NOALLOC_MAX_ELEMS)
        return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: %lld elements exceed the limit of %lld this entry point is built for; "
                                "use ktc_reduce_all", (long long)n, (long long)KTC_NOALLOC_MAX_ELEMS);
    Buf bo, bi;
    KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(in, &bi));
    if (bo.dev != bi.dev) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: buffers live on devices %d and %d", bo.dev, bi.dev);
    if (bi.n < n) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: in holds %lld floats, %lld needed", (long long)bi.n, (long long)n);
    if (bo.n < 1) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: out holds no float");
    if (bo.ptr >= bi.ptr && bo.ptr < bi.ptr + n) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: out lies inside the elements of in that are read");
    Device* d = device(bi.dev); if (!d) return KTC_ESTATE;
    if (!d->ready) return fail(KTC_ESTATE, "ktc_reduce_all_noalloc: device %d has no compute stream yet", d->id);
    KTC_CUDA(cudaSetDevice(d->id));
    double* partials = nullptr;
    KTC_TRY(scratch_for(d, &partials));

    // segment length: a multiple of 4, at least 8192 floats, at most kNoallocMaxPartials segments
    int64_t want = (int64_t)d->sm_count * 8;
    if (want > kNoallocMaxPartials) want = kNoallocMaxPartials;
    int64_t seg = (n + want - 1) / (want > 0 ? want : 1);
    if (seg < 8192) seg = 8192;
    seg = (seg + 3) & ~(int64_t)3;
    int64_t blocks = (n + seg - 1) / seg;
    if (blocks < 1) blocks = 1;
    if (blocks > kNoallocMaxPartials) return fail(KTC_EINVAL, "ktc_reduce_all_noalloc: internal segment count exceeds the scratch array");
    const int vec_ok = aligned16(bi.ptr) ? 1 : 0;
    std::lock_guard<std::mutex> pair_lock(g_call_mu[d->id]);           // the two launches enter the stream back to back
    k_noalloc_partial<<<(int)blocks, kNoallocThreads, 0, d->stream>>>(bi.ptr, n, seg, partials, vec_ok);
    k_noalloc_final<<<1, kNoallocThreads, 0, d->stream>>>(partials, (int)blocks, bo.ptr, op == KTC_MEAN ? 1 : 0, (double)n);
    count_launch(2);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KTC_ECUDA, "ktc_reduce_all_noalloc: launch failed: %s", cudaGetErrorString(e));
    return KTC_OK;
}
