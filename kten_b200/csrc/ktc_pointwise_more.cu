// ktc_pointwise_more.cu -- the unary maps, compares and NaN test of the raw-tensor SPI that are
// not on the benchmarked sweep (JVMRawTensor.kt:355-393, 401-435, 520-522).  Same streaming map
// kernels as the sweep's ops (ktc_map.cuh); only the per-element functors differ.
#include "ktc_map.cuh"
#include "ktc_math_more.cuh"

namespace ktc {

int launch_map1_more(Device* d, int op, float* out, const float* a, int64_t n) {
    switch (op) {
    case KTC_SINH:  return run_map1(d, out, a, n, UnOp<KTC_SINH>());
    case KTC_COSH:  return run_map1(d, out, a, n, UnOp<KTC_COSH>());
    case KTC_ABS:   return run_map1(d, out, a, n, UnOp<KTC_ABS>());
    case KTC_SIGN:  return run_map1(d, out, a, n, UnOp<KTC_SIGN>());
    case KTC_SQRT:  return run_map1(d, out, a, n, UnOp<KTC_SQRT>());
    case KTC_SIN:   return run_map1(d, out, a, n, UnOp<KTC_SIN>());
    case KTC_COS:   return run_map1(d, out, a, n, UnOp<KTC_COS>());
    case KTC_TAN:   return run_map1(d, out, a, n, UnOp<KTC_TAN>());
    case KTC_ASIN:  return run_map1(d, out, a, n, UnOp<KTC_ASIN>());
    case KTC_ACOS:  return run_map1(d, out, a, n, UnOp<KTC_ACOS>());
    case KTC_ATAN:  return run_map1(d, out, a, n, UnOp<KTC_ATAN>());
    case KTC_FLOOR: return run_map1(d, out, a, n, UnOp<KTC_FLOOR>());
    case KTC_CEIL:  return run_map1(d, out, a, n, UnOp<KTC_CEIL>());
    case KTC_ROUND: return run_map1(d, out, a, n, UnOp<KTC_ROUND>());
    case KTC_TRUNC: return run_map1(d, out, a, n, UnOp<KTC_TRUNC>());
    case KTC_RSQRT: return run_map1(d, out, a, n, UnOp<KTC_RSQRT>());
    }
    return fail(KTC_EINVAL, "unknown unary op %d", op);
}

int launch_eq_scalar(Device* d, int op, float* out, const float* a, int64_t n, float value, float eps) {
    if (op == KTC_EQ) return run_map1(d, out, a, n, EqScalar<false>{value, eps});
    if (op == KTC_NEQ) return run_map1(d, out, a, n, EqScalar<true>{value, eps});
    return fail(KTC_EINVAL, "unknown compare op %d", op);
}

int launch_compare_tensor(Device* d, int op, float* out, const float* a, const float* b, int64_t n, float eps) {
    switch (op) {
    case KTC_LT:  return run_map2(d, out, a, b, n, CompareT<KTC_LT>{eps});
    case KTC_LTE: return run_map2(d, out, a, b, n, CompareT<KTC_LTE>{eps});
    case KTC_GT:  return run_map2(d, out, a, b, n, CompareT<KTC_GT>{eps});
    case KTC_GTE: return run_map2(d, out, a, b, n, CompareT<KTC_GTE>{eps});
    case KTC_EQ:  return run_map2(d, out, a, b, n, CompareT<KTC_EQ>{eps});
    case KTC_NEQ: return run_map2(d, out, a, b, n, CompareT<KTC_NEQ>{eps});
    }
    return fail(KTC_EINVAL, "unknown compare op %d", op);
}

// any NaN in a[0, n): every thread looks at its elements and writes 1 to the flag if it saw one
// (all writers store the same value).  The host reads the flag back and clears it.
__global__ void __launch_bounds__(256) k_any_nan(const float* __restrict__ a, int64_t n, int* flag) {
    bool seen = false;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = a[i];
        seen |= (v != v);
    }
    if (seen) *flag = 1;
}

int launch_contains_nan(Device* d, const float* a, int64_t n, int* result) {
    int h = 0;
    if (n > 0) {
        k_any_nan<<<grid_for(d, n, 256 * 8, 16), 256, 0, d->stream>>>(a, n, d->err_flag);
        KTC_TRY(finish_launch("any_nan"));
        KTC_CUDA(cudaMemcpyAsync(&h, d->err_flag, sizeof(int), cudaMemcpyDeviceToHost, d->stream));
        KTC_CUDA(cudaMemsetAsync(d->err_flag, 0, sizeof(int), d->stream));
        KTC_CUDA(cudaStreamSynchronize(d->stream));
    }
    *result = h != 0;
    return KTC_OK;
}

}  // namespace ktc
