// ktc_api.cu -- extern "C" compute entry points: argument validation, the host
// side shape algebra (broadcast strides, [outer, axis, inner] collapse,
// sum-to-shape planning) and dispatch to the kernel launchers.
//
// Shape rules restate kten-api's host code:
//   right-aligned broadcast, mismatch is an error   ShapeFunctions.kt:168-201
//   row-major strides                                AbstractIndexing.kt:107-109
//   sum-to-shape = mayUnexpand                       autograd/functions/Utils.kt:14-41
#include "ktc_internal.hpp"

#include <algorithm>

using namespace ktc;

namespace {

struct Args {
    Device* d = nullptr;
    int dev = -1;
    int take(const Buf& b, const char* who) {
        if (dev < 0) { dev = b.dev; d = device(b.dev); if (!d) return KTC_ESTATE; return use_device(d); }
        if (b.dev != dev) return fail(KTC_EINVAL, "%s: operands live on different devices (%d and %d)", who, dev, b.dev);
        return KTC_OK;
    }
};

int need(const Buf& b, int64_t n, const char* who, const char* what) {
    if (n < 0) return fail(KTC_EINVAL, "%s: negative element count", who);
    if (b.n < n) return fail(KTC_EINVAL, "%s: %s holds %lld floats, %lld needed", who, what, (long long)b.n, (long long)n);
    return KTC_OK;
}

int check_shape(const int64_t* s, int n, const char* who, int64_t* volume) {
    if (n < 0 || n > KTC_MAX_DIMS) return fail(KTC_EINVAL, "%s: %d dimensions (at most %d supported)", who, n, KTC_MAX_DIMS);
    if (n > 0 && !s) return fail(KTC_EINVAL, "%s: shape is null", who);
    int64_t v = 1;
    for (int i = 0; i < n; ++i) {
        if (s[i] < 0) return fail(KTC_EINVAL, "%s: negative extent", who);
        v *= s[i];
        if (v > ((int64_t)1 << 40)) return fail(KTC_EINVAL, "%s: tensor too large", who);
    }
    *volume = v;
    return KTC_OK;
}

// element strides of `shape` seen through the right-aligned common shape `cs`
// (0 where the operand is broadcast)
void bcast_strides(const int64_t* shape, int n, const int64_t* cs, int cn, int64_t* out) {
    int64_t st = 1;
    for (int i = cn - 1; i >= 0; --i) {
        const int is = i - (cn - n);
        const int64_t ext = is >= 0 ? shape[is] : 1;
        out[i] = (ext == cs[i]) ? st : 0;
        st *= ext;
    }
}

}  // namespace

extern "C" {

int ktc_binary(int op, ktc_buf out, ktc_buf a, ktc_buf b, int64_t n) {
    Buf bo, ba, bb; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba)); KTC_TRY(resolve(b, &bb));
    Args g; KTC_TRY(g.take(bo, "ktc_binary")); KTC_TRY(g.take(ba, "ktc_binary")); KTC_TRY(g.take(bb, "ktc_binary"));
    KTC_TRY(need(bo, n, "ktc_binary", "out")); KTC_TRY(need(ba, n, "ktc_binary", "a")); KTC_TRY(need(bb, n, "ktc_binary", "b"));
    return launch_map2(g.d, op, bo.ptr, ba.ptr, bb.ptr, n);
}

int ktc_binary_inplace(int op, ktc_buf a, ktc_buf b, int64_t n) {
    // the JVM backend rejects unequal shapes for in-place ops (JVMRawTensor.kt:89-93);
    // the caller compares shapes, this call only sees the common element count
    return ktc_binary(op, a, a, b, n);
}

int ktc_binary_bcast(int op, ktc_buf out, ktc_buf a, const int64_t* a_shape, int a_ndim,
                     ktc_buf b, const int64_t* b_shape, int b_ndim) {
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_binary_bcast: unknown op %d", op);
    Buf bo, ba, bb; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba)); KTC_TRY(resolve(b, &bb));
    Args g; KTC_TRY(g.take(bo, "ktc_binary_bcast")); KTC_TRY(g.take(ba, "ktc_binary_bcast")); KTC_TRY(g.take(bb, "ktc_binary_bcast"));
    int64_t va, vb;
    KTC_TRY(check_shape(a_shape, a_ndim, "ktc_binary_bcast(a)", &va));
    KTC_TRY(check_shape(b_shape, b_ndim, "ktc_binary_bcast(b)", &vb));
    const int cn = std::max(a_ndim, b_ndim);
    int64_t cs[KTC_MAX_DIMS], as[KTC_MAX_DIMS], bs[KTC_MAX_DIMS];
    int64_t vol = 1;
    for (int i = 0; i < cn; ++i) {
        const int ia = i - (cn - a_ndim), ib = i - (cn - b_ndim);
        const int64_t da = ia >= 0 ? a_shape[ia] : 1, db = ib >= 0 ? b_shape[ib] : 1;
        if (!(da == db || da == 1 || db == 1))
            return fail(KTC_EINVAL, "Shapes must match for every non-singleton dimension (missing dimensions count as singleton "
                                    "dimensions at the beginning of the shapes): extent %lld vs %lld at aligned dimension %d",
                        (long long)da, (long long)db, i);
        cs[i] = std::max(da, db);
        vol *= cs[i];
    }
    KTC_TRY(need(ba, va, "ktc_binary_bcast", "a")); KTC_TRY(need(bb, vb, "ktc_binary_bcast", "b"));
    KTC_TRY(need(bo, vol, "ktc_binary_bcast", "out"));
    if (vol == 0) return KTC_OK;
    bcast_strides(a_shape, a_ndim, cs, cn, as);
    bcast_strides(b_shape, b_ndim, cs, cn, bs);
    return launch_bcast(g.d, op, bo.ptr, cs, cn, ba.ptr, as, bb.ptr, bs);
}

int ktc_broadcast_to(ktc_buf out, const int64_t* out_shape, int out_ndim, ktc_buf a, const int64_t* a_shape, int a_ndim) {
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_broadcast_to")); KTC_TRY(g.take(ba, "ktc_broadcast_to"));
    int64_t vo, va;
    KTC_TRY(check_shape(out_shape, out_ndim, "ktc_broadcast_to(out)", &vo));
    KTC_TRY(check_shape(a_shape, a_ndim, "ktc_broadcast_to(a)", &va));
    if (a_ndim > out_ndim)
        return fail(KTC_EINVAL, "Tensor with %d dimensions cannot be broadcasted to a shape with %d dimensions", a_ndim, out_ndim);
    for (int i = 0; i < a_ndim; ++i) {
        const int64_t da = a_shape[i], dt = out_shape[out_ndim - a_ndim + i];
        if (!(da == dt || da == 1))
            return fail(KTC_EINVAL, "Shape must match the target for every non-singleton dimension: extent %lld vs %lld", (long long)da, (long long)dt);
    }
    KTC_TRY(need(ba, va, "ktc_broadcast_to", "a")); KTC_TRY(need(bo, vo, "ktc_broadcast_to", "out"));
    if (vo == 0) return KTC_OK;
    int64_t as[KTC_MAX_DIMS];
    bcast_strides(a_shape, a_ndim, out_shape, out_ndim, as);
    return launch_bcast(g.d, -1, bo.ptr, out_shape, out_ndim, nullptr, nullptr, ba.ptr, as);
}

int ktc_scalar(int op, ktc_buf out, ktc_buf a, float s, int64_t n, int scalar_first) {
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_scalar: unknown op %d", op);
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_scalar")); KTC_TRY(g.take(ba, "ktc_scalar"));
    KTC_TRY(need(bo, n, "ktc_scalar", "out")); KTC_TRY(need(ba, n, "ktc_scalar", "a"));
    return launch_map1(g.d, scalar_first ? M1_SCALAR_L : M1_SCALAR_R, op, bo.ptr, ba.ptr, n, s, 0.f);
}

int ktc_scalar_inplace(int op, ktc_buf a, float s, int64_t n) { return ktc_scalar(op, a, a, s, n, 0); }

int ktc_unary(int op, ktc_buf out, ktc_buf a, int64_t n) {
    if (op < KTC_EXP || op > KTC_RSQRT) return fail(KTC_EINVAL, "ktc_unary: unknown op %d", op);
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_unary")); KTC_TRY(g.take(ba, "ktc_unary"));
    KTC_TRY(need(bo, n, "ktc_unary", "out")); KTC_TRY(need(ba, n, "ktc_unary", "a"));
    if (op > KTC_NEG) return launch_map1_more(g.d, op, bo.ptr, ba.ptr, n);
    return launch_map1(g.d, M1_UNARY, op, bo.ptr, ba.ptr, n, 0.f, 0.f);
}

int ktc_compare_scalar_eps(int op, ktc_buf out, ktc_buf a, float value, float epsilon, int64_t n) {
    if (op >= KTC_LT && op <= KTC_GTE) return ktc_compare_scalar(op, out, a, value, n);
    if (op != KTC_EQ && op != KTC_NEQ) return fail(KTC_EINVAL, "ktc_compare_scalar_eps: unknown op %d", op);
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_compare_scalar_eps")); KTC_TRY(g.take(ba, "ktc_compare_scalar_eps"));
    KTC_TRY(need(bo, n, "ktc_compare_scalar_eps", "out")); KTC_TRY(need(ba, n, "ktc_compare_scalar_eps", "a"));
    return launch_eq_scalar(g.d, op, bo.ptr, ba.ptr, n, value, epsilon);
}

int ktc_compare_tensor(int op, ktc_buf out, ktc_buf a, ktc_buf b, float epsilon, int64_t n) {
    if (op < KTC_LT || op > KTC_NEQ) return fail(KTC_EINVAL, "ktc_compare_tensor: unknown op %d", op);
    Buf bo, ba, bb; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba)); KTC_TRY(resolve(b, &bb));
    Args g; KTC_TRY(g.take(bo, "ktc_compare_tensor")); KTC_TRY(g.take(ba, "ktc_compare_tensor")); KTC_TRY(g.take(bb, "ktc_compare_tensor"));
    KTC_TRY(need(bo, n, "ktc_compare_tensor", "out")); KTC_TRY(need(ba, n, "ktc_compare_tensor", "a")); KTC_TRY(need(bb, n, "ktc_compare_tensor", "b"));
    return launch_compare_tensor(g.d, op, bo.ptr, ba.ptr, bb.ptr, n, epsilon);
}

int ktc_masked_fill(ktc_buf out, ktc_buf a, const int64_t* a_shape, int a_ndim,
                    ktc_buf mask, const int64_t* mask_shape, int mask_ndim, float value) {
    Buf bo, ba, bm; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba)); KTC_TRY(resolve(mask, &bm));
    Args g; KTC_TRY(g.take(bo, "ktc_masked_fill")); KTC_TRY(g.take(ba, "ktc_masked_fill")); KTC_TRY(g.take(bm, "ktc_masked_fill"));
    int64_t va, vm;
    KTC_TRY(check_shape(a_shape, a_ndim, "ktc_masked_fill(a)", &va));
    KTC_TRY(check_shape(mask_shape, mask_ndim, "ktc_masked_fill(mask)", &vm));
    if (mask_ndim > a_ndim)
        return fail(KTC_EINVAL, "Tensor with %d dimensions cannot be broadcasted to a shape with %d dimensions", mask_ndim, a_ndim);
    for (int i = 0; i < mask_ndim; ++i) {
        const int64_t dm = mask_shape[i], dt = a_shape[a_ndim - mask_ndim + i];
        if (!(dm == dt || dm == 1))
            return fail(KTC_EINVAL, "Shape must match the target for every non-singleton dimension: extent %lld vs %lld", (long long)dm, (long long)dt);
    }
    KTC_TRY(need(ba, va, "ktc_masked_fill", "a")); KTC_TRY(need(bm, vm, "ktc_masked_fill", "mask")); KTC_TRY(need(bo, va, "ktc_masked_fill", "out"));
    if (va == 0) return KTC_OK;
    int64_t as[KTC_MAX_DIMS], ms[KTC_MAX_DIMS];
    bcast_strides(a_shape, a_ndim, a_shape, a_ndim, as);
    bcast_strides(mask_shape, mask_ndim, a_shape, a_ndim, ms);
    return launch_bcast(g.d, kBcastMaskedFill, bo.ptr, a_shape, a_ndim, ba.ptr, as, bm.ptr, ms, value);
}

int ktc_contains_nan(ktc_buf a, int64_t n, int* result) {
    if (!result) return fail(KTC_EINVAL, "ktc_contains_nan: null result");
    Buf ba; KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(ba, "ktc_contains_nan"));
    KTC_TRY(need(ba, n, "ktc_contains_nan", "a"));
    return launch_contains_nan(g.d, ba.ptr, n, result);
}

int ktc_clamp(ktc_buf out, ktc_buf a, float lo, float hi, int64_t n) {
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_clamp")); KTC_TRY(g.take(ba, "ktc_clamp"));
    KTC_TRY(need(bo, n, "ktc_clamp", "out")); KTC_TRY(need(ba, n, "ktc_clamp", "a"));
    return launch_map1(g.d, M1_CLAMP, 0, bo.ptr, ba.ptr, n, lo, hi);
}

int ktc_compare_scalar(int op, ktc_buf out, ktc_buf a, float value, int64_t n) {
    if (op < KTC_LT || op > KTC_GTE) return fail(KTC_EINVAL, "ktc_compare_scalar: unknown op %d", op);
    Buf bo, ba; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(a, &ba));
    Args g; KTC_TRY(g.take(bo, "ktc_compare_scalar")); KTC_TRY(g.take(ba, "ktc_compare_scalar"));
    KTC_TRY(need(bo, n, "ktc_compare_scalar", "out")); KTC_TRY(need(ba, n, "ktc_compare_scalar", "a"));
    return launch_map1(g.d, M1_COMPARE, op, bo.ptr, ba.ptr, n, value, 0.f);
}

static int check_oai(int64_t outer, int64_t A, int64_t inner, const char* who) {
    if (outer < 0 || A < 0 || inner < 0) return fail(KTC_EINVAL, "%s: negative extent", who);
    if (outer > ((int64_t)1 << 40) || A > ((int64_t)1 << 40) || inner > ((int64_t)1 << 40)) return fail(KTC_EINVAL, "%s: extent too large", who);
    return KTC_OK;
}

int ktc_reduce_axis(int op, ktc_buf out, ktc_buf in, int64_t outer, int64_t axis_len, int64_t inner) {
    if (op < KTC_SUM || op > KTC_ARGMIN) return fail(KTC_EINVAL, "ktc_reduce_axis: unknown op %d", op);
    KTC_TRY(check_oai(outer, axis_len, inner, "ktc_reduce_axis"));
    Buf bo, bi; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(in, &bi));
    Args g; KTC_TRY(g.take(bo, "ktc_reduce_axis")); KTC_TRY(g.take(bi, "ktc_reduce_axis"));
    KTC_TRY(need(bi, outer * axis_len * inner, "ktc_reduce_axis", "in")); KTC_TRY(need(bo, outer * inner, "ktc_reduce_axis", "out"));
    if (bo.ptr == bi.ptr && outer * inner > 0) return fail(KTC_EINVAL, "ktc_reduce_axis: out aliases in");
    return launch_reduce_axis(g.d, op, bo.ptr, nullptr, bi.ptr, outer, axis_len, inner);
}

int ktc_reduce_axis_validx(int is_max, ktc_buf out_val, ktc_buf out_idx, ktc_buf in, int64_t outer, int64_t axis_len, int64_t inner) {
    KTC_TRY(check_oai(outer, axis_len, inner, "ktc_reduce_axis_validx"));
    Buf bv, bx, bi; KTC_TRY(resolve(out_val, &bv)); KTC_TRY(resolve(out_idx, &bx)); KTC_TRY(resolve(in, &bi));
    Args g; KTC_TRY(g.take(bv, "ktc_reduce_axis_validx")); KTC_TRY(g.take(bx, "ktc_reduce_axis_validx")); KTC_TRY(g.take(bi, "ktc_reduce_axis_validx"));
    KTC_TRY(need(bi, outer * axis_len * inner, "ktc_reduce_axis_validx", "in"));
    KTC_TRY(need(bv, outer * inner, "ktc_reduce_axis_validx", "out_val")); KTC_TRY(need(bx, outer * inner, "ktc_reduce_axis_validx", "out_idx"));
    if (outer * inner > 0 && (bv.ptr == bi.ptr || bx.ptr == bi.ptr || bv.ptr == bx.ptr)) return fail(KTC_EINVAL, "ktc_reduce_axis_validx: buffers alias");
    return launch_reduce_axis(g.d, is_max ? 100 : 101, bv.ptr, bx.ptr, bi.ptr, outer, axis_len, inner);
}

int ktc_reduce_all(int op, ktc_buf out, ktc_buf in, int64_t n) {
    if (op != KTC_SUM && op != KTC_MEAN) return fail(KTC_EINVAL, "ktc_reduce_all: op must be KTC_SUM or KTC_MEAN");
    return ktc_reduce_axis(op, out, in, 1, n, 1);
}

int ktc_sum_to_shape(ktc_buf out, const int64_t* old_shape, int old_ndim, ktc_buf in, const int64_t* in_shape, int in_ndim) {
    Buf bo, bi; KTC_TRY(resolve(out, &bo)); KTC_TRY(resolve(in, &bi));
    Args g; KTC_TRY(g.take(bo, "ktc_sum_to_shape")); KTC_TRY(g.take(bi, "ktc_sum_to_shape"));
    int64_t vo, vi;
    KTC_TRY(check_shape(old_shape, old_ndim, "ktc_sum_to_shape(old)", &vo));
    KTC_TRY(check_shape(in_shape, in_ndim, "ktc_sum_to_shape(in)", &vi));
    if (old_ndim > in_ndim) return fail(KTC_EINVAL, "ktc_sum_to_shape: target has more dimensions than the input");
    const int lead = in_ndim - old_ndim;
    for (int i = 0; i < old_ndim; ++i)
        if (!(old_shape[i] == in_shape[lead + i] || old_shape[i] == 1))
            return fail(KTC_EINVAL, "ktc_sum_to_shape: extent %lld cannot be reduced to %lld", (long long)in_shape[lead + i], (long long)old_shape[i]);
    KTC_TRY(need(bi, vi, "ktc_sum_to_shape", "in")); KTC_TRY(need(bo, vo, "ktc_sum_to_shape", "out"));
    if (vo == 0) return KTC_OK;
    if (bo.ptr == bi.ptr) return fail(KTC_EINVAL, "ktc_sum_to_shape: out aliases in");

    // collapse to alternating kept / reduced groups
    struct Grp { int64_t ext; bool red; };
    std::vector<Grp> grp;
    for (int i = 0; i < in_ndim; ++i) {
        const int64_t ext = in_shape[i];
        if (ext == 1) continue;
        const bool red = (i < lead) || (old_shape[i - lead] == 1);
        if (!grp.empty() && grp.back().red == red) grp.back().ext *= ext; else grp.push_back({ext, red});
    }
    bool any_red = false;
    for (auto& q : grp) any_red |= q.red;
    if (!any_red) {            // nothing to sum: plain copy
        KTC_CUDA(cudaMemcpyAsync(bo.ptr, bi.ptr, (size_t)vo * 4, cudaMemcpyDeviceToDevice, g.d->stream));
        return KTC_OK;
    }
    // one axis reduction per reduced group, largest extent first; intermediates come from the pool
    const float* cur = bi.ptr;
    Scratch tmp[2]; int flip = 0;
    while (true) {
        int best = -1;
        for (int i = 0; i < (int)grp.size(); ++i) if (grp[i].red && (best < 0 || grp[i].ext > grp[best].ext)) best = i;
        if (best < 0) break;
        int64_t outer = 1, inner = 1;
        for (int i = 0; i < best; ++i) outer *= grp[i].ext;
        for (int i = best + 1; i < (int)grp.size(); ++i) inner *= grp[i].ext;
        int n_red = 0; for (auto& q : grp) n_red += q.red ? 1 : 0;
        float* dst;
        if (n_red == 1) dst = bo.ptr;
        else {
            Scratch& s = tmp[flip];
            if (s.ptr) { pool_free(s.d, s.ptr, s.rounded); s.ptr = nullptr; }
            KTC_TRY(s.get(g.d, outer * inner));
            dst = s.ptr; flip ^= 1;
        }
        KTC_TRY(launch_reduce_axis(g.d, KTC_SUM, dst, nullptr, cur, outer, grp[best].ext, inner));
        cur = dst;
        grp.erase(grp.begin() + best);
        // merge the now adjacent kept groups
        for (int i = 0; i + 1 < (int)grp.size();)
            if (grp[i].red == grp[i + 1].red) { grp[i].ext *= grp[i + 1].ext; grp.erase(grp.begin() + i + 1); } else ++i;
    }
    return KTC_OK;
}

int ktc_scatter_axis(ktc_buf target, ktc_buf index, ktc_buf src, int64_t outer, int64_t axis_len, int64_t inner) {
    KTC_TRY(check_oai(outer, axis_len, inner, "ktc_scatter_axis"));
    Buf bt, bx, bs; KTC_TRY(resolve(target, &bt)); KTC_TRY(resolve(index, &bx)); KTC_TRY(resolve(src, &bs));
    Args g; KTC_TRY(g.take(bt, "ktc_scatter_axis")); KTC_TRY(g.take(bx, "ktc_scatter_axis")); KTC_TRY(g.take(bs, "ktc_scatter_axis"));
    KTC_TRY(need(bt, outer * axis_len * inner, "ktc_scatter_axis", "target"));
    KTC_TRY(need(bx, outer * inner, "ktc_scatter_axis", "index")); KTC_TRY(need(bs, outer * inner, "ktc_scatter_axis", "src"));
    return launch_scatter_axis(g.d, bt.ptr, bx.ptr, bs.ptr, outer, axis_len, inner);
}

}  // extern "C"
