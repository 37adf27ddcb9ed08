// kten_host.cpp -- a compiled host above the C ABI: the raw tensor and the caller of the sharded step.
//
// kten's host side is compiled code (Kotlin on a JVM); the Python mirror of it in this package costs
// about 0.2 ms per training step in interpreter time alone, which hides what the library below the C ABI
// can do once a step shrinks to tens of microseconds per GPU.  This file restates, in C++, the two host
// pieces a step of the sharded benchmark graph goes through, so that the per-step host cost can be
// measured as a JVM host would see it:
//
//   * Raw      -- the backend's RawTensor (backend/kten-cuda/.../store/CUDARawTensor.kt of this repo,
//                 AbstractRawTensor.kt:5-248): shape on the host, a reference-counted buffer handle or a
//                 cell of the expression recorder (ktc_lazy_*), one C-ABI call per method.  Only the
//                 methods the graph needs are here.
//   * the caller -- kten-api's define-by-run autograd for the nodes of
//                 loss = sum(sigmoid(x*w + b) pow 2): Function with its lazy forward, ref-counted outputs,
//                 saved values, fan-in cache and release walk (functions/Function.kt:8-215), Plus and Times
//                 with mayUnexpand (BasicFunctions.kt:7-55, Utils.kt:14-41), PowConstant
//                 (BasicFunctions.kt:182-204), Sigmoid (PointwiseFunctions.kt:66-81), Sum
//                 (AggregatingFunctions.kt:7-25), Variable.backwardWithGrad (Variable.kt:44-46), and the scoped
//                 garbage collector of the operations object (OCLTensorOperations.kt:72-94).
// The call sequence is the one kten_b200/autograd.py issues (checked against the reference's test vectors);
// a GPU test compares the two hosts bit for bit.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/kten_cuda.h"

namespace kten {

using Shape = std::vector<int64_t>;

static void check(int status) {
    if (status != KTC_OK) throw std::runtime_error(std::string("[") + std::to_string(status) + "] " + ktc_last_error());
}
static int64_t volume(const Shape& s) { int64_t v = 1; for (int64_t d : s) v *= d; return v; }

static Shape common_shape(const Shape& a, const Shape& b) {
    const size_t nd = std::max(a.size(), b.size());
    Shape out(nd);
    for (size_t i = 0; i < nd; ++i) {
        const int64_t da = i + a.size() >= nd ? a[i + a.size() - nd] : 1, db = i + b.size() >= nd ? b[i + b.size() - nd] : 1;
        if (da != db && da != 1 && db != 1) throw std::invalid_argument("shapes do not broadcast");
        out[i] = da == 1 ? db : da;
    }
    return out;
}

class Raw;
using RawP = std::shared_ptr<Raw>;

// The operations object: device, deferred mode, and the scoped collector that releases every raw tensor created
// while a scope is open (nested scopes are no-ops, OCLTensorOperations.kt:73-74).
struct Ops {
    int device = 0;
    bool lazy = false;
    bool defer_sums = true;
    std::vector<RawP>* collector = nullptr;
    std::vector<ktc_buf> pending_targets;      // buffers with a recorded `+= pending sum` update (may hold stale entries)

    bool is_pending_target(ktc_buf h) const { for (ktc_buf t : pending_targets) if (t == h) return true; return false; }
    void run_pending() { pending_targets.clear(); check(ktc_lazy_run_pending()); }
    RawP create(const Shape& shape);
    RawP create_fill(const Shape& shape, float v);
};

struct Scope {
    Ops& ops; std::vector<RawP> mine; bool owner;
    explicit Scope(Ops& o) : ops(o), owner(o.collector == nullptr) { if (owner) ops.collector = &mine; }
    ~Scope();
};

// storage slot: a buffer (one owned reference), a recorder cell, or both; shared by shallow copies of a pending tensor
struct Cell {
    ktc_buf store = 0;
    ktc_lazy_cell lz = 0;
    Shape lz_shape;
    ~Cell() { if (lz) ktc_lazy_free(lz); if (store) ktc_release(store); }
};

class Raw : public std::enable_shared_from_this<Raw> {
public:
    Shape shape;
    std::shared_ptr<Cell> cell;
    Ops* ops;
    int refCount = 1;
    bool mustSurviveGC = false, released = false;

    static RawP make(Ops* ops, const Shape& shape, std::shared_ptr<Cell> cell) {
        RawP r(new Raw());
        r->shape = shape; r->cell = std::move(cell); r->ops = ops;
        if (ops->collector) ops->collector->push_back(r);
        return r;
    }
    static RawP recorded(Ops* ops, const Shape& shape, ktc_lazy_cell lz) {
        auto c = std::make_shared<Cell>();
        c->lz = lz; c->lz_shape = shape;
        return make(ops, shape, c);
    }
    int64_t size() const { return volume(shape); }
    void incrementRef() { ++refCount; }
    bool release() {                                           // OCLRawTensor.release (OCLRawTensor.kt:37-48)
        if (released) return false;
        if (!mustSurviveGC) --refCount;
        if (refCount <= 0) { cell.reset(); released = true; return true; }
        return false;
    }
    ktc_buf buf() {                                            // the buffer handle; a pending value is computed first
        if (released) throw std::runtime_error("Raw tensor already released");
        Cell& c = *cell;
        if (!c.store) check(ktc_lazy_buffer(c.lz, &c.store));
        else if (!ops->pending_targets.empty() && ops->is_pending_target(c.store)) ops->run_pending();
        return c.store;
    }
    ktc_lazy_cell lz(bool apply_updates = true) {              // this tensor as an operand of a recorded call
        if (released) throw std::runtime_error("Raw tensor already released");
        Cell& c = *cell;
        if (!c.store) return c.lz;
        if (apply_updates && !ops->pending_targets.empty() && ops->is_pending_target(c.store)) ops->run_pending();
        if (!c.lz || c.lz_shape != shape) {
            if (c.lz) ktc_lazy_free(c.lz);
            check(ktc_lazy_leaf(c.store, shape.data(), (int)shape.size(), &c.lz));
            c.lz_shape = shape;
        }
        return c.lz;
    }
    bool isDeferred() const {
        if (cell->store || !cell->lz) return false;
        int pending = 0;
        check(ktc_lazy_info(cell->lz, &pending, nullptr, nullptr, nullptr));
        return pending != 0;
    }
    void after_assign(int state) {
        Cell& c = *cell;
        if (state == 1) { if (c.store) { check(ktc_release(c.store)); c.store = 0; } }
        else if (state == 2) ops->pending_targets.push_back(c.store);
        // state 3: the recorder gave the pending cell a buffer that receives 0f + sum; nothing to do here
    }
    void before_inplace_write() { if (cell->store) check(ktc_lazy_flush(cell->store)); }

    // ---- elementwise (JVMRawTensor.kt:75-140) ----
    RawP binary(int op, const RawP& o) {
        const Shape common = shape == o->shape ? shape : common_shape(shape, o->shape);
        if (ops->lazy) { ktc_lazy_cell out; check(ktc_lazy_binary(op, lz(), o->lz(), &out)); return recorded(ops, common, out); }
        RawP res = ops->create(common);
        if (shape == o->shape) check(ktc_binary(op, res->buf(), buf(), o->buf(), size()));
        else check(ktc_binary_bcast(op, res->buf(), buf(), shape.data(), (int)shape.size(), o->buf(), o->shape.data(), (int)o->shape.size()));
        return res;
    }
    RawP scalar(int op, float s, bool scalar_first = false) {
        if (ops->lazy) { ktc_lazy_cell out; check(ktc_lazy_scalar(op, lz(), s, scalar_first ? 1 : 0, &out)); return recorded(ops, shape, out); }
        RawP res = ops->create(shape);
        check(ktc_scalar(op, res->buf(), buf(), s, size(), scalar_first ? 1 : 0));
        return res;
    }
    RawP unary(int op) {
        if (ops->lazy && op <= KTC_NEG) { ktc_lazy_cell out; check(ktc_lazy_unary(op, lz(), &out)); return recorded(ops, shape, out); }
        RawP res = ops->create(shape);
        check(ktc_unary(op, res->buf(), buf(), size()));
        return res;
    }
    void binaryAssign(int op, const RawP& o) {                  // inplaceElementwiseOpOnTensors (JVMRawTensor.kt:89-97)
        if (shape != o->shape) throw std::invalid_argument("Shapes does not match for inplace operation on tensors");
        if (ops->lazy) { int st = 0; check(ktc_lazy_assign_binary(op, lz(), o->lz(), &st)); after_assign(st); return; }
        before_inplace_write();
        check(ktc_binary_inplace(op, buf(), o->buf(), size()));
    }
    void scalarAssign(int op, float s) {
        if (ops->lazy) { int st = 0; check(ktc_lazy_assign_scalar(op, lz(), s, &st)); after_assign(st); return; }
        before_inplace_write();
        check(ktc_scalar_inplace(op, buf(), s, size()));
    }
    RawP plus(const RawP& o) { return binary(KTC_PLUS, o); }
    RawP times(const RawP& o) { return binary(KTC_TIMES, o); }
    RawP times(float s) { return scalar(KTC_TIMES, s); }
    RawP pow(float s) { return scalar(KTC_POW, s); }
    RawP sigmoid() { return unary(KTC_SIGMOID); }
    RawP unaryMinus() { return unary(KTC_NEG); }
    void plusAssign(const RawP& o) { binaryAssign(KTC_PLUS, o); }
    void plusAssign(float s) { scalarAssign(KTC_PLUS, s); }
    void timesAssign(const RawP& o) { binaryAssign(KTC_TIMES, o); }

    RawP broadcastTo(const Shape& target) {                    // JVMRawTensor.kt:51-73: the same shape returns this
        if (shape == target) return shared_from_this();
        if (ops->lazy) { ktc_lazy_cell out; check(ktc_lazy_broadcast_to(lz(), target.data(), (int)target.size(), &out)); return recorded(ops, target, out); }
        RawP res = ops->create(target);
        check(ktc_broadcast_to(res->buf(), target.data(), (int)target.size(), buf(), shape.data(), (int)shape.size()));
        return res;
    }
    RawP copy(bool shallow) {                                   // JVMRawTensor.kt:257-262, OCLRawTensor.kt:252-258
        if (shallow) {
            if (isDeferred()) return make(ops, shape, cell);    // aliases share the pending value, later its storage
            auto c = std::make_shared<Cell>();
            check(ktc_retain(buf()));
            c->store = cell->store;
            return make(ops, shape, c);
        }
        if (isDeferred()) { ktc_lazy_cell out; check(ktc_lazy_broadcast_to(lz(), shape.data(), (int)shape.size(), &out)); return recorded(ops, shape, out); }
        RawP res = ops->create(shape);
        check(ktc_d2d(res->buf(), 0, buf(), 0, size()));
        return res;
    }
    void inplaceFill(float v) {
        if (ops->lazy && (cell->store || cell->lz)) {              // recorded: a pending constant where nobody else holds the buffer
            int st = 0;
            check(ktc_lazy_assign_fill(lz(), v, &st));
            after_assign(st);
            return;
        }
        if (isDeferred() || !cell->store) {                     // the pending value is overwritten: just take storage
            if (cell->lz) { ktc_lazy_free(cell->lz); cell->lz = 0; }
            check(ktc_alloc(ops->device, size(), &cell->store));
        }
        before_inplace_write();
        check(ktc_fill(buf(), 0, size(), v));
    }
    // ---- reductions (AbstractRawTensor.kt:92-119, JVMRawTensor.kt:146-152) ----
    RawP sum() {
        if (isDeferred()) { const Shape one{1}; ktc_lazy_cell out; check(ktc_lazy_sum(lz(), KTC_EXPR_SUM_ALL, 0, one.data(), 1, &out)); return recorded(ops, one, out); }
        RawP res = ops->create({1});
        check(ktc_reduce_all(KTC_SUM, res->buf(), buf(), size()));
        return res;
    }
    RawP sum(int axis, bool keepDimensions) {
        const int nd = (int)shape.size();
        const int a = axis < 0 ? axis + nd : axis;
        if (a < 0 || a >= nd) throw std::invalid_argument("axis out of range");
        Shape kept = shape; kept[a] = 1;
        Shape dropped = kept;
        if (nd > 1) dropped.erase(dropped.begin() + a);
        const Shape& final_shape = keepDimensions ? kept : dropped;
        if (isDeferred() && a == 0 && nd >= 2) {
            ktc_lazy_cell out; check(ktc_lazy_sum(lz(), KTC_EXPR_SUM_ROWS, 0, final_shape.data(), (int)final_shape.size(), &out));
            return recorded(ops, final_shape, out);
        }
        if (isDeferred() && a == nd - 1 && nd >= 2 && shape[a] > 1 && ops->defer_sums) {
            ktc_lazy_cell out; check(ktc_lazy_sum(lz(), KTC_EXPR_SUM_LAST, 0, final_shape.data(), (int)final_shape.size(), &out));
            return recorded(ops, final_shape, out);
        }
        int64_t outer = 1, inner = 1;
        for (int i = 0; i < a; ++i) outer *= shape[i];
        for (int i = a + 1; i < nd; ++i) inner *= shape[i];
        RawP res = ops->create(final_shape);
        check(ktc_reduce_axis(KTC_SUM, res->buf(), buf(), outer, shape[a], inner));
        return res;
    }
};

Scope::~Scope() {
    if (!owner) return;
    ops.collector = nullptr;
    for (RawP& r : mine) r->release();
}
RawP Ops::create(const Shape& shape) {
    auto c = std::make_shared<Cell>();
    check(ktc_alloc(device, volume(shape), &c->store));
    return Raw::make(this, shape, c);
}
RawP Ops::create_fill(const Shape& shape, float v) {
    if (lazy) {                                                 // a pending constant: no buffer, no fill kernel
        ktc_lazy_cell out;
        check(ktc_lazy_full(device, shape.data(), (int)shape.size(), v, &out));
        return Raw::recorded(this, shape, out);
    }
    RawP r = create(shape); r->inplaceFill(v); return r;
}

// Broadcast-gradient sum-to-shape (Utils.kt:14-41): leading axes are summed away, then every remaining axis whose
// extent differs is summed with the dimension kept; intermediates are released.
static RawP may_unexpand(RawP raw, const Shape& old_shape) {
    const int lead = (int)raw->shape.size() - (int)old_shape.size();
    std::vector<int> expanded;
    for (size_t i = 0; i < old_shape.size(); ++i) if (raw->shape[lead + i] != old_shape[i]) expanded.push_back((int)i);
    RawP res = raw;
    for (int i = 0; i < lead; ++i) { RawP prev = res; res = res->sum(0, false); if (i > 0) prev->release(); }
    for (size_t i = 0; i < expanded.size(); ++i) { RawP prev = res; res = res->sum(expanded[i], true); if (i > 0) prev->release(); }
    return res;
}

// ---- the caller: Tensor, Variable, Function (kten-api autograd) ---------------------------------------------
struct Tensor {
    Ops* ops;
    explicit Tensor(Ops* o) : ops(o) {}
    virtual ~Tensor() {}
    virtual bool requiresGrad() const { return false; }
    virtual Shape shape() = 0;
    virtual RawP getRawValue() = 0;
    virtual void backwardWithGrad(const RawP& gradient) = 0;
    virtual struct Function* asFunction() { return nullptr; }
};
using TensorP = std::shared_ptr<Tensor>;

struct NoGradVariable : Tensor {
    RawP raw;
    NoGradVariable(Ops* o, RawP r) : Tensor(o), raw(std::move(r)) {}
    Shape shape() override { return raw->shape; }
    RawP getRawValue() override { return raw; }
    void backwardWithGrad(const RawP&) override {}
};

struct Variable : Tensor {                                      // accumulates its gradient in place (Variable.kt:44-46)
    RawP value, gradient;
    Variable(Ops* o, RawP v) : Tensor(o), value(std::move(v)) { gradient = ops->create_fill(value->shape, 0.f); gradient->mustSurviveGC = true; }
    bool requiresGrad() const override { return true; }
    Shape shape() override { return value->shape; }
    RawP getRawValue() override { return value; }
    void backwardWithGrad(const RawP& g) override { gradient->plusAssign(g); }
    void zeroGrad() { gradient->inplaceFill(0.f); }
};

struct Function : Tensor {                                      // a lazily evaluated graph node (Function.kt)
    bool keepOutput = false, freeOutput = false, backwardRan = false;
    std::vector<RawP> valuesSaved;
    RawP output_;
    Shape cachedShape; bool haveShape = false;
    std::vector<Function*> registeredAsInputIn;
    RawP gradCache;

    using Tensor::Tensor;
    bool requiresGrad() const override { return true; }
    Function* asFunction() override { return this; }
    void setOutput(const RawP& v) { if (v) v->incrementRef(); output_ = v; }     // raises the ref-count (Function.kt:16-21)
    bool hasValue() const { return (bool)output_; }
    RawP getRawValue() override { return output_; }
    Shape shape() override {
        if (!haveShape) { if (!output_) internalForward(); cachedShape = output_->shape; haveShape = true; }
        return cachedShape;
    }
    virtual std::vector<TensorP> inputs() = 0;
    virtual void doForwardNode() = 0;
    virtual std::vector<RawP> doBackward(const RawP& gradient) = 0;

    void forward() { keepOutput = true; Scope scope(*ops); internalForward(); }
    virtual void internalForward() {
        gradCache.reset(); backwardRan = false;
        if (hasValue()) return;
        std::vector<TensorP> in = inputs();
        for (auto& t : in) if (Function* f = t->asFunction()) f->internalForward();
        if (!hasValue()) doForwardNode();
        for (auto& t : in) if (Function* f = t->asFunction()) f->mayFreeOutput();
    }
    void mayFreeOutput() { if (!keepOutput) freeOutput = true; }
    void saveForBackward(std::initializer_list<RawP> raws) {
        if (!hasValue() || valuesSaved.empty()) for (const RawP& r : raws) { r->incrementRef(); valuesSaved.push_back(r); }
    }
    void registerInputUsages() {
        for (auto& t : inputs()) if (Function* f = t->asFunction()) { f->registeredAsInputIn.push_back(this); f->registerInputUsages(); }
    }
    void backward() {                                           // backward() on a [1] result (Function.kt:54-89)
        if (shape() != Shape{1}) throw std::runtime_error("Backward is only allowed on singleton calculation results (tensors with shape [1])");
        registerInputUsages();
        Scope scope(*ops);
        if (!hasValue()) internalForward();
        RawP seed = ops->create_fill({1}, 1.0f);
        backwardWithGrad(seed);
        releaseUnusedInGraph();
    }
    void backwardWithGrad(const RawP& gradient) override {
        if (registeredAsInputIn.size() > 1) {                   // fan-in (Function.kt:108-120)
            if (!gradCache) gradCache = gradient->copy(false); else gradCache->plusAssign(gradient);
            for (Function* f : registeredAsInputIn) if (!f->backwardRan) return;
        }
        std::vector<RawP> grads = doBackward(gradCache ? gradCache : gradient);
        backwardRan = true;
        std::vector<TensorP> in = inputs();
        for (size_t i = 0; i < in.size(); ++i) if (in[i]->requiresGrad()) in[i]->backwardWithGrad(grads[i]);
        gradient->release();
        if (gradCache) gradCache->release();
    }
    void releaseUnusedInGraph() {
        if (freeOutput && output_) { output_->release(); output_.reset(); freeOutput = false; }
        for (RawP& v : valuesSaved) v->release();
        valuesSaved.clear();
        for (auto& t : inputs()) if (Function* f = t->asFunction()) f->releaseUnusedInGraph();
    }
};

struct BiFunction : Function {
    TensorP a, b; Shape aShape, bShape;
    BiFunction(Ops* o, TensorP x, TensorP y) : Function(o), a(std::move(x)), b(std::move(y)) { cachedShape = common_shape(a->shape(), b->shape()); haveShape = true; }
    std::vector<TensorP> inputs() override { return {a, b}; }
    void doForwardNode() override { RawP ra = a->getRawValue(), rb = b->getRawValue(); aShape = ra->shape; bShape = rb->shape; doForward(ra, rb); }
    virtual void doForward(const RawP& ra, const RawP& rb) = 0;
};
struct UnFunction : Function {
    TensorP t;
    UnFunction(Ops* o, TensorP x, bool same_shape = true) : Function(o), t(std::move(x)) { if (same_shape) { cachedShape = t->shape(); haveShape = true; } }
    std::vector<TensorP> inputs() override { return {t}; }
    void doForwardNode() override { doForward(t->getRawValue()); }
    virtual void doForward(const RawP& x) = 0;
};

struct Plus : BiFunction {                                      // BasicFunctions.kt:7-21
    using BiFunction::BiFunction;
    void doForward(const RawP& ra, const RawP& rb) override { setOutput(ra->plus(rb)); }
    std::vector<RawP> doBackward(const RawP& g) override { return {may_unexpand(g->copy(true), aShape), may_unexpand(g->copy(true), bShape)}; }
};
struct Times : BiFunction {                                     // BasicFunctions.kt:37-55
    using BiFunction::BiFunction;
    void doForward(const RawP& ra, const RawP& rb) override { saveForBackward({ra, rb}); setOutput(ra->times(rb)); }
    std::vector<RawP> doBackward(const RawP& g) override {
        RawP sa = valuesSaved[0], sb = valuesSaved[1];
        return {may_unexpand(g->times(sb), aShape), may_unexpand(g->times(sa), bShape)};
    }
};
struct PowConstant : UnFunction {                               // tensor pow constant (BasicFunctions.kt:182-204)
    float c;
    PowConstant(Ops* o, TensorP x, float constant) : UnFunction(o, std::move(x)), c(constant) {}
    void doForward(const RawP& x) override { saveForBackward({x}); setOutput(x->pow(c)); }
    std::vector<RawP> doBackward(const RawP& g) override {
        RawP grad = g->times(c);
        grad->timesAssign(valuesSaved[0]->pow(c - 1.0f));
        return {grad};
    }
};
struct Sigmoid : UnFunction {                                   // PointwiseFunctions.kt:66-81
    using UnFunction::UnFunction;
    void doForward(const RawP& x) override { RawP res = x->sigmoid(); saveForBackward({res}); setOutput(res); }
    std::vector<RawP> doBackward(const RawP& g) override {
        RawP res = valuesSaved[0];
        RawP grad = res->unaryMinus();
        grad->plusAssign(1.0f);
        grad->timesAssign(res);
        grad->timesAssign(g);
        return {grad};
    }
};
struct SumAll : UnFunction {                                    // AggregatingFunctions.kt:7-25, axis = everything
    Shape inputShape;
    SumAll(Ops* o, TensorP x) : UnFunction(o, std::move(x), false) { cachedShape = {1}; haveShape = true; }
    void doForward(const RawP& x) override { inputShape = x->shape; setOutput(x->sum()); }
    std::vector<RawP> doBackward(const RawP& g) override { return {g->broadcastTo(inputShape)}; }
};

// loss = sum(sigmoid(x*w + b) pow 2) over this rank's rows of x; backward accumulates the gradients of w [1, C] and
// b [C]; the three results are then summed over the ranks through the peer-memory exchange (or just looked up, in a
// world of one, so that whatever is pending is computed inside the step).
struct ShardedStep {
    Ops ops;
    std::shared_ptr<NoGradVariable> x;
    std::shared_ptr<Variable> w, b;
    std::shared_ptr<Function> last;
    ktc_p2p comm = 0;

    std::vector<RawP> step() {
        w->zeroGrad(); b->zeroGrad();
        auto xw = std::make_shared<Times>(&ops, x, w);
        auto z = std::make_shared<Plus>(&ops, xw, b);
        auto s = std::make_shared<Sigmoid>(&ops, z);
        auto p = std::make_shared<PowConstant>(&ops, s, 2.0f);
        auto loss = std::make_shared<SumAll>(&ops, p);
        loss->forward();                                        // keeps the loss value across backward()
        loss->backward();
        std::vector<RawP> out{loss->getRawValue(), w->gradient, b->gradient};
        if (comm) {                                             // through the recorder: what is pending runs first and takes the exchange along
            ktc_lazy_cell cells[3];
            for (int i = 0; i < 3; ++i) cells[i] = out[i]->lz(false);
            check(ktc_lazy_allreduce(comm, cells, 3));
            ops.pending_targets.clear();
        } else {
            for (int i = 0; i < 3; ++i) out[i]->buf();          // a world of one: the values are looked up, so pending work runs inside the step
        }
        last = loss;
        return out;
    }
    void release_step() {                                       // drop the graph of the last step (its retained loss value)
        if (!last) return;
        last->keepOutput = false; last->freeOutput = true;
        last->releaseUnusedInGraph();
        last.reset();
    }
};

}  // namespace kten

// ---- C entry points for the benchmark and the tests ---------------------------------------------------------------
using namespace kten;
static thread_local std::string g_host_error;
#define KTH_GUARD(body) try { body; return KTC_OK; } catch (const std::invalid_argument& e) { g_host_error = e.what(); return KTC_EINVAL; } \
    catch (const std::exception& e) { g_host_error = e.what(); return KTC_ESTATE; }

extern "C" {

KTC_API const char* kth_last_error(void) { return g_host_error.c_str(); }

// x [rows, cols], w [1, cols], b [cols]: buffers the caller keeps alive.  lazy != 0: elementwise calls and sums go
// through the expression recorder.  comm: a connected peer-memory communicator, or 0 for a world of one.
KTC_API int kth_sharded_create(int device, ktc_buf x, int64_t rows, int64_t cols, ktc_buf w, ktc_buf b, int lazy, ktc_p2p comm, void** out) {
    KTH_GUARD({
        auto* st = new ShardedStep();
        st->ops.device = device; st->ops.lazy = lazy != 0; st->comm = comm;
        auto wrap = [&](ktc_buf h, const Shape& s) { auto c = std::make_shared<Cell>(); check(ktc_retain(h)); c->store = h; RawP r = Raw::make(&st->ops, s, c); r->mustSurviveGC = true; return r; };
        st->x = std::make_shared<NoGradVariable>(&st->ops, wrap(x, {rows, cols}));
        st->w = std::make_shared<Variable>(&st->ops, wrap(w, {1, cols}));
        st->b = std::make_shared<Variable>(&st->ops, wrap(b, {cols}));
        *out = st;
    })
}

// n steps back to back, each in a scope of its own; the handles of the last step's results (loss [1], grad w
// [1, cols], grad b [cols]) are written to out3 when it is given -- they stay valid until the next call.
KTC_API int kth_sharded_run(void* handle, int n_steps, ktc_buf* out3) {
    KTH_GUARD({
        auto* st = static_cast<ShardedStep*>(handle);
        for (int i = 0; i < n_steps; ++i) {
            const bool last = i + 1 == n_steps;
            if (last && out3) {                                 // keep the last step's graph so that its loss buffer stays alive
                st->release_step();
                Scope scope(st->ops);
                std::vector<RawP> out = st->step();
                for (int k = 0; k < 3; ++k) out3[k] = out[k]->buf();
            } else {
                Scope scope(st->ops);
                st->step();
                st->release_step();
            }
        }
    })
}

KTC_API int kth_sharded_destroy(void* handle) {
    KTH_GUARD({
        auto* st = static_cast<ShardedStep*>(handle);
        st->release_step();
        delete st;
    })
}

}  // extern "C"
