// ktc_lazy.cpp -- the deferred-expression recorder behind the C ABI (ktc_lazy_*).
//
// kten's autograd issues one raw-tensor call per line of doForward / doBackward
// (kten-api/.../autograd/functions/BasicFunctions.kt, PointwiseFunctions.kt,
// AggregatingFunctions.kt, Utils.kt:14-41, Variable.kt:44-46); executed one by one, the
// sharded-graph step of the benchmark moves 34 tensor volumes through HBM.  A backend binding
// (the Kotlin CUDARawTensor, the Python mirror) can hand its elementwise calls to this recorder
// instead: a call returns a CELL -- the storage slot of a raw tensor -- that holds an expression
// node instead of a buffer.  The expression is compiled into a program for ktc_expr_eval when a
// value is needed: ktc_lazy_buffer (a host read or a call outside the elementwise set), a sum, an
// in-place write to one of its operands.  Every program instruction is one reference operation
// with its own rounding, so results equal the call-by-call execution bit for bit; only the
// order of summation inside a fused sum differs.
//
// Rules that keep the semantics of the eager backend:
//   * nodes are immutable values; an in-place call on a pending cell replaces its node, an
//     in-place call on a stored cell is evaluated into its own buffer (or recorded, see below);
//   * before a buffer is written in place (ktc_lazy_flush, or an in-place call here) every
//     pending expression that reads it is evaluated: a registry maps buffers to the cells whose
//     pending expressions depend on them;
//   * an interior value is recomputed inside at most `recompute_limit` programs; after that, if a
//     cell still waits for it, it is stored as a side output; a value behind a transcendental
//     (`store_cost`) is stored by the first program that computes it;
//   * with `defer_sums`, sums of pending cells are pending too and `stored += pending sum` is
//     remembered as an update of that buffer; the first need of any of them runs all pending
//     sums, those over one iteration space as ONE pass with several sinks;
//   * with `defer_inplace`, an in-place call with a pending operand on a stored cell whose
//     buffer nobody else holds makes the cell pending (its node reads the old buffer);
//   * compiled programs are cached by the structure of the expression DAG and re-bound to the
//     step's fresh nodes, so a training step that rebuilds the same graph pays for ordering and
//     register allocation once;
//   * the forward of SoftmaxCrossEntropy can be recorded too (ktc_lazy_softmax_xent_forward): its two
//     results stay pending, and an elementwise expression of the softmax's shape built on it -- the
//     function's backward -- is evaluated inside the forward's own kernel, which then writes the
//     softmax only if something else still wants it.
// Whatever ktc_expr_eval declines (KTC_ENOTSUP) runs as the library's separate calls.
//
// The file is plain C++ and reaches the rest of the library only through a table of the C ABI's
// own entry points, so that it can be compiled alone (KTC_LAZY_STANDALONE) and driven by a
// stand-in library on a machine without a GPU.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/kten_cuda.h"

namespace ktc {
#ifndef KTC_LAZY_STANDALONE
void set_error(const char* fmt, ...);
#endif
namespace lz {

// ---- the calls the recorder makes --------------------------------------------------------------
struct Backend {
    int (*alloc)(int, int64_t, ktc_buf*);
    int (*retain)(ktc_buf);
    int (*release)(ktc_buf);
    int (*refcount)(ktc_buf, int*);
    int (*buf_info)(ktc_buf, int*, int64_t*, void**);
    int (*d2d)(ktc_buf, int64_t, ktc_buf, int64_t, int64_t);
    int (*fill)(ktc_buf, int64_t, int64_t, float);
    int (*binary)(int, ktc_buf, ktc_buf, ktc_buf, int64_t);
    int (*binary_bcast)(int, ktc_buf, ktc_buf, const int64_t*, int, ktc_buf, const int64_t*, int);
    int (*binary_inplace)(int, ktc_buf, ktc_buf, int64_t);
    int (*scalar)(int, ktc_buf, ktc_buf, float, int64_t, int);
    int (*scalar_inplace)(int, ktc_buf, float, int64_t);
    int (*unary)(int, ktc_buf, ktc_buf, int64_t);
    int (*clamp)(ktc_buf, ktc_buf, float, float, int64_t);
    int (*compare_scalar)(int, ktc_buf, ktc_buf, float, int64_t);
    int (*broadcast_to)(ktc_buf, const int64_t*, int, ktc_buf, const int64_t*, int);
    int (*reduce_axis)(int, ktc_buf, ktc_buf, int64_t, int64_t, int64_t);
    int (*reduce_all)(int, ktc_buf, ktc_buf, int64_t);
    int (*expr_eval)(const uint32_t*, int, const float*, int, const int64_t*, int, const ktc_buf*, const int64_t*, int,
                     const ktc_buf*, int, int, ktc_buf, int);
    int (*expr_eval_multi_fused)(const uint32_t*, int, const float*, int, const int64_t*, int, const ktc_buf*, const int64_t*, int,
                                 const ktc_buf*, int, const int*, const ktc_buf*, const int*, int,
                                 const ktc_buf*, const int*, uint64_t, const ktc_buf*, const int64_t*, int);
    int (*p2p_allreduce_sum)(uint64_t, const ktc_buf*, const int64_t*, int);
    int (*softmax_fwd)(ktc_buf, ktc_buf, ktc_buf, ktc_buf, int64_t, int64_t, float, float);
    int (*softmax_fwd_expr)(ktc_buf, ktc_buf, ktc_buf, ktc_buf, int64_t, int64_t, float, float, const uint32_t*, int, const float*, int,
                            const ktc_buf*, const int64_t*, int, int, const ktc_buf*, int);
};
constexpr int kBackendEntries = sizeof(Backend) / sizeof(void*);

#ifdef KTC_LAZY_STANDALONE
static Backend B = {};
static thread_local char g_err[512];
static void set_error_v(const char* fmt, va_list ap) { vsnprintf(g_err, sizeof(g_err), fmt, ap); }
#else
static Backend B = {ktc_alloc, ktc_retain, ktc_release, ktc_refcount, ktc_buf_info, ktc_d2d, ktc_fill, ktc_binary, ktc_binary_bcast,
                    ktc_binary_inplace, ktc_scalar, ktc_scalar_inplace, ktc_unary, ktc_clamp, ktc_compare_scalar, ktc_broadcast_to,
                    ktc_reduce_axis, ktc_reduce_all, ktc_expr_eval, ktc_expr_eval_multi_fused, ktc_p2p_allreduce_sum,
                    ktc_softmax_xent_forward, ktc_softmax_xent_forward_expr};
static void set_error_v(const char* fmt, va_list ap) { char b[512]; vsnprintf(b, sizeof(b), fmt, ap); ::ktc::set_error("%s", b); }
#endif

static int fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); set_error_v(fmt, ap); va_end(ap);
    return code;
}
#define LZ_TRY(call) do { int s_ = (call); if (s_ != KTC_OK) return s_; } while (0)

constexpr int MAXD = KTC_MAX_DIMS;
enum Kind : uint8_t { K_LEAF = 0, K_CONST, K_UN, K_BIN, K_CLAMP, K_CMP, K_SQUARE, K_BCAST, K_REDUCE, K_SCATC, K_SOFTMAX, K_NLL };

struct Shape {
    int nd = 0;
    int64_t d[MAXD];
    int64_t volume() const { int64_t v = 1; for (int i = 0; i < nd; ++i) v *= d[i]; return v; }
    bool operator==(const Shape& o) const { return nd == o.nd && std::equal(d, d + nd, o.d); }
    bool operator!=(const Shape& o) const { return !(*this == o); }
};
static Shape make_shape(const int64_t* s, int nd) { Shape r; r.nd = nd; for (int i = 0; i < nd; ++i) r.d[i] = s[i]; return r; }

// K_SCATC: args[0] with `imm[0]` written at column (int)args[1] of every row -- inplaceScatter(-1, index, constant) with
// one index per row (JVMRawTensor.kt:317-332).
// A value.  `buf` is set once the value is in memory (the node then acts as a leaf and forgets how it was
// computed).  A K_REDUCE node is a sum that has not run yet: args[0] is the summed expression, op the sink
// kind, imm[0] != 0 a mean; it is never part of a program -- whoever needs its value runs the pending sums.
// K_SOFTMAX / K_NLL: the two results of SoftmaxCrossEntropy's forward that has not run yet (SoftmaxCrossEntropy.kt:40-59):
// K_SOFTMAX, args {logits, targets} (both in memory), imm {lo, hi}, is the [rows, cols] tensor the function saves for
// backward; K_NLL, args {the K_SOFTMAX node}, is the [rows] loss per row.  One kernel computes both; when the softmax is
// read by ONE recorded elementwise expression of its shape (the function's backward), that expression runs inside the same
// kernel and the softmax is written only if something else still wants it.
struct Node {
    int refs = 0;
    Kind kind = K_LEAF;
    int op = 0;
    int nargs = 0;
    Node* args[2] = {nullptr, nullptr};     // strong
    int nimm = 0;
    float imm[2] = {0.f, 0.f};
    Shape shape;
    ktc_buf buf = 0;                        // one reference while non-zero
    int dev = -1;
    int evals = 0;
    uint64_t owner = 0;                     // id of the cell that waits for this value (weak)
    std::vector<Node*> parents;             // nodes built on this one (weak; a dying node unlinks itself)
    bool has_sum = false;                   // a pending sum may sit underneath (never reset: a stale true only costs a look)
    bool has_row = false;                   // a pending K_SOFTMAX / K_NLL may sit underneath (never reset either)
    std::vector<ktc_buf> leaves;            // buffers this value is read from (sorted, unique)
    // scratch of the walks (valid for one epoch)
    uint32_t epoch = 0;
    int pos = -1, uses = 0, reg = -1, cost = 0;
    bool chosen = false;
    bool stored() const { return buf != 0; }
};

struct Cell {
    uint32_t gen = 1;
    bool live = false;
    Node* node = nullptr;                   // strong
};

struct Pending {
    Node* node;                             // weak until an update hangs on it (then one reference is held)
    bool strong;
    std::vector<ktc_buf> targets;           // buffers to which this sum is added when it has run (one reference each)
    std::vector<uint64_t> seq;              // request order of those updates
    std::vector<char> from_zero;            // the target was zeroed just before: it receives 0f + sum, its contents are not read
};

struct Cached {
    bool fusable = false;
    std::vector<uint32_t> code;
    std::vector<std::pair<int, int>> imm_src;            // (position in the order, index in node.imm)
    std::vector<std::pair<int, Shape>> leaf_plan;        // (position of the stored node, right-aligned shape)
    std::vector<int> store_plan;                         // positions of the nodes written by STORE
    int n_requested = 0;
};

struct Program {
    Shape shape;
    std::vector<uint32_t> code;
    std::vector<float> imm;
    std::vector<std::pair<ktc_buf, Shape>> leaves;
    std::vector<std::pair<int, int>> imm_src;
    std::vector<int> leaf_src;
    std::vector<int> free_regs;
    std::vector<Node*> order;
    bool ok = true;                                       // false: not fusable
};

// ---- state (one recorder per process, guarded by one mutex) ---------------------------------------
static std::mutex g_mu;
static std::vector<Cell> g_cells;
static std::vector<uint32_t> g_free_cells;
static std::unordered_map<ktc_buf, std::vector<uint64_t>> g_deps;      // buffer -> cells whose pending expressions read it
static size_t g_deps_purge_at = 1024;
static std::vector<Pending> g_pending;
static std::unordered_map<ktc_buf, int> g_pending_targets;            // buffer -> number of pending `+= sum` updates
static uint64_t g_update_seq = 0;
static std::unordered_map<std::string, Cached> g_cache;
static constexpr size_t kCacheMax = 4096;
static uint32_t g_epoch = 0;
static std::vector<struct Node*> g_evaluating;                        // values a caller further up the stack is computing right now
static int64_t g_live_nodes = 0;
static int opt_recompute_limit = 2, opt_store_cost = 8, opt_defer_sums = 1, opt_defer_inplace = 1;
static int64_t st_fused = 0, st_unfused = 0, st_multi = 0, st_cache_hits = 0, st_compiles = 0, st_fused_updates = 0, st_fused_exchanges = 0;

// ---- nodes ----------------------------------------------------------------------------------------
static void node_unref(Node* n);
static Node* node_ref(Node* n) { if (n) ++n->refs; return n; }

static void drop_args(Node* n, std::vector<Node*>& dead) {
    for (int i = 0; i < n->nargs; ++i) {
        Node* a = n->args[i];
        if (!a) continue;
        if (a->kind != K_CONST) {
            auto& ps = a->parents;
            auto it = std::find(ps.begin(), ps.end(), n);
            if (it != ps.end()) { *it = ps.back(); ps.pop_back(); }
        }
        if (--a->refs == 0) dead.push_back(a);
        n->args[i] = nullptr;
    }
    n->nargs = 0;
}

static void node_unref(Node* n) {
    if (!n || --n->refs > 0) return;
    std::vector<Node*> dead{n};
    while (!dead.empty()) {                               // iterative: chains can be long
        Node* d = dead.back(); dead.pop_back();
        if (d->kind == K_REDUCE) {
            for (size_t i = 0; i < g_pending.size(); ++i)
                if (g_pending[i].node == d) { g_pending.erase(g_pending.begin() + i); break; }
        }
        drop_args(d, dead);
        if (d->buf) B.release(d->buf);
        --g_live_nodes;
        delete d;
    }
}

static void merge_leaves(std::vector<ktc_buf>& into, const std::vector<ktc_buf>& from) {
    for (ktc_buf h : from) {
        auto it = std::lower_bound(into.begin(), into.end(), h);
        if (it == into.end() || *it != h) into.insert(it, h);
    }
}
static void add_leaf(std::vector<ktc_buf>& into, ktc_buf h) {
    auto it = std::lower_bound(into.begin(), into.end(), h);
    if (it == into.end() || *it != h) into.insert(it, h);
}
static bool has_leaf(const Node* n, ktc_buf h) { return std::binary_search(n->leaves.begin(), n->leaves.end(), h); }

// a new node holds one reference on each argument
static Node* new_node(Kind kind, const Shape& shape, int op, Node* a0, Node* a1, const float* imm, int nimm) {
    Node* n = new Node();
    ++g_live_nodes;
    n->kind = kind; n->op = op; n->shape = shape;
    n->nimm = nimm; for (int i = 0; i < nimm; ++i) n->imm[i] = imm[i];
    n->has_sum = kind == K_REDUCE;
    n->has_row = kind == K_SOFTMAX || kind == K_NLL;
    Node* as[2] = {a0, a1};
    for (int i = 0; i < 2; ++i) {
        Node* a = as[i];
        if (!a) continue;
        n->args[n->nargs++] = node_ref(a);
        if (a->has_sum && !a->stored()) n->has_sum = true;
        if (a->has_row && !a->stored()) n->has_row = true;
        if (a->dev >= 0) n->dev = a->dev;
        if (a->stored()) add_leaf(n->leaves, a->buf); else merge_leaves(n->leaves, a->leaves);
        if (a->kind != K_CONST) a->parents.push_back(n);
    }
    return n;
}

// takes over one reference on `buf`
static Node* new_leaf(ktc_buf buf, const Shape& shape, int dev) {
    Node* n = new Node();
    ++g_live_nodes;
    n->kind = K_LEAF; n->shape = shape; n->buf = buf; n->dev = dev;
    n->leaves.push_back(buf);
    return n;
}

static Node* new_const(float v) {
    Shape s; s.nd = 1; s.d[0] = 1;
    return new_node(K_CONST, s, 0, nullptr, nullptr, &v, 1);
}

static Node* strip(Node* n) {                             // look through broadcast markers: they change the shape, not the value
    while (n->kind == K_BCAST && !n->stored()) n = n->args[0];
    return n;
}

// ---- cells ----------------------------------------------------------------------------------------
static Cell* cell_of(uint64_t id) {
    const uint32_t idx = (uint32_t)(id & 0xffffffffu);
    if (idx == 0 || idx > g_cells.size()) return nullptr;
    Cell* c = &g_cells[idx - 1];
    return (c->live && c->gen == (uint32_t)(id >> 32)) ? c : nullptr;
}
static uint64_t cell_id(const Cell* c) { return ((uint64_t)c->gen << 32) | (uint64_t)((c - g_cells.data()) + 1); }

static uint64_t new_cell(Node* node /* one reference is taken over */) {
    uint32_t idx;
    if (!g_free_cells.empty()) { idx = g_free_cells.back(); g_free_cells.pop_back(); }
    else { g_cells.emplace_back(); idx = (uint32_t)g_cells.size() - 1; }
    Cell& c = g_cells[idx];
    c.live = true; c.node = node;
    return ((uint64_t)c.gen << 32) | (uint64_t)(idx + 1);
}

static bool waiting(const Node* n) {                      // a live cell still waits for exactly this value
    const Cell* c = cell_of(n->owner);
    return c && c->node == n && !n->stored();
}

static void register_cell(uint64_t id, Node* node) {
    node->owner = id;
    for (ktc_buf h : node->leaves) {
        auto& refs = g_deps[h];
        refs.push_back(id);
        const size_t k = refs.size();
        if (k > 64 && (k & (k - 1)) == 0)                 // at powers of two: drop the dead ones
            refs.erase(std::remove_if(refs.begin(), refs.end(), [](uint64_t r) { return cell_of(r) == nullptr; }), refs.end());
    }
    if (g_deps.size() > g_deps_purge_at) {
        for (auto it = g_deps.begin(); it != g_deps.end();) {
            auto& refs = it->second;
            refs.erase(std::remove_if(refs.begin(), refs.end(), [](uint64_t r) { return cell_of(r) == nullptr; }), refs.end());
            if (refs.empty()) it = g_deps.erase(it); else ++it;
        }
        g_deps_purge_at = std::max<size_t>(1024, 2 * g_deps.size());
    }
}

static uint64_t pending_cell(Kind kind, const Shape& shape, int op, Node* a0, Node* a1, const float* imm, int nimm) {
    Node* n = new_node(kind, shape, op, a0, a1, imm, nimm);
    const uint64_t id = new_cell(node_ref(n));
    register_cell(id, n);
    return id;
}

// The value of `node` now lives in `buf` (one reference is taken over): forget how it was computed, and make
// everything that is computed from it depend on the new buffer.
static void set_stored(Node* node, ktc_buf buf) {
    node->buf = buf;
    std::vector<Node*> dead;
    drop_args(node, dead);
    for (Node* d : dead) { ++d->refs; node_unref(d); }
    const uint32_t ep = ++g_epoch;
    std::vector<Node*> stack(node->parents.begin(), node->parents.end());
    while (!stack.empty()) {
        Node* a = stack.back(); stack.pop_back();
        if (a->epoch == ep) continue;
        a->epoch = ep;
        add_leaf(a->leaves, buf);
        if (cell_of(a->owner)) g_deps[buf].push_back(a->owner);
        stack.insert(stack.end(), a->parents.begin(), a->parents.end());
    }
}

// ---- shape algebra ----------------------------------------------------------------------------------
// right-aligned broadcast shape (ShapeFunctions.kt:168-185); false on a non-singleton mismatch
static bool common_shape(const Shape& a, const Shape& b, Shape* out) {
    out->nd = std::max(a.nd, b.nd);
    for (int i = 0; i < out->nd; ++i) {
        const int ia = i - (out->nd - a.nd), ib = i - (out->nd - b.nd);
        const int64_t da = ia >= 0 ? a.d[ia] : 1, db = ib >= 0 ? b.d[ib] : 1;
        if (da != db && da != 1 && db != 1) return false;
        out->d[i] = da == 1 ? db : da;
    }
    return true;
}

// ---- programs ---------------------------------------------------------------------------------------
static bool has_pending_sum(Node* const* roots, int n) {
    const uint32_t ep = ++g_epoch;
    std::vector<Node*> stack;
    for (int i = 0; i < n; ++i) if (roots[i] && roots[i]->has_sum) stack.push_back(roots[i]);
    while (!stack.empty()) {
        Node* x = stack.back(); stack.pop_back();
        if (x->epoch == ep || x->stored()) continue;
        x->epoch = ep;
        if (x->kind == K_REDUCE) return true;
        for (int i = 0; i < x->nargs; ++i) if (x->args[i]->has_sum) stack.push_back(x->args[i]);
    }
    return false;
}

// Children-first order of the unstored DAG under `roots` (broadcast markers looked through) and the number of
// uses of every node (one per consumer, one per root); positions and use counts are left in the nodes.
static void toposort(const std::vector<Node*>& roots, std::vector<Node*>& order) {
    const uint32_t ep = ++g_epoch;
    struct Item { Node* n; bool done; };
    std::vector<Item> stack;
    for (size_t i = roots.size(); i-- > 0;) stack.push_back({strip(roots[i]), false});
    while (!stack.empty()) {
        Item it = stack.back(); stack.pop_back();
        if (it.done) { it.n->pos = (int)order.size(); order.push_back(it.n); continue; }
        if (it.n->epoch == ep) { ++it.n->uses; continue; }
        it.n->epoch = ep; it.n->uses = 1; it.n->reg = -1; it.n->chosen = false;
        stack.push_back({it.n, true});
        if (!it.n->stored())
            for (int i = it.n->nargs; i-- > 0;) stack.push_back({strip(it.n->args[i]), false});
    }
}

static const int kHeavy[6] = {10, 10, 12, 16, 2, 1};      // rough issue cost of one element: exp log tanh sigmoid reciprocal neg
static int weight(const Node* n) {
    if (n->kind == K_UN) return (n->op >= 0 && n->op < 6) ? kHeavy[n->op] : (n->op == KTC_SQRT ? 3 : n->op == KTC_RSQRT ? 5 : 1);
    if (n->kind == K_BIN) return n->op == KTC_POW ? 30 : n->op == KTC_DIV ? 3 : 1;
    return (n->kind == K_LEAF || n->kind == K_CONST || n->kind == K_BCAST) ? 0 : 1;
}

static void emit(Program& p, int op, int d = 0, int a = 0, int b = 0, int k = 0) {
    if ((int)p.code.size() >= KTC_EXPR_MAX_INSTR) { p.ok = false; return; }
    p.code.push_back((uint32_t)op | ((uint32_t)d << 8) | ((uint32_t)a << 12) | ((uint32_t)b << 16) | ((uint32_t)k << 20));
}
static int imm_index(Program& p, const float* v, int n, int src) {
    if ((int)p.imm.size() + n > KTC_EXPR_MAX_IMM) { p.ok = false; return 0; }
    const int k = (int)p.imm.size();
    for (int j = 0; j < n; ++j) { p.imm.push_back(v[j]); p.imm_src.push_back({src, j}); }
    return k;
}
static bool pad_shape(const Shape& s, int nd, Shape* out) {
    if (s.nd > nd) return false;
    out->nd = nd;
    for (int i = 0; i < nd - s.nd; ++i) out->d[i] = 1;
    for (int i = 0; i < s.nd; ++i) out->d[nd - s.nd + i] = s.d[i];
    return true;
}
static int leaf_index(Program& p, ktc_buf h, const Shape& s, int src) {
    Shape padded;
    if (!pad_shape(s, p.shape.nd, &padded)) { p.ok = false; return 0; }
    for (size_t i = 0; i < p.leaves.size(); ++i)
        if (p.leaves[i].first == h && p.leaves[i].second == padded) return (int)i;
    if ((int)p.leaves.size() >= KTC_EXPR_MAX_LEAVES) { p.ok = false; return 0; }
    p.leaves.push_back({h, padded});
    p.leaf_src.push_back(src);
    return (int)p.leaves.size() - 1;
}
static int alloc_reg(Program& p) {
    if (p.free_regs.empty()) { p.ok = false; return 0; }
    const int r = p.free_regs.back(); p.free_regs.pop_back();
    return r;
}

static const int kBinX[5] = {KTC_X_ADD, KTC_X_SUB, KTC_X_MUL, KTC_X_DIV, KTC_X_POW};
static const int kUnX[6] = {KTC_X_EXP, KTC_X_LOG, KTC_X_TANH, KTC_X_SIGMOID, KTC_X_RCP, KTC_X_NEG};
// the unary operations that are expression instructions: exp .. neg, and sqrt, 1 / sqrt, abs
static bool unary_recordable(int op) { return (op >= KTC_EXP && op <= KTC_NEG) || op == KTC_SQRT || op == KTC_RSQRT || op == KTC_ABS; }
static int unary_x(int op) { return op <= KTC_NEG ? kUnX[op] : op == KTC_SQRT ? KTC_X_SQRT : op == KTC_RSQRT ? KTC_X_RSQRT : KTC_X_ABS; }
static const int kCmpX[4] = {KTC_X_CMP_LT, KTC_X_CMP_LTE, KTC_X_CMP_GT, KTC_X_CMP_GTE};

// The uncached compilation: side-output choice, register allocation, emission.
static void compile_uncached(Program& prog, std::vector<Node*>& store_nodes, const std::vector<Node*>& accs,
                             const std::vector<Node*>& sinks, const std::vector<Node*>& order, int recompute_limit, int store_cost) {
    const int64_t full_volume = prog.shape.volume();
    // Side outputs.  Recomputing a short chain from an operand that is read anyway costs no memory traffic, so
    // cheap values are recomputed (a bounded number of times); a value behind a transcendental is stored the
    // first time -- the kernel that computes it is issue-bound and the store rides along.  Chosen bottom-up (a
    // chosen value makes what is built on it cheap), then pruned top-down: nothing reaches below a stored value.
    if (recompute_limit > 0 || store_cost > 0) {
        for (Node* n : order) {
            if (n->stored() || n->kind == K_CONST || n->kind == K_LEAF) { n->cost = 0; continue; }
            int c = weight(n);
            for (int i = 0; i < n->nargs; ++i) c += strip(n->args[i])->cost;
            const bool requested = std::find(store_nodes.begin(), store_nodes.end(), n) != store_nodes.end();
            if (waiting(n) && n->shape.volume() == full_volume && !requested &&
                ((recompute_limit > 0 && n->evals >= recompute_limit) || (store_cost > 0 && c >= store_cost))) {
                n->chosen = true;
                c = 0;
            }
            n->cost = c;
        }
        const uint32_t ep = ++g_epoch;
        std::vector<Node*> stack(sinks.begin(), sinks.end());
        while (!stack.empty()) {
            Node* n = strip(stack.back()); stack.pop_back();
            if (n->epoch == ep || n->stored()) continue;
            n->epoch = ep;
            if (n->chosen && (int)store_nodes.size() < KTC_EXPR_MAX_STORES) { store_nodes.push_back(n); ++n->uses; continue; }
            for (int i = 0; i < n->nargs; ++i) stack.push_back(n->args[i]);
        }
    }
    auto release_use = [&](Node* n) { if (--n->uses == 0) prog.free_regs.push_back(n->reg); };
    for (Node* n : order) {
        int d;
        if (n->stored()) {
            d = alloc_reg(prog);
            emit(prog, KTC_X_LOAD, d, 0, 0, leaf_index(prog, n->buf, n->shape, n->pos));
        } else if (n->kind == K_CONST) {
            d = alloc_reg(prog);
            emit(prog, KTC_X_CONST, d, 0, 0, imm_index(prog, n->imm, 1, n->pos));
        } else {
            int srcs[2] = {0, 0};
            Node* kids[2] = {nullptr, nullptr};
            for (int i = 0; i < n->nargs; ++i) { kids[i] = strip(n->args[i]); srcs[i] = kids[i]->reg; }
            for (int i = 0; i < n->nargs; ++i) release_use(kids[i]);
            d = alloc_reg(prog);                          // may reuse a source register: the kernel reads before it writes
            switch (n->kind) {
            case K_BIN: emit(prog, kBinX[n->op], d, srcs[0], srcs[1]); break;
            case K_UN: emit(prog, unary_x(n->op), d, srcs[0]); break;
            case K_SQUARE: emit(prog, KTC_X_SQUARE, d, srcs[0]); break;
            case K_CLAMP: emit(prog, KTC_X_CLAMP, d, srcs[0], 0, imm_index(prog, n->imm, 2, n->pos)); break;
            case K_CMP: emit(prog, kCmpX[n->op], d, srcs[0], 0, imm_index(prog, n->imm, 1, n->pos)); break;
            case K_SCATC: emit(prog, KTC_X_SCATC, d, srcs[0], srcs[1], imm_index(prog, n->imm, 1, n->pos)); break;
            default: prog.ok = false; break;
            }
        }
        if (!prog.ok) return;
        n->reg = d;
        for (size_t k = 0; k < store_nodes.size(); ++k)
            if (store_nodes[k] == n) { emit(prog, KTC_X_STORE, 0, d, 0, (int)k); release_use(n); }
        for (size_t j = 0; j < accs.size(); ++j)
            if (accs[j] == n) { emit(prog, KTC_X_ACC, 0, d, 0, (int)j); release_use(n); }
        if (!prog.ok) return;
    }
}

static void key_put(std::string& k, int64_t v) { k.append(reinterpret_cast<const char*>(&v), sizeof(v)); }

// Linearise the DAG under `stores` + `accs` into a register program over the iteration space `shape`.
// accs: the summed node of a single-sink program, or one node per sink of a multi-sink program (the ACC of
// entry j carries sink index j).  store_nodes returns the nodes written by STORE, in store-index order; the
// first n_requested of them are the requested ones.  prog.ok == false: not fusable.
// The program depends on the structure of the DAG (operations, sharing, which values are in memory and which
// leaves are the same buffer) and on the per-node facts the side-output rule looks at -- not on buffer handles or
// constants.  Graphs are rebuilt with fresh nodes every step, so the compiled form is cached by that structure
// and re-bound to the current nodes: immediates, leaf handles and store nodes are looked up by position.
static void compile_program(Program& prog, const Shape& shape, const std::vector<Node*>& stores_in, const std::vector<Node*>& accs_in,
                            bool multi, int recompute_limit, int store_cost, std::vector<Node*>& store_nodes, int* n_requested) {
    prog.shape = shape;
    std::vector<Node*> accs, sinks;
    for (Node* n : stores_in) sinks.push_back(strip(n));
    for (Node* a : accs_in) { accs.push_back(strip(a)); sinks.push_back(accs.back()); }
    toposort(sinks, prog.order);
    const std::vector<Node*>& order = prog.order;
    const int64_t full_volume = shape.volume();
    std::string key;
    key.reserve(64 + order.size() * 48);
    key_put(key, shape.nd);
    for (int i = 0; i < shape.nd; ++i) key_put(key, shape.d[i]);
    key_put(key, (int64_t)stores_in.size());
    for (Node* n : stores_in) key_put(key, strip(n)->pos);
    key_put(key, (int64_t)accs.size());
    for (Node* a : accs) key_put(key, a->pos);
    key_put(key, multi ? 1 : 0); key_put(key, recompute_limit); key_put(key, store_cost);
    std::vector<std::pair<std::pair<ktc_buf, Shape>, int>> first_leaf;       // (buffer, right-aligned shape) -> first position
    for (Node* n : order) {
        if (n->stored()) {
            Shape padded;
            if (!pad_shape(n->shape, shape.nd, &padded)) { prog.ok = false; return; }
            int first = n->pos;
            for (auto& f : first_leaf) if (f.first.first == n->buf && f.first.second == padded) { first = f.second; break; }
            if (first == n->pos) first_leaf.push_back({{n->buf, padded}, n->pos});
            key_put(key, -1); key_put(key, n->shape.nd);
            for (int i = 0; i < n->shape.nd; ++i) key_put(key, n->shape.d[i]);
            key_put(key, first);
        } else if (n->kind == K_CONST) {
            key_put(key, -2);
        } else {
            key_put(key, n->kind); key_put(key, n->op); key_put(key, n->nimm); key_put(key, n->nargs);
            for (int i = 0; i < n->nargs; ++i) key_put(key, strip(n->args[i])->pos);
            key_put(key, (waiting(n) && n->shape.volume() == full_volume) ? 1 : 0);
            key_put(key, (recompute_limit > 0 && n->evals >= recompute_limit) ? 1 : 0);
        }
    }
    auto hit = g_cache.find(key);
    if (hit != g_cache.end()) {
        ++st_cache_hits;
        const Cached& c = hit->second;
        if (!c.fusable) { prog.ok = false; return; }
        prog.code = c.code;
        for (auto& s : c.imm_src) prog.imm.push_back(order[s.first]->imm[s.second]);
        for (auto& l : c.leaf_plan) prog.leaves.push_back({order[l.first]->buf, l.second});
        store_nodes.clear();
        for (int p : c.store_plan) store_nodes.push_back(order[p]);
        *n_requested = c.n_requested;
        return;
    }
    ++st_compiles;
    for (int r = KTC_EXPR_REGS - 1; r >= 0; --r) prog.free_regs.push_back(r);
    store_nodes.clear();
    for (Node* n : stores_in) store_nodes.push_back(strip(n));
    *n_requested = (int)store_nodes.size();
    compile_uncached(prog, store_nodes, accs, sinks, order, recompute_limit, store_cost);
    if (g_cache.size() < kCacheMax) {
        Cached c;
        c.fusable = prog.ok;
        if (prog.ok) {
            c.code = prog.code; c.imm_src = prog.imm_src; c.n_requested = *n_requested;
            for (size_t i = 0; i < prog.leaves.size(); ++i) c.leaf_plan.push_back({prog.leaf_src[i], prog.leaves[i].second});
            for (Node* n : store_nodes) c.store_plan.push_back(n->pos);
        }
        g_cache.emplace(std::move(key), std::move(c));
    }
}

// views the iteration space [A, ...] as [A, rest]: possible when every operand is either full or broadcast
// over the trailing dimensions
static bool as_rows(Program& prog, const Shape& shape) {
    int64_t rest = 1;
    for (int i = 1; i < shape.nd; ++i) rest *= shape.d[i];
    for (auto& l : prog.leaves) {
        const Shape& s = l.second;
        bool full = true, ones = true;
        for (int i = 1; i < shape.nd; ++i) { full = full && s.d[i] == shape.d[i]; ones = ones && s.d[i] == 1; }
        Shape r; r.nd = 2; r.d[0] = s.d[0];
        if (full) r.d[1] = rest; else if (ones) r.d[1] = 1; else return false;
        l.second = r;
    }
    prog.shape.nd = 2; prog.shape.d[0] = shape.d[0]; prog.shape.d[1] = rest;
    return true;
}

static void pack_leaves(const Program& prog, std::vector<ktc_buf>& hs, std::vector<int64_t>& shapes) {
    for (auto& l : prog.leaves) {
        hs.push_back(l.first);
        for (int i = 0; i < prog.shape.nd; ++i) shapes.push_back(l.second.d[i]);
    }
    if (hs.empty()) { hs.push_back(0); shapes.push_back(0); }
}

static int run_pending(struct Exchange* x = nullptr);
static int settle_rows(Node* const* roots, int n);
static int try_fused_softmax(const Shape& shape, const std::vector<Node*>& stores, const std::vector<ktc_buf>& handles, const std::vector<bool>& own,
                             Node* acc, int sink, int dev, bool* fused);
static int run_softmax(Node* sm, bool want_softmax);
static int force(Node* node, ktc_buf* h, Shape* shape);
static int eager_into(Node* node, const Shape& shape, ktc_buf out);

static int alloc_handle(int dev, int64_t n, ktc_buf* h) { return B.alloc(dev < 0 ? 0 : dev, n, h); }

// `handle` (one owned reference) now holds node's value
static void adopt(Node* node, ktc_buf handle) { set_stored(node, handle); }

// Compile `stores` (+ the summed node `acc`) and run them as one kernel.  handles[i] receives stores[i]; own[i]:
// the handle is a fresh buffer that node i adopts (its reference passes to the node).  Nodes stored on the side
// get fresh buffers.  *fused = false: not fusable, nothing was run.
static int try_fused(const Shape& shape, const std::vector<Node*>& stores, const std::vector<ktc_buf>& handles, const std::vector<bool>& own,
                     Node* acc, int sink, ktc_buf sink_out, bool mean, bool rows_view, int dev, bool* fused) {
    *fused = false;
    if (!g_pending.empty()) {
        std::vector<Node*> roots(stores);
        if (acc) roots.push_back(acc);
        if (has_pending_sum(roots.data(), (int)roots.size())) LZ_TRY(run_pending());
    }
    {
        bool rows_below = acc && acc->has_row;
        for (Node* n : stores) rows_below = rows_below || n->has_row;
        if (rows_below) {
            // a pending softmax forward underneath: this expression becomes its epilogue, or the forward runs first
            LZ_TRY(try_fused_softmax(shape, stores, handles, own, acc, sink, dev, fused));
            if (*fused) return KTC_OK;
            std::vector<Node*> roots(stores);
            if (acc) roots.push_back(acc);
            const size_t mark = g_evaluating.size();
            g_evaluating.insert(g_evaluating.end(), stores.begin(), stores.end());
            for (Node* n : stores) g_evaluating.push_back(strip(n));
            const int rs = settle_rows(roots.data(), (int)roots.size());
            g_evaluating.resize(mark);
            LZ_TRY(rs);
        }
    }
    Program prog;
    std::vector<Node*> store_nodes, accs;
    if (acc) accs.push_back(acc);
    int n_req = 0;
    compile_program(prog, shape, stores, accs, false, opt_recompute_limit, opt_store_cost, store_nodes, &n_req);
    if (!prog.ok) return KTC_OK;
    if (rows_view && !as_rows(prog, shape)) return KTC_OK;
    const int64_t total = shape.volume();
    std::vector<ktc_buf> all(handles);
    for (size_t i = n_req; i < store_nodes.size(); ++i) {
        ktc_buf h = 0;
        const int s = alloc_handle(dev, total, &h);
        if (s != KTC_OK) { for (size_t j = handles.size(); j < all.size(); ++j) B.release(all[j]); return s; }
        all.push_back(h);
    }
    std::vector<ktc_buf> lh; std::vector<int64_t> ls;
    pack_leaves(prog, lh, ls);
    const ktc_buf none = 0;
    const float zero = 0.f;
    const int rc = B.expr_eval(prog.code.data(), (int)prog.code.size(), prog.imm.empty() ? &zero : prog.imm.data(), (int)prog.imm.size(),
                               prog.shape.d, prog.shape.nd, lh.data(), ls.data(), (int)prog.leaves.size(),
                               all.empty() ? &none : all.data(), (int)all.size(), sink, sink_out, mean ? 1 : 0);
    if (rc != KTC_OK) {
        for (size_t j = handles.size(); j < all.size(); ++j) B.release(all[j]);
        return rc == KTC_ENOTSUP ? KTC_OK : rc;
    }
    ++st_fused;
    *fused = true;
    for (Node* n : prog.order) ++n->evals;
    for (int i = 0; i < n_req; ++i) if (own[i]) adopt(store_nodes[i], handles[i]);
    for (size_t i = n_req; i < store_nodes.size(); ++i) adopt(store_nodes[i], all[handles.size() + (i - n_req)]);
    return KTC_OK;
}

// Make sure the value under `node` (looking through broadcast markers) is in memory; the handle stays valid
// while the node is alive.
static int force(Node* node, ktc_buf* h, Shape* shape) {
    Node* nd = strip(node);
    if (nd->kind == K_REDUCE && !nd->stored()) {
        LZ_TRY(run_pending());
        if (!nd->stored()) return fail(KTC_ESTATE, "a pending sum was not evaluated");
    }
    if ((nd->kind == K_SOFTMAX || nd->kind == K_NLL) && !nd->stored()) {
        LZ_TRY(run_softmax(nd->kind == K_SOFTMAX ? nd : nd->args[0], nd->kind == K_SOFTMAX));
        if (!nd->stored()) return fail(KTC_ESTATE, "a pending softmax forward was not evaluated");
    }
    if (!nd->stored()) {
        ktc_buf fresh = 0;
        LZ_TRY(alloc_handle(nd->dev, nd->shape.volume(), &fresh));
        bool fused = false;
        int s = try_fused(nd->shape, {nd}, {fresh}, {true}, nullptr, KTC_EXPR_STORE_ONLY, 0, false, false, nd->dev, &fused);
        if (s == KTC_OK && !fused) {
            ++st_unfused;
            s = eager_into(nd, nd->shape, fresh);
            if (s == KTC_OK) adopt(nd, fresh);
        }
        if (s != KTC_OK) { if (!nd->stored()) B.release(fresh); return s; }
    }
    *h = nd->buf;
    if (shape) *shape = nd->shape;
    return KTC_OK;
}

// Give a pending cell storage.
static int materialize_cell(Cell* cell) {
    Node* node = cell->node;
    if (strip(node) == node) {
        if (node->stored()) return KTC_OK;
        ktc_buf h;
        return force(node, &h, nullptr);
    }
    // an alias of / a broadcast over another value: storage of its own
    node_ref(node);                                       // the cell may be re-pointed while its operands are evaluated
    ktc_buf h = 0;
    int s = alloc_handle(node->dev, node->shape.volume(), &h);
    if (s == KTC_OK) {
        bool fused = false;
        s = try_fused(node->shape, {node}, {h}, {false}, nullptr, KTC_EXPR_STORE_ONLY, 0, false, false, node->dev, &fused);
        if (s == KTC_OK && !fused) { ++st_unfused; s = eager_into(node, node->shape, h); }
        if (s == KTC_OK) {
            Node* leaf = new_leaf(h, node->shape, node->dev);
            leaf->owner = cell_id(cell);
            Node* old = cell->node;
            cell->node = node_ref(leaf);
            node_unref(old);
        } else {
            B.release(h);
        }
    }
    node_unref(node);
    return s;
}

// Before `handle` is written in place: every pending expression that reads it is evaluated.
static int flush_dependents(ktc_buf handle) {
    if (!g_pending.empty()) {
        bool hit = g_pending_targets.count(handle) != 0;
        for (size_t i = 0; !hit && i < g_pending.size(); ++i) hit = has_leaf(g_pending[i].node, handle);
        if (hit) LZ_TRY(run_pending());
    }
    auto it = g_deps.find(handle);
    if (it == g_deps.end()) return KTC_OK;
    std::vector<uint64_t> refs = std::move(it->second);
    g_deps.erase(it);
    for (uint64_t id : refs) {
        Cell* c = cell_of(id);
        if (c && c->node && !c->node->stored() && has_leaf(c->node, handle)) LZ_TRY(materialize_cell(c));
    }
    return KTC_OK;
}

// ---- call-by-call evaluation of what the kernel declines -----------------------------------------------
static int call_op(Node* nd, Node* const* kids, ktc_buf out, int64_t m) {
    if (nd->kind == K_BIN) {
        Node *a = kids[0], *b = kids[1];
        if (a->kind == K_CONST || b->kind == K_CONST) {
            const bool first = a->kind == K_CONST;
            ktc_buf h; LZ_TRY(force(first ? b : a, &h, nullptr));
            return B.scalar(nd->op, out, h, (first ? a : b)->imm[0], m, first ? 1 : 0);
        }
        ktc_buf ha, hb; Shape sa, sb;
        LZ_TRY(force(a, &ha, &sa)); LZ_TRY(force(b, &hb, &sb));
        if (sa == sb) return B.binary(nd->op, out, ha, hb, m);
        return B.binary_bcast(nd->op, out, ha, sa.d, sa.nd, hb, sb.d, sb.nd);
    }
    ktc_buf h; LZ_TRY(force(kids[0], &h, nullptr));
    switch (nd->kind) {
    case K_UN: return B.unary(nd->op, out, h, m);
    case K_SQUARE: return B.scalar(KTC_POW, out, h, 2.0f, m, 0);
    case K_CLAMP: return B.clamp(out, h, nd->imm[0], nd->imm[1], m);
    case K_CMP: return B.compare_scalar(nd->op, out, h, nd->imm[0], m);
    default: return fail(KTC_ESTATE, "cannot evaluate an expression node of kind %d", (int)nd->kind);
    }
}

// One step of the call-by-call evaluation: the operands of `node` are forced into memory (each as a fused
// program where possible), then the library call for `node` itself runs at the operation's natural shape --
// the common shape of its operands with broadcast markers looked through -- and the result is spread to
// `shape` if that is larger.
static int eager_into(Node* node, const Shape& shape, ktc_buf out) {
    Node* nd = strip(node);
    const int64_t n = shape.volume();
    auto spread = [&](ktc_buf h, const Shape& shp) -> int {
        if (shp.volume() == n) return B.d2d(out, 0, h, 0, n);
        return B.broadcast_to(out, shape.d, shape.nd, h, shp.d, shp.nd);
    };
    if ((nd->kind == K_REDUCE || nd->kind == K_SOFTMAX || nd->kind == K_NLL) && !nd->stored()) { ktc_buf h; LZ_TRY(force(nd, &h, nullptr)); }
    if (nd->stored()) return spread(nd->buf, nd->shape);
    if (nd->kind == K_CONST) return B.fill(out, 0, n, nd->imm[0]);
    node_ref(nd);
    Node* kids[2] = {nullptr, nullptr};
    Shape natural; bool have = false;
    for (int i = 0; i < nd->nargs; ++i) {
        kids[i] = strip(nd->args[i]);
        node_ref(kids[i]);
        if (kids[i]->kind == K_CONST) continue;
        if (!have) { natural = kids[i]->shape; have = true; }
        else if (natural != kids[i]->shape) { Shape c; common_shape(natural, kids[i]->shape, &c); natural = c; }
    }
    const int nk = nd->nargs;
    const int64_t m = natural.volume();
    int s;
    if (m == n) {
        s = call_op(nd, kids, out, m);
    } else {
        ktc_buf tmp = 0;
        s = alloc_handle(nd->dev, m, &tmp);
        if (s == KTC_OK) {
            s = call_op(nd, kids, tmp, m);
            if (s == KTC_OK) s = spread(tmp, natural);
            B.release(tmp);
        }
    }
    for (int i = 0; i < nk; ++i) node_unref(kids[i]);
    node_unref(nd);
    return s;
}

// ---- SoftmaxCrossEntropy's forward as a pending value ---------------------------------------------------
static Node* nll_of(Node* sm) {
    for (Node* p : sm->parents) if (p->kind == K_NLL && !p->stored()) return p;
    return nullptr;
}

// the pending K_SOFTMAX nodes under `roots`: `direct` are read by the expressions themselves, `via_nll` only through
// their K_NLL
static void find_rows(Node* const* roots, int n, std::vector<Node*>& direct, std::vector<Node*>& via_nll) {
    const uint32_t ep = ++g_epoch;
    struct Item { Node* n; bool from_nll; };
    std::vector<Item> stack;
    for (int i = 0; i < n; ++i) if (roots[i] && roots[i]->has_row) stack.push_back({roots[i], false});
    while (!stack.empty()) {
        Item it = stack.back(); stack.pop_back();
        Node* x = it.n;
        if (x->stored() || x->kind == K_REDUCE) continue;
        if (x->kind == K_SOFTMAX) {
            auto& into = it.from_nll ? via_nll : direct;
            if (std::find(into.begin(), into.end(), x) == into.end()) into.push_back(x);
            continue;
        }
        if (x->epoch == ep) continue;
        x->epoch = ep;
        for (int i = 0; i < x->nargs; ++i) if (x->args[i]->has_row) stack.push_back({x->args[i], x->kind == K_NLL});
    }
}

// Runs every pending softmax forward under `roots`, so that what is left is an ordinary expression.
static int settle_rows(Node* const* roots, int n) {
    bool any = false;
    for (int i = 0; i < n; ++i) any = any || (roots[i] && roots[i]->has_row);
    if (!any) return KTC_OK;
    std::vector<Node*> direct, via_nll;
    find_rows(roots, n, direct, via_nll);
    for (Node* sm : direct) node_ref(sm);
    for (Node* sm : via_nll) node_ref(sm);
    int s = KTC_OK;
    for (Node* sm : direct) if (s == KTC_OK && !sm->stored()) s = run_softmax(sm, true);
    for (Node* sm : via_nll) if (s == KTC_OK && !sm->stored()) s = run_softmax(sm, false);
    for (Node* sm : direct) node_unref(sm);
    for (Node* sm : via_nll) node_unref(sm);
    return s;
}

// After a program over `order` has run with the softmax in registers: does anything still need it in memory?  A cell
// that waits for it, or a reader outside the program.  (A cell that waits for an interior value of the program which the
// program did not store gets that value, if it ever asks, as any recomputed interior value: from the operands -- here
// the logits, through the forward once more.)
static bool softmax_needed_later(Node* sm, const std::vector<Node*>& order, const std::vector<Node*>& store_nodes) {
    if (waiting(sm)) return true;
    std::vector<Node*> seen, stack(sm->parents.begin(), sm->parents.end());
    while (!stack.empty()) {
        Node* p = stack.back(); stack.pop_back();
        if (p->kind == K_NLL || p->stored() || std::find(seen.begin(), seen.end(), p) != seen.end()) continue;
        seen.push_back(p);
        if (std::find(order.begin(), order.end(), p) == order.end()) return true;
        if (std::find(store_nodes.begin(), store_nodes.end(), p) != store_nodes.end()) continue;      // in memory from now on
        stack.insert(stack.end(), p->parents.begin(), p->parents.end());
    }
    return false;
}

static constexpr ktc_buf kSoftmaxInRegisters = ~(ktc_buf)0;      // stands for the softmax's buffer while a program is compiled around it
static std::vector<Node*> g_rows_busy;                            // K_SOFTMAX nodes whose evaluation is under way

// `stores` as the epilogue of the one pending softmax forward underneath them.  *fused = false: not of that form (or
// the library declined), nothing was run.
static int try_fused_softmax(const Shape& shape, const std::vector<Node*>& stores, const std::vector<ktc_buf>& handles, const std::vector<bool>& own,
                             Node* acc, int sink, int dev, bool* fused) {
    *fused = false;
    if (acc || sink != KTC_EXPR_STORE_ONLY || shape.nd != 2 || stores.empty() || !B.softmax_fwd_expr) return KTC_OK;
    std::vector<Node*> direct, via_nll;
    find_rows(stores.data(), (int)stores.size(), direct, via_nll);
    if (direct.size() != 1 || !via_nll.empty()) return KTC_OK;
    Node* sm = direct[0];
    if (sm->shape != shape) return KTC_OK;
    node_ref(sm);
    Node* nll = nll_of(sm);
    if (nll) node_ref(nll);
    auto done = [&](int s) { if (nll) node_unref(nll); node_unref(sm); return s; };
    const ktc_buf h_logits = sm->args[0]->buf, h_targets = sm->args[1]->buf;
    const float lo = sm->imm[0], hi = sm->imm[1];
    Program prog;
    std::vector<Node*> store_nodes;
    int n_req = 0;
    sm->buf = kSoftmaxInRegisters;                         // the program sees the softmax as a value in memory: one of its leaves
    compile_program(prog, shape, stores, {}, false, opt_recompute_limit, opt_store_cost, store_nodes, &n_req);
    sm->buf = 0;
    if (!prog.ok) return done(KTC_OK);
    int soft_leaf = -1, n_soft = 0;
    for (size_t i = 0; i < prog.leaves.size(); ++i) if (prog.leaves[i].first == kSoftmaxInRegisters) { soft_leaf = (int)i; ++n_soft; }
    if (n_soft != 1) return done(KTC_OK);
    const int64_t rows = shape.d[0], cols = shape.d[1], total = rows * cols;
    const bool keep = softmax_needed_later(sm, prog.order, store_nodes);
    std::vector<ktc_buf> fresh;                            // buffers allocated here, released on failure
    auto fail_with = [&](int s) { for (ktc_buf h : fresh) B.release(h); return done(s); };
    ktc_buf h_soft = 0, h_nll = 0;
    int s = KTC_OK;
    if (keep) { s = alloc_handle(dev, total, &h_soft); if (s != KTC_OK) return fail_with(s); fresh.push_back(h_soft); }
    s = alloc_handle(dev, rows, &h_nll); if (s != KTC_OK) return fail_with(s); fresh.push_back(h_nll);
    std::vector<ktc_buf> all(handles);
    for (size_t i = n_req; i < store_nodes.size(); ++i) {
        ktc_buf h = 0;
        s = alloc_handle(dev, total, &h); if (s != KTC_OK) return fail_with(s);
        fresh.push_back(h); all.push_back(h);
    }
    std::vector<ktc_buf> lh; std::vector<int64_t> ls;
    for (auto& l : prog.leaves) { lh.push_back(l.first == kSoftmaxInRegisters ? 0 : l.first); ls.push_back(l.second.d[0]); ls.push_back(l.second.d[1]); }
    const float zero = 0.f;
    const int rc = B.softmax_fwd_expr(h_soft, h_nll, h_logits, h_targets, rows, cols, lo, hi, prog.code.data(), (int)prog.code.size(),
                                      prog.imm.empty() ? &zero : prog.imm.data(), (int)prog.imm.size(), lh.data(), ls.data(), (int)lh.size(), soft_leaf,
                                      all.data(), (int)all.size());
    if (rc != KTC_OK) return fail_with(rc == KTC_ENOTSUP ? KTC_OK : rc);
    ++st_fused;
    *fused = true;
    for (Node* n : prog.order) ++n->evals;
    for (int i = 0; i < n_req; ++i) if (own[i]) adopt(store_nodes[i], handles[i]);
    for (size_t i = n_req; i < store_nodes.size(); ++i) adopt(store_nodes[i], all[handles.size() + (i - n_req)]);
    if (keep) adopt(sm, h_soft);
    if (nll && !nll->stored()) adopt(nll, h_nll); else B.release(h_nll);
    return done(KTC_OK);
}

// The forward on its own: softmax (if anything wants it in memory) and nll.
static int run_softmax_alone(Node* sm, Node* nll, bool want_softmax) {
    bool keep = want_softmax || waiting(sm);
    for (Node* p : sm->parents) keep = keep || p->kind != K_NLL;
    const int64_t rows = sm->shape.d[0], cols = sm->shape.d[1];
    ktc_buf h_soft = 0, h_nll = 0;
    if (keep) LZ_TRY(alloc_handle(sm->dev, rows * cols, &h_soft));
    int s = alloc_handle(sm->dev, rows, &h_nll);
    if (s == KTC_OK) s = B.softmax_fwd(h_soft, h_nll, sm->args[0]->buf, sm->args[1]->buf, rows, cols, sm->imm[0], sm->imm[1]);
    if (s != KTC_OK) { if (h_soft) B.release(h_soft); if (h_nll) B.release(h_nll); return s; }
    if (nll && !nll->stored()) adopt(nll, h_nll); else B.release(h_nll);
    if (keep) adopt(sm, h_soft);
    return KTC_OK;
}

// Evaluate a pending softmax forward because its softmax (want_softmax) or its nll is needed.  Recorded expressions
// that read the softmax go first: the one that has its shape takes the forward into its own kernel.
static int run_softmax(Node* sm, bool want_softmax) {
    if (sm->stored()) return KTC_OK;
    node_ref(sm);
    Node* nll = nll_of(sm);
    if (nll) node_ref(nll);
    int s = KTC_OK;
    const bool busy = std::find(g_rows_busy.begin(), g_rows_busy.end(), sm) != g_rows_busy.end();
    if (!busy) {
        g_rows_busy.push_back(sm);
        // the cells at the top of what has been built on the softmax
        std::vector<uint64_t> tops;
        std::vector<Node*> seen, stack(sm->parents.begin(), sm->parents.end());
        while (!stack.empty()) {
            Node* p = stack.back(); stack.pop_back();
            if (p->kind == K_NLL || p->kind == K_REDUCE || p->stored() || std::find(seen.begin(), seen.end(), p) != seen.end()) continue;
            seen.push_back(p);
            if (p->parents.empty() && waiting(p) && p->shape == sm->shape && std::find(g_evaluating.begin(), g_evaluating.end(), p) == g_evaluating.end())
                tops.push_back(p->owner);
            stack.insert(stack.end(), p->parents.begin(), p->parents.end());
        }
        for (uint64_t id : tops) {
            Cell* c = cell_of(id);
            if (s == KTC_OK && c && c->node && !c->node->stored() && !sm->stored()) s = materialize_cell(c);
        }
        g_rows_busy.erase(std::find(g_rows_busy.begin(), g_rows_busy.end(), sm));
    }
    const bool have = want_softmax ? sm->stored() : (sm->stored() || !nll || nll->stored());
    if (s == KTC_OK && !have) s = run_softmax_alone(sm, nll, want_softmax);
    if (nll) node_unref(nll);
    node_unref(sm);
    return s;
}

// ---- pending sums ---------------------------------------------------------------------------------------
// An all-reduce asked for while sums are pending (ktc_lazy_allreduce): when the sums turn out to be ONE pass whose
// second-pass kernel also applies every pending update, that kernel performs the exchange too.
struct Exchange {
    uint64_t comm = 0;
    std::vector<Node*> nodes;               // the values to sum over the ranks: stored nodes, or pending sums of the pass
    bool done = false;
};
struct Update { uint64_t seq; ktc_buf target; Node* nd; bool from_zero; };

// add_to[i]: the buffer node i's sum is also added to (0: none).  x: the exchange to fold in, or null.
static int try_fused_sums(const Shape& shape, const std::vector<Node*>& nodes, const std::vector<ktc_buf>& add_to, const std::vector<int>& add_mode,
                          Exchange* x, bool* fused) {
    *fused = false;
    std::vector<Node*> exprs; std::vector<int> kinds, means;
    bool any_rows = false;
    for (Node* nd : nodes) { exprs.push_back(nd->args[0]); kinds.push_back(nd->op); means.push_back(nd->imm[0] != 0.f ? 1 : 0); any_rows = any_rows || nd->op == KTC_EXPR_SUM_ROWS; }
    LZ_TRY(settle_rows(exprs.data(), (int)exprs.size()));
    Program prog;
    std::vector<Node*> store_nodes; int n_req = 0;
    // every consumer known so far sits in this pass: nothing is stored on the side for its cost alone
    compile_program(prog, shape, {}, exprs, true, opt_recompute_limit, 0, store_nodes, &n_req);
    if (!prog.ok) return KTC_OK;
    if (any_rows && !as_rows(prog, shape)) return KTC_OK;
    const int dev = nodes[0]->dev;
    std::vector<ktc_buf> outs, extra;
    auto drop = [&]() { for (ktc_buf h : outs) B.release(h); for (ktc_buf h : extra) B.release(h); };
    for (Node* nd : nodes) { ktc_buf h = 0; const int s = alloc_handle(dev, nd->shape.volume(), &h); if (s != KTC_OK) { drop(); return s; } outs.push_back(h); }
    for (size_t i = 0; i < store_nodes.size(); ++i) { ktc_buf h = 0; const int s = alloc_handle(dev, shape.volume(), &h); if (s != KTC_OK) { drop(); return s; } extra.push_back(h); }
    std::vector<ktc_buf> lh; std::vector<int64_t> ls;
    pack_leaves(prog, lh, ls);
    const ktc_buf none = 0; const float zero = 0.f;
    std::vector<ktc_buf> xb; std::vector<int64_t> xc;
    if (x) {
        for (Node* n : x->nodes) {
            ktc_buf h = n->buf;
            for (size_t i = 0; !h && i < nodes.size(); ++i) if (nodes[i] == n) h = outs[i];
            if (!h) { x = nullptr; break; }               // not a value of this pass: the exchange runs on its own afterwards
            xb.push_back(h); xc.push_back(n->shape.volume());
        }
    }
    const int rc = B.expr_eval_multi_fused(prog.code.data(), (int)prog.code.size(), prog.imm.empty() ? &zero : prog.imm.data(), (int)prog.imm.size(),
                                           prog.shape.d, prog.shape.nd, lh.data(), ls.data(), (int)prog.leaves.size(),
                                           extra.empty() ? &none : extra.data(), (int)extra.size(), kinds.data(), outs.data(), means.data(), (int)nodes.size(),
                                           add_to.data(), add_mode.data(), x ? x->comm : 0, x ? xb.data() : nullptr, x ? xc.data() : nullptr, x ? (int)xb.size() : 0);
    if (rc != KTC_OK) { drop(); return rc == KTC_ENOTSUP ? KTC_OK : rc; }
    ++st_fused; ++st_multi;
    if (x) { x->done = true; ++st_fused_exchanges; }
    *fused = true;
    for (Node* n : prog.order) ++n->evals;
    for (size_t i = 0; i < store_nodes.size(); ++i) adopt(store_nodes[i], extra[i]);
    for (size_t i = 0; i < nodes.size(); ++i) adopt(nodes[i], outs[i]);
    return KTC_OK;
}

// A single pending sum: fused with its expression, else the expression is evaluated and reduced by the
// library's reduction call.
static int run_one_sum(Node* nd) {
    Node* expr = node_ref(nd->args[0]);
    const Shape shape = expr->shape;
    const bool mean = nd->imm[0] != 0.f;
    ktc_buf out = 0;
    int s = alloc_handle(nd->dev, nd->shape.volume(), &out);
    if (s != KTC_OK) { node_unref(expr); return s; }
    bool ok = false;
    s = try_fused(shape, {}, {}, {}, expr, nd->op, out, mean, nd->op == KTC_EXPR_SUM_ROWS, nd->dev, &ok);
    if (s == KTC_OK && !ok) {
        ++st_unfused;
        ktc_buf h; Shape shp;
        s = force(expr, &h, &shp);
        const int64_t n = shape.volume();
        ktc_buf tmp = 0;
        if (s == KTC_OK && shp.volume() != n) {           // a broadcast marker over a smaller value
            s = alloc_handle(nd->dev, n, &tmp);
            if (s == KTC_OK) { h = tmp; s = eager_into(expr, shape, tmp); }
        }
        if (s == KTC_OK) {
            if (nd->op == KTC_EXPR_SUM_ALL) s = B.reduce_all(mean ? KTC_MEAN : KTC_SUM, out, h, n);
            else if (nd->op == KTC_EXPR_SUM_LAST) s = B.reduce_axis(KTC_SUM, out, h, n / shape.d[shape.nd - 1], shape.d[shape.nd - 1], 1);
            else s = B.reduce_axis(KTC_SUM, out, h, 1, shape.d[0], n / shape.d[0]);
        }
        if (tmp) B.release(tmp);
    }
    node_unref(expr);
    if (s != KTC_OK) { B.release(out); return s; }
    adopt(nd, out);
    return KTC_OK;
}

// Evaluate every pending sum that is still wanted, then apply the pending updates in the order they were
// requested.  Sums over the same iteration space run as one multi-sink pass (up to KTC_EXPR_MAX_SINKS per
// pass); a sum whose expression contains another pending sum waits for it.
static int run_pending(Exchange* x) {
    std::vector<Pending> entries;
    entries.swap(g_pending);
    std::unordered_map<ktc_buf, int> target_count;
    target_count.swap(g_pending_targets);
    struct Todo { Node* nd; };
    std::vector<Node*> todo;
    std::vector<Update> ups;
    for (Pending& e : entries) {
        if (!e.strong) node_ref(e.node);                  // keep every sum alive until this call is over
        if (!e.node->stored()) todo.push_back(e.node);
        for (size_t i = 0; i < e.targets.size(); ++i) ups.push_back({e.seq[i], e.targets[i], e.node, e.from_zero[i] != 0});
    }
    std::sort(ups.begin(), ups.end(), [](const Update& a, const Update& b) { return a.seq < b.seq; });
    // an update is folded into the second pass of its sum when it is the only update of its buffer and the only one
    // hanging on its sum (then its place in the order of the calls cannot matter), and the sum is not read by the pass
    auto foldable = [&](const Update& u) {
        if (target_count[u.target] != 1) return false;
        int n = 0;
        for (const Update& v : ups) n += v.nd == u.nd;
        return n == 1 && !u.nd->stored() && u.nd->op != KTC_EXPR_SUM_LAST;
    };
    std::vector<char> folded(ups.size(), 0);
    int status = KTC_OK;
    std::vector<Node*> waiting_nodes(todo);
    int passes = 0;
    while (status == KTC_OK && !waiting_nodes.empty()) {
        std::vector<Node*> ready, rest;
        for (Node* nd : waiting_nodes) { Node* e = nd->args[0]; (has_pending_sum(&e, 1) ? rest : ready).push_back(nd); }
        if (ready.empty()) { status = fail(KTC_ESTATE, "pending sums depend on one another"); break; }
        waiting_nodes.swap(rest);
        // one pass per iteration space; leading-axis sums view the space as [A, rest], last-axis sums need its
        // innermost dimension, so the two kinds do not share a pass (full sums join either)
        std::vector<std::pair<Shape, std::vector<Node*>>> by_shape;
        for (Node* nd : ready) {
            const Shape& s = nd->args[0]->shape;
            auto it = std::find_if(by_shape.begin(), by_shape.end(), [&](const std::pair<Shape, std::vector<Node*>>& p) { return p.first == s; });
            if (it == by_shape.end()) { by_shape.push_back({s, {}}); it = by_shape.end() - 1; }
            it->second.push_back(nd);
        }
        std::vector<std::pair<Shape, std::vector<Node*>>> groups;
        for (auto& bs : by_shape) {
            std::vector<Node*> last, rows, full;
            for (Node* nd : bs.second) (nd->op == KTC_EXPR_SUM_LAST ? last : nd->op == KTC_EXPR_SUM_ROWS ? rows : full).push_back(nd);
            if (!rows.empty() || last.empty()) { rows.insert(rows.end(), full.begin(), full.end()); groups.push_back({bs.first, rows}); full.clear(); }
            if (!last.empty()) { last.insert(last.end(), full.begin(), full.end()); groups.push_back({bs.first, last}); }
        }
        for (auto& g : groups) {
            for (size_t i = 0; status == KTC_OK && i < g.second.size(); i += KTC_EXPR_MAX_SINKS) {
                std::vector<Node*> chunk(g.second.begin() + i, g.second.begin() + std::min(g.second.size(), i + KTC_EXPR_MAX_SINKS));
                bool fused = false;
                ++passes;
                if (chunk.size() > 1) {
                    std::vector<ktc_buf> add_to(chunk.size(), 0);
                    std::vector<int> add_mode(chunk.size(), 0);
                    std::vector<size_t> which(chunk.size(), 0);
                    size_t n_fold = 0;
                    for (size_t k = 0; k < ups.size(); ++k)
                        for (size_t c = 0; c < chunk.size(); ++c)
                            if (ups[k].nd == chunk[c] && foldable(ups[k])) { add_to[c] = ups[k].target; add_mode[c] = ups[k].from_zero ? 2 : 1; which[c] = k; ++n_fold; }
                    // the exchange joins only when this is the whole of the pending work: one pass, every update in it
                    const bool whole = passes == 1 && waiting_nodes.empty() && groups.size() == 1 && g.second.size() == chunk.size() && n_fold == ups.size();
                    status = try_fused_sums(g.first, chunk, add_to, add_mode, (x && whole) ? x : nullptr, &fused);
                    if (status == KTC_OK && fused)
                        for (size_t c = 0; c < chunk.size(); ++c) if (add_to[c]) { folded[which[c]] = 1; ++st_fused_updates; }
                }
                for (size_t j = 0; status == KTC_OK && !fused && j < chunk.size(); ++j) status = run_one_sum(chunk[j]);
            }
        }
    }
    for (size_t k = 0; status == KTC_OK && k < ups.size(); ++k) {
        if (folded[k]) continue;
        const int64_t n = ups[k].nd->shape.volume();
        if (ups[k].from_zero) status = B.fill(ups[k].target, 0, n, 0.f);
        if (status == KTC_OK) status = B.binary_inplace(KTC_PLUS, ups[k].target, ups[k].nd->buf, n);
    }
    for (Pending& e : entries) {
        for (ktc_buf h : e.targets) B.release(h);
        node_unref(e.node);
    }
    return status;
}

// Remember `buffer handle += node` (node: a pending sum).  The node is kept alive from here on.
static bool add_pending_update(Node* node, ktc_buf handle, bool from_zero = false) {
    for (Pending& e : g_pending) {
        if (e.node != node) continue;
        if (B.retain(handle) != KTC_OK) return false;
        if (!e.strong) { e.strong = true; node_ref(node); }
        e.targets.push_back(handle);
        e.seq.push_back(++g_update_seq);
        e.from_zero.push_back(from_zero ? 1 : 0);
        ++g_pending_targets[handle];
        return true;
    }
    return false;
}

static uint64_t defer_sum(Node* expr, int kind, bool mean, const Shape& res_shape) {
    const float m = mean ? 1.f : 0.f;
    Node* n = new_node(K_REDUCE, res_shape, kind, expr, nullptr, &m, 1);
    const uint64_t id = new_cell(node_ref(n));
    register_cell(id, n);
    g_pending.push_back({n, false, {}, {}, {}});
    return id;
}

// ---- operands -------------------------------------------------------------------------------------------
// the node under a cell as an operand of a new expression
static int operand(uint64_t id, Node** out) {
    Cell* c = cell_of(id);
    if (!c || !c->node) return fail(KTC_ESTATE, "stale or unknown expression cell");
    Node* n = c->node;
    if (n->stored() && !g_pending_targets.empty() && g_pending_targets.count(n->buf)) {
        LZ_TRY(run_pending());                            // a `+= pending sum` update of this buffer is due
        c = cell_of(id);
        n = c->node;
    }
    *out = n;
    return KTC_OK;
}

// target = f(target, ...) in place.  state: 0 the target's buffer was written (or will be, by a recorded
// update: 2); 1 the cell is pending now (a caller that held the buffer drops its reference).
static int assign(uint64_t target_id, Kind kind, int op, Node* a0, Node* a1, const float* imm, int nimm, int* state) {
    Cell* cell = cell_of(target_id);
    Node* own = cell->node;
    if (!own->stored() && own->has_row) {
        // The target is an expression over a pending softmax forward, and so is the operand (a gradient accumulated over two
        // steps): in one expression neither forward could take its consumer along, so the target is evaluated first -- with
        // its own forward -- and the new expression starts from the stored result.
        Node* other = a0 == own ? a1 : a0;
        if (other && other != own && other->has_row && !other->stored()) {
            const bool first = a0 == own, second = a1 == own;
            node_ref(other);
            const int ms = materialize_cell(cell);
            cell = cell_of(target_id);
            if (ms == KTC_OK && cell) {
                own = cell->node;
                if (first) a0 = own;
                if (second) a1 = own;
            }
            node_unref(other);                            // still held by the caller's cell
            if (ms != KTC_OK) return ms;
            if (!cell) return fail(KTC_ESTATE, "in-place call on a cell that went away");
        }
    }
    Node* node = new_node(kind, own->shape, op, a0, a1, imm, nimm);
    node_ref(node);
    auto done = [&](int s, int st) { if (state) *state = st; node_unref(node); return s; };
    if (!own->stored() && kind == K_BIN && op == KTC_PLUS && !g_pending.empty()) {
        // zeroed pending target += pending sum (a gradient cleared with zeroGrad, then accumulated into): the cell gets a
        // buffer of its own that receives 0f + sum when the sums run -- in the second pass of their kernel where possible
        Node* zero = strip(own);
        Node* other = strip(a1);
        if (zero->kind == K_CONST && zero->imm[0] == 0.f && !std::signbit(zero->imm[0]) && a0 == own && other->kind == K_REDUCE && !other->stored()
            && other->shape.volume() == own->shape.volume()) {
            ktc_buf h = 0;
            const int s = alloc_handle(other->dev, own->shape.volume(), &h);
            if (s != KTC_OK) return done(s, 0);
            if (add_pending_update(other, h, true)) {
                Node* leaf = new_leaf(h, own->shape, other->dev);
                leaf->owner = target_id;
                cell->node = node_ref(leaf);
                node_unref(own);
                return done(KTC_OK, 3);
            }
            B.release(h);
        }
    }
    if (!own->stored()) {                                 // a pending target takes the new value
        cell->node = node_ref(node);
        register_cell(target_id, node);
        node_unref(own);
        return done(KTC_OK, 1);
    }
    if (strip(own) != own) return done(fail(KTC_ESTATE, "in-place call on a broadcast marker"), 0);
    const ktc_buf h = own->buf;
    const int64_t n = own->shape.volume();
    node_ref(own);
    auto finish = [&](int s, int st) { node_unref(own); return done(s, st); };
    int s = flush_dependents(h);
    if (s != KTC_OK) return finish(s, 0);
    Node* other = kind == K_BIN ? strip(a1) : nullptr;
    if (node->has_sum && !g_pending.empty()) {
        if (other && op == KTC_PLUS && other->kind == K_REDUCE && !other->stored() && other->shape.volume() == n && strip(a0)->stored()
            && add_pending_update(other, h))
            return finish(KTC_OK, 2);                     // target += pending sum: applied when the sums run
        s = run_pending();
        if (s != KTC_OK) return finish(s, 0);
    }
    if (other && (other->kind == K_CONST || (other->stored() && other->shape.volume() == n))) {
        // nothing to fuse: the operand is already in memory (a gradient accumulated into a Variable, ...)
        if (other->kind == K_CONST) return finish(B.scalar_inplace(op, h, other->imm[0], n), 0);
        return finish(B.binary_inplace(op, h, other->buf, n), 0);
    }
    cell = cell_of(target_id);
    if (opt_defer_inplace && cell->node == own && (a0 == own || a1 == own)) {
        // Nobody else holds the buffer (this cell's node, and the caller's reference if it ever asked for it): instead of a pass that
        // rewrites the buffer now, the cell becomes pending -- its node reads the old buffer as an operand -- so that
        // the in-place calls that follow join one program.  A buffer with another holder (a view, a shallow copy, a
        // pending expression that still reads it) is written in place as before.
        int cnt = 0;
        s = B.refcount(h, &cnt);
        if (s != KTC_OK) return finish(s, 0);
        if (cnt == 2 || cnt == 1) {
            cell->node = node_ref(node);
            register_cell(target_id, node);
            node_unref(own);                              // the cell's reference; `node` keeps the leaf and its buffer
            return finish(KTC_OK, 1);
        }
    }
    bool fused = false;
    s = try_fused(own->shape, {node}, {h}, {false}, nullptr, KTC_EXPR_STORE_ONLY, 0, false, false, own->dev, &fused);
    if (s != KTC_OK || fused) return finish(s, 0);
    ++st_unfused;
    if (kind == K_SQUARE) return finish(B.scalar_inplace(KTC_POW, h, 2.0f, n), 0);
    if (kind == K_SCATC) return finish(fail(KTC_ENOTSUP, "this scatter is not fusable here: use ktc_scatter_axis_nd on the buffers"), 0);
    if (kind != K_BIN) return finish(fail(KTC_ESTATE, "in-place call of kind %d", (int)kind), 0);
    if (other->kind == K_CONST) return finish(B.scalar_inplace(op, h, other->imm[0], n), 0);
    ktc_buf hb; Shape shp;
    s = force(other, &hb, &shp);
    if (s != KTC_OK) return finish(s, 0);
    if (shp.volume() != n) {                              // a broadcast marker over a smaller value
        ktc_buf tmp = 0;
        s = alloc_handle(own->dev, n, &tmp);
        if (s == KTC_OK) { s = eager_into(a1, own->shape, tmp); if (s == KTC_OK) s = B.binary_inplace(op, h, tmp, n); B.release(tmp); }
        return finish(s, 0);
    }
    return finish(B.binary_inplace(op, h, hb, n), 0);
}

}  // namespace lz
}  // namespace ktc

// ---- the C ABI ------------------------------------------------------------------------------------------
using namespace ktc::lz;
#define LZ_LOCK std::lock_guard<std::mutex> lock_(g_mu)

extern "C" {

#ifdef KTC_LAZY_STANDALONE
KTC_API int ktc_lazy_test_set_backend(void* const* table, int n) {
    if (n != kBackendEntries) return KTC_EINVAL;
    memcpy(&B, table, sizeof(B));
    return KTC_OK;
}
KTC_API const char* ktc_last_error(void) { return g_err; }
#endif

KTC_API int ktc_lazy_leaf(ktc_buf buf, const int64_t* shape, int ndim, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (!out || ndim < 0 || ndim > MAXD) return fail(KTC_EINVAL, "ktc_lazy_leaf: bad arguments");
    int dev = 0; int64_t n = 0;
    LZ_TRY(B.buf_info(buf, &dev, &n, nullptr));
    const Shape s = make_shape(shape, ndim);
    if (s.volume() > n) return fail(KTC_EINVAL, "ktc_lazy_leaf: shape holds %lld elements, the buffer %lld", (long long)s.volume(), (long long)n);
    LZ_TRY(B.retain(buf));
    Node* leaf = new_leaf(buf, s, dev);
    *out = new_cell(node_ref(leaf));
    leaf->owner = *out;
    return KTC_OK;
}

KTC_API int ktc_lazy_free(ktc_lazy_cell cell) {
    LZ_LOCK;
    Cell* c = cell_of(cell);
    if (!c) return fail(KTC_ESTATE, "ktc_lazy_free: stale or unknown cell");
    Node* n = c->node;
    c->node = nullptr; c->live = false; ++c->gen;
    g_free_cells.push_back((uint32_t)(c - g_cells.data()));
    node_unref(n);
    return KTC_OK;
}

KTC_API int ktc_lazy_unary(int op, ktc_lazy_cell a, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (!unary_recordable(op)) return fail(KTC_ENOTSUP, "ktc_lazy_unary: op %d is not an expression instruction", op);
    Node* na; LZ_TRY(operand(a, &na));
    *out = pending_cell(K_UN, na->shape, op, na, nullptr, nullptr, 0);
    return KTC_OK;
}

KTC_API int ktc_lazy_binary(int op, ktc_lazy_cell a, ktc_lazy_cell b, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_lazy_binary: unknown op %d", op);
    Node *na, *nb;
    LZ_TRY(operand(a, &na)); LZ_TRY(operand(b, &nb)); LZ_TRY(operand(a, &na));
    Shape common;
    if (!common_shape(na->shape, nb->shape, &common)) return fail(KTC_EINVAL, "ktc_lazy_binary: shapes do not broadcast");
    *out = pending_cell(K_BIN, common, op, na, nb, nullptr, 0);
    return KTC_OK;
}

static int scalar_node(int op, Node* me, float s, int scalar_first, Kind* kind, Node** a0, Node** a1) {
    if (op == KTC_POW && !scalar_first && s == 2.0f) { *kind = K_SQUARE; *a0 = me; *a1 = nullptr; return 0; }
    Node* c = new_const(s);
    *kind = K_BIN;
    *a0 = scalar_first ? c : me; *a1 = scalar_first ? me : c;
    return 1;                                             // a constant node was created (one floating reference to drop)
}

KTC_API int ktc_lazy_scalar(int op, ktc_lazy_cell a, float s, int scalar_first, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_lazy_scalar: unknown op %d", op);
    Node* na; LZ_TRY(operand(a, &na));
    if (op == KTC_POW && !scalar_first && s == 1.0f) {    // x pow 1 is x: a deep copy that is not made yet
        *out = pending_cell(K_BCAST, na->shape, 0, na, nullptr, nullptr, 0);
        return KTC_OK;
    }
    Kind kind; Node *a0, *a1;
    const int made = scalar_node(op, na, s, scalar_first, &kind, &a0, &a1);
    Node* c = made ? (scalar_first ? a0 : a1) : nullptr;
    if (c) node_ref(c);
    *out = pending_cell(kind, na->shape, kind == K_SQUARE ? 0 : op, a0, a1, nullptr, 0);
    if (c) node_unref(c);
    return KTC_OK;
}

KTC_API int ktc_lazy_clamp(ktc_lazy_cell a, float lo, float hi, ktc_lazy_cell* out) {
    LZ_LOCK;
    Node* na; LZ_TRY(operand(a, &na));
    const float imm[2] = {lo, hi};
    *out = pending_cell(K_CLAMP, na->shape, 0, na, nullptr, imm, 2);
    return KTC_OK;
}

KTC_API int ktc_lazy_compare_scalar(int op, ktc_lazy_cell a, float value, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (op < KTC_LT || op > KTC_GTE) return fail(KTC_ENOTSUP, "ktc_lazy_compare_scalar: op %d is not an expression instruction", op);
    Node* na; LZ_TRY(operand(a, &na));
    *out = pending_cell(K_CMP, na->shape, op, na, nullptr, &value, 1);
    return KTC_OK;
}

KTC_API int ktc_lazy_broadcast_to(ktc_lazy_cell a, const int64_t* shape, int ndim, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (ndim < 0 || ndim > MAXD) return fail(KTC_EINVAL, "ktc_lazy_broadcast_to: bad rank");
    Node* na; LZ_TRY(operand(a, &na));
    const Shape s = make_shape(shape, ndim);
    Shape common;
    if (!common_shape(na->shape, s, &common) || common != s) return fail(KTC_EINVAL, "ktc_lazy_broadcast_to: shape cannot be broadcast to the target");
    *out = pending_cell(K_BCAST, s, 0, na, nullptr, nullptr, 0);
    return KTC_OK;
}

KTC_API int ktc_lazy_assign_binary(int op, ktc_lazy_cell target, ktc_lazy_cell other, int* state) {
    LZ_LOCK;
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_lazy_assign_binary: unknown op %d", op);
    Node *nt, *no;
    LZ_TRY(operand(target, &nt)); LZ_TRY(operand(other, &no)); LZ_TRY(operand(target, &nt));
    if (nt->shape != no->shape) return fail(KTC_EINVAL, "Shapes does not match for inplace operation on tensors");
    node_ref(no);
    const int s = assign(target, K_BIN, op, nt, no, nullptr, 0, state);
    node_unref(no);
    return s;
}

KTC_API int ktc_lazy_assign_scalar(int op, ktc_lazy_cell target, float s, int* state) {
    LZ_LOCK;
    if (op < KTC_PLUS || op > KTC_POW) return fail(KTC_EINVAL, "ktc_lazy_assign_scalar: unknown op %d", op);
    Node* nt; LZ_TRY(operand(target, &nt));
    Kind kind; Node *a0, *a1;
    const int made = scalar_node(op, nt, s, 0, &kind, &a0, &a1);
    if (made) node_ref(a1);
    const int st = assign(target, kind, kind == K_SQUARE ? 0 : op, a0, a1, nullptr, 0, state);
    if (made) node_unref(a1);
    return st;
}

// a pending constant of the given shape
static Node* constant_node(const Shape& s, float value, int dev) {
    Node* c = new_const(value);
    node_ref(c);
    Node* b = new_node(K_BCAST, s, 0, c, nullptr, nullptr, 0);
    b->dev = dev;
    node_unref(c);
    return b;
}

KTC_API int ktc_lazy_full(int dev, const int64_t* shape, int ndim, float value, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (!out || ndim < 0 || ndim > MAXD) return fail(KTC_EINVAL, "ktc_lazy_full: bad arguments");
    Node* n = constant_node(make_shape(shape, ndim), value, dev);
    *out = new_cell(node_ref(n));
    register_cell(*out, n);
    return KTC_OK;
}

KTC_API int ktc_lazy_assign_fill(ktc_lazy_cell target, float value, int* state) {
    LZ_LOCK;
    Cell* cell = cell_of(target);
    if (!cell || !cell->node) return fail(KTC_ESTATE, "ktc_lazy_assign_fill: stale or unknown cell");
    Node* own = cell->node;
    if (own->stored()) {
        const ktc_buf h = own->buf;
        node_ref(own);
        int s = flush_dependents(h);                      // pending readers of the old contents, pending updates of it
        cell = cell_of(target);
        int cnt = 0;
        if (s == KTC_OK) s = B.refcount(h, &cnt);
        // the holders of a buffer nobody else uses: this cell's node, and the caller's tensor if it ever asked for the buffer
        if (s != KTC_OK || !(opt_defer_inplace && cell->node == own && (cnt == 2 || cnt == 1))) {
            if (s == KTC_OK) s = B.fill(h, 0, own->shape.volume(), value);
            node_unref(own);
            if (state) *state = 0;
            return s;
        }
        node_unref(own);
    }
    Node* n = constant_node(own->shape, value, own->dev);
    cell->node = node_ref(n);
    register_cell(target, n);
    node_unref(own);
    if (state) *state = 1;
    return KTC_OK;
}

KTC_API int ktc_lazy_assign_scatter_const(ktc_lazy_cell target, ktc_lazy_cell index, float value, int* state) {
    LZ_LOCK;
    Node *nt, *ni;
    LZ_TRY(operand(target, &nt)); LZ_TRY(operand(index, &ni)); LZ_TRY(operand(target, &nt));
    const Shape &st = nt->shape, &si = ni->shape;
    bool ok = st.nd >= 1 && si.nd == st.nd && si.d[si.nd - 1] == 1 && st.d[st.nd - 1] > 1;
    for (int i = 0; ok && i + 1 < st.nd; ++i) ok = si.d[i] == st.d[i];
    if (!ok) return fail(KTC_ENOTSUP, "ktc_lazy_assign_scatter_const: the index must have the target's shape with a last extent of 1");
    if (!strip(ni)->stored()) { ktc_buf h; LZ_TRY(force(ni, &h, nullptr)); LZ_TRY(operand(target, &nt)); }
    node_ref(ni);
    const int s = assign(target, K_SCATC, 0, nt, ni, &value, 1, state);
    node_unref(ni);
    return s;
}

// The forward of SoftmaxCrossEntropy (SoftmaxCrossEntropy.kt:40-59) on logits [rows, cols] and targets (rows class indices),
// recorded: *softmax is the tensor the function saves for backward, *nll the loss per row.  Nothing runs until one of them
// is needed; an elementwise expression of the softmax's shape recorded meanwhile (the function's backward and what is
// accumulated from it) is then evaluated inside the forward's kernel, and the softmax itself is written only if a tensor
// still holds it.  KTC_ENOTSUP: rows the one-pass kernel does not take -- issue the calls.
KTC_API int ktc_lazy_softmax_xent_forward(ktc_lazy_cell logits, ktc_lazy_cell targets, float lo, float hi, ktc_lazy_cell* softmax, ktc_lazy_cell* nll) {
    LZ_LOCK;
    if (!softmax || !nll) return fail(KTC_EINVAL, "ktc_lazy_softmax_xent_forward: null output");
    if (!B.softmax_fwd) return fail(KTC_ENOTSUP, "ktc_lazy_softmax_xent_forward: the library has no one-pass forward");
    Node *lg, *tg;
    LZ_TRY(operand(logits, &lg)); LZ_TRY(operand(targets, &tg)); LZ_TRY(operand(logits, &lg));
    if (lg->shape.nd != 2) return fail(KTC_EINVAL, "ktc_lazy_softmax_xent_forward: logits of %d dimensions", lg->shape.nd);
    const int64_t rows = lg->shape.d[0], cols = lg->shape.d[1];
    if (tg->shape.volume() != rows) return fail(KTC_EINVAL, "ktc_lazy_softmax_xent_forward: %lld targets for %lld rows", (long long)tg->shape.volume(), (long long)rows);
    if (rows < 1 || cols <= 64 || cols > 12288 || (cols & 3) || strip(lg)->shape.volume() != rows * cols || strip(tg)->shape.volume() != rows)
        return fail(KTC_ENOTSUP, "ktc_lazy_softmax_xent_forward: [%lld, %lld] logits are not handled in one pass", (long long)rows, (long long)cols);
    node_ref(lg); node_ref(tg);
    ktc_buf hl = 0, ht = 0;
    int s = force(lg, &hl, nullptr);
    if (s == KTC_OK) s = force(tg, &ht, nullptr);
    void* ptr = nullptr; int dev = 0; int64_t n = 0;
    if (s == KTC_OK) s = B.buf_info(hl, &dev, &n, &ptr);
    if (s == KTC_OK && (reinterpret_cast<uintptr_t>(ptr) & 15)) s = fail(KTC_ENOTSUP, "ktc_lazy_softmax_xent_forward: the logits are not 16-byte aligned");
    if (s == KTC_OK) {
        const float imm[2] = {lo, hi};
        Node* sm = new_node(K_SOFTMAX, strip(lg)->shape, 0, strip(lg), strip(tg), imm, 2);
        Shape rs; rs.nd = 1; rs.d[0] = rows;
        Node* nl = new_node(K_NLL, rs, 0, sm, nullptr, nullptr, 0);
        *softmax = new_cell(node_ref(sm)); register_cell(*softmax, sm);
        *nll = new_cell(node_ref(nl)); register_cell(*nll, nl);
    }
    node_unref(lg); node_unref(tg);
    return s;
}

// kind: KTC_EXPR_SUM_ALL (sum() / mean()), KTC_EXPR_SUM_ROWS (sum over axis 0 of [A, ...]), KTC_EXPR_SUM_LAST
// (sum over the innermost axis); res_shape is the shape of the result.
KTC_API int ktc_lazy_sum(ktc_lazy_cell a, int kind, int mean, const int64_t* res_shape, int res_ndim, ktc_lazy_cell* out) {
    LZ_LOCK;
    if (kind != KTC_EXPR_SUM_ALL && kind != KTC_EXPR_SUM_ROWS && kind != KTC_EXPR_SUM_LAST) return fail(KTC_EINVAL, "ktc_lazy_sum: unknown kind %d", kind);
    if (res_ndim < 0 || res_ndim > MAXD) return fail(KTC_EINVAL, "ktc_lazy_sum: bad rank");
    Node* na; LZ_TRY(operand(a, &na));
    const Shape rs = make_shape(res_shape, res_ndim);
    const Shape shape = na->shape;
    if (shape.nd < 1 || (kind != KTC_EXPR_SUM_ALL && shape.nd < 2)) return fail(KTC_EINVAL, "ktc_lazy_sum: rank %d has no such axis", shape.nd);
    const int64_t n = shape.volume();
    const int64_t want = kind == KTC_EXPR_SUM_ALL ? 1 : kind == KTC_EXPR_SUM_ROWS ? n / std::max<int64_t>(1, shape.d[0]) : n / std::max<int64_t>(1, shape.d[shape.nd - 1]);
    if (rs.volume() != want) return fail(KTC_EINVAL, "ktc_lazy_sum: result shape holds %lld elements, the sum %lld", (long long)rs.volume(), (long long)want);
    Node* expr = strip(na);
    const bool pending_expr = !expr->stored() && expr->kind != K_REDUCE;
    if (opt_defer_sums && pending_expr) { *out = defer_sum(na, kind, mean != 0, rs); return KTC_OK; }
    // the sum runs now: fused with the pending expression where possible, else over the evaluated operand
    node_ref(na);
    ktc_buf res = 0;
    int s = alloc_handle(na->dev, rs.volume(), &res);
    bool fused = false;
    if (s == KTC_OK && pending_expr)
        s = try_fused(shape, {}, {}, {}, na, kind, res, mean != 0, kind == KTC_EXPR_SUM_ROWS, na->dev, &fused);
    if (s == KTC_OK && !fused) {
        ktc_buf h; Shape shp;
        s = force(na, &h, &shp);
        ktc_buf tmp = 0;
        if (s == KTC_OK && shp.volume() != n) { s = alloc_handle(na->dev, n, &tmp); if (s == KTC_OK) { h = tmp; s = eager_into(na, shape, tmp); } }
        if (s == KTC_OK) {
            if (kind == KTC_EXPR_SUM_ALL) s = B.reduce_all(mean ? KTC_MEAN : KTC_SUM, res, h, n);
            else if (kind == KTC_EXPR_SUM_LAST) s = B.reduce_axis(KTC_SUM, res, h, n / shape.d[shape.nd - 1], shape.d[shape.nd - 1], 1);
            else s = B.reduce_axis(KTC_SUM, res, h, 1, shape.d[0], n / shape.d[0]);
        }
        if (tmp) B.release(tmp);
    }
    node_unref(na);
    if (s != KTC_OK) { if (res) B.release(res); return s; }
    Node* leaf = new_leaf(res, rs, na->dev);
    *out = new_cell(node_ref(leaf));
    leaf->owner = *out;
    return KTC_OK;
}

// The buffer that holds the cell's value; a pending value is computed first.  One reference on the buffer is
// added for the caller (to be dropped with ktc_release).
KTC_API int ktc_lazy_buffer(ktc_lazy_cell cell, ktc_buf* out) {
    LZ_LOCK;
    Cell* c = cell_of(cell);
    if (!c || !c->node) return fail(KTC_ESTATE, "ktc_lazy_buffer: stale or unknown cell");
    if (!c->node->stored()) {
        LZ_TRY(materialize_cell(c));
        c = cell_of(cell);
    } else if (!g_pending_targets.empty() && g_pending_targets.count(c->node->buf)) {
        LZ_TRY(run_pending());
        c = cell_of(cell);
    }
    if (!c->node->stored()) return fail(KTC_ESTATE, "a pending value did not receive its storage");
    LZ_TRY(B.retain(c->node->buf));
    *out = c->node->buf;
    return KTC_OK;
}

// pending: 1 while the cell's value is not in memory; is_sum: 1 while it is a sum that has not run
KTC_API int ktc_lazy_info(ktc_lazy_cell cell, int* pending, int* is_sum, int64_t* shape, int* ndim) {
    LZ_LOCK;
    Cell* c = cell_of(cell);
    if (!c || !c->node) return fail(KTC_ESTATE, "ktc_lazy_info: stale or unknown cell");
    if (pending) *pending = c->node->stored() ? 0 : 1;
    if (is_sum) *is_sum = (!c->node->stored() && strip(c->node)->kind == K_REDUCE && !strip(c->node)->stored()) ? 1 : 0;
    if (ndim) *ndim = c->node->shape.nd;
    if (shape) for (int i = 0; i < c->node->shape.nd; ++i) shape[i] = c->node->shape.d[i];
    return KTC_OK;
}

// To be called before `buf` is written by any call that is not recorded here: pending expressions that read
// it -- and pending `+= sum` updates of it -- run first.
KTC_API int ktc_lazy_flush(ktc_buf buf) {
    LZ_LOCK;
    return flush_dependents(buf);
}

KTC_API int ktc_lazy_run_pending(void) {
    LZ_LOCK;
    if (g_pending.empty()) return KTC_OK;
    return run_pending();
}

// Sum the values of `cells` over the ranks of a peer-memory communicator, in place (ktc_p2p_allreduce_sum on their
// buffers).  Pending values are computed first; when all the pending work is one pass with several sums -- the loss
// and the gradients of a training step -- the exchange runs inside that pass's second-pass kernel.
KTC_API int ktc_lazy_allreduce(uint64_t comm, const ktc_lazy_cell* cells, int n) {
    LZ_LOCK;
    if (!cells || n < 1 || n > 8) return fail(KTC_EINVAL, "ktc_lazy_allreduce: 1..8 cells per call");
    Exchange x;
    x.comm = comm;
    for (int i = 0; i < n; ++i) {
        Cell* c = cell_of(cells[i]);
        if (!c || !c->node) return fail(KTC_ESTATE, "ktc_lazy_allreduce: stale or unknown cell");
        Node* nd = strip(c->node);
        if (!nd->stored() && nd->kind != K_REDUCE) { ktc_buf h; LZ_TRY(force(nd, &h, nullptr)); }      // an elementwise value: computed now
        x.nodes.push_back(node_ref(nd));
    }
    int s = KTC_OK;
    if (!g_pending.empty()) s = run_pending(&x);
    if (s == KTC_OK && !x.done) {
        std::vector<ktc_buf> bufs; std::vector<int64_t> counts;
        for (Node* nd : x.nodes) {
            ktc_buf h = 0;
            s = force(nd, &h, nullptr);
            if (s != KTC_OK) break;
            bufs.push_back(h); counts.push_back(nd->shape.volume());
        }
        if (s == KTC_OK) s = B.p2p_allreduce_sum(comm, bufs.data(), counts.data(), n);
    }
    for (Node* nd : x.nodes) node_unref(nd);
    return s;
}

// recompute_limit, store_cost, defer_sums, defer_inplace
KTC_API int ktc_lazy_option(const char* name, int value) {
    LZ_LOCK;
    if (!name) return fail(KTC_EINVAL, "ktc_lazy_option: no name");
    if (!strcmp(name, "recompute_limit")) opt_recompute_limit = value;
    else if (!strcmp(name, "store_cost")) opt_store_cost = value;
    else if (!strcmp(name, "defer_sums")) opt_defer_sums = value;
    else if (!strcmp(name, "defer_inplace")) opt_defer_inplace = value;
    else return fail(KTC_EINVAL, "ktc_lazy_option: unknown option %s", name);
    return KTC_OK;
}

// out10: programs run, expressions that fell back to separate calls, passes with several sums, sums pending now,
// program-cache hits, programs compiled, live nodes, live cells, `+= sum` updates applied by a second-pass kernel,
// all-reduces performed by a second-pass kernel
KTC_API int ktc_lazy_stats(int64_t* out10) {
    LZ_LOCK;
    if (!out10) return fail(KTC_EINVAL, "ktc_lazy_stats: no output");
    out10[0] = st_fused; out10[1] = st_unfused; out10[2] = st_multi; out10[3] = (int64_t)g_pending.size();
    out10[4] = st_cache_hits; out10[5] = st_compiles; out10[6] = g_live_nodes;
    out10[7] = (int64_t)g_cells.size() - (int64_t)g_free_cells.size();
    out10[8] = st_fused_updates; out10[9] = st_fused_exchanges;
    return KTC_OK;
}

}  // extern "C"
