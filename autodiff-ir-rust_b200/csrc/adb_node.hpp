// Lazy expression DAG used by the lowering.
//
// The reference lowers every IR command to its own kernel and then fuses adjacent kernels of equal
// size (src/kernel/fusion/elw_expr.rs:15-144); index math for aliases is kept as `Expression` trees
// built by applying the data commands in reverse (src/kernel/helper/shape.rs:51-76,
// src/kernel/indexing/matrix.rs:11-132).  Here every value is a node over its own index space:
//   LOAD   a strided read of a buffer (mixed-radix strides per axis, so merges of axes never fail)
//   CONST  a scalar broadcast to the node's shape (CreateConstant, src/core/ir.rs:11)
//   OP     + * exp2 log2 sin recip sqrt ==0 >0 <0 applied element by element
//   PIECE  concatenation of children along one axis (Concat, src/core/ir.rs:65), kept in a normal
//          form where PIECE is hoisted above OP so each piece is a plain expression
// View / Index / Permute / Broadcast are pushed down to the leaves, which is what makes them free.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

namespace adb {

using Shape = std::vector<int64_t>;

inline int64_t numel(const Shape& s) {
    int64_t n = 1;
    for (auto x : s) n *= x;
    return n;
}

struct Sub {
    int64_t size, stride;
    bool operator==(const Sub& o) const { return size == o.size && stride == o.stride; }
};

// offset + for every axis of the node a row-major list of (size, stride) digits whose sizes
// multiply to the axis length (an empty list means the axis has length 1).
struct View {
    int64_t offset = 0;
    std::vector<std::vector<Sub>> dims;
    bool operator==(const View& o) const { return offset == o.offset && dims == o.dims; }
};

inline void canon_subs(std::vector<Sub>& v) {
    std::vector<Sub> out;
    for (auto s : v) {
        if (s.size == 1) continue;
        if (!out.empty() && out.back().stride == s.stride * s.size) {
            out.back().size *= s.size;
            out.back().stride = s.stride;
        } else
            out.push_back(s);
    }
    v.swap(out);
}

inline View contiguous_view(const Shape& shape, int64_t offset = 0) {
    View v;
    v.offset = offset;
    v.dims.resize(shape.size());
    int64_t st = 1;
    for (int i = int(shape.size()) - 1; i >= 0; i--) {
        if (shape[i] != 1) v.dims[i].push_back({shape[i], st});
        st *= shape[i];
    }
    return v;
}

// all digits of a view in row-major order, canonicalised
inline std::vector<Sub> flat_subs(const View& v) {
    std::vector<Sub> all;
    for (auto& d : v.dims)
        for (auto& s : d) all.push_back(s);
    canon_subs(all);
    return all;
}

inline bool view_is_contiguous(const View& v, const Shape& shape) {
    auto f = flat_subs(v);
    int64_t n = numel(shape);
    if (n == 1) return true;
    return f.size() == 1 && f[0].stride == 1 && f[0].size == n;
}

// largest element offset touched (exclusive upper bound needs +1)
inline int64_t view_max_offset(const View& v) {
    int64_t m = v.offset;
    for (auto& d : v.dims)
        for (auto& s : d)
            if (s.stride > 0) m += (s.size - 1) * s.stride;
    return m;
}

enum NodeKind : uint8_t { N_LOAD, N_CONST, N_OP, N_PIECE };
enum EOp : uint8_t { E_ADD, E_MUL, E_EXP2, E_LOG2, E_SIN, E_RECIP, E_SQRT, E_EQZ, E_GTZ, E_LTZ };

inline bool eop_is_binary(EOp o) { return o == E_ADD || o == E_MUL; }

struct Node {
    NodeKind kind = N_CONST;
    Shape shape;
    // LOAD
    int buf = -1;
    uint32_t version = 0;
    View view;
    // CONST
    float cval = 0.f;
    // OP
    EOp op = E_ADD;
    Node* a = nullptr;
    Node* b = nullptr;
    // PIECE: kids[i] covers [ends[i-1], ends[i]) along axis pdim
    int pdim = 0;
    std::vector<int64_t> ends;
    std::vector<Node*> kids;
    // once a lazy value has been written to memory, readers are forwarded to that LOAD
    Node* fwd = nullptr;
    int64_t nops = 0;  // size of the expression as a tree (saturating); a cheap upper bound on DAG size
    uint32_t serial = 0;
};

inline float eval_unary(EOp op, float x) {
    switch (op) {
    case E_EXP2: return exp2f(x);
    case E_LOG2: return log2f(x);
    case E_SIN: return sinf(x);
    case E_RECIP: return 1.0f / x;
    case E_SQRT: return sqrtf(fabsf(x));
    case E_EQZ: return x == 0.0f ? 1.0f : 0.0f;
    case E_GTZ: return x > 0.0f ? 1.0f : 0.0f;
    case E_LTZ: return x < 0.0f ? 1.0f : 0.0f;
    default: return x;
    }
}

class Graph {
  public:
    static constexpr int64_t NOPS_CAP = int64_t(1) << 40;

    // current version of every buffer; a LOAD is valid while its version matches
    std::vector<uint32_t> buf_version;

    bool load_valid(const Node* n) const { return n->kind != N_LOAD || buf_version[n->buf] == n->version; }

    // follow forwarding pointers left behind by materialisation
    Node* canon(Node* n) const {
        while (n->fwd && load_valid(n->fwd)) n = n->fwd;
        return n;
    }

    Node* load(int buf, const Shape& shape, const View& view) { return load_cons(buf, buf_version[buf], shape, view); }

    Node* constant(float v, const Shape& shape) {
        // identical constants share one node so that common sub-expressions over them are found
        uint32_t bits;
        std::memcpy(&bits, &v, 4);
        auto range = consts_.equal_range(bits);
        for (auto it = range.first; it != range.second; ++it)
            if (it->second->shape == shape) return it->second;
        Node* n = fresh();
        consts_.emplace(bits, n);
        n->kind = N_CONST;
        n->shape = shape;
        n->cval = v;
        n->nops = 0;
        return n;
    }

    // ---- element-wise ops (with constant folding, x+0 / x*1 removal, CSE and PIECE hoisting).
    // Returns nullptr when an operand could not be cut to the pieces of the other one; the caller
    // then materialises the operands and retries.
    Node* op1(EOp op, Node* a) {
        a = canon(a);
        if (a->kind == N_CONST) return constant(eval_unary(op, a->cval), a->shape);
        if (a->kind == N_PIECE) {
            std::vector<Node*> kids;
            for (auto k : a->kids) {
                Node* r = op1(op, k);
                if (!r) return nullptr;
                kids.push_back(r);
            }
            return piece(a->pdim, kids);
        }
        OpKey key{op, a, nullptr};
        auto it = cse_.find(key);
        if (it != cse_.end()) return it->second;
        Node* n = fresh();
        n->kind = N_OP;
        n->shape = a->shape;
        n->op = op;
        n->a = a;
        n->nops = std::min(NOPS_CAP, a->nops + 1);
        cse_[key] = n;
        return n;
    }

    Node* op2(EOp op, Node* a, Node* b) {
        a = canon(a);
        b = canon(b);
        if (a->kind == N_CONST && b->kind == N_CONST)
            return constant(op == E_ADD ? a->cval + b->cval : a->cval * b->cval, a->shape);
        // identities: x * 1 -> x and x + (-0) -> x are exact; x + (+0) -> x differs only in the sign
        // of a zero result (-0 + +0 = +0), which no comparison or later op here can observe
        float ident = op == E_ADD ? 0.0f : 1.0f;
        if (b->kind == N_CONST && b->cval == ident) return a;
        if (a->kind == N_CONST && a->cval == ident) return b;
        if (a->kind == N_PIECE || b->kind == N_PIECE) {
            Node* p = a->kind == N_PIECE ? a : b;
            Node* o = a->kind == N_PIECE ? b : a;
            std::vector<Node*> kids;
            int64_t start = 0;
            for (size_t i = 0; i < p->kids.size(); i++) {
                Node* os = slice(o, p->pdim, start, p->ends[i]);
                if (!os) return nullptr;
                Node* r = (p == a) ? op2(op, p->kids[i], os) : op2(op, os, p->kids[i]);
                if (!r) return nullptr;
                kids.push_back(r);
                start = p->ends[i];
            }
            return piece(p->pdim, kids);
        }
        // + and * commute exactly in IEEE arithmetic: order operands for CSE
        if (a->serial > b->serial) std::swap(a, b);
        OpKey key{op, a, b};
        auto it = cse_.find(key);
        if (it != cse_.end()) return it->second;
        Node* n = fresh();
        n->kind = N_OP;
        n->shape = a->kind == N_CONST ? b->shape : a->shape;
        n->op = op;
        n->a = a;
        n->b = b;
        n->nops = std::min(NOPS_CAP, a->nops + b->nops + 1);
        cse_[key] = n;
        return n;
    }

    // ---- concatenation in normal form
    Node* piece(int dim, const std::vector<Node*>& kids_in) {
        std::vector<Node*> kids;
        for (auto k0 : kids_in) {
            Node* k = canon(k0);
            if (k->shape[dim] == 0) continue;
            if (k->kind == N_PIECE && k->pdim == dim) {
                for (auto kk : k->kids) kids.push_back(kk);
            } else
                kids.push_back(k);
        }
        if (kids.empty()) return canon(kids_in[0]);
        // merge neighbours that are the same expression shifted along `dim`
        std::vector<Node*> merged;
        for (auto k : kids) {
            if (!merged.empty()) {
                Node* m = try_merge(merged.back(), k, dim, 0);
                if (m) {
                    merged.back() = m;
                    continue;
                }
            }
            merged.push_back(k);
        }
        if (merged.size() == 1) return merged[0];
        Node* n = fresh();
        n->kind = N_PIECE;
        n->pdim = dim;
        n->shape = merged[0]->shape;
        int64_t e = 0;
        int64_t ops = 0;
        for (auto k : merged) {
            e += k->shape[dim];
            n->ends.push_back(e);
            ops = std::min(NOPS_CAP, ops + k->nops);
        }
        n->shape[dim] = e;
        n->kids = merged;
        n->nops = ops;
        return n;
    }

    // ---- data commands, pushed down to the leaves -------------------------------------------
    Node* permute(Node* n, const std::vector<uint32_t>& p) {
        Memo memo;
        return permute_rec(n, p, memo);
    }
    Node* index(Node* n, int dim, int64_t k) {
        Memo memo;
        return index_rec(n, dim, k, memo);
    }
    Node* broadcast(Node* n, int dim, int64_t r) {
        Memo memo;
        return broadcast_rec(n, dim, r, memo);
    }
    // nullptr: not expressible without copying
    Node* slice(Node* n, int dim, int64_t lo, int64_t hi) {
        n = canon(n);
        if (lo == 0 && hi == n->shape[dim]) return n;
        Memo memo;
        return slice_rec(n, dim, lo, hi, memo);
    }
    Node* reshape(Node* n, const Shape& shape) {
        n = canon(n);
        if (n->shape == shape) return n;
        Memo memo;
        return reshape_rec(n, shape, memo);
    }

    size_t size() const { return pool_.size(); }

    // number of distinct OP/LOAD nodes reachable from n (exact DAG size)
    int64_t dag_size(Node* n) {
        std::unordered_map<Node*, char> seen;
        int64_t cnt = 0;
        std::vector<Node*> st{canon(n)};
        while (!st.empty()) {
            Node* x = st.back();
            st.pop_back();
            if (seen.count(x)) continue;
            seen[x] = 1;
            if (x->kind == N_OP) {
                cnt++;
                st.push_back(canon(x->a));
                if (x->b) st.push_back(canon(x->b));
            } else if (x->kind == N_LOAD)
                cnt++;
            else if (x->kind == N_PIECE)
                for (auto k : x->kids) st.push_back(canon(k));
        }
        return cnt;
    }

  private:
    using Memo = std::unordered_map<Node*, Node*>;
    struct OpKey {
        EOp op;
        Node *a, *b;
        bool operator==(const OpKey& o) const { return op == o.op && a == o.a && b == o.b; }
    };
    struct OpKeyHash {
        size_t operator()(const OpKey& k) const {
            return std::hash<const void*>()(k.a) * 1000003u ^ std::hash<const void*>()(k.b) * 31u ^ size_t(k.op);
        }
    };
    std::deque<Node> pool_;
    std::unordered_map<OpKey, Node*, OpKeyHash> cse_;
    std::unordered_multimap<uint32_t, Node*> consts_;
    std::unordered_map<std::string, Node*> loads_;
    uint32_t serial_ = 0;

    Node* fresh() {
        pool_.emplace_back();
        pool_.back().serial = serial_++;
        return &pool_.back();
    }

    Node* rebuild_op(Node* n, Node* a, Node* b) {
        if (!a || (n->b && !b)) return nullptr;
        return n->b ? op2(n->op, a, b) : op1(n->op, a);
    }

    Node* permute_rec(Node* n, const std::vector<uint32_t>& p, Memo& memo) {
        n = canon(n);
        auto it = memo.find(n);
        if (it != memo.end()) return it->second;
        Shape ns(p.size());
        for (size_t i = 0; i < p.size(); i++) ns[i] = n->shape[p[i]];
        Node* r = nullptr;
        switch (n->kind) {
        case N_CONST: r = constant(n->cval, ns); break;
        case N_LOAD: {
            View v;
            v.offset = n->view.offset;
            v.dims.resize(p.size());
            for (size_t i = 0; i < p.size(); i++) v.dims[i] = n->view.dims[p[i]];
            r = load_v(n, ns, v);
            break;
        }
        case N_OP: r = rebuild_op(n, permute_rec(n->a, p, memo), n->b ? permute_rec(n->b, p, memo) : nullptr); break;
        case N_PIECE: {
            std::vector<Node*> kids;
            for (auto k : n->kids) kids.push_back(permute_rec(k, p, memo));
            int nd = 0;
            for (size_t i = 0; i < p.size(); i++)
                if (int(p[i]) == n->pdim) nd = int(i);
            r = piece(nd, kids);
            break;
        }
        }
        memo[n] = r;
        return r;
    }

    Node* index_rec(Node* n, int dim, int64_t k, Memo& memo) {
        n = canon(n);
        auto it = memo.find(n);
        if (it != memo.end()) return it->second;
        Shape ns = n->shape;
        ns.erase(ns.begin() + dim);
        Node* r = nullptr;
        switch (n->kind) {
        case N_CONST: r = constant(n->cval, ns); break;
        case N_LOAD: {
            View v = n->view;
            int64_t rem = k;
            auto& subs = v.dims[dim];
            for (int i = int(subs.size()) - 1; i >= 0; i--) {
                v.offset += (rem % subs[i].size) * subs[i].stride;
                rem /= subs[i].size;
            }
            v.dims.erase(v.dims.begin() + dim);
            r = load_v(n, ns, v);
            break;
        }
        case N_OP: r = rebuild_op(n, index_rec(n->a, dim, k, memo), n->b ? index_rec(n->b, dim, k, memo) : nullptr); break;
        case N_PIECE: {
            if (dim == n->pdim) {
                int64_t start = 0;
                for (size_t i = 0; i < n->kids.size(); i++) {
                    if (k < n->ends[i]) {
                        Memo m2;
                        r = index_rec(n->kids[i], dim, k - start, m2);
                        break;
                    }
                    start = n->ends[i];
                }
            } else {
                std::vector<Node*> kids;
                for (auto kid : n->kids) kids.push_back(index_rec(kid, dim, k, memo));
                r = piece(n->pdim - (dim < n->pdim ? 1 : 0), kids);
            }
            break;
        }
        }
        memo[n] = r;
        return r;
    }

    Node* broadcast_rec(Node* n, int dim, int64_t rep, Memo& memo) {
        n = canon(n);
        auto it = memo.find(n);
        if (it != memo.end()) return it->second;
        Shape ns = n->shape;
        ns[dim] = rep;
        Node* r = nullptr;
        switch (n->kind) {
        case N_CONST: r = constant(n->cval, ns); break;
        case N_LOAD: {
            View v = n->view;
            v.dims[dim].clear();
            if (rep != 1) v.dims[dim].push_back({rep, 0});
            r = load_v(n, ns, v);
            break;
        }
        case N_OP: r = rebuild_op(n, broadcast_rec(n->a, dim, rep, memo), n->b ? broadcast_rec(n->b, dim, rep, memo) : nullptr); break;
        case N_PIECE: {
            std::vector<Node*> kids;
            for (auto kid : n->kids) kids.push_back(broadcast_rec(kid, dim, rep, memo));
            r = piece(n->pdim, kids);
            break;
        }
        }
        memo[n] = r;
        return r;
    }

    Node* slice_rec(Node* n, int dim, int64_t lo, int64_t hi, Memo& memo) {
        n = canon(n);
        auto it = memo.find(n);
        if (it != memo.end()) return it->second;
        Shape ns = n->shape;
        ns[dim] = hi - lo;
        Node* r = nullptr;
        switch (n->kind) {
        case N_CONST: r = constant(n->cval, ns); break;
        case N_LOAD: {
            View v = n->view;
            auto& subs = v.dims[dim];
            if (subs.empty()) {
                // axis of length 1 (lo == 0, hi == 1 handled by the caller) -- nothing to cut
            } else if (subs.size() == 1) {
                v.offset += lo * subs[0].stride;
                subs[0].size = hi - lo;
            } else {
                int64_t inner = 1;
                for (size_t i = 1; i < subs.size(); i++) inner *= subs[i].size;
                if (lo % inner == 0 && hi % inner == 0) {
                    v.offset += (lo / inner) * subs[0].stride;
                    subs[0].size = (hi - lo) / inner;
                } else {
                    memo[n] = nullptr;
                    return nullptr;
                }
            }
            r = load_v(n, ns, v);
            break;
        }
        case N_OP: {
            Node* a = slice_rec(n->a, dim, lo, hi, memo);
            Node* b = n->b ? slice_rec(n->b, dim, lo, hi, memo) : nullptr;
            r = rebuild_op(n, a, b);
            break;
        }
        case N_PIECE: {
            std::vector<Node*> kids;
            if (dim == n->pdim) {
                int64_t start = 0;
                for (size_t i = 0; i < n->kids.size(); i++) {
                    int64_t s = std::max(lo, start), e = std::min(hi, n->ends[i]);
                    if (s < e) {
                        Node* kid = canon(n->kids[i]);
                        Node* ks = (s == start && e == n->ends[i]) ? kid : slice(kid, dim, s - start, e - start);
                        if (!ks) { memo[n] = nullptr; return nullptr; }
                        kids.push_back(ks);
                    }
                    start = n->ends[i];
                }
            } else {
                for (auto kid : n->kids) {
                    Node* ks = slice_rec(kid, dim, lo, hi, memo);
                    if (!ks) { memo[n] = nullptr; return nullptr; }
                    kids.push_back(ks);
                }
            }
            r = piece(n->pdim, kids);
            break;
        }
        }
        memo[n] = r;
        return r;
    }

    static bool regroup(const View& v, const Shape& shape, View& out) {
        std::vector<Sub> all;
        for (auto& d : v.dims)
            for (auto& s : d) all.push_back(s);
        canon_subs(all);  // digits that are contiguous across an axis boundary may be cut anywhere
        out.offset = v.offset;
        out.dims.assign(shape.size(), {});
        size_t pos = 0;
        for (size_t i = 0; i < shape.size(); i++) {
            int64_t need = shape[i];
            while (need > 1) {
                if (pos >= all.size()) return false;
                Sub& s = all[pos];
                if (s.size <= need) {
                    if (need % s.size) return false;
                    out.dims[i].push_back(s);
                    need /= s.size;
                    pos++;
                } else {
                    if (s.size % need) return false;
                    int64_t inner = s.size / need;
                    out.dims[i].push_back({need, s.stride * inner});
                    s.size = inner;
                    need = 1;
                }
            }
        }
        return pos == all.size();
    }

    Node* reshape_rec(Node* n, const Shape& shape, Memo& memo) {
        n = canon(n);
        auto it = memo.find(n);
        if (it != memo.end()) return it->second;
        Node* r = nullptr;
        switch (n->kind) {
        case N_CONST: r = constant(n->cval, shape); break;
        case N_LOAD: {
            View v;
            if (regroup(n->view, shape, v)) r = load_v(n, shape, v);
            break;
        }
        case N_OP: {
            Node* a = reshape_rec(n->a, shape, memo);
            Node* b = n->b ? reshape_rec(n->b, shape, memo) : nullptr;
            r = rebuild_op(n, a, b);
            break;
        }
        case N_PIECE: {
            // pieces survive a reshape when the cut axis is the outermost non-trivial axis on both
            // sides (then every piece stays one contiguous range of the new outermost axis), or
            // when only length-1 axes are added / removed.
            auto strip = [](const Shape& s) {
                Shape o;
                for (auto x : s)
                    if (x != 1) o.push_back(x);
                return o;
            };
            int new_dim = -1;
            int64_t scale_num = 1, scale_den = 1;
            if (strip(n->shape) == strip(shape)) {
                int rank_before = 0;
                for (int i = 0; i < n->pdim; i++)
                    if (n->shape[i] != 1) rank_before++;
                int seen = 0;
                for (size_t i = 0; i < shape.size(); i++) {
                    if (shape[i] == 1) continue;
                    if (seen == rank_before) { new_dim = int(i); break; }
                    seen++;
                }
            } else {
                bool outer_old = true;
                for (int i = 0; i < n->pdim; i++)
                    if (n->shape[i] != 1) outer_old = false;
                if (outer_old) {
                    int64_t inner_old = 1;
                    for (size_t i = n->pdim + 1; i < n->shape.size(); i++) inner_old *= n->shape[i];
                    for (size_t i = 0; i < shape.size(); i++)
                        if (shape[i] != 1) { new_dim = int(i); break; }
                    if (new_dim >= 0) {
                        int64_t inner_new = 1;
                        for (size_t i = new_dim + 1; i < shape.size(); i++) inner_new *= shape[i];
                        if (inner_old % inner_new == 0) { scale_num = inner_old / inner_new; }
                        else if (inner_new % inner_old == 0) { scale_den = inner_new / inner_old; }
                        else new_dim = -1;
                    }
                }
            }
            if (new_dim >= 0) {
                std::vector<Node*> kids;
                bool ok = true;
                for (auto kid0 : n->kids) {
                    Node* kid = canon(kid0);
                    int64_t ext = kid->shape[n->pdim] * scale_num;
                    if (ext % scale_den) { ok = false; break; }
                    Shape ks = shape;
                    ks[new_dim] = ext / scale_den;
                    Node* kr = reshape(kid, ks);
                    if (!kr) { ok = false; break; }
                    kids.push_back(kr);
                }
                if (ok) r = piece(new_dim, kids);
            }
            break;
        }
        }
        memo[n] = r;
        return r;
    }

    Node* load_v(Node* src, const Shape& shape, const View& v) { return load_cons(src->buf, src->version, shape, v); }

    // structurally equal reads of one buffer version share a node, so that repeated aliases of the
    // same data (two `.t()` of one weight, say) meet in the CSE tables
    Node* load_cons(int buf, uint32_t version, const Shape& shape, const View& view) {
        View v = view;
        for (auto& d : v.dims) canon_subs(d);
        std::string key;
        auto put = [&](int64_t x) { key.append(reinterpret_cast<const char*>(&x), sizeof x); };
        put(buf); put(version); put(v.offset); put(int64_t(shape.size()));
        for (auto x : shape) put(x);
        for (auto& d : v.dims) {
            put(int64_t(d.size()));
            for (auto& sub : d) { put(sub.size); put(sub.stride); }
        }
        auto it = loads_.find(key);
        if (it != loads_.end()) return it->second;
        Node* n = fresh();
        n->kind = N_LOAD;
        n->shape = shape;
        n->buf = buf;
        n->version = version;
        n->view = std::move(v);
        n->nops = 1;
        loads_.emplace(std::move(key), n);
        return n;
    }

    // two neighbours along `dim` that are one expression shifted -> the joined expression
    Node* try_merge(Node* a, Node* b, int dim, int depth) {
        a = canon(a);
        b = canon(b);
        if (a->kind != b->kind || depth > 48) return nullptr;
        if (a->shape.size() != b->shape.size()) return nullptr;
        for (size_t i = 0; i < a->shape.size(); i++)
            if (int(i) != dim && a->shape[i] != b->shape[i]) return nullptr;
        Shape ns = a->shape;
        ns[dim] = a->shape[dim] + b->shape[dim];
        switch (a->kind) {
        case N_CONST:
            if (a->cval == b->cval && std::signbit(a->cval) == std::signbit(b->cval)) return constant(a->cval, ns);
            return nullptr;
        case N_LOAD: {
            if (a->buf != b->buf || a->version != b->version) return nullptr;
            for (size_t i = 0; i < a->view.dims.size(); i++)
                if (int(i) != dim && !(a->view.dims[i] == b->view.dims[i])) return nullptr;
            auto& sa = a->view.dims[dim];
            auto& sb = b->view.dims[dim];
            if (sa.size() > 1 || sb.size() > 1) return nullptr;
            int64_t na = a->shape[dim], nb = b->shape[dim];
            int64_t stride;
            if (!sa.empty()) {
                stride = sa[0].stride;
                if (!sb.empty() && sb[0].stride != stride) return nullptr;
            } else if (!sb.empty())
                stride = sb[0].stride;
            else
                stride = b->view.offset - a->view.offset;
            if (b->view.offset != a->view.offset + na * stride) return nullptr;
            if (stride < 0) return nullptr;
            View v = a->view;
            v.dims[dim].clear();
            v.dims[dim].push_back({na + nb, stride});
            return load_v(a, ns, v);
        }
        case N_OP: {
            if (a->op != b->op || a->nops > 64) return nullptr;
            if ((a->b == nullptr) != (b->b == nullptr)) return nullptr;
            if (!a->b) {
                Node* ma = try_merge(a->a, b->a, dim, depth + 1);
                return ma ? op1(a->op, ma) : nullptr;
            }
            // operands were ordered for CSE, so try both pairings of a commutative op
            Node* ma = try_merge(a->a, b->a, dim, depth + 1);
            Node* mb = ma ? try_merge(a->b, b->b, dim, depth + 1) : nullptr;
            if (!ma || !mb) {
                ma = try_merge(a->a, b->b, dim, depth + 1);
                mb = ma ? try_merge(a->b, b->a, dim, depth + 1) : nullptr;
            }
            if (!ma || !mb) return nullptr;
            return op2(a->op, ma, mb);
        }
        default: return nullptr;
        }
    }
};

}  // namespace adb
