// IR -> plan.  Plays the role of the reference's `to_kernel` pipeline (src/kernel/to_kernel.rs:34-107):
// instruction selection (src/kernel/to_instr/*.rs), alias tracking (src/kernel/trackers/kernel.rs),
// the three fusion passes (src/kernel/fusion/*.rs), reordering for in-place chains
// (src/kernel/memory/*.rs) and alloc insertion (src/kernel/alloc/*.rs) -- but organised differently:
// values stay lazy expression DAGs until something needs them in memory, so fusion, common
// sub-expression sharing, dead-code removal and "temporaries never touch HBM" fall out of one
// mechanism instead of a sequence of rewriting passes.
#include "adb_lower.hpp"

#include <algorithm>
#include <cstdio>
#include <limits>
#include <map>
#include <set>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

namespace adb {

namespace {

struct IdInfo {
    int ndefs = 0;
    int def_seg = -1;
    bool cross = false;    // read outside the straight-line segment that defines it (or by the host)
    bool is_cond = false;
    bool needed = false;   // reachable from the dep list / a condition (dead-code elimination)
    int64_t uses = 0;      // remaining reads by live commands
    int buf = -1;          // persistent buffer once allocated
    std::vector<uint32_t> alias_kids;
    // an id owns a persistent buffer when its value must survive the straight-line segment that
    // computes it; ids that are redefined but only used inside one segment stay in registers
    bool needs_buffer() const { return cross || is_cond; }
};

struct Binding {
    enum Kind : uint8_t { UNDEF, VALUE, ALIAS } kind = UNDEF;
    Node* node = nullptr;      // VALUE
    bool pending = false;      // VALUE that still has to be written to the id's persistent buffer
    const Cmd* cmd = nullptr;  // ALIAS: the View / Index / Permute / Broadcast / Concat command
    Node* cache = nullptr;
    Node* cache_pa = nullptr;
    Node* cache_pb = nullptr;
};

bool is_alias_op(uint8_t op) {
    return op == OP_VIEW || op == OP_INDEX || op == OP_PERMUTE || op == OP_BROADCAST || op == OP_CONCAT;
}

bool has_result(uint8_t op) {
    switch (op) {
    case OP_WHILE: case OP_IF: case OP_EX: case OP_HEADING: return false;
    default: return true;
    }
}

// operands read by a command (in-place forms also read their target)
void cmd_reads(const Cmd& c, uint32_t out[2], int& n) {
    n = 0;
    switch (c.op) {
    case OP_MUL: case OP_ADD: case OP_DOT: case OP_BATCH_DOT: case OP_CONCAT: case OP_MUL_EQ: case OP_ADD_EQ:
        out[n++] = c.a; out[n++] = c.b; break;
    case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_SUM: case OP_MAX: case OP_CONTIG: case OP_EXP2: case OP_LOG2:
    case OP_SIN: case OP_RECIP: case OP_SQRT: case OP_VIEW: case OP_INDEX: case OP_PERMUTE:
    case OP_BROADCAST: case OP_ALLREDUCE:
        out[n++] = c.a; break;
    default: break;
    }
}

struct StoreTask {
    Node* node;    // plain expression (no PIECE)
    int buf;
    View view;     // destination access over node->shape
};

class Lowerer {
  public:
    Lowerer(Program& prog, Plan& plan, const LowerOptions& opt) : prog_(prog), plan_(plan), opt_(opt) {
        info_.resize(prog.ids.size());
        bind_.resize(prog.ids.size());
    }

    void run() {
        plan_.ir_commands = prog_.n_cmds;
        plan_.exact_div = opt_.exact_div;
        is_dep_.assign(prog_.ids.size(), 0);
        for (auto d : prog_.dep) { info_[d].cross = true; is_dep_[d] = 1; }
        int seg = 0;
        analyze(prog_.main, seg);
        dce();
        count_uses(prog_.main);
        // aliases keep their parents alive and make them cross-segment when they are
        propagate_alias_cross(prog_.main);
        index_mats(prog_.main);
        {
            std::vector<uint32_t> all;
            collect_assigned(prog_.main, all);
        }
        cur_ = &plan_.main;
        bool stopped = lower_block(prog_.main, true);
        (void)stopped;
        finalize_results();
        plan_.n_steps = pos_;
        fuse_reductions();
        if (!opt_.no_fusion && !opt_.no_dot_epilogue) fuse_dot_epilogues(plan_.main);
        if (!opt_.no_fusion) drop_unread_outputs();
        if (opt_.bucket_collectives && opt_.world > 1 && scale_all(4)) bucket_collectives(plan_.main);
        if (!opt_.no_fusion && !opt_.no_grouping) {
            std::vector<int> uses(plan_.kernels.size(), 0);
            count_kernel_uses(plan_.main, uses);
            group_kernels(plan_.main, uses);
        }
        plan_arena();
    }

  private:
    Program& prog_;
    Plan& plan_;
    LowerOptions opt_;
    Graph g_;
    std::vector<IdInfo> info_;
    std::vector<Binding> bind_;
    std::vector<char> is_dep_;
    std::vector<uint32_t> lazy_ids_;   // ids bound to values that do not live in their own buffer yet
    std::vector<uint32_t> materializing_;  // ids whose values are being written out (materialize_ids calls in progress)
    StepBlock* cur_ = nullptr;
    int pos_ = 0;
    int tmp_counter_ = 0;
    std::vector<std::pair<int, int>> loop_spans_;  // [first,last] step positions of While bodies
    bool results_done_ = false;

    std::unordered_map<const Cmd*, int> mat_index_;  // CreateMat -> ordinal in program order
    std::map<std::pair<Node*, Node*>, Node*> dot_cse_;  // (A, B) -> product still in memory
    std::map<Node*, Node*> sum_cse_;                    // summand -> row sums still in memory
    std::map<Node*, Node*> max_cse_;                    // the same for row maxima

    void index_mats(Block& b) {
        for (auto& c : b.cmds) {
            if (c.op == OP_CREATE_MAT) { int n = int(mat_index_.size()); mat_index_[&c] = n; }
            else if (c.op == OP_WHILE) index_mats(*c.block);
            else if (c.op == OP_IF) {
                for (auto& cb : c.conds) index_mats(*cb.second);
                if (c.else_block) index_mats(*c.else_block);
            }
        }
    }

    [[noreturn]] void fail(const std::string& msg) { throw LowerError(msg); }
    const std::string& name(uint32_t id) const { return prog_.ids[id]; }

    // ------------------------------------------------------------------ views at control-flow joins
    // An id bound to a View / Index / Permute / Broadcast / Concat is not a value but a window: it shows whatever its
    // source holds when it is read.  Straight-line code resolves that at lowering time.  Where paths meet -- a loop
    // body that runs zero, one or many times, a branch that is taken or not -- an id must look the same whichever
    // path was taken, and the only common form is "the value sits in the id's own buffer".  So an id that is a window
    // in front of a While / If and is assigned somewhere inside, or that a block leaves behind as a window, is
    // frozen: its current contents are copied into its buffer.  A frozen copy stops following its source, which is
    // only right when nothing reads the id (or a view of it) after its source has changed while it would still be a
    // window; `check_freeze` walks the rest of the program (loop back-edges included) and the lowering refuses the
    // program when that can happen.
    struct Frame { const Block* blk; size_t idx; bool is_while; };
    std::vector<Frame> frames_;                                          // blocks being lowered, outermost first
    std::unordered_map<const Block*, std::vector<uint32_t>> assigned_;   // ids assigned anywhere inside a block

    void collect_assigned(Block& b, std::vector<uint32_t>& out) {
        auto nested = [&](Block& inner) {
            std::vector<uint32_t>& v = assigned_[&inner];
            collect_assigned(inner, v);
            out.insert(out.end(), v.begin(), v.end());
        };
        for (auto& c : b.cmds) {
            if (c.op == OP_WHILE) nested(*c.block);
            else if (c.op == OP_IF) {
                for (auto& cb : c.conds) nested(*cb.second);
                if (c.else_block) nested(*c.else_block);
            } else if (has_result(c.op)) out.push_back(c.res);
        }
        std::sort(out.begin(), out.end());
        out.erase(std::unique(out.begin(), out.end()), out.end());
    }

    enum : uint8_t { S_WINDOW = 1, S_STALE = 2, S_REBOUND = 4 };   // possible states of a frozen id along the paths that reach a point
    struct FreezeScan {
        uint32_t id;
        std::unordered_set<uint32_t> sources;   // ids the window looks through, transitively
        std::unordered_set<uint32_t> readers;   // the id and the views derived from it afterwards
        bool conflict = false;
        uint32_t where = 0;
    };
    void scan_read(uint32_t r, uint8_t st, FreezeScan& f) {
        if ((st & S_STALE) && f.readers.count(r) && !f.conflict) { f.conflict = true; f.where = r; }
    }
    uint8_t scan_loop(const Cmd& c, uint8_t st, FreezeScan& f) {
        uint8_t acc = st;
        for (int it = 0; it < 4; it++) {
            uint8_t out = scan_cmds(*c.block, 0, acc, f);
            scan_read(c.a, out, f);
            if ((acc | out) == acc) break;
            acc |= out;
        }
        return acc;
    }
    uint8_t scan_cmd(const Cmd& c, uint8_t st, FreezeScan& f) {
        if (c.op == OP_WHILE) {
            scan_read(c.a, st, f);
            return scan_loop(c, st, f);
        }
        if (c.op == OP_IF) {
            for (auto& cb : c.conds) scan_read(cb.first, st, f);
            uint8_t out = 0;
            for (auto& cb : c.conds) out |= scan_cmds(*cb.second, 0, st, f);
            out |= c.else_block ? scan_cmds(*c.else_block, 0, st, f) : st;
            return out;
        }
        if (!has_result(c.op) || !live(c)) return st;
        uint32_t r[2];
        int n;
        cmd_reads(c, r, n);
        for (int k = 0; k < n; k++) {
            if (!f.readers.count(r[k])) continue;
            if (is_alias_op(c.op)) { if (c.res != f.id) f.readers.insert(c.res); }
            else scan_read(r[k], st, f);
        }
        if (c.res == f.id) return S_REBOUND;
        if (f.sources.count(c.res) && (st & S_WINDOW)) st = uint8_t((st & ~S_WINDOW) | S_STALE);
        return st;
    }
    uint8_t scan_cmds(const Block& b, size_t from, uint8_t st, FreezeScan& f) {
        for (size_t i = from; i < b.cmds.size() && !f.conflict; i++) st = scan_cmd(b.cmds[i], st, f);
        return st;
    }

    // `id` is bound to a view and is about to be frozen in front of command `from` of `blk` (frames_ = the blocks
    // around it): refuse when a later read could tell the copy from the window
    void check_freeze(uint32_t id, const Block& blk, size_t from) {
        FreezeScan f;
        f.id = id;
        f.readers.insert(id);
        std::vector<uint32_t> st{id};
        while (!st.empty()) {
            uint32_t x = st.back();
            st.pop_back();
            if (bind_[x].kind != Binding::ALIAS) continue;
            const Cmd& c = *bind_[x].cmd;
            if (f.sources.insert(c.a).second) st.push_back(c.a);
            if (c.op == OP_CONCAT && f.sources.insert(c.b).second) st.push_back(c.b);
        }
        // ids that already look through `id` (views of the view made earlier) read the copy from now on as well
        {
            std::vector<uint32_t> up{id};
            while (!up.empty()) {
                uint32_t x = up.back();
                up.pop_back();
                for (uint32_t k : info_[x].alias_kids) {
                    if (bind_[k].kind != Binding::ALIAS || !bind_[k].cmd) continue;
                    const Cmd& kc = *bind_[k].cmd;
                    if (kc.a != x && !(kc.op == OP_CONCAT && kc.b == x)) continue;
                    if (f.readers.insert(k).second) up.push_back(k);
                }
            }
        }
        uint8_t state = scan_cmds(blk, from, S_WINDOW, f);
        for (size_t d = frames_.size(); d-- > 0 && !f.conflict;) {
            const Frame& fr = frames_[d];
            if (fr.is_while) state = scan_loop(fr.blk->cmds[fr.idx], state, f);
            state = scan_cmds(*fr.blk, fr.idx + 1, state, f);
        }
        for (auto d : prog_.dep) scan_read(d, state, f);
        if (f.conflict)
            fail("'" + name(id) + "' is a view when control flow joins and is read (through '" + name(f.where) +
                 "') after its source changes; whether it still follows the source then depends on the path taken, "
                 "which a lowered program cannot express -- make it a tensor of its own (Contigious) first");
    }

    void freeze_alias(uint32_t id, const Block& blk, size_t from) {
        check_freeze(id, blk, from);
        Node* n = resolve(id);
        bind_value(id, n);   // pending: the next flush copies it into the id's own buffer
    }

    // in front of a While / If: ids that are views now and are assigned somewhere inside
    void freeze_for_blocks(const std::vector<const Block*>& inner, const Block& blk, size_t at) {
        for (const Block* b : inner) {
            auto it = assigned_.find(b);
            if (it == assigned_.end()) continue;
            for (uint32_t id : it->second)
                if (bind_[id].kind == Binding::ALIAS && info_[id].needed && info_[id].needs_buffer()) freeze_alias(id, blk, at);
        }
    }
    // at the end of a block: ids it leaves behind as views
    void freeze_at_end(const Block& blk) {
        auto it = assigned_.find(&blk);
        if (it == assigned_.end()) return;
        for (uint32_t id : it->second)
            if (bind_[id].kind == Binding::ALIAS && info_[id].needed && info_[id].needs_buffer()) freeze_alias(id, blk, blk.cmds.size());
    }

    // ------------------------------------------------------------------ analysis
    void def(uint32_t id, int seg) {
        auto& i = info_[id];
        i.ndefs++;
        if (i.def_seg < 0) i.def_seg = seg;
    }
    void use(uint32_t id, int seg) {
        auto& i = info_[id];
        if (i.def_seg != seg) i.cross = true;
    }

    void analyze(Block& b, int& seg) {
        int cur = ++seg;
        for (auto& c : b.cmds) {
            if (c.op == OP_WHILE) {
                info_[c.a].is_cond = true;
                analyze(*c.block, seg);
                cur = ++seg;
            } else if (c.op == OP_IF) {
                for (auto& cb : c.conds) {
                    info_[cb.first].is_cond = true;
                    analyze(*cb.second, seg);
                }
                if (c.else_block) analyze(*c.else_block, seg);
                cur = ++seg;
            } else if (has_result(c.op)) {
                uint32_t r[2];
                int n;
                cmd_reads(c, r, n);
                for (int k = 0; k < n; k++) use(r[k], cur);
                def(c.res, cur);
                if (c.op == OP_ALLREDUCE) info_[c.a].cross = true;
            }
        }
    }

    // flow-insensitive liveness: a command is live when its result can reach the dep list,
    // a condition or a collective
    void dce() {
        for (auto d : prog_.dep) info_[d].needed = true;
        for (size_t i = 0; i < info_.size(); i++)
            if (info_[i].is_cond) info_[i].needed = true;
        bool changed = true;
        std::function<void(Block&)> walk = [&](Block& b) {
            for (auto& c : b.cmds) {
                if (c.op == OP_WHILE) walk(*c.block);
                else if (c.op == OP_IF) {
                    for (auto& cb : c.conds) walk(*cb.second);
                    if (c.else_block) walk(*c.else_block);
                } else if (has_result(c.op) && info_[c.res].needed) {
                    uint32_t r[2];
                    int n;
                    cmd_reads(c, r, n);
                    for (int k = 0; k < n; k++)
                        if (!info_[r[k]].needed) { info_[r[k]].needed = true; changed = true; }
                }
            }
        };
        while (changed) {
            changed = false;
            walk(prog_.main);
        }
    }
    bool live(const Cmd& c) const { return !has_result(c.op) || info_[c.res].needed; }

    void count_uses(Block& b) {
        for (auto& c : b.cmds) {
            if (c.op == OP_WHILE) { info_[c.a].uses += 1; count_uses(*c.block); }
            else if (c.op == OP_IF) {
                for (auto& cb : c.conds) { info_[cb.first].uses += 1; count_uses(*cb.second); }
                if (c.else_block) count_uses(*c.else_block);
            } else if (has_result(c.op) && live(c)) {
                uint32_t r[2];
                int n;
                cmd_reads(c, r, n);
                for (int k = 0; k < n; k++) info_[r[k]].uses++;
            }
        }
    }

    void propagate_alias_cross(Block& b) {
        for (size_t ii = b.cmds.size(); ii-- > 0;) {
            auto& c = b.cmds[ii];
            if (c.op == OP_WHILE) propagate_alias_cross(*c.block);
            else if (c.op == OP_IF) {
                if (c.else_block) propagate_alias_cross(*c.else_block);
                for (size_t k = c.conds.size(); k-- > 0;) propagate_alias_cross(*c.conds[k].second);
            } else if (is_alias_op(c.op) && live(c)) {
                if (info_[c.res].cross || info_[c.res].is_cond) {
                    info_[c.a].cross = true;
                    if (c.op == OP_CONCAT) info_[c.b].cross = true;
                }
                info_[c.a].alias_kids.push_back(c.res);
                if (c.op == OP_CONCAT) info_[c.b].alias_kids.push_back(c.res);
            }
        }
    }

    bool id_live(uint32_t id, int depth = 0) const {
        const auto& i = info_[id];
        if (i.uses > 0) return true;
        if (bind_[id].pending) return true;
        if (results_pending_(id)) return true;
        if (depth > 64) return true;
        for (auto k : i.alias_kids)
            if (bind_[k].kind == Binding::ALIAS && id_live(k, depth + 1)) return true;
        return false;
    }
    bool results_pending_(uint32_t id) const {
        return !results_done_ && is_dep_[id];
    }

    // ------------------------------------------------------------------ buffers and steps
    int new_buffer(int64_t n, const std::string& nm, bool persistent) {
        BufferInfo b;
        b.numel = n;
        b.name = nm;
        b.persistent = persistent;
        plan_.bufs.push_back(b);
        g_.buf_version.push_back(0);
        return int(plan_.bufs.size()) - 1;
    }
    int temp_buffer(int64_t n) { return new_buffer(n, "tmp" + std::to_string(tmp_counter_++), false); }

    int id_buffer(uint32_t id, const Shape& shape) {
        auto& i = info_[id];
        int64_t n = numel(shape);
        if (i.buf >= 0) {
            if (plan_.bufs[i.buf].numel != n)
                fail("id '" + name(id) + "' is redefined with a different size; a buffer keeps one size "
                     "(the reference asserts the same, src/devices/opencl/context.rs:62-64)");
            return i.buf;
        }
        i.buf = new_buffer(n, name(id), true);
        return i.buf;
    }

    void touch(int buf, int pos) {
        auto& b = plan_.bufs[buf];
        b.first = std::min(b.first, pos);
        b.last = std::max(b.last, pos);
    }

    Step& push_step(Step::Kind k) {
        cur_->steps.emplace_back();
        Step& s = cur_->steps.back();
        s.kind = k;
        s.pos = pos_++;
        return s;
    }

    // ------------------------------------------------------------------ bindings
    Node* resolve(uint32_t id, int depth = 0) {
        Binding& b = bind_[id];
        if (depth > 4096) fail("alias chain too deep at '" + name(id) + "'");
        if (b.kind == Binding::UNDEF) fail("id '" + name(id) + "' is read before it is defined");
        if (b.kind == Binding::VALUE) {
            Node* n = g_.canon(b.node);
            if (!g_.load_valid(n)) fail("internal: stale binding for '" + name(id) + "'");
            return n;
        }
        const Cmd& c = *b.cmd;
        Node* pa = resolve(c.a, depth + 1);
        Node* pb = c.op == OP_CONCAT ? resolve(c.b, depth + 1) : nullptr;
        if (b.cache && b.cache_pa == pa && b.cache_pb == pb) return g_.canon(b.cache);
        Node* r = nullptr;
        switch (c.op) {
        case OP_VIEW: {
            if (numel(c.dims) != numel(pa->shape)) fail("View of '" + name(c.a) + "' changes the element count");
            r = g_.reshape(pa, c.dims);
            if (!r) {
                Node* m = materialize_node(pa);
                r = g_.reshape(m, c.dims);
                if (!r) fail("internal: reshape of a contiguous value failed");
            }
            break;
        }
        case OP_INDEX:
            if (c.dim >= pa->shape.size() || int64_t(c.index) >= pa->shape[c.dim]) fail("Index out of range on '" + name(c.a) + "'");
            r = g_.index(pa, int(c.dim), int64_t(c.index));
            break;
        case OP_PERMUTE: {
            if (c.perm.size() != pa->shape.size()) fail("Permute rank mismatch on '" + name(c.a) + "'");
            std::vector<char> seen(c.perm.size(), 0);
            for (auto p : c.perm) {
                if (p >= c.perm.size() || seen[p]) fail("Permute is not a permutation");
                seen[p] = 1;
            }
            r = g_.permute(pa, c.perm);
            break;
        }
        case OP_BROADCAST:
            if (c.dim >= pa->shape.size() || pa->shape[c.dim] != 1) fail("Broadcast needs a length-1 axis on '" + name(c.a) + "'");
            r = g_.broadcast(pa, int(c.dim), int64_t(c.count));
            break;
        case OP_CONCAT: {
            if (pa->shape.size() != pb->shape.size() || c.dim >= pa->shape.size()) fail("Concat rank mismatch");
            for (size_t i = 0; i < pa->shape.size(); i++)
                if (i != c.dim && pa->shape[i] != pb->shape[i]) fail("Dim misaligned at concat");
            r = g_.piece(int(c.dim), {pa, pb});
            break;
        }
        default: fail("internal: bad alias command");
        }
        b.cache = r;
        b.cache_pa = pa;
        b.cache_pb = pb;
        return r;
    }

    void consume(uint32_t id) {
        if (info_[id].uses > 0) info_[id].uses--;
    }

    void bind_value(uint32_t id, Node* n) {
        Binding& b = bind_[id];
        b.kind = Binding::VALUE;
        b.node = n;
        b.cmd = nullptr;
        b.cache = nullptr;
        b.pending = false;
        n = g_.canon(n);
        bool own = false;
        if (n->kind == N_LOAD && info_[id].buf == n->buf && view_is_contiguous(n->view, n->shape) && n->view.offset == 0) own = true;
        if (info_[id].needs_buffer() && !own) b.pending = true;
        if (!own) lazy_ids_.push_back(id);
    }

    void bind_own_buffer(uint32_t id, int buf, const Shape& shape) {
        Binding& b = bind_[id];
        b.kind = Binding::VALUE;
        b.node = g_.load(buf, shape, contiguous_view(shape));
        b.pending = false;
        b.cmd = nullptr;
        b.cache = nullptr;
    }

    // ------------------------------------------------------------------ hazards
    bool depends_on(Node* n, int buf) {
        std::unordered_set<Node*> seen;
        std::vector<Node*> st{g_.canon(n)};
        while (!st.empty()) {
            Node* x = st.back();
            st.pop_back();
            if (!seen.insert(x).second) continue;
            switch (x->kind) {
            case N_LOAD: if (x->buf == buf) return true; break;
            case N_OP:
                st.push_back(g_.canon(x->a));
                if (x->b) st.push_back(g_.canon(x->b));
                break;
            case N_PIECE: for (auto k : x->kids) st.push_back(g_.canon(k)); break;
            default: break;
            }
        }
        return false;
    }

    // called before a kernel overwrites live contents of `buf`: every lazy value that still reads
    // the old contents and is needed later is written out first
    void before_write(int buf, const std::vector<uint32_t>& exclude) {
        if (g_.buf_version[buf] == 0) return;  // nothing could have read it yet
        std::vector<uint32_t> todo;
        std::vector<uint32_t> keep;
        std::unordered_set<uint32_t> seen;
        for (auto id : lazy_ids_) {
            if (!seen.insert(id).second) continue;
            Binding& b = bind_[id];
            if (b.kind != Binding::VALUE) continue;
            Node* n = g_.canon(b.node);
            bool own = n->kind == N_LOAD && info_[id].buf == n->buf;
            if (own && !b.pending) continue;  // already in its own buffer
            if (!id_live(id)) continue;
            keep.push_back(id);
            if (std::find(exclude.begin(), exclude.end(), id) != exclude.end()) continue;
            if (depends_on(n, buf)) todo.push_back(id);
        }
        lazy_ids_.swap(keep);
        if (!todo.empty()) materialize_ids(todo);
    }

    // ------------------------------------------------------------------ materialisation
    static bool slice_view(View& v, int dim, int64_t lo, int64_t hi) {
        auto& subs = v.dims[dim];
        if (subs.empty()) return lo == 0;
        if (subs.size() == 1) {
            v.offset += lo * subs[0].stride;
            subs[0].size = hi - lo;
            return true;
        }
        int64_t inner = 1;
        for (size_t i = 1; i < subs.size(); i++) inner *= subs[i].size;
        if (lo % inner || hi % inner) return false;
        v.offset += (lo / inner) * subs[0].stride;
        subs[0].size = (hi - lo) / inner;
        return true;
    }

    void collect_stores(Node* n, int buf, const View& view, std::vector<StoreTask>& out) {
        n = g_.canon(n);
        if (numel(n->shape) == 0) return;
        if (n->kind == N_PIECE) {
            int64_t start = 0;
            for (size_t i = 0; i < n->kids.size(); i++) {
                View v = view;
                if (!slice_view(v, n->pdim, start, n->ends[i])) fail("internal: destination view cannot be cut");
                for (auto& d : v.dims) canon_subs(d);
                collect_stores(n->kids[i], buf, v, out);
                start = n->ends[i];
            }
            return;
        }
        out.push_back({n, buf, view});
    }

    // write lazy values of ids into their buffers (persistent buffer for ids that need one, else a temp)
    void materialize_ids(std::vector<uint32_t> ids) {
        // ids whose value already sits in its own buffer need nothing
        std::vector<uint32_t> work;
        for (auto id : ids) {
            Binding& b = bind_[id];
            if (b.kind != Binding::VALUE) continue;
            Node* n = g_.canon(b.node);
            bool own = n->kind == N_LOAD && info_[id].buf == n->buf && view_is_contiguous(n->view, n->shape) && n->view.offset == 0;
            if (own) { b.pending = false; continue; }
            if (std::find(work.begin(), work.end(), id) == work.end()) work.push_back(id);
        }
        if (work.empty()) return;
        std::vector<int> dst(work.size());
        std::vector<char> parked(work.size(), 0);
        for (size_t k = 0; k < work.size(); k++) {
            uint32_t id = work[k];
            Node* n = g_.canon(bind_[id].node);
            bool own = info_[id].needs_buffer();
            int target = own ? id_buffer(id, n->shape) : -1;
            // x' = f(y), y' = g(x), each written out on its own (an all-reduce of x): writing x needs y' out of the way
            // first (it reads the old x), and y' cannot go to y's buffer because x' still reads the old y.  A value
            // that something further up this call chain still reads the target of goes to a temporary for now and
            // reaches its own buffer at the next flush.
            for (size_t q = 0; own && q < materializing_.size(); q++) {
                const uint32_t other = materializing_[q];
                if (other != id && bind_[other].kind == Binding::VALUE && depends_on(bind_[other].node, target)) own = false;
            }
            parked[k] = info_[id].needs_buffer() && !own;
            dst[k] = own ? target : temp_buffer(numel(n->shape));
        }
        // old contents of the targets may still be needed by other lazy values
        const size_t depth = materializing_.size();
        materializing_.insert(materializing_.end(), work.begin(), work.end());
        for (size_t k = 0; k < work.size(); k++) before_write(dst[k], work);
        materializing_.resize(depth);
        std::vector<StoreTask> tasks;
        std::vector<std::pair<size_t, size_t>> span(work.size());
        for (size_t k = 0; k < work.size(); k++) {
            Node* n = g_.canon(bind_[work[k]].node);
            span[k].first = tasks.size();
            collect_stores(n, dst[k], contiguous_view(n->shape), tasks);
            span[k].second = tasks.size();
        }
        emit_stores(tasks);
        for (size_t k = 0; k < work.size(); k++) {
            uint32_t id = work[k];
            Node* old = bind_[id].node;
            Node* oldc = g_.canon(old);
            g_.buf_version[dst[k]]++;
            Node* ld = g_.load(dst[k], oldc->shape, contiguous_view(oldc->shape));
            if (oldc->kind == N_OP || oldc->kind == N_PIECE) oldc->fwd = ld;
            if (parked[k]) {
                bind_value(id, ld);      // still owes its own buffer a copy
                continue;
            }
            bind_[id].node = ld;
            bind_[id].pending = false;
        }
    }

    // write an arbitrary node to a fresh temp and forward the node to it
    Node* materialize_node(Node* n) {
        n = g_.canon(n);
        if (n->kind == N_LOAD && view_is_contiguous(n->view, n->shape)) return n;
        int buf = temp_buffer(numel(n->shape));
        std::vector<StoreTask> tasks;
        collect_stores(n, buf, contiguous_view(n->shape), tasks);
        emit_stores(tasks);
        g_.buf_version[buf]++;
        Node* ld = g_.load(buf, n->shape, contiguous_view(n->shape));
        if (n->kind == N_OP || n->kind == N_PIECE) n->fwd = ld;
        return ld;
    }

    void flush_pending() {
        std::vector<uint32_t> ids;
        std::unordered_set<uint32_t> seen;
        for (auto id : lazy_ids_)
            if (bind_[id].kind == Binding::VALUE && bind_[id].pending && seen.insert(id).second) ids.push_back(id);
        if (!ids.empty()) materialize_ids(ids);
        // everything else that is still lazy is local to the finished segment
        std::vector<uint32_t> keep;
        for (auto id : lazy_ids_)
            if (bind_[id].kind == Binding::VALUE && bind_[id].pending) keep.push_back(id);
        lazy_ids_.swap(keep);
    }

    // group store tasks of equal size into fused kernels; a task whose destination is still read
    // by the group with another access pattern (or from another kernel of the group) is written to
    // a temporary first and copied over afterwards
    struct CopyBack {
        int tmp, buf;
        View view;
        Shape shape;
    };
    void emit_stores(std::vector<StoreTask>& tasks) {
        if (tasks.empty()) return;
        std::vector<CopyBack> copies;
        for (auto& t : tasks) {
            if (g_.buf_version[t.buf] == 0) continue;  // fresh buffer: nobody reads it
            bool conflict = false;
            for (auto& u : tasks) {
                if (!depends_on(u.node, t.buf)) continue;
                if (numel(u.node->shape) != numel(t.node->shape) || reads_other_access(u.node, t.buf, t.view)) {
                    conflict = true;
                    break;
                }
            }
            if (conflict) {
                int tmp = temp_buffer(numel(t.node->shape));
                copies.push_back({tmp, t.buf, t.view, t.node->shape});
                t.buf = tmp;
                t.view = contiguous_view(t.node->shape);
            }
        }
        std::map<int64_t, std::vector<StoreTask*>> groups;
        for (auto& t : tasks) groups[numel(t.node->shape)].push_back(&t);
        for (auto& kv : groups) {
            // keep kernels bounded: split a group when its combined DAG gets too large
            std::vector<StoreTask*> cur;
            int64_t sz = 0;
            for (auto* t : kv.second) {
                int64_t s = std::min<int64_t>(t->node->nops, opt_.fuse_limit);
                if (!cur.empty() && (sz + s > opt_.fuse_limit * 2 || cur.size() >= 16)) {
                    emit_elw(cur);
                    cur.clear();
                    sz = 0;
                }
                cur.push_back(t);
                sz += s;
            }
            if (!cur.empty()) emit_elw(cur);
        }
        for (auto& c : copies) {
            g_.buf_version[c.tmp]++;
            StoreTask t{g_.load(c.tmp, c.shape, contiguous_view(c.shape)), c.buf, c.view};
            std::vector<StoreTask*> one{&t};
            emit_elw(one);
        }
    }

    bool reads_other_access(Node* n, int buf, const View& view) {
        std::unordered_set<Node*> seen;
        std::vector<Node*> st{g_.canon(n)};
        auto want = flat_subs(view);
        while (!st.empty()) {
            Node* x = st.back();
            st.pop_back();
            if (!seen.insert(x).second) continue;
            if (x->kind == N_LOAD) {
                if (x->buf == buf && !(x->view.offset == view.offset && flat_subs(x->view) == want)) return true;
            } else if (x->kind == N_OP) {
                st.push_back(g_.canon(x->a));
                if (x->b) st.push_back(g_.canon(x->b));
            }
        }
        return false;
    }

    // ------------------------------------------------------------------ kernel construction
    struct SsaBuilder {
        Lowerer& L;
        KernelSpec& k;
        bool reduce;
        std::unordered_map<Node*, int> memo;
        std::map<uint32_t, int> consts;
        SsaBuilder(Lowerer& l, KernelSpec& ks, bool red) : L(l), k(ks), reduce(red) {}

        Operand make_operand(int buf, const View& v) {
            Operand o;
            o.buf = buf;
            o.offset = v.offset;
            if (reduce) {
                o.xsubs = v.dims[0];
                o.subs = v.dims[1];
                canon_subs(o.xsubs);
                canon_subs(o.subs);
            } else
                o.subs = flat_subs(v);
            return o;
        }

        int build(Node* n0) {
            // iterative post-order so very deep chains cannot overflow the stack
            std::vector<std::pair<Node*, int>> st;
            st.push_back({L.g_.canon(n0), 0});
            while (!st.empty()) {
                Node* n = st.back().first;
                int phase = st.back().second;
                if (memo.count(n)) { st.pop_back(); continue; }
                if (n->kind == N_PIECE) L.fail("internal: piecewise value inside a kernel expression");
                if (n->kind == N_LOAD) {
                    if (!L.g_.load_valid(n)) L.fail("internal: kernel reads overwritten data");
                    Operand o = make_operand(n->buf, n->view);
                    int oi = -1;
                    for (size_t i = 0; i < k.ins.size(); i++)
                        if (k.ins[i].same_access(o)) { oi = int(i); break; }
                    if (oi < 0) { k.ins.push_back(o); oi = int(k.ins.size()) - 1; }
                    Ssa s; s.kind = Ssa::LOAD; s.operand = oi;
                    k.ssa.push_back(s);
                    memo[n] = int(k.ssa.size()) - 1;
                    st.pop_back();
                } else if (n->kind == N_CONST) {
                    uint32_t bits;
                    std::memcpy(&bits, &n->cval, 4);
                    auto it = consts.find(bits);
                    if (it == consts.end()) {
                        Ssa s; s.kind = Ssa::CONST; s.c = n->cval;
                        k.ssa.push_back(s);
                        it = consts.emplace(bits, int(k.ssa.size()) - 1).first;
                    }
                    memo[n] = it->second;
                    st.pop_back();
                } else {
                    Node* a = L.g_.canon(n->a);
                    Node* b = n->b ? L.g_.canon(n->b) : nullptr;
                    if (phase == 0) {
                        st.back().second = 1;
                        if (b && !memo.count(b)) st.push_back({b, 0});
                        if (!memo.count(a)) st.push_back({a, 0});
                    } else {
                        Ssa s; s.kind = Ssa::OP; s.op = n->op; s.a = memo[a]; s.b = b ? memo[b] : -1;
                        k.ssa.push_back(s);
                        memo[n] = int(k.ssa.size()) - 1;
                        st.pop_back();
                    }
                }
            }
            return memo[L.g_.canon(n0)];
        }
    };

    void emit_elw(std::vector<StoreTask*>& tasks) {
        KernelSpec k;
        k.type = KernelSpec::ELW;
        k.n = numel(tasks[0]->node->shape);
        SsaBuilder sb(*this, k, false);
        for (auto* t : tasks) {
            int v = sb.build(t->node);
            KernelSpec::Out o;
            o.ssa = v;
            o.dst.buf = t->buf;
            o.dst.offset = t->view.offset;
            o.dst.subs = flat_subs(t->view);
            k.outs.push_back(o);
        }
        plan_.kernels.push_back(std::move(k));
        Step& s = push_step(Step::ELW);
        s.kernel = int(plan_.kernels.size()) - 1;
        auto& ks = plan_.kernels.back();
        for (auto& o : ks.ins) touch(o.buf, s.pos);
        for (auto& o : ks.outs) touch(o.dst.buf, s.pos);
    }

    // ------------------------------------------------------------------ commands
    Node* elementwise2(EOp op, Node* a, Node* b) {
        Node* r = g_.op2(op, a, b);
        if (!r) {
            a = materialize_node(a);
            b = materialize_node(b);
            r = g_.op2(op, a, b);
            if (!r) fail("internal: element-wise op on materialised operands failed");
        }
        return r;
    }

    void after_op(uint32_t id, Node* r) {
        bind_value(id, r);
        r = g_.canon(r);
        bool too_big = false;
        if (r->nops > opt_.fuse_limit) {
            int64_t exact = g_.dag_size(r);
            if (exact > opt_.fuse_limit) too_big = true;
            else if (r->kind == N_OP) r->nops = exact;
        }
        if ((opt_.no_fusion && (r->kind == N_OP || r->kind == N_PIECE)) || too_big) materialize_ids({id});
    }

    void check_same_numel(const Cmd& c, Node* a, Node* b) {
        if (a->kind != N_CONST && b->kind != N_CONST && a->shape != b->shape) {
            if (numel(a->shape) != numel(b->shape))
                fail("element-wise operands '" + name(c.a) + "' and '" + name(c.b) + "' differ in size");
        }
    }

    void lower_cmd(const Cmd& c) {
        switch (c.op) {
        case OP_HEADING: return;
        case OP_CREATE_MAT: return lower_create_mat(c);
        case OP_CREATE_CONST: {
            bind_value(c.res, g_.constant(c.cval, c.dims));
            return;
        }
        case OP_MUL: case OP_ADD: case OP_MUL_EQ: case OP_ADD_EQ: {
            Node* a = resolve(c.a);
            Node* b = resolve(c.b);
            check_same_numel(c, a, b);
            if (a->kind != N_CONST && b->kind != N_CONST && a->shape != b->shape) {
                // same element count, different shape: align the right operand to the left one
                Node* rb = g_.reshape(b, a->shape);
                if (!rb) rb = g_.reshape(materialize_node(b), a->shape);
                b = rb;
            }
            if (a->kind == N_CONST && b->kind != N_CONST && a->shape != b->shape) a = g_.constant(a->cval, b->shape);
            if (b->kind == N_CONST && a->shape != b->shape) b = g_.constant(b->cval, a->shape);
            EOp op = (c.op == OP_MUL || c.op == OP_MUL_EQ) ? E_MUL : E_ADD;
            Node* r = elementwise2(op, a, b);
            consume(c.a);
            consume(c.b);
            after_op(c.res, r);
            return;
        }
        case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_EXP2: case OP_LOG2: case OP_SIN: case OP_RECIP: case OP_SQRT: {
            static const EOp map[] = {E_EQZ, E_GTZ, E_LTZ};
            EOp op;
            switch (c.op) {
            case OP_EQZ: case OP_GTZ: case OP_LTZ: op = map[c.op - OP_EQZ]; break;
            case OP_EXP2: op = E_EXP2; break;
            case OP_LOG2: op = E_LOG2; break;
            case OP_SIN: op = E_SIN; break;
            case OP_RECIP: op = E_RECIP; break;
            default: op = E_SQRT; break;
            }
            Node* a = resolve(c.a);
            Node* r = g_.op1(op, a);
            if (!r) r = g_.op1(op, materialize_node(a));
            consume(c.a);
            after_op(c.res, r);
            return;
        }
        case OP_CONTIG: {
            Node* a = resolve(c.a);
            consume(c.a);
            bind_value(c.res, a);
            return;
        }
        case OP_VIEW: case OP_INDEX: case OP_PERMUTE: case OP_BROADCAST: case OP_CONCAT: {
            if (c.res == c.a || (c.op == OP_CONCAT && c.res == c.b))
                fail("alias command writes onto its own operand ('" + name(c.res) + "')");
            // parents stay referenced for as long as the alias is; their reads are counted when the
            // alias itself is consumed, so only validate now
            (void)resolve(c.a);
            consume(c.a);
            if (c.op == OP_CONCAT) { (void)resolve(c.b); consume(c.b); }
            Binding& b = bind_[c.res];
            b.kind = Binding::ALIAS;
            b.cmd = &c;
            b.node = nullptr;
            b.cache = nullptr;
            b.pending = false;
            (void)resolve(c.res);  // shape / range checks happen at definition
            return;
        }
        case OP_SUM: return lower_sum(c, 0);
        case OP_MAX: return lower_sum(c, 1);
        case OP_DOT: return lower_dot(c);
        case OP_BATCH_DOT: return lower_batch_dot(c);
        case OP_ALLREDUCE: return lower_allreduce(c);
        default: fail("internal: unexpected command in straight-line code");
        }
    }

    static bool uniform_payload(const float* p, int64_t n, float& v) {
        if (n == 0) return false;
        uint32_t first;
        std::memcpy(&first, p, 4);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(p);
        for (int64_t i = 1; i < n; i++)
            if (u[i] != first) return false;
        v = p[0];
        return true;
    }

    void lower_create_mat(const Cmd& c) {
        int64_t n = numel(c.dims);
        if (int64_t(c.count) != n) fail("CreateMat '" + name(c.res) + "': # of values doesn't match dim size");
        PayloadSlot slot;
        slot.kind = c.payload_kind;
        slot.addr = c.payload;
        slot.count = n;
        slot.cmd_index = mat_index_.at(&c);
        plan_.payloads.push_back(slot);
        int slot_idx = int(plan_.payloads.size()) - 1;
        if (n == 0) {
            bind_value(c.res, g_.constant(0.f, c.dims));
            return;
        }
        float cv;
        if (c.payload_kind != PAYLOAD_DEVICE && info_[c.res].ndefs == 1 &&
            uniform_payload(reinterpret_cast<const float*>(uintptr_t(c.payload)), n, cv)) {
            // a constant-filled tensor (backward seeds, zero padding) never needs to exist in memory
            plan_.payloads.back().assumed_const = true;  // a cached plan re-checks this on reuse
            plan_.payloads.back().const_val = cv;
            bind_value(c.res, g_.constant(cv, c.dims));
            return;
        }
        bool persistent = info_[c.res].needs_buffer();
        if (c.payload_kind == PAYLOAD_DEVICE && info_[c.res].ndefs == 1 && (c.payload % 16) == 0) {
            // resident and never written: read the caller's memory in place
            int buf = new_buffer(n, name(c.res), true);
            plan_.bufs[buf].external = true;
            plan_.bufs[buf].payload = slot_idx;
            info_[c.res].buf = buf;
            g_.buf_version[buf] = 1;
            bind_own_buffer(c.res, buf, c.dims);
            return;
        }
        int buf = persistent ? id_buffer(c.res, c.dims) : new_buffer(n, name(c.res), false);
        if (!persistent) info_[c.res].buf = buf;
        before_write(buf, {c.res});
        Step& s = push_step(Step::UPLOAD);
        s.buf = buf;
        s.payload = slot_idx;
        s.nelem = n;
        touch(buf, s.pos);
        g_.buf_version[buf]++;
        bind_own_buffer(c.res, buf, c.dims);
    }

    // destination buffer of a kernel-producing command (Sum, DotProduct)
    int result_buffer(uint32_t id, const Shape& shape) {
        int buf;
        if (info_[id].needs_buffer()) buf = id_buffer(id, shape);
        else {
            buf = new_buffer(numel(shape), name(id), false);
            info_[id].buf = buf;
        }
        return buf;
    }

    // Sum (red_op 0) and Max (red_op 1) over the last axis of a 2-d value
    void lower_sum(const Cmd& c, int red_op) {
        Node* a = resolve(c.a);
        if (a->shape.size() != 2) fail(std::string("Reduce (") + (red_op ? "max" : "sum") + ") node needs dim=2 ('" + name(c.a) + "')");
        consume(c.a);
        lower_sum_node(c, a, red_op);
    }

    // the row reduction of a 2-d value `a` into the id c.res (also used by matrix-vector products)
    void lower_sum_node(const Cmd& c, Node* a, int red_op) {
        int64_t V = a->shape[0], R = a->shape[1];
        if (R == 0) {
            // nothing to reduce: the identity of the operation (the oracle's accumulators start there as well)
            after_op(c.res, g_.constant(red_op == 1 ? -std::numeric_limits<float>::infinity() : 0.0f, {V}));
            return;
        }
        if (a->kind == N_CONST && (red_op == 1 || a->cval == 0.0f)) {
            after_op(c.res, g_.constant(a->cval, {V}));   // maximum of a constant row; sum of zeros
            return;
        }
        // the same reduction of the same value was computed before and is still in memory
        // (what the reference's repeat_opt does on the IR, src/ir/opts/repeat_opt.rs:5-71)
        std::map<Node*, Node*>& cse = red_op ? max_cse_ : sum_cse_;
        {
            auto it = cse.find(a);
            if (it != cse.end() && g_.load_valid(it->second)) {
                bind_value(c.res, it->second);
                return;
            }
        }
        Node* sum_key = a;
        if (a->kind == N_PIECE && a->pdim != 0) a = materialize_node(a);
        if (a->nops > opt_.fuse_limit && g_.dag_size(a) > opt_.fuse_limit) a = materialize_node(a);
        int buf = result_buffer(c.res, {V});
        // `Sum a -> a` (a row of length 1): blocks of the reduce kernels read rows that other blocks already wrote
        const bool overlaps = depends_on(a, buf);
        if (overlaps) buf = temp_buffer(V);
        before_write(buf, {c.res});
        std::vector<StoreTask> parts;
        if (a->kind == N_PIECE) {
            int64_t start = 0;
            for (size_t i = 0; i < a->kids.size(); i++) {
                Node* kid = g_.canon(a->kids[i]);
                if (kid->kind == N_PIECE) kid = materialize_node(kid);
                View v = contiguous_view({V});
                slice_view(v, 0, start, a->ends[i]);
                parts.push_back({kid, buf, v});
                start = a->ends[i];
            }
        } else
            parts.push_back({a, buf, contiguous_view({V})});
        for (auto& p : parts) {
            KernelSpec k;
            k.type = KernelSpec::REDUCE;
            k.n = p.node->shape[0];
            k.r = R;
            k.red_op = red_op;
            if (k.n == 0) continue;
            SsaBuilder sb(*this, k, true);
            KernelSpec::Out o;
            o.ssa = sb.build(p.node);
            o.dst.buf = buf;
            o.dst.offset = p.view.offset;
            o.dst.xsubs = p.view.dims[0];
            k.outs.push_back(o);
            plan_reduce(k, opt_.sm_count);
            if (k.split > 1) {
                // two passes: `split` partial sums per row into scratch memory, then a small reduce of
                // the partials (row mode keeps them next to each other, column mode one row per part)
                KernelSpec::Out final_out = k.outs[0];
                int scratch = temp_buffer(k.n * k.split);
                k.scratch = scratch;
                k.outs[0].dst = Operand();
                k.outs[0].dst.buf = scratch;
                if (k.n > 1) k.outs[0].dst.xsubs = {{k.n, 1}};
                KernelSpec k2;
                k2.type = KernelSpec::REDUCE;
                k2.n = k.n;
                k2.r = k.split;
                k2.red_op = red_op;
                Operand in;
                in.buf = scratch;
                if (k.mode == 0) {
                    if (k.n > 1) in.xsubs = {{k.n, k.split}};
                    in.subs = {{k.split, 1}};
                } else {
                    if (k.n > 1) in.xsubs = {{k.n, 1}};
                    in.subs = {{k.split, k.n}};
                }
                k2.ins.push_back(in);
                Ssa ld;
                ld.kind = Ssa::LOAD;
                ld.operand = 0;
                k2.ssa.push_back(ld);
                final_out.ssa = 0;
                k2.outs.push_back(final_out);
                plan_reduce(k2, opt_.sm_count);
                k2.split = 1;
                plan_.kernels.push_back(std::move(k));
                Step& s1 = push_step(Step::REDUCE);
                s1.kernel = int(plan_.kernels.size()) - 1;
                for (auto& in1 : plan_.kernels.back().ins) touch(in1.buf, s1.pos);
                touch(scratch, s1.pos);
                plan_.kernels.push_back(std::move(k2));
                Step& s2 = push_step(Step::REDUCE);
                s2.kernel = int(plan_.kernels.size()) - 1;
                touch(scratch, s2.pos);
                touch(buf, s2.pos);
                continue;
            }
            plan_.kernels.push_back(std::move(k));
            Step& s = push_step(Step::REDUCE);
            s.kernel = int(plan_.kernels.size()) - 1;
            for (auto& in : plan_.kernels.back().ins) touch(in.buf, s.pos);
            touch(buf, s.pos);
        }
        g_.buf_version[buf]++;
        if (overlaps) bind_value(c.res, g_.load(buf, {V}, contiguous_view({V})));
        else bind_own_buffer(c.res, buf, {V});
        cse[sum_key] = bind_[c.res].node;
        cse[g_.canon(sum_key)] = bind_[c.res].node;
    }

    // a GEMM operand: 2-d strided read of a buffer (anything else is copied out first)
    struct MatOperand {
        int buf;
        int64_t off, rs, cs;
    };
    MatOperand matrix_operand(Node* n) {
        n = g_.canon(n);
        bool ok = n->kind == N_LOAD && n->view.dims[0].size() <= 1 && n->view.dims[1].size() <= 1;
        if (ok) {
            int64_t rs = n->view.dims[0].empty() ? 0 : n->view.dims[0][0].stride;
            int64_t cs = n->view.dims[1].empty() ? 0 : n->view.dims[1][0].stride;
            // a broadcast (stride-0) axis of length > 1 is not a matrix in memory
            if ((rs == 0 && n->shape[0] > 1) || (cs == 0 && n->shape[1] > 1)) ok = false;
            if (ok) {
                if (n->shape[0] == 1) rs = n->shape[1] * (cs ? cs : 1);
                if (n->shape[1] == 1) cs = 1;
                return {n->buf, n->view.offset, rs, cs};
            }
        }
        Node* m = materialize_node(n);
        return {m->buf, 0, n->shape[1], 1};
    }

    // The tensor-core kernels fetch operands with TMA, which wants one unit stride and the other stride a multiple of four
    // elements (16 bytes).  A big operand that misses that (1001 columns, a slice starting at an odd column) is copied
    // once into a temporary whose rows are padded to a multiple of four; the padding is never read (the tensor map
    // knows the true extent).  Without it the product would fall back to the CUDA-core kernel, ten times slower.
    MatOperand aligned_operand(Node* n, const MatOperand& m, int64_t flops) {
        const bool unit_r = m.rs == 1, unit_c = m.cs == 1;
        const int64_t other = unit_c ? m.rs : m.cs;
        const bool ok = (unit_r || unit_c) && other % 4 == 0 && m.off % 4 == 0;
        if (ok || flops < (int64_t(1) << 24) || opt_.no_fusion) return m;
        n = g_.canon(n);
        const int64_t rows = n->shape[0], cols = n->shape[1];
        if (rows < 32 || cols < 8) return m;
        // keep the operand's majorness when it has one (a transposed view stays a transposed copy: no strided gather)
        const bool col_major = unit_r && !unit_c;
        const int64_t ld = ((col_major ? rows : cols) + 3) / 4 * 4;
        const int buf = temp_buffer(col_major ? cols * ld : rows * ld);
        View v;
        v.offset = 0;
        v.dims.resize(2);
        if (rows > 1) v.dims[0].push_back({rows, col_major ? 1 : ld});
        if (cols > 1) v.dims[1].push_back({cols, col_major ? ld : 1});
        std::vector<StoreTask> tasks;
        collect_stores(n, buf, v, tasks);
        emit_stores(tasks);
        g_.buf_version[buf]++;
        return {buf, 0, col_major ? 1 : ld, col_major ? ld : 1};
    }

    void lower_dot(const Cmd& c) {
        Node* a = resolve(c.a);
        Node* b = resolve(c.b);
        if (a->shape.size() != 2) fail("A must be a 2d array");
        if (b->shape.size() != 2) fail("B must be a 2d array");
        if (a->shape[1] != b->shape[0]) fail("A's second dimension must equal B's first dimension");
        int64_t M = a->shape[0], K = a->shape[1], N = b->shape[1];
        consume(c.a);
        consume(c.b);
        // nothing to sum over, or nothing to produce: the product is all zeros / has no elements
        if (K == 0 || M * N == 0) {
            after_op(c.res, g_.constant(0.0f, {M, N}));
            return;
        }
        // Matrix times vector (or vector times matrix) is a row sum of products: one pass over the matrix at memory
        // speed through the reduce kernels, instead of a tile kernel that would keep one column of its tiles busy.
        // (Summation order differs from the dot kernels' k-ascending one, like every other reduction here.)
        if ((N == 1 || M == 1) && M * N * K >= (int64_t(1) << 16) && K > 1 && !opt_.no_fusion) {
            Node* summand = nullptr;
            if (N == 1) {
                Node* row = g_.reshape(b, {1, K});
                if (!row) row = g_.reshape(materialize_node(b), {1, K});
                Node* rep = row ? g_.broadcast(row, 0, M) : nullptr;
                if (rep) summand = g_.op2(E_MUL, a, rep);
            } else {
                Node* bt = g_.permute(b, {1, 0});
                Node* rep = g_.broadcast(a, 0, N);
                if (bt && rep) summand = g_.op2(E_MUL, rep, bt);
            }
            if (summand) {
                lower_sum_node(c, summand, 0);
                Node* r = g_.reshape(resolve(c.res), {M, N});
                if (!r) fail("internal: matrix-vector result cannot be reshaped");
                bind_value(c.res, r);
                return;
            }
        }
        // A product of a few hundred multiply-adds is an element-wise expression: sum over k of (column k of A, repeated
        // along the columns) * (row k of B, repeated along the rows), k ascending like the dot kernels.  It then fuses with
        // whatever surrounds it (the whole training step of a 2 x 5 network becomes a handful of kernels instead of one
        // launch per product), and the expression limit of after_op keeps chains of such products from growing.
        if (!opt_.no_fusion && !opt_.no_tiny_dot && K <= TINY_DOT_K && M * N * K <= TINY_DOT_WORK) {
            Node* acc = nullptr;
            bool ok = true;
            for (int64_t k = 0; k < K && ok; k++) {
                Node* ak = g_.index(a, 1, k);
                if (ak) ak = g_.reshape(ak, {M, 1});
                if (ak) ak = g_.broadcast(ak, 1, N);
                Node* bk = g_.index(b, 0, k);
                if (bk) bk = g_.reshape(bk, {1, N});
                if (bk) bk = g_.broadcast(bk, 0, M);
                if (!ak || !bk) { ok = false; break; }
                Node* t = elementwise2(E_MUL, ak, bk);
                acc = acc ? elementwise2(E_ADD, acc, t) : t;
                if (!acc) ok = false;
            }
            if (ok && acc) {
                after_op(c.res, acc);
                return;
            }
        }
        std::pair<Node*, Node*> dot_key{a, b};
        {
            auto it = dot_cse_.find(dot_key);
            if (it != dot_cse_.end() && g_.load_valid(it->second)) {
                bind_value(c.res, it->second);
                return;
            }
        }
        MatOperand ma = matrix_operand(a);
        MatOperand mb = matrix_operand(b);
        if (M >= 32 && N >= 32 && K >= 8) {
            ma = aligned_operand(a, ma, M * N * K);
            mb = aligned_operand(b, mb, M * N * K);
        }
        Shape rs{M, N};
        int buf = result_buffer(c.res, rs);
        // `DotProduct v w -> v`: the kernels read A and B while other tiles of C are already being written (and a
        // split k loop zeroes C first), so the product never lands in a buffer it reads from; it goes to a
        // temporary and the id is bound to that (copied into the id's own buffer at the next flush if it needs one)
        const bool overlaps = buf == ma.buf || buf == mb.buf;
        const int own = buf;
        if (overlaps) buf = temp_buffer(M * N);
        before_write(buf, {c.res});
        Step& s = push_step(Step::GEMM);
        s.gemm.a = ma.buf; s.gemm.b = mb.buf; s.gemm.c = buf;
        s.gemm.M = M; s.gemm.N = N; s.gemm.K = K;
        s.gemm.a_off = ma.off; s.gemm.b_off = mb.off; s.gemm.c_off = 0;
        s.gemm.a_rs = ma.rs; s.gemm.a_cs = ma.cs; s.gemm.b_rs = mb.rs; s.gemm.b_cs = mb.cs;
        touch(ma.buf, s.pos);
        touch(mb.buf, s.pos);
        touch(buf, s.pos);
        g_.buf_version[buf]++;
        if (overlaps) {
            (void)own;
            bind_value(c.res, g_.load(buf, rs, contiguous_view(rs)));
        } else
            bind_own_buffer(c.res, buf, rs);
        dot_cse_[dot_key] = bind_[c.res].node;
        // operands that were just written to memory are found under their new identity as well
        dot_cse_[{g_.canon(a), g_.canon(b)}] = bind_[c.res].node;
    }

    // BatchDot (extension; the reference lists batched matmul as missing, TODO.md:22, and runs one 2-d DotProduct per
    // attention head, src/nn/transformer.rs:10-18): [B,M,K] x [B,K,N] -> [B,M,N] as ONE step; the slices of an operand
    // are a fixed number of elements apart, so transposed / permuted operands need no copy as long as every axis of
    // the view is a single stride.
    void lower_batch_dot(const Cmd& c) {
        Node* a = resolve(c.a);
        Node* b = resolve(c.b);
        if (a->shape.size() != 3 || b->shape.size() != 3) fail("BatchDot needs 3-d operands");
        if (a->shape[0] != b->shape[0]) fail("BatchDot operands differ in their batch size");
        if (a->shape[2] != b->shape[1]) fail("A's last dimension must equal B's second dimension");
        const int64_t B = a->shape[0], M = a->shape[1], K = a->shape[2], N = b->shape[2];
        consume(c.a);
        consume(c.b);
        if (K == 0 || B * M * N == 0) {
            after_op(c.res, g_.constant(0.0f, {B, M, N}));
            return;
        }
        struct Op3 { int buf; int64_t off, bs, rs, cs; };
        auto operand = [&](Node* n) -> Op3 {
            n = g_.canon(n);
            bool ok = n->kind == N_LOAD;
            for (int d = 0; ok && d < 3; d++) ok = n->view.dims[size_t(d)].size() <= 1;
            if (ok) {
                auto st = [&](int d) { return n->view.dims[size_t(d)].empty() ? int64_t(0) : n->view.dims[size_t(d)][0].stride; };
                int64_t bs = st(0), rs = st(1), cs = st(2);
                if ((rs == 0 && n->shape[1] > 1) || (cs == 0 && n->shape[2] > 1)) ok = false;
                if (ok) {
                    if (n->shape[1] == 1) rs = n->shape[2] * (cs ? cs : 1);
                    if (n->shape[2] == 1) cs = 1;
                    return {n->buf, n->view.offset, bs, rs, cs};
                }
            }
            Node* m = materialize_node(n);
            return {m->buf, 0, n->shape[1] * n->shape[2], n->shape[2], 1};
        };
        Op3 oa = operand(a), ob = operand(b);
        Shape rs{B, M, N};
        int buf = result_buffer(c.res, rs);
        const bool overlaps = buf == oa.buf || buf == ob.buf;
        if (overlaps) buf = temp_buffer(B * M * N);
        before_write(buf, {c.res});
        Step& s = push_step(Step::GEMM);
        s.gemm.a = oa.buf; s.gemm.b = ob.buf; s.gemm.c = buf;
        s.gemm.M = M; s.gemm.N = N; s.gemm.K = K;
        s.gemm.a_off = oa.off; s.gemm.b_off = ob.off; s.gemm.c_off = 0;
        s.gemm.a_rs = oa.rs; s.gemm.a_cs = oa.cs; s.gemm.b_rs = ob.rs; s.gemm.b_cs = ob.cs;
        s.gemm.batch = B; s.gemm.a_bs = oa.bs; s.gemm.b_bs = ob.bs; s.gemm.c_bs = M * N;
        touch(oa.buf, s.pos);
        touch(ob.buf, s.pos);
        touch(buf, s.pos);
        g_.buf_version[buf]++;
        if (overlaps) bind_value(c.res, g_.load(buf, rs, contiguous_view(rs)));
        else bind_own_buffer(c.res, buf, rs);
    }

    void lower_allreduce(const Cmd& c) {
        if (bind_[c.a].kind != Binding::VALUE) fail("AllReduce target '" + name(c.a) + "' must be a tensor, not a view");
        consume(c.a);
        materialize_ids({c.a});  // the id is cross-segment by construction, so this is its own buffer
        Node* a = resolve(c.a);
        if (a->kind != N_LOAD || info_[c.a].buf != a->buf) fail("internal: AllReduce target has no buffer");
        int buf = a->buf;
        before_write(buf, {c.a});
        Step& s = push_step(Step::ALLREDUCE);
        s.buf = buf;
        s.off = 0;
        s.nelem = numel(a->shape);
        touch(buf, s.pos);
        g_.buf_version[buf]++;
        bind_own_buffer(c.a, buf, a->shape);
    }

    std::pair<int, int64_t> condition_location(uint32_t id) {
        Node* n = resolve(id);
        if (numel(n->shape) != 1) fail("condition '" + name(id) + "' must have dim of [1]");
        if (n->kind != N_LOAD) {
            bind_[id].pending = true;
            if (bind_[id].kind == Binding::ALIAS) {
                Node* m = materialize_node(n);
                return {m->buf, m->view.offset};
            }
            materialize_ids({id});
            n = resolve(id);
        }
        return {n->buf, n->view.offset};
    }

    // What was computed on one side of a control-flow boundary cannot be reused on the other by identity: an
    // expression evaluated in front of a loop is out of date once the body has changed its operands, and one
    // evaluated inside a body or a branch may never have been evaluated at all.  Forwarded nodes and remembered
    // sums / products are only followed while the buffer they were written to keeps its version, so advancing every
    // version cuts all of those links; ids keep their buffers (refresh_bindings rebinds them at the new version).
    void forget_computed_values() {
        // an id bound to an expression that has been written out (the expression forwards to a load of the buffer) is
        // bound to that load first: once the versions move, the forward is no longer followed and the expression's own
        // operands are out of date as well
        for (auto& b : bind_)
            if (b.kind == Binding::VALUE && b.node) {
                Node* n = g_.canon(b.node);
                if (n->kind == N_LOAD) b.node = n;
            }
        for (auto& v : g_.buf_version) v++;
        refresh_bindings();
    }

    void refresh_bindings() {
        for (auto& b : bind_) {
            if (b.kind == Binding::VALUE && b.node) {
                Node* n = g_.canon(b.node);
                if (n->kind == N_LOAD && !g_.load_valid(n)) b.node = g_.load(n->buf, n->shape, n->view);
            }
            b.cache = nullptr;
        }
    }

    // returns true when an EX was reached at this level
    bool lower_block(Block& blk, bool top) {
        for (size_t ci = 0; ci < blk.cmds.size(); ci++) {
            auto& c = blk.cmds[ci];
            if (c.op == OP_EX) {
                flush_pending();
                if (top) {
                    finalize_results();
                    push_step(Step::EXIT);
                    return true;
                }
                push_step(Step::EXIT);
                continue;
            }
            if (c.op == OP_WHILE) {
                freeze_for_blocks({c.block.get()}, blk, ci);
                flush_pending();
                auto loc = condition_location(c.a);
                consume(c.a);
                StepBlock* saved = cur_;
                Step& s = push_step(Step::WHILE);
                s.cond_buf = loc.first;
                s.cond_off = loc.second;
                touch(loc.first, s.pos);
                s.body = std::make_unique<StepBlock>();
                int first = pos_;
                StepBlock* body = s.body.get();
                forget_computed_values();
                cur_ = body;
                frames_.push_back({&blk, ci, true});
                lower_block(*c.block, false);
                freeze_at_end(*c.block);
                frames_.pop_back();
                flush_pending();
                cur_ = saved;
                loop_spans_.push_back({first, pos_});
                auto loc2 = condition_location(c.a);
                if (loc2 != loc) fail("While condition '" + name(c.a) + "' moves to another buffer inside the loop");
                forget_computed_values();
                continue;
            }
            if (c.op == OP_IF) {
                {
                    std::vector<const Block*> inner;
                    for (auto& cb : c.conds) inner.push_back(cb.second.get());
                    if (c.else_block) inner.push_back(c.else_block.get());
                    freeze_for_blocks(inner, blk, ci);
                }
                flush_pending();
                StepBlock* saved = cur_;
                std::vector<std::pair<int, int64_t>> locs;
                for (auto& cb : c.conds) {
                    locs.push_back(condition_location(cb.first));
                    consume(cb.first);
                }
                Step& s = push_step(Step::IF);
                Step* sp = &s;
                for (auto& loc : locs) {
                    touch(loc.first, sp->pos);
                    Step::Branch br;
                    br.cond_buf = loc.first;
                    br.cond_off = loc.second;
                    sp->branches.push_back(std::move(br));
                }
                std::vector<Binding> snapshot = bind_;
                for (size_t k = 0; k < c.conds.size(); k++) {
                    sp->branches[k].body = std::make_unique<StepBlock>();
                    cur_ = sp->branches[k].body.get();
                    frames_.push_back({&blk, ci, false});
                    lower_block(*c.conds[k].second, false);
                    freeze_at_end(*c.conds[k].second);
                    frames_.pop_back();
                    flush_pending();
                    restore_after_branch(snapshot);
                }
                if (c.else_block) {
                    sp->else_body = std::make_unique<StepBlock>();
                    cur_ = sp->else_body.get();
                    frames_.push_back({&blk, ci, false});
                    lower_block(*c.else_block, false);
                    freeze_at_end(*c.else_block);
                    frames_.pop_back();
                    flush_pending();
                    restore_after_branch(snapshot);
                }
                cur_ = saved;
                continue;
            }
            if (!live(c)) continue;
            lower_cmd(c);
        }
        return false;
    }

    // after a conditional branch: ids (re)defined inside live in their persistent buffers, everything
    // else looks as it did before the branch
    void restore_after_branch(const std::vector<Binding>& snapshot) {
        for (size_t id = 0; id < bind_.size(); id++) {
            Binding& b = bind_[id];
            const Binding& s = snapshot[id];
            bool changed = b.kind != s.kind || b.node != s.node || b.cmd != s.cmd;
            if (!changed) continue;
            if (info_[id].buf >= 0 && info_[id].needs_buffer() && b.kind == Binding::VALUE) {
                Node* n = g_.canon(b.node);
                b.node = g_.load(info_[id].buf, n->shape, contiguous_view(n->shape));
                b.pending = false;
            } else
                b = s;
        }
        forget_computed_values();
    }

    void finalize_results() {
        if (results_done_) return;
        flush_pending();
        for (auto id : prog_.dep) {
            ResultInfo r;
            r.id = name(id);
            Binding& b = bind_[id];
            if (b.kind == Binding::UNDEF) {
                plan_.results.push_back(r);
                continue;
            }
            Node* n = resolve(id);
            if (!(n->kind == N_LOAD && view_is_contiguous(n->view, n->shape))) n = materialize_node(n);
            r.shape = n->shape;
            r.buf = n->buf;
            r.off = n->view.offset;
            plan_.bufs[n->buf].persistent = true;
            plan_.results.push_back(r);
        }
        results_done_ = true;
    }

    // ------------------------------------------------------------------ sums fused into element-wise passes
    // A Sum whose summand is built from the operands an element-wise kernel streams anyway (or from a value that
    // kernel writes) costs a second pass over the same memory when it runs as a kernel of its own: config 2's
    // loss and bias gradient re-read both 256 MB inputs, a bias gradient re-reads the activation gradient that the
    // kernel before it wrote.  This pass moves such a reduce step into the element-wise kernel as a side sum
    // (KernelSpec::reds) when the two walk the same index space and no other step gets in the way.  The reference
    // fuses in the other direction only (a reduce followed by element-wise work on its result,
    // src/kernel/fusion/reduce_elw.rs:12-144).
    static constexpr int POS_SCALE = 64;       // room between two original step positions for moved / added steps
    static constexpr int64_t FUSE_MIN_ELEMS = int64_t(1) << 18;

    void step_rw(const Step& s, std::vector<int>& rd, std::vector<int>& wr) const {
        rd.clear();
        wr.clear();
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE:
            kernel_rw(plan_, s.kernel, rd, wr);
            break;
        case Step::GEMM:
            rd = {s.gemm.a, s.gemm.b};
            wr = {s.gemm.c};
            if (s.gemm.accumulate) rd.push_back(s.gemm.c);
            if (s.gemm.colvec >= 0) rd.push_back(s.gemm.colvec);
            if (s.gemm.out >= 0) wr.push_back(s.gemm.out);
            break;
        case Step::UPLOAD: wr = {s.buf}; break;
        case Step::ALLREDUCE:
            rd = {s.buf};
            rd.insert(rd.end(), s.more_bufs.begin(), s.more_bufs.end());
            wr = rd;
            break;
        default: break;
        }
    }
    static bool hits(const std::vector<int>& a, const std::vector<int>& b) {
        for (int x : a)
            for (int y : b)
                if (x == y) return true;
        return false;
    }
    static bool is_barrier(const Step& s) { return s.kind == Step::WHILE || s.kind == Step::IF || s.kind == Step::EXIT; }

    void scale_positions(StepBlock& blk, int f) {
        for (auto& s : blk.steps) {
            s.pos *= f;
            if (s.body) scale_positions(*s.body, f);
            for (auto& br : s.branches) scale_positions(*br.body, f);
            if (s.else_body) scale_positions(*s.else_body, f);
        }
    }
    // multiplies every step position (and everything measured in positions) by f: room for steps that passes add
    bool scale_all(int f) {
        if (pos_ >= INT_MAX / f - 1) return false;
        scale_positions(plan_.main, f);
        for (auto& b : plan_.bufs) {
            if (b.first != INT_MAX) b.first *= f;
            if (b.last >= 0) b.last *= f;
        }
        for (auto& sp : loop_spans_) { sp.first *= f; sp.second *= f; }
        pos_ *= f;
        return true;
    }

    void fuse_reductions() {
        if (opt_.no_fusion || opt_.no_reduce_fusion) return;
        if (!scale_all(POS_SCALE)) return;
        fuse_rows(plan_.main);
        fuse_block(plan_.main);
        if (opt_.world > 1) hoist_collectives(plan_.main);
    }

    // ------------------------------------------------------------------ collectives next to their producers
    // The frontend's optimiser step comes after the whole backward pass, so every gradient all-reduce (and the small
    // kernel that scales its operand) sits at the end of the step, behind the last dot product.  Each such pair is
    // moved up to right behind the step that produces the gradient: a runtime that issues collectives on their own
    // stream can then overlap them with the remaining dot products.  On a single stream the order is immaterial.
    static int last_pos(const Step& s) {
        int p = s.pos;
        if (s.body && !s.body->steps.empty()) p = std::max(p, last_pos(s.body->steps.back()));
        for (auto& br : s.branches)
            if (!br.body->steps.empty()) p = std::max(p, last_pos(br.body->steps.back()));
        if (s.else_body && !s.else_body->steps.empty()) p = std::max(p, last_pos(s.else_body->steps.back()));
        return p;
    }
    void hoist_collectives(StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (s.body) hoist_collectives(*s.body);
            for (auto& br : s.branches) hoist_collectives(*br.body);
            if (s.else_body) hoist_collectives(*s.else_body);
        }
        auto& steps = blk.steps;
        std::vector<int> rd, wr, prd, pwr;
        for (size_t j = 1; j < steps.size(); j++) {
            if (steps[j].kind != Step::ALLREDUCE || steps[j - 1].kind != Step::ELW) continue;
            const KernelSpec& pk = plan_.kernels[size_t(steps[j - 1].kernel)];
            if (pk.type != KernelSpec::ELW || pk.outs.size() != 1 || !pk.reds.empty() || pk.outs[0].dst.buf != steps[j].buf) continue;
            step_rw(steps[j - 1], prd, pwr);   // the pair reads prd, writes pwr (the all-reduce works in place on pwr)
            // how far up can the pair go?
            size_t i = j - 1;                  // the pair ends up right behind steps[i - 1]
            while (i > 0) {
                const Step& q = steps[i - 1];
                if (is_barrier(q)) break;
                step_rw(q, rd, wr);
                if (hits(wr, prd) || hits(wr, pwr) || hits(rd, pwr)) break;
                i--;
            }
            // never to the very head of a block: positions in front of a body's first step belong to the enclosing block
            // (its While / If step sits right there), and the pair is as early behind the first step
            if (i == 0) i = 1;
            if (i + 1 >= j) continue;          // nowhere to go (also: i == j - 1 means "stay")
            // positions right behind steps[i - 1] (behind everything nested in it, when it is a While / If)
            const int base = last_pos(steps[i - 1]);
            int next_pos = base + 1;
            size_t ins_at = i;
            while (ins_at < steps.size() && steps[ins_at].pos < base + POS_SCALE && ins_at < j - 1) { next_pos = steps[ins_at].pos + 1; ins_at++; }
            if (ins_at >= j - 1 || next_pos + 2 >= base + POS_SCALE - 1 || (ins_at < steps.size() && next_pos + 1 >= steps[ins_at].pos)) continue;
            Step a = std::move(steps[j - 1]), b = std::move(steps[j]);
            steps.erase(steps.begin() + long(j - 1), steps.begin() + long(j + 1));
            a.pos = next_pos;
            b.pos = next_pos + 1;
            for (int x : prd) touch(x, a.pos);
            for (int x : pwr) { touch(x, a.pos); touch(x, b.pos); }
            steps.insert(steps.begin() + long(ins_at), std::move(b));
            steps.insert(steps.begin() + long(ins_at), std::move(a));
        }
    }

    // ------------------------------------------------------------------ row reductions chained with their consumers
    // mean -> variance -> normalise, max -> sum of exponentials -> divide: consecutive steps over the same [P, Q]
    // space in which later ones read the per-row results of earlier ones.  As separate kernels every step streams
    // the input again; as one ROWS kernel (one block per row, section "gen_rows" of the code generator) the input
    // comes from HBM once.  Only adjacent steps are chained, rows of 512 .. 16384 elements, and the per-row results
    // are still written out (other steps may read them).
    void fuse_rows(StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (s.body) fuse_rows(*s.body);
            for (auto& br : s.branches) fuse_rows(*br.body);
            if (s.else_body) fuse_rows(*s.else_body);
        }
        auto& steps = blk.steps;
        for (size_t i = 0; i < steps.size(); i++) {
            if (steps[i].kind != Step::REDUCE) continue;
            const KernelSpec& first = plan_.kernels[size_t(steps[i].kernel)];
            if (first.scratch >= 0 || first.split != 1 || first.mode != 0) continue;
            const int64_t P = first.n, Q = first.r;
            const bool small_ok = opt_.fuse_small_sums;
            if (!small_ok && (P < 64 || Q < 512 || Q > 16384 || P * Q < FUSE_MIN_ELEMS)) continue;
            if (P < 1 || Q < 1) continue;

            KernelSpec rk;
            rk.type = KernelSpec::ROWS;
            rk.n = P * Q;
            rk.p2 = P;
            rk.q2 = Q;
            std::map<std::tuple<int, int, uint32_t, int, int, int>, int> known;
            auto key_of = [](const Ssa& v) {
                uint32_t bits;
                std::memcpy(&bits, &v.c, 4);
                int a = v.kind == Ssa::OP ? v.a : -1, b = v.kind == Ssa::OP ? v.b : -1;
                if (v.kind == Ssa::OP && b >= 0 && a > b) std::swap(a, b);
                return std::make_tuple(int(v.kind), (v.kind == Ssa::LOAD || v.kind == Ssa::RED) ? v.operand : -1,
                                       v.kind == Ssa::CONST ? bits : 0u, v.kind == Ssa::OP ? int(v.op) : -1, a, b);
            };
            auto intern = [&](Ssa v) {
                auto it = known.find(key_of(v));
                if (it != known.end()) return it->second;
                rk.ssa.push_back(v);
                known.emplace(key_of(v), int(rk.ssa.size()) - 1);
                return int(rk.ssa.size()) - 1;
            };
            std::vector<int> written;   // buffers the chain writes (phase results, final outputs)
            auto phase_of = [&](const Operand& o, const std::vector<Sub>& flat) -> int {
                // a load of an earlier phase's per-row result, broadcast along the row?
                std::vector<Sub> want;
                if (P > 1) want.push_back({P, 1});
                if (Q > 1) want.push_back({Q, 0});
                canon_subs(want);
                for (size_t k = 0; k < rk.phases.size(); k++)
                    if (rk.phases[k].dst.buf == o.buf && rk.phases[k].dst.offset == o.offset && flat == want) return int(k);
                return -1;
            };
            // adds one step to the ROWS kernel under construction; false = the chain ends before it
            auto absorb = [&](const KernelSpec& k) {
                const bool is_reduce = k.type == KernelSpec::REDUCE;
                if (is_reduce) {
                    // lanes along the summed axis only: a column sum walks memory with a large stride per row
                    if (k.mode != 0 || k.n != P || k.r != Q || k.scratch >= 0 || k.split != 1) return false;
                    std::vector<Sub> d = k.outs[0].dst.xsubs;
                    canon_subs(d);
                    std::vector<Sub> contiguous;
                    if (P > 1) contiguous.push_back({P, 1});
                    if (d != contiguous) return false;
                } else {
                    if (k.type != KernelSpec::ELW || k.n != P * Q || !k.reds.empty()) return false;
                }
                // operands
                std::vector<int> in_of(k.ins.size(), -1), red_of(k.ins.size(), -1);
                const size_t ins_before = rk.ins.size();
                for (size_t t = 0; t < k.ins.size(); t++) {
                    const Operand& o = k.ins[t];
                    std::vector<Sub> flat = is_reduce ? flat_digits(o, true) : o.subs;
                    canon_subs(flat);
                    const bool chain_written = std::find(written.begin(), written.end(), o.buf) != written.end();
                    if (chain_written) {
                        red_of[t] = phase_of(o, flat);
                        if (red_of[t] < 0) { rk.ins.resize(ins_before); return false; }
                        continue;
                    }
                    Operand no;
                    no.buf = o.buf;
                    no.offset = o.offset;
                    no.subs = flat;
                    for (size_t u = 0; u < rk.ins.size(); u++)
                        if (rk.ins[u].same_access(no)) in_of[t] = int(u);
                    if (in_of[t] < 0) {
                        rk.ins.push_back(no);
                        in_of[t] = int(rk.ins.size()) - 1;
                    }
                }
                // outputs must not touch anything the chain reads or wrote
                for (auto& out : k.outs) {
                    for (auto& in : rk.ins)
                        if (in.buf == out.dst.buf) { rk.ins.resize(ins_before); return false; }
                    if (std::find(written.begin(), written.end(), out.dst.buf) != written.end()) { rk.ins.resize(ins_before); return false; }
                }
                // splice the SSA
                std::vector<int> remap(k.ssa.size(), -1);
                for (size_t t = 0; t < k.ssa.size(); t++) {
                    Ssa v = k.ssa[t];
                    if (v.kind == Ssa::LOAD) {
                        if (red_of[size_t(v.operand)] >= 0) { v.kind = Ssa::RED; v.operand = red_of[size_t(v.operand)]; }
                        else v.operand = in_of[size_t(v.operand)];
                    } else if (v.kind == Ssa::OP) {
                        v.a = remap[size_t(v.a)];
                        if (v.b >= 0) v.b = remap[size_t(v.b)];
                    }
                    remap[t] = intern(v);
                }
                if (is_reduce) {
                    KernelSpec::Phase ph;
                    ph.red_op = k.red_op;
                    ph.ssa = remap[size_t(k.outs[0].ssa)];
                    ph.dst = k.outs[0].dst;
                    rk.phases.push_back(ph);
                    written.push_back(ph.dst.buf);
                } else {
                    for (auto& out : k.outs) {
                        KernelSpec::Out no = out;
                        no.ssa = remap[size_t(out.ssa)];
                        rk.outs.push_back(no);
                        written.push_back(out.dst.buf);
                    }
                }
                return true;
            };

            size_t j = i;
            bool uses_result = false;
            while (j < steps.size() && rk.phases.size() < 4) {
                const Step& st = steps[j];
                if (st.kind != Step::REDUCE && st.kind != Step::ELW) break;
                const KernelSpec& k = plan_.kernels[size_t(st.kernel)];
                if (!absorb(k)) break;
                j++;
                if (st.kind == Step::ELW) break;   // the store loop closes the chain
            }
            for (auto& v : rk.ssa) uses_result = uses_result || v.kind == Ssa::RED;
            const size_t count = j - i;
            if (count < 2 || !uses_result || rk.phases.empty()) continue;

            // commit: one ROWS step at the position of the last chain member
            const int pos = steps[j - 1].pos;
            for (size_t q = i; q < j; q++) plan_.kernels[size_t(steps[q].kernel)].dead = true;
            plan_.kernels.push_back(std::move(rk));
            Step ns;
            ns.kind = Step::ELW;
            ns.pos = pos;
            ns.kernel = int(plan_.kernels.size()) - 1;
            {
                std::vector<int> rd, wr;
                const KernelSpec& nk = plan_.kernels.back();
                for (auto& in : nk.ins) touch(in.buf, pos);
                for (auto& out : nk.outs) touch(out.dst.buf, pos);
                for (auto& ph : nk.phases) touch(ph.dst.buf, pos);
            }
            steps.erase(steps.begin() + long(i), steps.begin() + long(j));
            steps.insert(steps.begin() + long(i), std::move(ns));
        }
    }

    void fuse_block(StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (s.body) fuse_block(*s.body);
            for (auto& br : s.branches) fuse_block(*br.body);
            if (s.else_body) fuse_block(*s.else_body);
        }
        for (size_t e = 0; e < blk.steps.size(); e++) {
            if (blk.steps[e].kind != Step::ELW) continue;
            if (plan_.kernels[size_t(blk.steps[e].kernel)].type != KernelSpec::ELW) continue;
            if (plan_.kernels[size_t(blk.steps[e].kernel)].n < (opt_.fuse_small_sums ? 1 : FUSE_MIN_ELEMS)) continue;
            bool again = true;
            while (again && plan_.kernels[size_t(blk.steps[e].kernel)].reds.size() < 4) {
                again = false;
                // straight-line neighbourhood of the kernel
                size_t lo = e, hi = e;
                while (lo > 0 && !is_barrier(blk.steps[lo - 1]) && e - (lo - 1) <= 48) lo--;
                while (hi + 1 < blk.steps.size() && !is_barrier(blk.steps[hi + 1]) && (hi + 1) - e <= 48) hi++;
                for (size_t r = lo; r <= hi && !again; r++) {
                    if (r == e || blk.steps[r].kind != Step::REDUCE) continue;
                    size_t e_now = e;
                    if (try_fuse(blk, r, e_now)) {
                        e = e_now;
                        again = true;
                    }
                }
            }
        }
    }

    // flat digits of a reduce operand when the reduce's [V, R] space is laid over the flat index with the kept axis
    // outermost (x_major) or innermost
    static std::vector<Sub> flat_digits(const Operand& o, bool x_major) {
        std::vector<Sub> d;
        if (x_major) { d = o.xsubs; d.insert(d.end(), o.subs.begin(), o.subs.end()); }
        else { d = o.subs; d.insert(d.end(), o.xsubs.begin(), o.xsubs.end()); }
        canon_subs(d);
        return d;
    }

    // tries to turn the reduce at index r into a side sum of the element-wise kernel at index e; on success the
    // step list is rewritten and e is updated to the kernel's new index
    bool try_fuse(StepBlock& blk, size_t r, size_t& e) {
        auto& steps = blk.steps;
        const KernelSpec& rk0 = plan_.kernels[size_t(steps[r].kernel)];
        if (rk0.red_op != 0) return false;  // side sums only
        // second pass of a split reduce: handled together with its first pass
        if (r > 0 && steps[r - 1].kind == Step::REDUCE && r - 1 != e) {
            const KernelSpec& prev = plan_.kernels[size_t(steps[r - 1].kernel)];
            if (prev.scratch >= 0 && rk0.ins.size() == 1 && rk0.ins[0].buf == prev.scratch) return false;
        }
        size_t r_end = r;  // last step of the reduce group
        Operand final_dst = rk0.outs[0].dst;
        int old_scratch = -1;
        if (rk0.scratch >= 0) {
            if (r + 1 >= steps.size() || steps[r + 1].kind != Step::REDUCE || r + 1 == e) return false;
            const KernelSpec& k2 = plan_.kernels[size_t(steps[r + 1].kernel)];
            if (k2.ins.size() != 1 || k2.ins[0].buf != rk0.scratch) return false;
            r_end = r + 1;
            final_dst = k2.outs[0].dst;
            old_scratch = rk0.scratch;
        }
        if (r < e && r_end >= e) return false;
        const bool sink = r < e;  // the reduce runs before the kernel today and moves down to it
        KernelSpec& ek = plan_.kernels[size_t(steps[e].kernel)];
        const int64_t V = rk0.n, R = rk0.r;
        if (V <= 0 || R <= 0 || V * R != ek.n) return false;

        // dependences
        std::vector<int> rd, wr, e_rd, e_wr, r_rd;
        step_rw(steps[e], e_rd, e_wr);
        for (auto& in : rk0.ins) r_rd.push_back(in.buf);
        const std::vector<int> r_wr = {final_dst.buf};
        if (hits(e_rd, r_wr) && sink) return false;  // the kernel consumes the sum
        std::vector<size_t> moved;                    // sink: steps between the reduce and the kernel that depend on the sum
        if (sink) {
            // (a summand input that the kernel overwrites is looked at below: allowed only as an in-place update
            //  of the very elements the same thread reads)
            std::vector<int> tainted = r_wr;
            for (size_t q = r_end + 1; q < e; q++) {
                step_rw(steps[q], rd, wr);
                if (hits(rd, tainted)) {
                    moved.push_back(q);
                    tainted.insert(tainted.end(), wr.begin(), wr.end());
                }
            }
            if (hits(e_rd, tainted)) return false;
            if (moved.size() > 24) return false;
            // a moved step must not cross a step it conflicts with; the summand's inputs must stay untouched
            for (size_t q = r_end + 1; q <= e; q++) {
                if (std::find(moved.begin(), moved.end(), q) != moved.end()) continue;
                step_rw(steps[q], rd, wr);
                if (q != e && hits(wr, r_rd)) return false;
                if (hits(wr, r_wr)) return false;
                for (size_t m : moved) {
                    if (m > q) continue;
                    std::vector<int> mrd, mwr;
                    step_rw(steps[m], mrd, mwr);
                    if (hits(wr, mrd) || hits(wr, mwr) || hits(rd, mwr)) return false;
                }
            }
        } else {
            for (size_t q = e + 1; q < r; q++) {
                step_rw(steps[q], rd, wr);
                if (hits(wr, r_rd) || hits(rd, r_wr) || hits(wr, r_wr)) return false;
            }
            if (hits(e_wr, r_wr)) return false;
        }

        // steps that earlier fusions parked right behind the kernel: the new ones line up after them, so they must
        // not depend on each other in either direction; and there must be positions left
        const int e_pos = steps[e].pos;
        {
            int used = 0;
            std::vector<int> nrd = {final_dst.buf}, nwr = {final_dst.buf};
            for (size_t m : moved) {
                std::vector<int> mrd, mwr;
                step_rw(steps[m], mrd, mwr);
                nrd.insert(nrd.end(), mrd.begin(), mrd.end());
                nwr.insert(nwr.end(), mwr.begin(), mwr.end());
            }
            for (size_t q = e + 1; q < steps.size() && steps[q].pos < e_pos + POS_SCALE; q++) {
                used++;
                step_rw(steps[q], rd, wr);
                if (hits(rd, nwr) || hits(wr, nrd) || hits(wr, nwr)) return false;
            }
            if (used + 1 + int(moved.size()) >= POS_SCALE - 2) return false;
        }
        std::vector<int> dead_kernels;
        for (size_t q = r; q <= r_end; q++) dead_kernels.push_back(steps[q].kernel);

        // index spaces: which of the two layouts of [V, R] over the flat index matches the kernel's operands?
        struct Match { bool ok = false; std::vector<int> in_of; std::vector<int> val_of; };
        auto match = [&](bool x_major) {
            Match m;
            m.in_of.assign(rk0.ins.size(), -1);
            m.val_of.assign(rk0.ins.size(), -1);
            for (size_t i = 0; i < rk0.ins.size(); i++) {
                const Operand& o = rk0.ins[i];
                std::vector<Sub> d = flat_digits(o, x_major);
                const bool written_by_e = std::find(e_wr.begin(), e_wr.end(), o.buf) != e_wr.end();
                if (written_by_e && sink) {
                    // in-place update: the summand wants the old value, which the kernel loads from the same
                    // element before it stores the new one -- every access of the kernel to this buffer must be
                    // this very access
                    for (size_t j = 0; j < ek.ins.size(); j++) {
                        std::vector<Sub> ed = ek.ins[j].subs;
                        canon_subs(ed);
                        if (ek.ins[j].buf == o.buf && ek.ins[j].offset == o.offset && ed == d) m.in_of[i] = int(j);
                    }
                    if (m.in_of[i] < 0) return m;
                    for (auto& in2 : ek.ins)
                        if (in2.buf == o.buf && !in2.same_access(ek.ins[size_t(m.in_of[i])])) return m;
                    for (auto& o2 : ek.outs) {
                        if (o2.dst.buf != o.buf) continue;
                        std::vector<Sub> od = o2.dst.subs;
                        canon_subs(od);
                        if (o2.dst.offset != o.offset || od != d) return m;
                    }
                } else if (written_by_e) {
                    for (size_t j = 0; j < ek.outs.size(); j++) {
                        std::vector<Sub> ed = ek.outs[j].dst.subs;
                        canon_subs(ed);
                        if (ek.outs[j].dst.buf == o.buf && ek.outs[j].dst.offset == o.offset && ed == d) m.val_of[i] = ek.outs[j].ssa;
                    }
                    if (m.val_of[i] < 0) return m;
                } else {
                    for (size_t j = 0; j < ek.ins.size(); j++) {
                        std::vector<Sub> ed = ek.ins[j].subs;
                        canon_subs(ed);
                        if (ek.ins[j].buf == o.buf && ek.ins[j].offset == o.offset && ed == d) m.in_of[i] = int(j);
                    }
                    if (m.in_of[i] < 0) return m;
                }
            }
            m.ok = true;
            return m;
        };
        int axis = -1;
        int64_t P = 0, Q = 0;
        Match mt;
        for (int t = 0; t < 2 && axis < 0; t++) {
            const bool x_major = t == 0;
            const int64_t p = x_major ? V : R, q = x_major ? R : V;
            if (!ek.reds.empty() && (p != ek.p2 || q != ek.q2)) continue;
            if (!opt_.fuse_small_sums && (q < 128 || p < 8)) continue;
            Match m = match(x_major);
            if (!m.ok) continue;
            mt = std::move(m);
            axis = x_major ? 0 : 1;
            P = p;
            Q = q;
        }
        if (axis < 0) return false;
        // the kernel must keep its vector width
        {
            KernelSpec probe;
            probe.n = ek.n;
            probe.ins = ek.ins;
            probe.outs = ek.outs;
            if (elw_vec(probe) == 4 && Q % 4) return false;
        }

        // splice the summand into the kernel's SSA
        std::map<std::tuple<int, int, uint32_t, int, int, int>, int> known;
        auto key_of = [](const Ssa& s) {
            uint32_t bits;
            std::memcpy(&bits, &s.c, 4);
            // + and * commute exactly: the two kernels may have ordered the same operands differently
            int a = s.kind == Ssa::OP ? s.a : -1, b = s.kind == Ssa::OP ? s.b : -1;
            if (s.kind == Ssa::OP && b >= 0 && a > b) std::swap(a, b);
            return std::make_tuple(int(s.kind), s.kind == Ssa::LOAD ? s.operand : -1, s.kind == Ssa::CONST ? bits : 0u,
                                   s.kind == Ssa::OP ? int(s.op) : -1, a, b);
        };
        for (size_t i = 0; i < ek.ssa.size(); i++) known.emplace(key_of(ek.ssa[i]), int(i));
        std::vector<int> remap(rk0.ssa.size(), -1);
        for (size_t i = 0; i < rk0.ssa.size(); i++) {
            Ssa s = rk0.ssa[i];
            if (s.kind == Ssa::LOAD) {
                if (mt.val_of[size_t(s.operand)] >= 0) { remap[i] = mt.val_of[size_t(s.operand)]; continue; }
                s.operand = mt.in_of[size_t(s.operand)];
            } else if (s.kind == Ssa::OP) {
                s.a = remap[size_t(s.a)];
                if (s.b >= 0) s.b = remap[size_t(s.b)];
            }
            auto it = known.find(key_of(s));
            if (it != known.end()) { remap[i] = it->second; continue; }
            ek.ssa.push_back(s);
            remap[i] = int(ek.ssa.size()) - 1;
            known.emplace(key_of(s), remap[i]);
        }

        // launch geometry and the partial-sum buffer
        if (ek.reds.empty()) {
            ek.p2 = P;
            ek.q2 = Q;
            const int vec = elw_vec(ek) == 4 && Q % 4 == 0 ? 4 : 1;
            const int64_t tiles_q = (Q + 32 * vec - 1) / (32 * vec);
            // at least 32 rows per block so that the cross-warp combine and the partial store are amortised
            int64_t chunks = std::max<int64_t>(1, std::min<int64_t>((int64_t(opt_.sm_count) * 16 + tiles_q - 1) / tiles_q, (P + 31) / 32));
            int64_t rows = (P + chunks - 1) / chunks;
            ek.row_chunk = (rows + 7) / 8 * 8;
        }
        KernelSpec::Red red;
        red.ssa = remap[size_t(rk0.outs[0].ssa)];
        red.axis = axis;
        ek.reds.push_back(red);  // from here on elw_vec() also requires q2 % 4 == 0 for 128-bit lanes
        const int vec = elw_vec(ek);
        const int64_t tiles_q = (Q + 32 * vec - 1) / (32 * vec);
        const int64_t chunks_p = (P + ek.row_chunk - 1) / ek.row_chunk;
        const int64_t parts = axis == 0 ? tiles_q : chunks_p;
        const int64_t kept = axis == 0 ? P : Q;
        const int scratch = temp_buffer(kept * parts);
        ek.reds.back().dst.buf = scratch;
        ek.reds.back().dst.subs = {{kept * parts, 1}};

        // second pass: partials -> the reduce's own destination
        KernelSpec k2;
        k2.type = KernelSpec::REDUCE;
        k2.n = kept;
        k2.r = parts;
        Operand in;
        in.buf = scratch;
        if (axis == 0) {
            if (kept > 1) in.xsubs = {{kept, parts}};
            if (parts > 1) in.subs = {{parts, 1}};
        } else {
            if (kept > 1) in.xsubs = {{kept, 1}};
            if (parts > 1) in.subs = {{parts, kept}};
        }
        k2.ins.push_back(in);
        Ssa ld;
        ld.kind = Ssa::LOAD;
        ld.operand = 0;
        k2.ssa.push_back(ld);
        KernelSpec::Out fo;
        fo.ssa = 0;
        fo.dst = final_dst;
        k2.outs.push_back(fo);
        plan_reduce(k2, opt_.sm_count);
        k2.split = 1;
        k2.chunk = k2.r;
        plan_.kernels.push_back(std::move(k2));
        const int k2_index = int(plan_.kernels.size()) - 1;

        // rewrite the step list: [.. reduce group .. moved .. E ..] -> [.. E, (earlier tails), second pass, moved ..]
        std::vector<Step> tail;
        {
            Step s2;
            s2.kind = Step::REDUCE;
            s2.kernel = k2_index;
            tail.push_back(std::move(s2));
        }
        for (size_t m : moved) tail.push_back(std::move(steps[m]));
        std::vector<size_t> drop = moved;
        for (size_t q = r; q <= r_end; q++) drop.push_back(q);
        std::sort(drop.begin(), drop.end());
        std::vector<Step> out;
        out.reserve(steps.size() + 1);
        size_t new_e = 0;
        for (size_t q = 0; q < steps.size(); q++) {
            if (std::binary_search(drop.begin(), drop.end(), q)) continue;
            if (q == e) new_e = out.size();
            out.push_back(std::move(steps[q]));
        }
        size_t ins_at = new_e + 1;
        int next_pos = e_pos + 1;
        while (ins_at < out.size() && out[ins_at].pos < e_pos + POS_SCALE) { next_pos = out[ins_at].pos + 1; ins_at++; }
        for (auto& t : tail) {
            t.pos = next_pos++;
            std::vector<int> trd, twr;
            step_rw(t, trd, twr);
            for (int b : trd) touch(b, t.pos);
            for (int b : twr) touch(b, t.pos);
        }
        touch(scratch, e_pos);
        out.insert(out.begin() + long(ins_at), std::make_move_iterator(tail.begin()), std::make_move_iterator(tail.end()));
        steps = std::move(out);
        for (size_t q = 0; q < dead_kernels.size(); q++) plan_.kernels[size_t(dead_kernels[q])].dead = true;
        if (old_scratch >= 0) { plan_.bufs[size_t(old_scratch)].first = INT_MAX; plan_.bufs[size_t(old_scratch)].last = -1; }
        e = new_e;
        return true;
    }

    // ------------------------------------------------------------------ element-wise work folded into dot products
    // The reference fuses a dot product with the element-wise kernels that follow it (`DPElwExpr`,
    // src/kernel/fusion/dp_elw.rs:13-150) and then drops buffers that only live inside the fused region
    // (src/kernel/alloc/alloc_temp_opt.rs:37-122).  Here: an output of an element-wise kernel that is a chain
    // v = product; v = op(v, constant | bias[column] | v itself) moves into the dot product's epilogue, where the
    // accumulator is still in registers.  Three shapes come out of it (Step::Gemm):
    //   out = chain(product)                       Linear + bias + activation: the activation never re-reads the product
    //   t = c1 * c2 * product                      the scaled gradient that an all-reduce wants: no scale pass
    //   W = W + c1 * c2 * product                  the SGD update: the gradient never exists in memory
    // A kernel whose outputs all moved away disappears; otherwise it is pruned to what is left.
    bool all_readers(const StepBlock& blk, int buf, const Step* except, int& n) const {
        std::vector<int> rd, wr;
        for (auto& st : blk.steps) {
            if (&st != except) {
                step_rw(st, rd, wr);
                for (int b : rd) n += b == buf;
                if ((st.kind == Step::WHILE && st.cond_buf == buf)) n++;
                for (auto& br : st.branches) n += br.cond_buf == buf;
            }
            if (st.body) all_readers(*st.body, buf, except, n);
            for (auto& br : st.branches) all_readers(*br.body, buf, except, n);
            if (st.else_body) all_readers(*st.else_body, buf, except, n);
        }
        return n > 0;
    }
    bool buffer_escapes(int buf) const {
        if (plan_.bufs[size_t(buf)].persistent || plan_.bufs[size_t(buf)].external) return true;
        for (auto& r : plan_.results) if (r.buf == buf) return true;
        return false;
    }

    // drops SSA values and operands that no output, side sum or phase of `k` uses any more
    static void prune_kernel(KernelSpec& k) {
        std::vector<char> live(k.ssa.size(), 0);
        std::vector<int> st;
        for (auto& o : k.outs) st.push_back(o.ssa);
        for (auto& r : k.reds) st.push_back(r.ssa);
        for (auto& ph : k.phases) st.push_back(ph.ssa);
        while (!st.empty()) {
            int i = st.back();
            st.pop_back();
            if (i < 0 || live[size_t(i)]) continue;
            live[size_t(i)] = 1;
            if (k.ssa[size_t(i)].kind == Ssa::OP) { st.push_back(k.ssa[size_t(i)].a); st.push_back(k.ssa[size_t(i)].b); }
        }
        std::vector<int> in_map(k.ins.size(), -1), ssa_map(k.ssa.size(), -1);
        std::vector<Operand> ins;
        std::vector<Ssa> ssa;
        for (size_t i = 0; i < k.ssa.size(); i++) {
            if (!live[i]) continue;
            Ssa v = k.ssa[i];
            if (v.kind == Ssa::LOAD) {
                if (in_map[size_t(v.operand)] < 0) { ins.push_back(k.ins[size_t(v.operand)]); in_map[size_t(v.operand)] = int(ins.size()) - 1; }
                v.operand = in_map[size_t(v.operand)];
            } else if (v.kind == Ssa::OP) {
                v.a = ssa_map[size_t(v.a)];
                if (v.b >= 0) v.b = ssa_map[size_t(v.b)];
            }
            ssa.push_back(v);
            ssa_map[i] = int(ssa.size()) - 1;
        }
        for (auto& o : k.outs) o.ssa = ssa_map[size_t(o.ssa)];
        for (auto& r : k.reds) r.ssa = ssa_map[size_t(r.ssa)];
        for (auto& ph : k.phases) ph.ssa = ssa_map[size_t(ph.ssa)];
        k.ins.swap(ins);
        k.ssa.swap(ssa);
    }

    struct EpiChain {
        std::vector<Step::Gemm::EpiOp> ops;
        int colvec = -1;
        int64_t colvec_off = 0;
        bool acc_mat = false;      // the chain ends with "+ destination" (in-place accumulate)
        bool ok = false;
    };

    // the value `idx` of kernel `k` as a chain over the load of `cb` (identity access over M*N elements)
    bool chain_of(const KernelSpec& k, int idx, int cb, int64_t M, int64_t N, const Operand& dst, EpiChain& out, int depth = 0) const {
        if (depth > 64) return false;
        const Ssa& v = k.ssa[size_t(idx)];
        auto is_product = [&](int i) {
            const Ssa& x = k.ssa[size_t(i)];
            if (x.kind != Ssa::LOAD) return false;
            const Operand& o = k.ins[size_t(x.operand)];
            std::vector<Sub> want;
            if (M * N > 1) want.push_back({M * N, 1});
            std::vector<Sub> have = o.subs;
            canon_subs(have);
            return o.buf == cb && o.offset == 0 && have == want;
        };
        if (v.kind == Ssa::LOAD) return is_product(idx);
        if (v.kind != Ssa::OP) return false;
        Step::Gemm::EpiOp op;
        op.op = v.op;
        if (!eop_is_binary(v.op)) {
            if (!chain_of(k, v.a, cb, M, N, dst, out, depth + 1)) return false;
            op.operand = 0;
            out.ops.push_back(op);
            return true;
        }
        if (v.a == v.b) {   // x op x
            if (!chain_of(k, v.a, cb, M, N, dst, out, depth + 1)) return false;
            if (v.op == E_ADD) {   // x + x is 2 x, exactly
                op.op = E_MUL;
                op.operand = 1;
                op.c = 2.0f;
                out.ops.push_back(op);
                return true;
            }
            Step::Gemm::EpiOp save;
            save.operand = 4;
            out.ops.push_back(save);
            op.operand = 3;
            out.ops.push_back(op);
            return true;
        }
        // which side carries the product?
        auto side_operand = [&](int i, Step::Gemm::EpiOp& o2, bool& is_acc, EpiChain& out) {
            const Ssa& x = k.ssa[size_t(i)];
            is_acc = false;
            if (x.kind == Ssa::CONST) { o2.operand = 1; o2.c = x.c; return true; }
            if (x.kind != Ssa::LOAD) return false;
            const Operand& o = k.ins[size_t(x.operand)];
            std::vector<Sub> have = o.subs;
            canon_subs(have);
            std::vector<Sub> colv;
            if (M > 1) colv.push_back({M, 0});
            if (N > 1) colv.push_back({N, 1});
            canon_subs(colv);
            if (o.buf != cb && have == colv && N > 1) {
                if (out.colvec >= 0 && (out.colvec != o.buf || out.colvec_off != o.offset)) return false;
                out.colvec = o.buf;
                out.colvec_off = o.offset;
                o2.operand = 2;
                return true;
            }
            std::vector<Sub> full;
            if (M * N > 1) full.push_back({M * N, 1});
            std::vector<Sub> dsubs = dst.subs;
            canon_subs(dsubs);
            if (o.buf == dst.buf && o.offset == dst.offset && have == full && dsubs == full) { is_acc = true; return true; }
            return false;
        };
        for (int t = 0; t < 2; t++) {
            const int chain_side = t == 0 ? v.a : v.b, other = t == 0 ? v.b : v.a;
            EpiChain trial = out;
            bool is_acc = false;
            Step::Gemm::EpiOp o2 = op;
            if (!side_operand(other, o2, is_acc, trial)) continue;
            if (!chain_of(k, chain_side, cb, M, N, dst, trial, depth + 1)) continue;
            if (is_acc) {
                if (v.op != E_ADD || depth != 0 || trial.acc_mat) continue;   // only "destination + chain" at the very end
                trial.acc_mat = true;
            } else
                trial.ops.push_back(o2);
            out = trial;
            return true;
        }
        return false;
    }

    void fuse_dot_epilogues(StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (s.body) fuse_dot_epilogues(*s.body);
            for (auto& br : s.branches) fuse_dot_epilogues(*br.body);
            if (s.else_body) fuse_dot_epilogues(*s.else_body);
        }
        auto& steps = blk.steps;
        std::vector<int> rd, wr;
        for (size_t gi = 0; gi < steps.size(); gi++) {
            if (steps[gi].kind != Step::GEMM || steps[gi].gemm.epi != Step::Gemm::EPI_NONE || steps[gi].gemm.c_off != 0 || steps[gi].gemm.batch != 1) continue;
            const int cb = steps[gi].gemm.c;
            const int64_t M = steps[gi].gemm.M, N = steps[gi].gemm.N;
            if (M * N <= 0) continue;
            // the first step behind the product that reads it
            size_t ei = 0;
            bool found = false;
            for (size_t j = gi + 1; j < steps.size() && j - gi <= 64; j++) {
                if (is_barrier(steps[j])) break;
                step_rw(steps[j], rd, wr);
                const bool reads = std::find(rd.begin(), rd.end(), cb) != rd.end();
                const bool writes = std::find(wr.begin(), wr.end(), cb) != wr.end();
                if (reads) { found = !writes; ei = j; break; }
                if (writes) break;
            }
            if (!found || steps[ei].kind != Step::ELW) continue;
            KernelSpec& k = plan_.kernels[size_t(steps[ei].kernel)];
            if (k.type != KernelSpec::ELW || !k.reds.empty() || k.n != M * N) continue;
            // one output at a time (several parameters of equal size share one update kernel)
            for (size_t oi = 0; oi < k.outs.size(); oi++) {
                const KernelSpec::Out o = k.outs[oi];
                std::vector<Sub> dsubs = o.dst.subs, full;
                canon_subs(dsubs);
                if (M * N > 1) full.push_back({M * N, 1});
                if (dsubs != full) continue;
                EpiChain ch;
                if (!chain_of(k, o.ssa, cb, M, N, o.dst, ch)) continue;
                if (ch.ops.empty() && !ch.acc_mat) continue;
                if (ch.ops.size() > 12) continue;
                bool scale_only = true;
                for (auto& op : ch.ops) scale_only = scale_only && op.op == E_MUL && op.operand == 1;
                if (ch.acc_mat && !scale_only) continue;
                // `W += s * product` inside the product would add every k chunk's partial sum to W on its own: each add
                // rounds at the precision of W, and an update of a hundred ulps of W spread over 64 chunks comes out
                // percents off (measured on the first layer of the benchmark network at batch 65536).  With more than
                // one chunk the gradient is finished first and added once, by the element-wise kernel, as written.
                if (ch.acc_mat && steps[gi].gemm.K > DOT_CHUNK_K) continue;
                // who else reads the plain product?
                int other_readers = 0;
                all_readers(plan_.main, cb, nullptr, other_readers);
                // (this kernel counts once however many of its outputs read it: look at its other outputs)
                bool k_still_reads = false;
                for (size_t q = 0; q < k.outs.size(); q++) {
                    if (q == oi) continue;
                    EpiChain dummy;
                    std::vector<int> stq{k.outs[q].ssa};
                    std::vector<char> seen(k.ssa.size(), 0);
                    while (!stq.empty()) {
                        int i = stq.back();
                        stq.pop_back();
                        if (i < 0 || seen[size_t(i)]) continue;
                        seen[size_t(i)] = 1;
                        const Ssa& x = k.ssa[size_t(i)];
                        if (x.kind == Ssa::LOAD && k.ins[size_t(x.operand)].buf == cb) k_still_reads = true;
                        if (x.kind == Ssa::OP) { stq.push_back(x.a); stq.push_back(x.b); }
                    }
                }
                const bool raw_needed = buffer_escapes(cb) || other_readers > 1 || k_still_reads;
                if (scale_only && raw_needed) continue;   // the scaled product replaces the plain one: nobody may want the latter
                // few tiles and a long k loop: the dot kernels would split k over the SMs, which a chain on the finished
                // sum rules out (one owner per tile) -- the split is worth more than the saved pass
                if (!scale_only && ((M + 255) / 256) * ((N + 255) / 256) * 4 <= opt_.sm_count && steps[gi].gemm.K >= 2048) continue;
                // the output's value appears at the product's position instead of the kernel's: nothing in between may
                // look at the destination, overwrite the bias, or -- when the kernel itself goes away -- mind the move
                bool hoist_ok = true;
                for (size_t j = gi + 1; j < ei && hoist_ok; j++) {
                    step_rw(steps[j], rd, wr);
                    for (int b : rd) if (b == o.dst.buf) hoist_ok = false;
                    for (int b : wr) if (b == o.dst.buf || b == ch.colvec) hoist_ok = false;
                }
                // the kernel's other inputs are not needed by the epilogue, and the destination must not be one of the
                // product's own operands
                if (o.dst.buf == steps[gi].gemm.a || o.dst.buf == steps[gi].gemm.b) hoist_ok = false;
                if (!hoist_ok) continue;

                Step::Gemm& g = steps[gi].gemm;
                g.ops = ch.ops;
                g.colvec = ch.colvec;
                g.colvec_off = ch.colvec_off;
                if (scale_only) {
                    g.epi = Step::Gemm::EPI_SCALE;
                    g.accumulate = ch.acc_mat;
                    g.c = o.dst.buf;
                    g.c_off = o.dst.offset;
                    touch(g.c, steps[gi].pos);
                    plan_.bufs[size_t(cb)].first = INT_MAX;
                    plan_.bufs[size_t(cb)].last = -1;
                } else {
                    g.epi = Step::Gemm::EPI_CHAIN;
                    g.store_raw = raw_needed;
                    g.out = o.dst.buf;
                    g.out_off = o.dst.offset;
                    touch(g.out, steps[gi].pos);
                    if (g.colvec >= 0) touch(g.colvec, steps[gi].pos);
                    if (!raw_needed) {
                        // partial sums accumulate in the destination itself; the last chunk overwrites them with the chain
                        g.c = g.out;
                        g.c_off = g.out_off;
                        plan_.bufs[size_t(cb)].first = INT_MAX;
                        plan_.bufs[size_t(cb)].last = -1;
                    }
                }
                k.outs.erase(k.outs.begin() + long(oi));
                break;   // one epilogue per product
            }
            if (steps[gi].gemm.epi == Step::Gemm::EPI_NONE) continue;
            if (k.outs.empty()) {
                k.dead = true;
                steps.erase(steps.begin() + long(ei));
            } else
                prune_kernel(k);
        }
    }

    // ------------------------------------------------------------------ outputs nobody reads
    // A value can be written to a temporary because one consumer needed it in memory and then lose that consumer to a
    // later pass (or never have had one: the zero padding that Index backward concatenates and a slice cuts away
    // again).  An element-wise output into a temporary that no step of the whole plan reads is dropped; a kernel that
    // is left without outputs goes with it.
    void collect_reads(const StepBlock& blk, std::vector<char>& read) const {
        std::vector<int> rd, wr;
        for (auto& st : blk.steps) {
            step_rw(st, rd, wr);
            for (int b : rd) read[size_t(b)] = 1;
            if (st.kind == Step::WHILE) read[size_t(st.cond_buf)] = 1;
            for (auto& br : st.branches) read[size_t(br.cond_buf)] = 1;
            if (st.body) collect_reads(*st.body, read);
            for (auto& br : st.branches) collect_reads(*br.body, read);
            if (st.else_body) collect_reads(*st.else_body, read);
        }
    }
    bool drop_in_block(StepBlock& blk, const std::vector<char>& read) {
        bool changed = false;
        for (auto& st : blk.steps) {
            if (st.body) changed |= drop_in_block(*st.body, read);
            for (auto& br : st.branches) changed |= drop_in_block(*br.body, read);
            if (st.else_body) changed |= drop_in_block(*st.else_body, read);
        }
        for (size_t i = 0; i < blk.steps.size();) {
            Step& st = blk.steps[i];
            if (st.kind != Step::ELW) { i++; continue; }
            KernelSpec& k = plan_.kernels[size_t(st.kernel)];
            if (k.type != KernelSpec::ELW || !k.reds.empty()) { i++; continue; }
            const size_t before = k.outs.size();
            for (size_t o = 0; o < k.outs.size();) {
                const int b = k.outs[o].dst.buf;
                // (two outputs may share a buffer: the other halves of a concatenation keep it alive through `read`)
                bool result = plan_.bufs[size_t(b)].external;
                for (auto& r : plan_.results) result = result || r.buf == b;
                // (a buffer that lives for the whole program but is neither read by any step nor handed back is as dead
                //  as a temporary: ids that views of kept tensors refer to get such buffers)
                if (!read[size_t(b)] && !result) k.outs.erase(k.outs.begin() + long(o));
                else o++;
            }
            if (k.outs.size() == before) { i++; continue; }
            changed = true;
            if (k.outs.empty()) {
                k.dead = true;
                blk.steps.erase(blk.steps.begin() + long(i));
            } else {
                prune_kernel(k);
                i++;
            }
        }
        return changed;
    }
    void drop_unread_outputs() {
        for (int round = 0; round < 8; round++) {
            std::vector<char> read(plan_.bufs.size(), 0);
            collect_reads(plan_.main, read);
            if (!drop_in_block(plan_.main, read)) break;
        }
    }

    // ------------------------------------------------------------------ neighbouring collectives as one
    // Data-parallel training all-reduces every gradient: four weight matrices and four bias vectors per step in the
    // benchmark network, each collective paying its own latency and none of them long enough to reach the link's peak.
    // An all-reduce of a temporary is held back until a step needs the buffer (or a block ends); the collectives held
    // back together become one ALLREDUCE over buffers that the arena places side by side.  Kept tensors and buffers
    // of the caller stay as they are.  (With collectives on their own stream the pass is off: there each collective
    // should start as early as it can.)
    bool bucketable(const Step& s) const {
        if (s.kind != Step::ALLREDUCE || !s.more_bufs.empty() || s.off != 0) return false;
        const BufferInfo& b = plan_.bufs[size_t(s.buf)];
        if (b.external || s.nelem != b.numel || b.numel <= 0) return false;
        for (auto& r : plan_.results)
            if (r.buf == s.buf) return false;
        for (auto& pk : plan_.packs)
            for (int x : pk)
                if (x == s.buf) return false;
        return true;
    }
    void bucket_collectives(StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (s.body) bucket_collectives(*s.body);
            for (auto& br : s.branches) bucket_collectives(*br.body);
            if (s.else_body) bucket_collectives(*s.else_body);
        }
        std::vector<Step> out;
        std::vector<Step> held;            // collectives waiting for the first step that needs one of their buffers
        std::vector<int> rd, wr;
        auto flush = [&](int pos_before) {
            if (held.empty()) return;
            if (held.size() == 1) {
                held[0].pos = std::max(held[0].pos, pos_before);
                touch(held[0].buf, held[0].pos);
                out.push_back(std::move(held[0]));
                held.clear();
                return;
            }
            Step m = std::move(held[0]);
            std::vector<int> pack = {m.buf};
            int64_t span = ((plan_.bufs[size_t(m.buf)].numel * 4 + 255) / 256) * 256;
            for (size_t i = 1; i < held.size(); i++) {
                m.more_bufs.push_back(held[i].buf);
                pack.push_back(held[i].buf);
                const int64_t bytes = plan_.bufs[size_t(held[i].buf)].numel * 4;
                span += i + 1 < held.size() ? ((bytes + 255) / 256) * 256 : bytes;
                m.pos = std::max(m.pos, held[i].pos);
            }
            m.pos = std::max(m.pos, pos_before);
            m.nelem = span / 4;
            for (int b : pack) touch(b, m.pos);
            plan_.packs.push_back(std::move(pack));
            out.push_back(std::move(m));
            held.clear();
        };
        for (auto& s : blk.steps) {
            if (bucketable(s)) {
                bool dup = false;
                for (auto& h : held) dup = dup || h.buf == s.buf;
                if (!dup) { held.push_back(std::move(s)); continue; }
            }
            if (!held.empty()) {
                bool needed = is_barrier(s);
                if (!needed) {
                    step_rw(s, rd, wr);
                    for (auto& h : held)
                        for (int b : {h.buf})
                            needed = needed || std::find(rd.begin(), rd.end(), b) != rd.end() || std::find(wr.begin(), wr.end(), b) != wr.end();
                }
                // the merged collective takes the position of the last one held back; it must still lie in front of `s`
                if (needed) flush(out.empty() ? INT_MIN : last_pos(out.back()) + 1);
            }
            out.push_back(std::move(s));
        }
        flush(out.empty() ? INT_MIN : last_pos(out.back()) + 1);
        blk.steps = std::move(out);
    }

    // ------------------------------------------------------------------ independent kernels in one launch
    // A step list often holds runs of small kernels that do not depend on one another (the bias updates of an
    // optimiser step, the pieces of a concat, a gradient that is a constant fill next to the sums that feed the
    // next layer).  Launched one after another each pays a launch and leaves most SMs idle; here they become one
    // GROUP kernel whose grid is the concatenation of the members' grids.  A member may be picked from further down
    // the step list when nothing it would jump over (or join) writes what it reads or touches what it writes.  Only
    // small kernels are grouped: a large one would hold back everything that waits for the group, and the executor
    // already lets independent kernels of a captured graph run side by side.  The reference's fusion passes merge
    // kernels only along producer -> consumer edges (src/kernel/fusion/elw.rs, reduce_elw.rs); it has no counterpart.
    static constexpr int64_t TINY_DOT_K = 8, TINY_DOT_WORK = 256;
    static constexpr int64_t GROUP_BIG = int64_t(1) << 22;
    static constexpr size_t GROUP_MAX = 8, GROUP_LOOKAHEAD = 24, GROUP_ARG_WORDS = 384;
    static int64_t kernel_work(const KernelSpec& k) {
        if (k.type == KernelSpec::REDUCE) return k.n * std::max<int64_t>(1, k.r);
        if (k.type == KernelSpec::ROWS) return k.p2 * k.q2;
        return k.n;
    }
    void count_kernel_uses(const StepBlock& blk, std::vector<int>& uses) const {
        for (auto& s : blk.steps) {
            if ((s.kind == Step::ELW || s.kind == Step::REDUCE) && s.kernel >= 0) uses[size_t(s.kernel)]++;
            if (s.body) count_kernel_uses(*s.body, uses);
            for (auto& br : s.branches) count_kernel_uses(*br.body, uses);
            if (s.else_body) count_kernel_uses(*s.else_body, uses);
        }
    }
    bool groupable(const std::vector<Step>& steps, size_t i, const std::vector<int>& uses) const {
        const Step& s = steps[i];
        if (s.kind != Step::ELW && s.kind != Step::REDUCE) return false;
        if (size_t(s.kernel) >= uses.size() || uses[size_t(s.kernel)] != 1) return false;
        const KernelSpec& k = plan_.kernels[size_t(s.kernel)];
        if (k.dead || k.type == KernelSpec::GROUP || kernel_work(k) > GROUP_BIG) return false;
        if (k.type == KernelSpec::ELW && (!k.reds.empty() || elw_uses_tile(k))) return false;   // 2-d grids, 16 KB of shared memory
        if (k.type == KernelSpec::REDUCE && (k.split != 1 || k.scratch >= 0)) return false;
        // the kernel that scales the operand of a collective stays next to it (the runtime moves the pair to the
        // communication stream)
        if (opt_.world > 1 && i + 1 < steps.size() && steps[i + 1].kind == Step::ALLREDUCE) return false;
        return true;
    }
    void group_kernels(StepBlock& blk, const std::vector<int>& uses) {
        for (auto& s : blk.steps) {
            if (s.body) group_kernels(*s.body, uses);
            for (auto& br : s.branches) group_kernels(*br.body, uses);
            if (s.else_body) group_kernels(*s.else_body, uses);
        }
        auto& steps = blk.steps;
        std::vector<int> rd, wr, seen_rd, seen_wr;
        for (size_t i = 0; i < steps.size(); i++) {
            if (!groupable(steps, i, uses)) continue;
            std::vector<size_t> members = {i};
            step_rw(steps[i], seen_rd, seen_wr);
            // the members' argument blocks travel in one kernel parameter block: keep it well under 4 KB
            auto arg_words = [&](const Step& st) {
                const KernelSpec& k = plan_.kernels[size_t(st.kernel)];
                return k.ins.size() + k.outs.size() + k.phases.size() + 2;
            };
            size_t words = arg_words(steps[i]);
            if (words > GROUP_ARG_WORDS) continue;
            for (size_t j = i + 1; j < steps.size() && j <= i + GROUP_LOOKAHEAD && members.size() < GROUP_MAX; j++) {
                if (is_barrier(steps[j])) break;
                step_rw(steps[j], rd, wr);
                bool ok = groupable(steps, j, uses) && !hits(seen_wr, rd) && !hits(seen_wr, wr) && !hits(wr, seen_rd);
                if (ok && words + arg_words(steps[j]) > GROUP_ARG_WORDS) ok = false;
                if (ok) {
                    members.push_back(j);
                    words += arg_words(steps[j]);
                }
                seen_rd.insert(seen_rd.end(), rd.begin(), rd.end());
                seen_wr.insert(seen_wr.end(), wr.begin(), wr.end());
            }
            if (members.size() < 2) continue;
            KernelSpec g;
            g.type = KernelSpec::GROUP;
            const int head_pos = steps[i].pos;
            for (size_t m : members) {
                const int ki = steps[m].kernel;
                g.members.push_back(ki);
                g.n += kernel_work(plan_.kernels[size_t(ki)]);
                plan_.kernels[size_t(ki)].grouped = true;
                step_rw(steps[m], rd, wr);
                for (int x : rd) touch(x, head_pos);
                for (int x : wr) touch(x, head_pos);
            }
            // small members first: their blocks are scheduled ahead of a large member's
            std::stable_sort(g.members.begin(), g.members.end(), [&](int a, int b) {
                return kernel_work(plan_.kernels[size_t(a)]) < kernel_work(plan_.kernels[size_t(b)]);
            });
            for (size_t q = members.size(); q-- > 1;) steps.erase(steps.begin() + long(members[q]));
            steps[i].kind = Step::ELW;
            steps[i].kernel = int(plan_.kernels.size());
            plan_.kernels.push_back(std::move(g));
        }
    }

    // ------------------------------------------------------------------ arena
    void plan_arena() {
        auto& bufs = plan_.bufs;
        // a buffer touched inside a loop and also outside of it must survive the whole loop
        for (int pass = 0; pass < 3; pass++)
        for (auto& b : bufs) {
            if (b.persistent || b.external || b.last < 0) continue;
            for (auto& sp : loop_spans_) {
                bool inside = b.first >= sp.first && b.last < sp.second;
                bool overlaps = b.last >= sp.first && b.first < sp.second;
                if (overlaps && !inside) {
                    b.first = std::min(b.first, sp.first);
                    b.last = std::max(b.last, sp.second);
                }
            }
        }
        std::vector<int> order;
        for (size_t i = 0; i < bufs.size(); i++)
            if (!bufs[i].external && (bufs[i].last >= 0 || bufs[i].persistent) && bufs[i].numel > 0) order.push_back(int(i));
        std::sort(order.begin(), order.end(), [&](int x, int y) {
            if (bufs[x].numel != bufs[y].numel) return bufs[x].numel > bufs[y].numel;
            return x < y;
        });
        struct Placed { int64_t off, size; int first, last; };
        std::vector<Placed> placed;
        int64_t top = 0;
        // Kept tensors first, side by side, when they are small: the host then reads all of them back with one copy
        // (a program like the README's MLP step keeps eight tensors of a few floats each; eight copies of a few bytes
        // cost more than the kernels that made them).
        std::vector<char> is_result(bufs.size(), 0);
        {
            int64_t total = 0;
            std::vector<int> res;
            for (auto& r : plan_.results)
                if (r.buf >= 0 && !bufs[size_t(r.buf)].external && !is_result[size_t(r.buf)]) {
                    is_result[size_t(r.buf)] = 1;
                    res.push_back(r.buf);
                    total += ((bufs[size_t(r.buf)].numel * 4 + 255) / 256) * 256;
                }
            if (!res.empty() && total <= (int64_t(1) << 20)) {
                for (int i : res) {
                    auto& b = bufs[size_t(i)];
                    const int64_t size = ((b.numel * 4 + 255) / 256) * 256;
                    b.arena_off = top;
                    placed.push_back({top, size, INT_MIN, INT_MAX});
                    top += size;
                }
                plan_.results_bytes = top;
            } else
                std::fill(is_result.begin(), is_result.end(), 0);
        }
        auto lowest_fit = [&](int64_t size, int first, int last) {
            std::vector<std::pair<int64_t, int64_t>> busy;
            for (auto& p : placed)
                if (!(p.last < first || last < p.first)) busy.push_back({p.off, p.off + p.size});
            std::sort(busy.begin(), busy.end());
            int64_t off = 0;
            for (auto& iv : busy) {
                if (off + size <= iv.first) break;
                off = std::max(off, iv.second);
            }
            return off;
        };
        // buffers that one collective covers: one block, members in order, alive for as long as any member is
        std::vector<char> packed(bufs.size(), 0);
        for (auto& pk : plan_.packs) {
            int64_t size = 0;
            int first = INT_MAX, last = INT_MIN;
            for (int i : pk) {
                size += ((bufs[size_t(i)].numel * 4 + 255) / 256) * 256;
                first = std::min(first, bufs[size_t(i)].persistent ? INT_MIN : bufs[size_t(i)].first);
                last = std::max(last, bufs[size_t(i)].persistent ? INT_MAX : bufs[size_t(i)].last);
            }
            int64_t off = lowest_fit(size, first, last);
            placed.push_back({off, size, first, last});
            top = std::max(top, off + size);
            for (int i : pk) {
                bufs[size_t(i)].arena_off = off;
                off += ((bufs[size_t(i)].numel * 4 + 255) / 256) * 256;
                packed[size_t(i)] = 1;
            }
        }
        for (int i : order) {
            if (is_result[size_t(i)] || packed[size_t(i)]) continue;
            auto& b = bufs[i];
            int first = b.persistent ? INT_MIN : b.first;
            int last = b.persistent ? INT_MAX : b.last;
            int64_t size = ((b.numel * 4 + 255) / 256) * 256;
            std::vector<std::pair<int64_t, int64_t>> busy;
            for (auto& p : placed)
                if (!(p.last < first || last < p.first)) busy.push_back({p.off, p.off + p.size});
            std::sort(busy.begin(), busy.end());
            int64_t off = 0;
            for (auto& iv : busy) {
                if (off + size <= iv.first) break;
                off = std::max(off, iv.second);
            }
            b.arena_off = off;
            placed.push_back({off, size, first, last});
            top = std::max(top, off + size);
        }
        plan_.arena_bytes = top;
    }
};

}  // namespace

void lower_program(Program& prog, Plan& plan, const LowerOptions& opt) {
    Lowerer l(prog, plan, opt);
    l.run();
}

// ---------------------------------------------------------------------- listing
static const char* eop_name(EOp o) {
    switch (o) {
    case E_ADD: return "+";
    case E_MUL: return "*";
    case E_EXP2: return "exp2";
    case E_LOG2: return "log2";
    case E_SIN: return "sin";
    case E_RECIP: return "recip";
    case E_SQRT: return "sqrt_abs";
    case E_EQZ: return "eqz";
    case E_GTZ: return "gtz";
    case E_LTZ: return "ltz";
    }
    return "?";
}

static std::string subs_str(const std::vector<Sub>& s) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < s.size(); i++) o << (i ? " " : "") << s[i].size << "x" << s[i].stride;
    o << "]";
    return o.str();
}

static void dump_kernel(const Plan& p, const KernelSpec& k, const std::string& label, const std::string& pad, bool src,
                        std::ostringstream& o) {
    const bool is_reduce = k.type == KernelSpec::REDUCE;
    int nops = 0;
    for (auto& x : k.ssa) nops += x.kind == Ssa::OP;
    if (k.type == KernelSpec::ROWS) o << pad << label << " rows [" << k.p2 << "," << k.q2 << "] phases=" << k.phases.size();
    else if (!is_reduce) o << pad << label << " elw n=" << k.n;
    else o << pad << label << (k.red_op ? " reduce(max) rows=" : " reduce rows=") << k.n << " len=" << k.r << " mode=" << (k.mode ? "col" : "row") << " split=" << k.split;
    o << " ops=" << nops << " vec=" << k.vec << " ins=" << k.ins.size() << " outs=" << k.outs.size() << " " << k.entry << "\n";
    for (auto& in : k.ins)
        o << pad << "    in  " << p.bufs[in.buf].name << "+" << in.offset << " " << (is_reduce ? subs_str(in.xsubs) + "," : "") << subs_str(in.subs) << "\n";
    for (auto& out : k.outs)
        o << pad << "    out " << p.bufs[out.dst.buf].name << "+" << out.dst.offset << " " << (is_reduce ? subs_str(out.dst.xsubs) : subs_str(out.dst.subs)) << "\n";
    for (auto& ph : k.phases)
        o << pad << "    " << (ph.red_op ? "max" : "sum") << " v" << ph.ssa << " along each row -> " << p.bufs[ph.dst.buf].name << "+"
          << ph.dst.offset << "\n";
    for (auto& rd : k.reds)
        o << pad << "    sum v" << rd.ssa << " over " << (rd.axis == 0 ? "columns" : "rows") << " of [" << k.p2 << "," << k.q2
          << "] -> " << p.bufs[rd.dst.buf].name << " " << subs_str(rd.dst.subs) << " (rows per block " << k.row_chunk << ")\n";
    if (src) {
        for (size_t i = 0; i < k.ssa.size(); i++) {
            auto& x = k.ssa[i];
            o << pad << "      v" << i << " = ";
            if (x.kind == Ssa::LOAD) o << "load in" << x.operand;
            else if (x.kind == Ssa::RED) o << "row result " << x.operand;
            else if (x.kind == Ssa::CONST) o << x.c;
            else if (x.b >= 0) o << "v" << x.a << " " << eop_name(x.op) << " v" << x.b;
            else o << eop_name(x.op) << "(v" << x.a << ")";
            o << "\n";
        }
    }
}

static void dump_block(const Plan& p, const StepBlock& b, int ind, bool src, std::ostringstream& o) {
    std::string pad(size_t(ind) * 2, ' ');
    for (auto& s : b.steps) {
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE: {
            auto& k = p.kernels[s.kernel];
            const std::string label = "#" + std::to_string(s.pos);
            if (k.type == KernelSpec::GROUP) {
                o << pad << label << " group of " << k.members.size() << " kernels in one launch " << k.entry << "\n";
                for (int m : k.members) dump_kernel(p, p.kernels[size_t(m)], "  -", pad + "  ", src, o);
            } else {
                dump_kernel(p, k, label, pad, src, o);
            }
            break;
        }
        case Step::GEMM:
            o << pad << "#" << s.pos << (s.gemm.batch > 1 ? " gemm x" + std::to_string(s.gemm.batch) + " " : " gemm ") << p.bufs[s.gemm.c].name << "[" << s.gemm.M << "," << s.gemm.N << "] = "
              << p.bufs[s.gemm.a].name << "+" << s.gemm.a_off << "(" << s.gemm.a_rs << "," << s.gemm.a_cs << ") . "
              << p.bufs[s.gemm.b].name << "+" << s.gemm.b_off << "(" << s.gemm.b_rs << "," << s.gemm.b_cs << ") K=" << s.gemm.K << "\n";
            if (s.gemm.epi != Step::Gemm::EPI_NONE) {
                o << pad << "    epilogue: ";
                if (s.gemm.epi == Step::Gemm::EPI_SCALE) o << p.bufs[s.gemm.c].name << (s.gemm.accumulate ? " += " : " = ") << "product";
                else o << p.bufs[s.gemm.out].name << "+" << s.gemm.out_off << " = product";
                for (auto& op : s.gemm.ops) {
                    if (op.operand == 4) { o << " ; save"; continue; }
                    o << " ; " << eop_name(op.op);
                    if (op.operand == 1) o << " " << op.c;
                    else if (op.operand == 2) o << " " << p.bufs[s.gemm.colvec].name << "[col]";
                    else if (op.operand == 3) o << " saved";
                }
                if (s.gemm.epi == Step::Gemm::EPI_CHAIN) o << (s.gemm.store_raw ? "  (plain product kept in " + p.bufs[s.gemm.c].name + ")" : "  (plain product not kept)");
                o << "\n";
            }
            break;
        case Step::UPLOAD:
            o << pad << "#" << s.pos << " upload " << p.bufs[s.buf].name << " n=" << s.nelem << "\n";
            break;
        case Step::ALLREDUCE:
            o << pad << "#" << s.pos << " allreduce " << p.bufs[s.buf].name;
            for (int b : s.more_bufs) o << " + " << p.bufs[size_t(b)].name;
            o << " n=" << s.nelem << "\n";
            break;
        case Step::WHILE:
            o << pad << "#" << s.pos << " while (" << p.bufs[s.cond_buf].name << "+" << s.cond_off << " != 0) {\n";
            dump_block(p, *s.body, ind + 1, src, o);
            o << pad << "}\n";
            break;
        case Step::IF:
            for (size_t k = 0; k < s.branches.size(); k++) {
                o << pad << "#" << s.pos << (k ? " else if (" : " if (") << p.bufs[s.branches[k].cond_buf].name << "+" << s.branches[k].cond_off << " == 1) {\n";
                dump_block(p, *s.branches[k].body, ind + 1, src, o);
                o << pad << "}\n";
            }
            if (s.else_body) {
                o << pad << "else {\n";
                dump_block(p, *s.else_body, ind + 1, src, o);
                o << pad << "}\n";
            }
            break;
        case Step::EXIT: o << pad << "#" << s.pos << " exit\n"; break;
        }
    }
}

std::string dump_plan(const Plan& plan, bool with_source) {
    std::ostringstream o;
    size_t live = 0;
    for (auto& k : plan.kernels) live += !k.dead && !k.grouped;
    o << "plan: " << plan.ir_commands << " IR commands -> " << plan.n_steps << " steps, " << live
      << " kernels, arena " << plan.arena_bytes << " B, " << plan.bufs.size() << " buffers\n";
    dump_block(plan, plan.main, 0, with_source, o);
    o << "results:";
    for (auto& r : plan.results) o << " " << r.id << (r.buf >= 0 ? "@" + plan.bufs[r.buf].name : "(none)");
    o << "\n";
    if (with_source) {
        std::set<std::string> seen;
        for (auto& k : plan.kernels)
            if (!k.source.empty() && seen.insert(k.entry).second) o << "// ---- " << k.entry << "\n" << k.source << "\n";
    }
    return o.str();
}

}  // namespace adb
