// Data-parallel rewrite of an IR program: one process per GPU, the batch axis split across ranks,
// parameters replicated, gradients summed with an all-reduce before they meet replicated values.
// The reference is single-device and has nothing comparable; this pass works on the same IR commands
// (src/core/ir.rs:8-105) and inserts the extension command AllReduce.
//
// Every id gets a tag while the program is walked in order:
//   REP        the same value on every rank (parameters, scalars)
//   SHARD(d)   the rank holds its 1/world slice of axis d (the batch, wherever views / permutes moved it)
//   PART       per-rank partial sum whose true value is the sum over ranks (a contraction over the batch)
//   CONST      CreateConstant: conforms to anything
// Linear ops keep PART (scaling by a constant, adding two partial sums, Sum); everything else forces an
// AllReduce of the partial operand first.  That puts the collective where the SGD update consumes the
// gradient: `p += -1 * (lr * grad)` all-reduces the scaled gradient right before the in-place add.
//
// Which CreateMat tensors hold the batch is either given (their ids) or guessed from the first dimension.  Constants
// and broadcasts carry no such information: a CreateConstant with a dimension equal to the batch, or a broadcast to
// that many entries, is first assumed to be batch-shaped and the assumption is checked where the value meets a
// tensor whose distribution is known.  When it does not fit (a constant shaped like a parameter whose width happens
// to equal the batch), the decision is recorded and the rewrite starts over with it; the program that is finally
// rewritten in place uses the decisions found that way.
#include "adb_shard.hpp"

#include <algorithm>
#include <functional>
#include <map>
#include <set>

namespace adb {

namespace {

enum Tag : uint8_t { T_UNDEF, T_REP, T_SHARD, T_PART, T_CONST };

struct Info {
    Tag tag = T_UNDEF;
    int axis = 0;
    std::vector<int64_t> dims;   // global shape
    std::vector<int64_t> ldims;  // CONST: the shape the command was given (possibly cut along the batch)
    int origin = -1;             // ordinal of the guessed decision this value's distribution rests on (-1: none)
};

// thrown when a guessed decision turns out wrong: command number `ordinal` must cut `axis` instead (-1: nothing)
struct Decide {
    int ordinal;
    int axis;
};

struct Sharder {
    Program& prog;
    int rank, world;
    int64_t batch;
    std::vector<Info> info;
    std::vector<char> needed, is_dep;
    const std::vector<std::string>* only = nullptr;   // ids of the CreateMat tensors that hold the batch (optional)
    const std::map<int, int>* decided = nullptr;      // command ordinal -> axis to cut (-1: none), found by earlier attempts
    int ordinal_ = 0;                                  // counts the commands that went through step()
    int pending_origin_ = -1;                          // origin the result of the current command inherits

    Sharder(Program& p, int r, int w, int64_t b) : prog(p), rank(r), world(w), batch(b) {
        info.resize(p.ids.size());
        needed.assign(p.ids.size(), 0);
        is_dep.assign(p.ids.size(), 0);
    }

    [[noreturn]] void fail(const std::string& m) { throw IrError("data-parallel rewrite: " + m); }
    const std::string& name(uint32_t id) { return prog.ids[id]; }

    static void reads(const Cmd& c, uint32_t out[2], int& n) {
        n = 0;
        switch (c.op) {
        case OP_MUL: case OP_ADD: case OP_DOT: case OP_BATCH_DOT: case OP_CONCAT: case OP_MUL_EQ: case OP_ADD_EQ: out[n++] = c.a; out[n++] = c.b; break;
        case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_SUM: case OP_MAX: case OP_CONTIG: case OP_EXP2: case OP_LOG2: case OP_SIN:
        case OP_RECIP: case OP_SQRT: case OP_VIEW: case OP_INDEX: case OP_PERMUTE: case OP_BROADCAST: case OP_ALLREDUCE:
            out[n++] = c.a; break;
        default: break;
        }
    }
    static bool has_result(uint8_t op) { return !(op == OP_WHILE || op == OP_IF || op == OP_EX || op == OP_HEADING); }

    // commands whose result cannot reach the dep list or a condition are left alone (no collectives for dead values)
    void mark_needed() {
        for (auto d : prog.dep) { needed[d] = 1; is_dep[d] = 1; }
        std::function<void(Block&)> conds = [&](Block& b) {
            for (auto& c : b.cmds) {
                if (c.op == OP_WHILE) { needed[c.a] = 1; conds(*c.block); }
                else if (c.op == OP_IF) {
                    for (auto& cb : c.conds) { needed[cb.first] = 1; conds(*cb.second); }
                    if (c.else_block) conds(*c.else_block);
                }
            }
        };
        conds(prog.main);
        bool changed = true;
        std::function<void(Block&)> walk = [&](Block& b) {
            for (auto& c : b.cmds) {
                if (c.op == OP_WHILE) walk(*c.block);
                else if (c.op == OP_IF) {
                    for (auto& cb : c.conds) walk(*cb.second);
                    if (c.else_block) walk(*c.else_block);
                } else if (has_result(c.op) && needed[c.res]) {
                    uint32_t r[2];
                    int n;
                    reads(c, r, n);
                    for (int k = 0; k < n; k++)
                        if (!needed[r[k]]) { needed[r[k]] = 1; changed = true; }
                }
            }
        };
        while (changed) { changed = false; walk(prog.main); }
    }

    Cmd make_allreduce(uint32_t id) {
        Cmd c;
        c.op = OP_ALLREDUCE;
        c.a = id;
        c.res = id;
        return c;
    }

    // make sure `id` is a full value before a non-linear use
    void resolve_partial(uint32_t id, std::vector<Cmd>& out) {
        if (info[id].tag == T_PART) {
            out.push_back(make_allreduce(id));
            info[id].tag = T_REP;
            prog.n_cmds++;
        }
    }

    void set(uint32_t id, Tag t, int axis, const std::vector<int64_t>& dims, const Cmd&) {
        Info& i = info[id];
        // an id that is assigned again (loop-carried state, op-assign) must stay sharded / unsharded as it was
        const bool was = i.tag == T_SHARD, now = t == T_SHARD;
        if (i.tag != T_UNDEF && (was != now || (now && i.axis != axis)))
            fail("id '" + name(id) + "' changes its distribution between assignments");
        i.tag = t;
        i.axis = axis;
        i.dims = dims;
        i.ldims.clear();
        i.origin = (t == T_SHARD || t == T_CONST) ? pending_origin_ : -1;
    }

    std::vector<int64_t> local_dims(const Info& i) const {
        if (i.tag == T_CONST) return i.ldims;
        std::vector<int64_t> d = i.dims;
        if (i.tag == T_SHARD && size_t(i.axis) < d.size()) d[size_t(i.axis)] /= world;
        return d;
    }
    // a guessed decision (if there is one behind `i`) is replaced by `axis`; otherwise the program is refused
    [[noreturn]] void redecide(const Info& i, int axis, const std::string& why) {
        if (i.origin >= 0) {
            auto it = decided ? decided->find(i.origin) : std::map<int, int>::const_iterator();
            if (!decided || it == decided->end() || it->second != axis) throw Decide{i.origin, axis};
        }
        fail(why);
    }

    // Where control flow joins, the tags must hold whichever path ran: a loop body runs zero, one or many times, a
    // branch is taken or not.  A partial value is the one state that an AllReduce placed by a single walk gets wrong
    // there (inside a loop it would be summed again on every iteration; behind a branch that was not taken the
    // value would still be partial, or be summed although it was already complete).  So partial values do not cross
    // block boundaries: every partial id that a block reads or assigns is completed in front of the block, and every
    // id that a block leaves partial is completed at its end when anything can still read it (the next iteration
    // before it is assigned again, code outside the block, or the host).
    struct BlockRefs {
        std::map<uint32_t, int> reads;   // id -> reading commands inside (conditions and nested blocks included)
        std::set<uint32_t> defs;         // ids assigned inside
        std::set<uint32_t> exposed;      // ids read before the block itself has certainly assigned them
    };
    void gather(const Block& b, BlockRefs& out) {
        std::set<uint32_t> defined;
        auto rd = [&](uint32_t id) {
            out.reads[id]++;
            if (!defined.count(id)) out.exposed.insert(id);
        };
        for (auto& c : b.cmds) {
            if (c.op == OP_WHILE || c.op == OP_IF) {
                BlockRefs in;
                if (c.op == OP_WHILE) {
                    rd(c.a);
                    gather(*c.block, in);
                    in.reads[c.a]++;   // the condition is read again after every pass
                    in.exposed.insert(c.a);
                } else {
                    for (auto& cb : c.conds) rd(cb.first);
                    for (auto& cb : c.conds) gather(*cb.second, in);
                    if (c.else_block) gather(*c.else_block, in);
                }
                for (auto& kv : in.reads) out.reads[kv.first] += kv.second;
                for (auto id : in.exposed)
                    if (!defined.count(id)) out.exposed.insert(id);
                out.defs.insert(in.defs.begin(), in.defs.end());
                continue;
            }
            if (!has_result(c.op) || !needed[c.res]) continue;
            uint32_t r[2];
            int n;
            reads(c, r, n);
            for (int k = 0; k < n; k++) rd(r[k]);
            out.defs.insert(c.res);
            defined.insert(c.res);
        }
    }
    std::map<uint32_t, int> total_reads_;
    bool have_totals_ = false;
    void complete_before(const BlockRefs& br, std::vector<Cmd>& out) {
        for (auto& kv : br.reads) resolve_partial(kv.first, out);
        for (auto id : br.defs) resolve_partial(id, out);
    }
    void complete_at_end(Block& inner, const BlockRefs& br) {
        if (!have_totals_) {
            BlockRefs all;
            gather(prog.main, all);
            total_reads_ = all.reads;
            have_totals_ = true;
        }
        for (auto id : br.defs) {
            if (info[id].tag != T_PART) continue;
            auto in = br.reads.find(id);
            auto tot = total_reads_.find(id);
            const int inside = in == br.reads.end() ? 0 : in->second, total = tot == total_reads_.end() ? 0 : tot->second;
            if (br.exposed.count(id) || total > inside || is_dep[id]) {
                inner.cmds.push_back(make_allreduce(id));
                info[id].tag = T_REP;
                prog.n_cmds++;
            }
        }
    }

    void block(Block& b) {
        std::vector<Cmd> out;
        out.reserve(b.cmds.size() + 8);
        for (auto& c : b.cmds) {
            if (c.op == OP_WHILE) {
                if (info[c.a].tag == T_SHARD) fail("loop condition '" + name(c.a) + "' is sharded");
                BlockRefs br;
                gather(*c.block, br);
                br.reads[c.a]++;
                br.exposed.insert(c.a);
                complete_before(br, out);
                block(*c.block);
                // (the condition is recomputed inside the body into the same id: it counts as read by the next pass)
                complete_at_end(*c.block, br);
                out.push_back(std::move(c));
                continue;
            }
            if (c.op == OP_IF) {
                BlockRefs all;
                for (auto& cb : c.conds) {
                    if (info[cb.first].tag == T_SHARD) fail("condition '" + name(cb.first) + "' is sharded");
                    all.reads[cb.first]++;
                    gather(*cb.second, all);
                }
                if (c.else_block) gather(*c.else_block, all);
                complete_before(all, out);
                for (auto& cb : c.conds) {
                    BlockRefs br;
                    gather(*cb.second, br);
                    block(*cb.second);
                    complete_at_end(*cb.second, br);
                }
                if (c.else_block) {
                    BlockRefs br;
                    gather(*c.else_block, br);
                    block(*c.else_block);
                    complete_at_end(*c.else_block, br);
                }
                out.push_back(std::move(c));
                continue;
            }
            if (!has_result(c.op) || !needed[c.res]) {
                out.push_back(std::move(c));
                continue;
            }
            step(c, out);
            uint32_t res = c.res;
            out.push_back(std::move(c));
            if (is_dep[res] && info[res].tag == T_PART) {
                // a kept partial value is completed right where it is produced
                out.push_back(make_allreduce(res));
                info[res].tag = T_REP;
                prog.n_cmds++;
            }
        }
        b.cmds = std::move(out);
    }

    static int64_t prod(const std::vector<int64_t>& d, size_t from, size_t to) {
        int64_t p = 1;
        for (size_t i = from; i < to; i++) p *= d[i];
        return p;
    }

    void step(Cmd& c, std::vector<Cmd>& out) {
        const int ord = ordinal_++;
        {
            // the result inherits the guess behind the operand that fixes its distribution
            uint32_t r[2];
            int n;
            reads(c, r, n);
            pending_origin_ = -1;
            for (int k = 0; k < n && pending_origin_ < 0; k++)
                if (info[r[k]].tag == T_SHARD) pending_origin_ = info[r[k]].origin;
            for (int k = 0; k < n && pending_origin_ < 0; k++)
                if (info[r[k]].tag == T_CONST) pending_origin_ = info[r[k]].origin;
            // constants only ever meet tensors in element-wise commands; anywhere else a cut constant is a wrong guess
            const bool elementwise = c.op == OP_MUL || c.op == OP_ADD || c.op == OP_MUL_EQ || c.op == OP_ADD_EQ || c.op == OP_EQZ ||
                                     c.op == OP_GTZ || c.op == OP_LTZ || c.op == OP_EXP2 || c.op == OP_LOG2 || c.op == OP_SIN ||
                                     c.op == OP_RECIP || c.op == OP_SQRT || c.op == OP_CONTIG;
            if (!elementwise)
                for (int k = 0; k < n; k++) {
                    const Info& x = info[r[k]];
                    if (x.tag == T_CONST && x.ldims != x.dims) redecide(x, -1, "constant '" + name(r[k]) + "' is reshaped after it was cut along the batch");
                }
        }
        switch (c.op) {
        case OP_CREATE_MAT: {
            std::vector<int64_t> g = c.dims;
            int64_t n = prod(g, 0, g.size());
            const bool listed = !only || std::find(only->begin(), only->end(), name(c.res)) != only->end();
            if (only && listed && (g.empty() || g[0] != batch))
                fail("CreateMat '" + name(c.res) + "' is listed as holding the batch but its first dimension is not the batch");
            if (!g.empty() && g[0] == batch && listed) {
                if (batch % world) fail("batch is not divisible by the number of ranks");
                int64_t local = n / world;
                if (int64_t(c.count) == n) {
                    c.payload += uint64_t(rank) * uint64_t(local) * 4;  // this rank's rows of the full tensor
                } else if (int64_t(c.count) != local) {
                    fail("CreateMat '" + name(c.res) + "' holds neither the full batch nor this rank's share");
                }
                c.count = uint64_t(local);
                c.dims[0] = batch / world;
                set(c.res, T_SHARD, 0, g, c);
            } else
                set(c.res, T_REP, 0, g, c);
            return;
        }
        case OP_CREATE_CONST: {
            std::vector<int64_t> g = c.dims;
            // guess: the first dimension that equals the batch is the batch (unless an earlier attempt found otherwise)
            int cut = -1;
            for (size_t k = 0; k < g.size() && cut < 0; k++)
                if (g[k] == batch) cut = int(k);
            const bool guessed = cut >= 0;
            if (decided) {
                auto it = decided->find(ord);
                if (it != decided->end()) cut = it->second;
            }
            if (cut >= 0) {
                if (size_t(cut) >= g.size() || g[size_t(cut)] % world) fail("constant '" + name(c.res) + "' cannot be cut along axis " + std::to_string(cut));
                c.dims[size_t(cut)] = g[size_t(cut)] / world;
            }
            pending_origin_ = (guessed || cut >= 0) ? ord : -1;
            set(c.res, T_CONST, std::max(cut, 0), g, c);
            info[c.res].ldims = c.dims;
            return;
        }
        case OP_MUL: case OP_ADD: case OP_MUL_EQ: case OP_ADD_EQ: {
            const bool mul = c.op == OP_MUL || c.op == OP_MUL_EQ;
            Info a = info[c.a], b = info[c.b];
            if (a.tag == T_UNDEF || b.tag == T_UNDEF) fail("'" + name(a.tag == T_UNDEF ? c.a : c.b) + "' is read before it is defined");
            // linear cases keep partial sums partial
            bool keep_partial = (mul && ((a.tag == T_PART && b.tag == T_CONST) || (a.tag == T_CONST && b.tag == T_PART))) ||
                                (!mul && a.tag == T_PART && b.tag == T_PART);
            if (!keep_partial) {
                resolve_partial(c.a, out);
                resolve_partial(c.b, out);
                a = info[c.a];
                b = info[c.b];
            }
            const Info& shape_src = a.tag == T_CONST ? b : a;
            // a constant must have the local shape of the tensor it meets
            if ((a.tag == T_CONST) != (b.tag == T_CONST)) {
                const Info& k = a.tag == T_CONST ? a : b;
                const Info& t = a.tag == T_CONST ? b : a;
                if (k.dims == t.dims && k.ldims != local_dims(t))
                    redecide(k, t.tag == T_SHARD ? t.axis : -1,
                             "constant '" + name(a.tag == T_CONST ? c.a : c.b) + "' does not have the shape of the tensor it is combined with");
            }
            if (keep_partial) { set(c.res, T_PART, 0, shape_src.dims, c); return; }
            if (a.tag == T_CONST && b.tag == T_CONST) {
                if (a.dims == b.dims && a.ldims != b.ldims) {
                    if (b.origin >= 0) redecide(b, a.ldims == a.dims ? -1 : a.axis, "constants of different local shapes are combined");
                    redecide(a, b.ldims == b.dims ? -1 : b.axis, "constants of different local shapes are combined");
                }
                set(c.res, T_CONST, a.axis, a.dims, c);
                info[c.res].ldims = a.ldims;
                return;
            }
            if (a.tag == T_SHARD || b.tag == T_SHARD) {
                const Info& s = a.tag == T_SHARD ? a : b;
                const Info& o = a.tag == T_SHARD ? b : a;
                if (o.tag == T_REP && s.origin >= 0) redecide(s, -1, "a broadcast along the batch meets a replicated tensor");
                if (o.tag == T_SHARD && o.axis != s.axis) {
                    if (o.origin >= 0) redecide(o, -1, "operands are sharded along different axes");
                    if (s.origin >= 0) redecide(s, -1, "operands are sharded along different axes");
                }
                if (o.tag == T_REP) fail("'" + name(c.a) + "' and '" + name(c.b) + "' mix a sharded and a replicated tensor of the same shape");
                if (o.tag == T_SHARD && o.axis != s.axis) fail("operands are sharded along different axes (tensors are recognised as batch tensors by their first dimension: a "
                                                                 "parameter with as many rows as the batch is mistaken for one -- name the batch tensors (adb_config.shard_ids) or use a batch size that differs from the layer widths)");
                set(c.res, T_SHARD, s.axis, s.dims, c);
                return;
            }
            set(c.res, T_REP, 0, shape_src.dims, c);
            return;
        }
        case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_EXP2: case OP_LOG2: case OP_SIN: case OP_RECIP: case OP_SQRT: case OP_CONTIG: {
            if (info[c.a].tag == T_UNDEF) fail("'" + name(c.a) + "' is read before it is defined");
            resolve_partial(c.a, out);
            Info a = info[c.a];
            set(c.res, a.tag, a.axis, a.dims, c);
            if (a.tag == T_CONST) info[c.res].ldims = a.ldims;
            return;
        }
        case OP_SUM: {
            Info a = info[c.a];
            if (a.dims.size() != 2) fail("Sum needs a 2-d operand");
            std::vector<int64_t> g{a.dims[0]};
            if (a.tag == T_SHARD) {
                if (a.axis == 0) set(c.res, T_SHARD, 0, g, c);
                else set(c.res, T_PART, 0, g, c);
            } else if (a.tag == T_PART) set(c.res, T_PART, 0, g, c);
            else set(c.res, T_REP, 0, g, c);
            return;
        }
        case OP_MAX: {
            // not linear: a partial operand is summed over the ranks first; a maximum along the batch itself
            // would need a max-reduction across ranks, which this rewrite does not have
            resolve_partial(c.a, out);
            Info a = info[c.a];
            if (a.dims.size() != 2) fail("Max needs a 2-d operand");
            std::vector<int64_t> g{a.dims[0]};
            if (a.tag == T_SHARD) {
                if (a.axis != 0) fail("Max of '" + name(c.a) + "' runs along the sharded batch axis");
                set(c.res, T_SHARD, 0, g, c);
            } else set(c.res, T_REP, 0, g, c);
            return;
        }
        case OP_DOT: {
            resolve_partial(c.a, out);
            resolve_partial(c.b, out);
            Info a = info[c.a], b = info[c.b];
            if (a.dims.size() != 2 || b.dims.size() != 2) fail("DotProduct needs 2-d operands");
            std::vector<int64_t> g{a.dims[0], b.dims[1]};
            bool a_rep = a.tag == T_REP || a.tag == T_CONST, b_rep = b.tag == T_REP || b.tag == T_CONST;
            if (a.tag == T_SHARD && a.axis == 0 && b_rep) set(c.res, T_SHARD, 0, g, c);
            else if (a.tag == T_SHARD && a.axis == 1 && b.tag == T_SHARD && b.axis == 0) set(c.res, T_PART, 0, g, c);
            else if (a_rep && b.tag == T_SHARD && b.axis == 1) set(c.res, T_SHARD, 1, g, c);
            else if (a_rep && b_rep) set(c.res, T_REP, 0, g, c);
            else {
                if (b.tag == T_SHARD && b.origin >= 0) redecide(b, -1, "DotProduct operand is a broadcast along the batch");
                if (a.tag == T_SHARD && a.origin >= 0) redecide(a, -1, "DotProduct operand is a broadcast along the batch");
                fail("DotProduct of '" + name(c.a) + "' and '" + name(c.b) + "' cannot be split over the batch");
            }
            return;
        }
        case OP_BATCH_DOT: {
            resolve_partial(c.a, out);
            resolve_partial(c.b, out);
            Info a = info[c.a], b = info[c.b];
            if (a.dims.size() != 3 || b.dims.size() != 3) fail("BatchDot needs 3-d operands");
            std::vector<int64_t> g{a.dims[0], a.dims[1], b.dims[2]};
            const bool a_rep = a.tag == T_REP || a.tag == T_CONST, b_rep = b.tag == T_REP || b.tag == T_CONST;
            // the slices are independent: both operands cut along the slice axis stay cut, anything else is refused
            if (a_rep && b_rep) set(c.res, T_REP, 0, g, c);
            else if (a.tag == T_SHARD && b.tag == T_SHARD && a.axis == 0 && b.axis == 0) set(c.res, T_SHARD, 0, g, c);
            else fail("BatchDot of '" + name(c.a) + "' and '" + name(c.b) + "' cannot be split over the batch");
            return;
        }
        case OP_VIEW: {
            Info a = info[c.a];
            std::vector<int64_t> g = c.dims;
            if (a.tag == T_SHARD) {
                int64_t before = prod(a.dims, 0, size_t(a.axis));
                int64_t p = 1;
                int nd = -1;
                for (size_t i = 0; i < g.size(); i++) {
                    if (p == before && g[i] != 1) { nd = int(i); break; }
                    p *= g[i];
                }
                if (nd < 0) fail("View of '" + name(c.a) + "' loses the sharded axis");
                int64_t old_ext = a.dims[a.axis], new_ext = g[nd];
                bool ok = new_ext % world == 0 && (new_ext % old_ext == 0 || old_ext % new_ext == 0);
                if (!ok) fail("View of '" + name(c.a) + "' cuts through the sharded axis");
                c.dims[nd] = new_ext / world;
                set(c.res, T_SHARD, nd, g, c);
            } else {
                set(c.res, a.tag, 0, g, c);
                if (a.tag == T_CONST) info[c.res].ldims = g;   // only uncut constants get this far: local = global shape
            }
            return;
        }
        case OP_INDEX: {
            Info a = info[c.a];
            std::vector<int64_t> g = a.dims;
            if (c.dim >= g.size()) fail("Index axis out of range");
            g.erase(g.begin() + c.dim);
            if (a.tag == T_SHARD) {
                if (int(c.dim) == a.axis) fail("Index into the sharded axis of '" + name(c.a) + "'");
                set(c.res, T_SHARD, a.axis - (int(c.dim) < a.axis ? 1 : 0), g, c);
            } else {
                set(c.res, a.tag, 0, g, c);
                if (a.tag == T_CONST) info[c.res].ldims = g;
            }
            return;
        }
        case OP_PERMUTE: {
            Info a = info[c.a];
            std::vector<int64_t> g(c.perm.size());
            int nd = 0;
            for (size_t i = 0; i < c.perm.size(); i++) {
                if (c.perm[i] >= a.dims.size()) fail("Permute index out of bounds");
                g[i] = a.dims[c.perm[i]];
                if (int(c.perm[i]) == a.axis) nd = int(i);
            }
            set(c.res, a.tag, a.tag == T_SHARD ? nd : 0, g, c);
            if (a.tag == T_CONST) info[c.res].ldims = g;
            return;
        }
        case OP_BROADCAST: {
            resolve_partial(c.a, out);
            Info a = info[c.a];
            std::vector<int64_t> g = a.dims;
            if (c.dim >= g.size()) fail("Broadcast axis out of range");
            g[c.dim] = int64_t(c.count);
            if (a.tag == T_SHARD) {
                if (int(c.dim) == a.axis) fail("Broadcast along the sharded axis");
                set(c.res, T_SHARD, a.axis, g, c);
            } else if (int64_t(c.count) == batch && !(decided && decided->count(ord) && decided->at(ord) < 0)) {
                // a replicated value repeated along the batch (a guess: the count could be a layer width that
                // happens to equal the batch): every rank materialises only its rows
                c.count = uint64_t(batch / world);
                pending_origin_ = ord;
                set(c.res, T_SHARD, int(c.dim), g, c);
            } else {
                set(c.res, a.tag, 0, g, c);
                if (a.tag == T_CONST) info[c.res].ldims = g;
            }
            return;
        }
        case OP_CONCAT: {
            resolve_partial(c.a, out);
            resolve_partial(c.b, out);
            Info a = info[c.a], b = info[c.b];
            std::vector<int64_t> g = a.dims;
            if (c.dim >= g.size() || b.dims.size() != g.size()) fail("Concat rank mismatch");
            g[c.dim] += b.dims[c.dim];
            if (a.tag == T_SHARD || b.tag == T_SHARD) {
                if (a.tag != b.tag || a.axis != b.axis || a.axis == int(c.dim)) fail("Concat of differently distributed tensors");
                set(c.res, T_SHARD, a.axis, g, c);
            } else
                set(c.res, T_REP, 0, g, c);
            return;
        }
        case OP_ALLREDUCE:
            info[c.a].tag = T_REP;
            return;
        default: return;
        }
    }
};

}  // namespace

void shard_program(Program& prog, int rank, int world, int64_t batch, const std::vector<std::string>* only) {
    if (world <= 1) return;
    if (batch <= 0) throw IrError("data-parallel rewrite: shard_batch must be positive");
    if (rank < 0 || rank >= world) throw IrError("data-parallel rewrite: rank out of range");
    if (only && only->empty()) only = nullptr;
    // attempts on scratch copies find out which guesses about constants / broadcasts do not hold ...
    std::map<int, int> decided;
    const std::vector<uint8_t> bytes = serialize_program(prog);
    for (int attempt = 0;; attempt++) {
        Program scratch = parse_program(bytes.data(), bytes.size());
        Sharder s(scratch, rank, world, batch);
        s.only = only;
        s.decided = &decided;
        try {
            s.mark_needed();
            s.block(scratch.main);
            break;
        } catch (const Decide& d) {
            if (attempt >= 256) throw IrError("data-parallel rewrite: the shapes of constants and broadcasts cannot be reconciled");
            decided[d.ordinal] = d.axis;
        }
    }
    // ... and the program itself is rewritten in place with what they found
    Sharder s(prog, rank, world, batch);
    s.only = only;
    s.decided = &decided;
    try {
        s.mark_needed();
        s.block(prog.main);
    } catch (const Decide&) {
        throw IrError("data-parallel rewrite: internal inconsistency while applying decisions");
    }
}

}  // namespace adb
