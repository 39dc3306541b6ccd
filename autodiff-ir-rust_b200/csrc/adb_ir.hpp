// HLIR program as received over the C-ABI: the reference's `enum IRCmds` / `IRProcedure`
// (src/core/ir.rs:8-112) with string ids replaced by indices into an id table.
#pragma once
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace adb {

enum Op : uint8_t {
    OP_CREATE_MAT = 1, OP_CREATE_CONST = 2,
    OP_MUL = 3, OP_ADD = 4, OP_MUL_EQ = 5, OP_ADD_EQ = 6,
    OP_EQZ = 7, OP_GTZ = 8, OP_LTZ = 9,
    OP_SUM = 10, OP_DOT = 11,
    OP_VIEW = 12, OP_INDEX = 13, OP_CONCAT = 14, OP_PERMUTE = 15, OP_BROADCAST = 16, OP_CONTIG = 17,
    OP_EXP2 = 18, OP_LOG2 = 19, OP_SIN = 20, OP_RECIP = 21, OP_SQRT = 22,
    OP_WHILE = 23, OP_IF = 24, OP_EX = 25, OP_HEADING = 26, OP_ALLREDUCE = 27,
    OP_MAX = 28,  // extension: row maximum of a 2-d tensor, same shape contract as OP_SUM
    OP_BATCH_DOT = 29,  // extension: [B,M,K] x [B,K,N] -> [B,M,N]
};

enum PayloadKind : uint8_t { PAYLOAD_INLINE = 0, PAYLOAD_HOST = 1, PAYLOAD_DEVICE = 2 };

struct Block;

struct Cmd {
    uint8_t op = 0;
    uint32_t a = 0, b = 0, res = 0;
    std::vector<int64_t> dims;      // CreateMat / CreateConstant / View
    std::vector<uint32_t> perm;     // Permute
    uint64_t index = 0;             // Index
    uint64_t count = 0;             // CreateMat n / Broadcast r
    uint32_t dim = 0;               // Index / Concat / Broadcast
    float cval = 0.f;               // CreateConstant
    uint8_t payload_kind = 0;       // CreateMat
    uint64_t payload = 0;           // CreateMat: address (host or device) of the data
    std::unique_ptr<Block> block;   // While
    std::vector<std::pair<uint32_t, std::unique_ptr<Block>>> conds;  // If
    std::unique_ptr<Block> else_block;
    std::string text;               // Heading
};

struct Block {
    std::vector<Cmd> cmds;
};

struct Program {
    std::vector<std::string> ids;
    std::vector<uint32_t> dep;
    Block main;
    size_t n_cmds = 0;
};

struct IrError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Reader {
  public:
    Reader(const uint8_t* p, size_t n) : base_(p), p_(p), end_(p + n) {}
    template <class T> T get() {
        if (p_ + sizeof(T) > end_) throw IrError("truncated blob");
        T v;
        std::memcpy(&v, p_, sizeof(T));
        p_ += sizeof(T);
        return v;
    }
    std::string str(size_t n) {
        if (p_ + n > end_) throw IrError("truncated blob");
        std::string s(reinterpret_cast<const char*>(p_), n);
        p_ += n;
        return s;
    }
    const uint8_t* base() const { return base_; }
    size_t size() const { return size_t(end_ - base_); }

  private:
    const uint8_t *base_, *p_, *end_;
};

inline std::vector<int64_t> read_dims(Reader& r) {
    uint8_t nd = r.get<uint8_t>();
    if (nd > 8) throw IrError("more than 8 dimensions");
    std::vector<int64_t> d(nd);
    for (auto& x : d) {
        uint64_t v = r.get<uint64_t>();
        if (v > (uint64_t(1) << 40)) throw IrError("dimension too large");
        x = int64_t(v);
    }
    return d;
}

void parse_block(Reader& r, Program& prog, Block& out, int depth);

inline void parse_cmd(Reader& r, Program& prog, Cmd& c, int depth) {
    c.op = r.get<uint8_t>();
    auto id = [&]() {
        uint32_t v = r.get<uint32_t>();
        if (v >= prog.ids.size()) throw IrError("id index out of range");
        return v;
    };
    switch (c.op) {
    case OP_CREATE_MAT: {
        c.res = id();
        c.dims = read_dims(r);
        c.payload_kind = r.get<uint8_t>();
        uint64_t where = r.get<uint64_t>();
        c.count = r.get<uint64_t>();
        if (c.payload_kind == PAYLOAD_INLINE) {
            if (where > r.size() || c.count > (r.size() - where) / 4) throw IrError("inline payload out of range");
            c.payload = uint64_t(uintptr_t(r.base() + where));
        } else if (c.payload_kind == PAYLOAD_HOST || c.payload_kind == PAYLOAD_DEVICE) {
            c.payload = where;
        } else
            throw IrError("unknown payload kind");
        break;
    }
    case OP_CREATE_CONST: c.res = id(); c.cval = r.get<float>(); c.dims = read_dims(r); break;
    case OP_MUL: case OP_ADD: case OP_DOT: case OP_BATCH_DOT: c.a = id(); c.b = id(); c.res = id(); break;
    case OP_MUL_EQ: case OP_ADD_EQ: c.a = id(); c.b = id(); c.res = c.a; break;
    case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_SUM: case OP_MAX: case OP_CONTIG:
    case OP_EXP2: case OP_LOG2: case OP_SIN: case OP_RECIP: case OP_SQRT:
        c.a = id(); c.res = id(); break;
    case OP_VIEW: c.a = id(); c.res = id(); c.dims = read_dims(r); break;
    case OP_INDEX: c.a = id(); c.res = id(); c.index = r.get<uint64_t>(); c.dim = r.get<uint32_t>(); break;
    case OP_CONCAT: c.a = id(); c.b = id(); c.res = id(); c.dim = r.get<uint32_t>(); break;
    case OP_PERMUTE: {
        c.a = id(); c.res = id();
        uint8_t n = r.get<uint8_t>();
        if (n > 8) throw IrError("permute rank > 8");
        c.perm.resize(n);
        for (auto& p : c.perm) p = r.get<uint32_t>();
        break;
    }
    case OP_BROADCAST: c.a = id(); c.res = id(); c.dim = r.get<uint32_t>(); c.count = r.get<uint64_t>(); break;
    case OP_WHILE:
        c.a = id();
        c.block = std::make_unique<Block>();
        parse_block(r, prog, *c.block, depth + 1);
        break;
    case OP_IF: {
        uint32_t n = r.get<uint32_t>();
        if (n > (1u << 20)) throw IrError("too many If conditions");
        for (uint32_t i = 0; i < n; i++) {
            uint32_t cid = id();
            auto blk = std::make_unique<Block>();
            parse_block(r, prog, *blk, depth + 1);
            c.conds.emplace_back(cid, std::move(blk));
        }
        if (r.get<uint8_t>()) {
            c.else_block = std::make_unique<Block>();
            parse_block(r, prog, *c.else_block, depth + 1);
        }
        break;
    }
    case OP_EX: break;
    case OP_HEADING: c.text = r.str(r.get<uint16_t>()); break;
    case OP_ALLREDUCE: c.a = id(); c.res = c.a; break;
    default: throw IrError("unknown opcode " + std::to_string(int(c.op)));
    }
    prog.n_cmds++;
}

inline void parse_block(Reader& r, Program& prog, Block& out, int depth) {
    if (depth > 64) throw IrError("blocks nested too deeply");
    uint32_t n = r.get<uint32_t>();
    if (n > (1u << 28)) throw IrError("procedure too long");
    out.cmds.resize(n);
    for (auto& c : out.cmds) parse_cmd(r, prog, c, depth);
}

inline Program parse_program(const uint8_t* blob, size_t nbytes) {
    Reader r(blob, nbytes);
    Program p;
    if (r.get<uint32_t>() != 0x52494441u) throw IrError("bad magic");
    if (r.get<uint32_t>() != 1u) throw IrError("unsupported wire version");
    (void)r.get<uint32_t>();
    uint32_t n_ids = r.get<uint32_t>();
    if (n_ids > (1u << 28)) throw IrError("id table too large");
    p.ids.reserve(n_ids);
    for (uint32_t i = 0; i < n_ids; i++) p.ids.push_back(r.str(r.get<uint16_t>()));
    uint32_t n_dep = r.get<uint32_t>();
    if (n_dep > n_ids) throw IrError("dep list longer than id table");
    p.dep.resize(n_dep);
    for (auto& d : p.dep) {
        d = r.get<uint32_t>();
        if (d >= n_ids) throw IrError("dep id out of range");
    }
    parse_block(r, p, p.main, 0);
    return p;
}

// ---- serialiser (used by the data-parallel rewrite, which returns a new blob) ----
class Writer {
  public:
    template <class T> void put(T v) {
        size_t n = buf.size();
        buf.resize(n + sizeof(T));
        std::memcpy(buf.data() + n, &v, sizeof(T));
    }
    void dims(const std::vector<int64_t>& d) {
        put<uint8_t>(uint8_t(d.size()));
        for (auto x : d) put<uint64_t>(uint64_t(x));
    }
    std::vector<uint8_t> buf;
};

inline void write_block(Writer& w, const Block& b, std::vector<std::pair<size_t, const Cmd*>>& inline_fix);

inline void write_cmd(Writer& w, const Cmd& c, std::vector<std::pair<size_t, const Cmd*>>& inline_fix) {
    w.put<uint8_t>(c.op);
    switch (c.op) {
    case OP_CREATE_MAT:
        w.put<uint32_t>(c.res); w.dims(c.dims);
        w.put<uint8_t>(c.payload_kind);
        if (c.payload_kind == PAYLOAD_INLINE) inline_fix.emplace_back(w.buf.size(), &c);
        w.put<uint64_t>(c.payload); w.put<uint64_t>(c.count);
        break;
    case OP_CREATE_CONST: w.put<uint32_t>(c.res); w.put<float>(c.cval); w.dims(c.dims); break;
    case OP_MUL: case OP_ADD: case OP_DOT: case OP_BATCH_DOT: w.put<uint32_t>(c.a); w.put<uint32_t>(c.b); w.put<uint32_t>(c.res); break;
    case OP_MUL_EQ: case OP_ADD_EQ: w.put<uint32_t>(c.a); w.put<uint32_t>(c.b); break;
    case OP_EQZ: case OP_GTZ: case OP_LTZ: case OP_SUM: case OP_MAX: case OP_CONTIG:
    case OP_EXP2: case OP_LOG2: case OP_SIN: case OP_RECIP: case OP_SQRT:
        w.put<uint32_t>(c.a); w.put<uint32_t>(c.res); break;
    case OP_VIEW: w.put<uint32_t>(c.a); w.put<uint32_t>(c.res); w.dims(c.dims); break;
    case OP_INDEX: w.put<uint32_t>(c.a); w.put<uint32_t>(c.res); w.put<uint64_t>(c.index); w.put<uint32_t>(c.dim); break;
    case OP_CONCAT: w.put<uint32_t>(c.a); w.put<uint32_t>(c.b); w.put<uint32_t>(c.res); w.put<uint32_t>(c.dim); break;
    case OP_PERMUTE:
        w.put<uint32_t>(c.a); w.put<uint32_t>(c.res); w.put<uint8_t>(uint8_t(c.perm.size()));
        for (auto p : c.perm) w.put<uint32_t>(p);
        break;
    case OP_BROADCAST: w.put<uint32_t>(c.a); w.put<uint32_t>(c.res); w.put<uint32_t>(c.dim); w.put<uint64_t>(c.count); break;
    case OP_WHILE: w.put<uint32_t>(c.a); write_block(w, *c.block, inline_fix); break;
    case OP_IF:
        w.put<uint32_t>(uint32_t(c.conds.size()));
        for (auto& cb : c.conds) { w.put<uint32_t>(cb.first); write_block(w, *cb.second, inline_fix); }
        w.put<uint8_t>(c.else_block ? 1 : 0);
        if (c.else_block) write_block(w, *c.else_block, inline_fix);
        break;
    case OP_EX: break;
    case OP_HEADING:
        w.put<uint16_t>(uint16_t(c.text.size()));
        w.buf.insert(w.buf.end(), c.text.begin(), c.text.end());
        break;
    case OP_ALLREDUCE: w.put<uint32_t>(c.a); break;
    }
}

inline void write_block(Writer& w, const Block& b, std::vector<std::pair<size_t, const Cmd*>>& inline_fix) {
    w.put<uint32_t>(uint32_t(b.cmds.size()));
    for (auto& c : b.cmds) write_cmd(w, c, inline_fix);
}

inline std::vector<uint8_t> serialize_program(const Program& p) {
    Writer w;
    w.put<uint32_t>(0x52494441u); w.put<uint32_t>(1u); w.put<uint32_t>(0u); w.put<uint32_t>(uint32_t(p.ids.size()));
    for (auto& s : p.ids) {
        w.put<uint16_t>(uint16_t(s.size()));
        w.buf.insert(w.buf.end(), s.begin(), s.end());
    }
    w.put<uint32_t>(uint32_t(p.dep.size()));
    for (auto d : p.dep) w.put<uint32_t>(d);
    std::vector<std::pair<size_t, const Cmd*>> fix;
    write_block(w, p.main, fix);
    for (auto& f : fix) {
        while (w.buf.size() % 16) w.buf.push_back(0);
        uint64_t off = w.buf.size();
        std::memcpy(w.buf.data() + f.first, &off, 8);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(uintptr_t(f.second->payload));
        w.buf.insert(w.buf.end(), src, src + f.second->count * 4);
    }
    return w.buf;
}

}  // namespace adb
