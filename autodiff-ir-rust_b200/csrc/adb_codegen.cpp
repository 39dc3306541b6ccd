// CUDA source for the fused kernels of a plan.
//
// The reference emits one OpenCL C string per kernel and builds it at first use
// (src/devices/opencl/kernels/{unary,binary,movement,reduce,fuse_elw,fuse_reduce_elw}.rs,
// cache in src/devices/opencl/context.rs:90-106): one work-item per output element, scalar loads,
// index expressions spelled out with / and %.  Here the skeletons are hand-written for sm_100a
// (128-bit loads/stores, grid-stride loops sized to the 148 SMs, warp-shuffle + shared-memory
// reduction trees, a column-sum variant whose lanes run along the contiguous axis) and only the
// straight-line SSA body between load and store is spliced in from the plan.
//
// Arithmetic contract (matches the CPU restatement of the reference semantics):
//   + and * are __fadd_rn / __fmul_rn (never contracted into FMA), 1/x and sqrt(fabsf(x)) are the
//   <= 1 ulp rcp.approx / sqrt.approx (or __frcp_rn / __fsqrt_rn when the plan asks for correctly rounded
//   division), comparisons give 1.0f / 0.0f against 0.0f
//   (src/devices/opencl/kernels/unary.rs:3-17), exp2f / log2f / sinf are CUDA's (<= 2 ulp).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <sstream>

#include "adb_lower.hpp"

namespace adb {

namespace {

struct Access {
    enum Mode { SCALAR, VEC4, GATHER } mode = SCALAR;
    int64_t lane_stride = 0;  // GATHER: element stride between the 4 lanes
};

// set for the duration of generate_kernels
thread_local bool g_exact_div = false;

// 1/x and sqrt(x) through the special-function unit: rcp.approx.f32 / sqrt.approx.f32 keep subnormal inputs and
// results and are within 1 ulp, inside the 2-ulp bound the element-wise primitives are held to; the correctly
// rounded forms cost 10 and 11 issue slots per element in kernels that are issue-bound
const char* helpers() {
    if (g_exact_div) return "";
    return "__device__ __forceinline__ float adb_rcp(float x) { float r; asm(\"rcp.approx.f32 %0, %1;\" : \"=f\"(r) : \"f\"(x)); return r; }\n"
           "__device__ __forceinline__ float adb_sqrt(float x) { float r; asm(\"sqrt.approx.f32 %0, %1;\" : \"=f\"(r) : \"f\"(x)); return r; }\n";
}

std::string hexf(float v) {
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    char buf[48];
    std::snprintf(buf, sizeof buf, "__int_as_float(0x%08x)", bits);
    return buf;
}

bool needs_wide(int64_t n, const std::vector<const Operand*>& ops) {
    if (n >= (int64_t(1) << 31) - 1024) return true;
    for (auto* o : ops) {
        int64_t m = 0;
        for (auto& s : o->subs) m += (s.size - 1) * std::max<int64_t>(s.stride, 0);
        for (auto& s : o->xsubs) m += (s.size - 1) * std::max<int64_t>(s.stride, 0);
        if (m >= (int64_t(1) << 31) - 1024) return true;
    }
    return false;
}

// offset expression of a digit list from index variable `iv` (outermost digit needs no modulo)
std::string offset_expr(const std::vector<Sub>& subs, const std::string& iv, std::ostringstream& pre,
                        const std::string& tag, const char* idx_t) {
    if (subs.empty()) return "0";
    if (subs.size() == 1) {
        if (subs[0].stride == 0) return "0";
        if (subs[0].stride == 1) return iv;
        return iv + " * " + std::to_string(subs[0].stride);
    }
    std::string r = "r_" + tag;
    pre << "      " << idx_t << " " << r << " = " << iv << ";\n";
    std::string expr;
    for (size_t t = subs.size(); t-- > 1;) {
        std::string d = "d_" + tag + "_" + std::to_string(t);
        pre << "      " << idx_t << " " << d << " = " << r << " % " << subs[t].size << "; " << r << " /= " << subs[t].size << ";\n";
        if (subs[t].stride != 0) {
            if (!expr.empty()) expr += " + ";
            expr += subs[t].stride == 1 ? d : d + " * " + std::to_string(subs[t].stride);
        }
    }
    if (subs[0].stride != 0) {
        if (!expr.empty()) expr += " + ";
        expr += subs[0].stride == 1 ? r : r + " * " + std::to_string(subs[0].stride);
    }
    return expr.empty() ? "0" : expr;
}

Access classify(const std::vector<Sub>& subs, int64_t offset, int vec, bool is_store) {
    Access a;
    if (vec == 1) return a;
    if (subs.empty()) { a.mode = Access::SCALAR; return a; }
    const Sub& in = subs.back();
    if (in.stride == 0 && !is_store) { a.mode = Access::SCALAR; return a; }
    bool aligned = offset % 4 == 0;
    for (size_t i = 0; i + 1 < subs.size(); i++)
        if (subs[i].stride % 4) aligned = false;
    if (in.stride == 1 && aligned) { a.mode = Access::VEC4; return a; }
    a.mode = Access::GATHER;
    a.lane_stride = in.stride;
    return a;
}

// can the innermost digit of every operand hold 4 consecutive lanes?
bool lanes_ok(const std::vector<Sub>& subs) { return subs.empty() || subs.back().size % 4 == 0; }

void emit_ssa(std::ostringstream& o, const KernelSpec& k, int vec, const std::vector<std::string>& load_names,
              const std::vector<Access>& acc, const char* ind, const std::vector<char>* need = nullptr) {
    static const char L[4] = {'x', 'y', 'z', 'w'};
    for (size_t i = 0; i < k.ssa.size(); i++) {
        if (need && !(*need)[i]) continue;
        const Ssa& s = k.ssa[i];
        for (int l = 0; l < vec; l++) {
            std::string lhs = "v" + std::to_string(i) + "_" + std::to_string(l);
            o << ind << "const float " << lhs << " = ";
            if (s.kind == Ssa::LOAD) {
                const std::string& nm = load_names[s.operand];
                if (vec == 1 || acc[s.operand].mode == Access::SCALAR) o << nm;
                else if (acc[s.operand].mode == Access::VEC4) o << nm << "." << L[l];
                else o << nm << "_" << l;
            } else if (s.kind == Ssa::CONST) {
                o << hexf(s.c);
            } else if (s.kind == Ssa::RED) {
                o << "red" << s.operand;
            } else {
                std::string a = "v" + std::to_string(s.a) + "_" + std::to_string(l);
                std::string b = s.b >= 0 ? "v" + std::to_string(s.b) + "_" + std::to_string(l) : "";
                switch (s.op) {
                case E_ADD: o << "__fadd_rn(" << a << ", " << b << ")"; break;
                case E_MUL: o << "__fmul_rn(" << a << ", " << b << ")"; break;
                case E_EXP2: o << "exp2f(" << a << ")"; break;
                case E_LOG2: o << "log2f(" << a << ")"; break;
                case E_SIN: o << "sinf(" << a << ")"; break;
                case E_RECIP: o << (g_exact_div ? "__frcp_rn(" : "adb_rcp(") << a << ")"; break;
                case E_SQRT: o << (g_exact_div ? "__fsqrt_rn(fabsf(" : "adb_sqrt(fabsf(") << a << "))"; break;
                case E_EQZ: o << "(" << a << " == 0.0f ? 1.0f : 0.0f)"; break;
                case E_GTZ: o << "(" << a << " > 0.0f ? 1.0f : 0.0f)"; break;
                case E_LTZ: o << "(" << a << " < 0.0f ? 1.0f : 0.0f)"; break;
                }
            }
            o << ";\n";
        }
    }
}

void emit_loads(std::ostringstream& o, const KernelSpec& k, int vec, const std::vector<Access>& acc,
                const std::vector<std::string>& off, std::vector<std::string>& names, const char* ind,
                const std::vector<char>* need = nullptr, const std::vector<char>* cached = nullptr) {
    names.resize(k.ins.size());
    for (size_t i = 0; i < k.ins.size(); i++) {
        std::string nm = "l" + std::to_string(i);
        names[i] = nm;
        if (need && !(*need)[i]) continue;
        if (cached && (*cached)[i]) {
            // the value was loaded into registers at the start of the row (ROWS kernels, loop index t)
            o << ind << "const " << (vec == 4 ? "float4 " : "float ") << nm << " = c" << i << "[t];\n";
            continue;
        }
        std::string p = "a.in[" + std::to_string(i) + "]";
        if (vec == 1 || acc[i].mode == Access::SCALAR)
            o << ind << "const float " << nm << " = " << p << "[" << off[i] << "];\n";
        else if (acc[i].mode == Access::VEC4)
            o << ind << "const float4 " << nm << " = *reinterpret_cast<const float4*>(" << p << " + (" << off[i] << "));\n";
        else
            for (int l = 0; l < 4; l++)
                o << ind << "const float " << nm << "_" << l << " = " << p << "[(" << off[i] << ") + " << l * acc[i].lane_stride << "];\n";
    }
}

uint64_t fnv(const std::string& s) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

void finish(KernelSpec& k, const std::string& body, const char* prefix) {
    char name[64];
    std::snprintf(name, sizeof name, "%s_%016llx", prefix, (unsigned long long)fnv(body));
    k.entry = name;
    std::string src = body;
    size_t p;
    while ((p = src.find("@ENTRY@")) != std::string::npos) src.replace(p, 7, name);
    k.source = src;
}

// -------------------------------------------------------------------------------- element-wise
int elw_vec_impl(const KernelSpec& k) {
    int vec = 4;
    if (k.n % 4) vec = 1;
    for (auto& i : k.ins)
        if (!lanes_ok(i.subs)) vec = 1;
    for (auto& o : k.outs) {
        if (!lanes_ok(o.dst.subs)) vec = 1;
        if (o.dst.subs.empty() || o.dst.subs.back().stride == 0) vec = 1;
    }
    if (!k.reds.empty() && k.q2 % 4) vec = 1;
    return vec;
}

void gen_elw_red(KernelSpec& k);

// Materialised axis swap (`x.t().contigious()`, `x.permute(0, 2, 1)` made contiguous, with or without element-wise work
// on the way): the reference's Movement kernel reads with the permuted index expression, one scattered 4-byte load per
// element (src/devices/opencl/kernels/movement.rs:7-46).  When the one input is contiguous along an axis P that is not
// the output's innermost axis Q, a 64 x 64 tile of the (P, Q) plane goes through shared memory instead: 128-bit loads
// along P, 128-bit stores along Q, every other axis is a batch index.  Returns false when the kernel is not of that form.
bool gen_transpose(KernelSpec& k) {
    if (k.ins.size() != 1 || k.outs.empty() || !k.reds.empty() || k.n < (int64_t(1) << 16)) return false;
    for (auto& v : k.ssa)
        if (v.kind == Ssa::RED) return false;
    std::vector<Sub> full;
    full.push_back({k.n, 1});
    for (auto& o : k.outs) {
        std::vector<Sub> d = o.dst.subs;
        canon_subs(d);
        if (d != full) return false;
    }
    const std::vector<Sub>& dg = k.ins[0].subs;   // digits over the output's linear index, outermost first
    if (dg.size() < 2) return false;
    const size_t qi = dg.size() - 1;
    const int64_t Q = dg[qi].size, SQ = dg[qi].stride;
    if (SQ <= 1 || Q < 32) return false;
    size_t pi = dg.size();
    for (size_t t = 0; t + 1 < dg.size(); t++)
        if (dg[t].stride == 1 && dg[t].size >= 32) pi = t;
    if (pi == dg.size()) return false;
    const int64_t P = dg[pi].size;
    // 128-bit accesses need 4-element alignment of every row start on both sides
    std::vector<int64_t> ostride(dg.size(), 1);
    for (size_t t = dg.size() - 1; t-- > 0;) ostride[t] = ostride[t + 1] * dg[t + 1].size;
    bool vec_ok = P % 4 == 0 && Q % 4 == 0 && SQ % 4 == 0 && k.ins[0].offset % 4 == 0 && ostride[pi] % 4 == 0;
    for (size_t t = 0; t < dg.size(); t++)
        if (t != pi && t != qi && (dg[t].stride % 4 || ostride[t] % 4)) vec_ok = false;
    for (auto& o : k.outs)
        if (o.dst.offset % 4) vec_ok = false;
    if (!vec_ok) return false;
    int64_t batch = 1;
    for (size_t t = 0; t < dg.size(); t++)
        if (t != pi && t != qi) batch *= dg[t].size;
    const int64_t tiles_p = (P + 63) / 64, tiles_q = (Q + 63) / 64;
    k.tr_tiles = tiles_p * tiles_q * batch;
    k.vec = 4;
    k.threads = 256;
    k.wide_index = true;

    std::ostringstream o;
    o << helpers() << "struct Args { const float* in[1]; float* out[" << k.outs.size() << "]; long long n; };\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
    // tile[q][p]; the 128-bit column slots of row q are rotated by an XOR with (q / 4) % 8, so rows stay 128-bit aligned
    // for the writes and the transposed reads (rows 4 apart, same column) spread over the banks (2-way at worst)
    o << "  __shared__ __align__(16) float tile[64][64];\n";
    o << "  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 values each way\n";
    o << "  for (long long t = blockIdx.x; t < " << k.tr_tiles << "ll; t += gridDim.x) {\n";
    o << "    long long r = t;\n";
    o << "    const int q0 = int(r % " << tiles_q << ") * 64; r /= " << tiles_q << ";\n";
    o << "    const int p0 = int(r % " << tiles_p << ") * 64; r /= " << tiles_p << ";\n";
    o << "    long long ib = 0, ob = 0;\n";
    for (size_t t = dg.size(); t-- > 0;) {
        if (t == pi || t == qi) continue;
        o << "    { const long long d = r % " << dg[t].size << "; r /= " << dg[t].size << "; ib += d * " << dg[t].stride << "ll; ob += d * "
          << ostride[t] << "ll; }\n";
    }
    // read: thread (tx, ty) loads 4 consecutive p for rows q = ty, ty + 16, ...
    o << "    for (int j = ty; j < 64; j += 16) {\n";
    o << "      const int q = q0 + j, p = p0 + tx * 4;\n";
    o << "      if (q < " << Q << " && p < " << P << ")\n";
    o << "        *reinterpret_cast<float4*>(&tile[j][(tx * 4) ^ (((j >> 2) & 7) << 2)]) = *reinterpret_cast<const float4*>(a.in[0] + ib + (long long)q * " << SQ << "ll + p);\n";
    o << "    }\n";
    o << "    __syncthreads();\n";
    // write: thread (tx, ty) stores 4 consecutive q for rows p = ty, ty + 16, ...
    o << "    for (int j = ty; j < 64; j += 16) {\n";
    o << "      const int p = p0 + j, q = q0 + tx * 4;\n";
    o << "      if (p < " << P << " && q < " << Q << ") {\n";
    for (int l = 0; l < 4; l++) o << "        const float t_" << l << " = tile[tx * 4 + " << l << "][j ^ ((tx & 7) << 2)];\n";
    std::vector<std::string> names{"t"};
    std::vector<Access> acc(1);
    acc[0].mode = Access::GATHER;   // emit_ssa reads lane l of a gathered operand as <name>_<l>
    emit_ssa(o, k, 4, names, acc, "        ");
    for (size_t i = 0; i < k.outs.size(); i++) {
        const std::string v = "v" + std::to_string(k.outs[i].ssa);
        o << "        *reinterpret_cast<float4*>(a.out[" << i << "] + ob + (long long)p * " << ostride[pi] << "ll + q) = make_float4(" << v << "_0, " << v
          << "_1, " << v << "_2, " << v << "_3);\n";
    }
    o << "      }\n    }\n";
    o << "    __syncthreads();\n";
    o << "  }\n}\n";
    finish(k, o.str(), "adb_transpose");
    return true;
}

void gen_elw(KernelSpec& k) {
    if (!k.reds.empty()) { gen_elw_red(k); return; }
    if (gen_transpose(k)) return;
    std::vector<const Operand*> ops;
    for (auto& i : k.ins) ops.push_back(&i);
    for (auto& o : k.outs) ops.push_back(&o.dst);
    k.wide_index = needs_wide(k.n, ops);
    const char* idx_t = k.wide_index ? "long long" : "unsigned int";
    const int vec = elw_vec_impl(k);
    k.vec = vec;
    k.threads = 256;

    std::vector<Access> in_acc(k.ins.size()), out_acc(k.outs.size());
    for (size_t i = 0; i < k.ins.size(); i++) in_acc[i] = classify(k.ins[i].subs, k.ins[i].offset, vec, false);
    for (size_t i = 0; i < k.outs.size(); i++) out_acc[i] = classify(k.outs[i].dst.subs, k.outs[i].dst.offset, vec, true);

    std::ostringstream o;
    o << helpers() << "struct Args { const float* in[" << std::max<size_t>(1, k.ins.size()) << "]; float* out[" << k.outs.size()
      << "]; long long n; };\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
    o << "  const " << idx_t << " nv = (" << idx_t << ")(a.n / " << vec << ");\n";
    o << "  for (" << idx_t << " j = blockIdx.x * 256u + threadIdx.x; j < nv; j += (" << idx_t << ")gridDim.x * 256u) {\n";
    o << "      const " << idx_t << " i = j * " << vec << ";\n";
    // offsets, shared between operands with the same digits
    std::vector<std::pair<std::vector<Sub>, std::string>> seen;
    auto offset_of = [&](const std::vector<Sub>& subs) {
        for (auto& s : seen)
            if (s.first == subs) return s.second;
        std::ostringstream pre;
        std::string tag = std::to_string(seen.size());
        std::string e = offset_expr(subs, "i", pre, tag, idx_t);
        o << pre.str();
        std::string var = "o" + tag;
        o << "      const " << idx_t << " " << var << " = " << e << ";\n";
        seen.push_back({subs, var});
        return var;
    };
    std::vector<std::string> in_off(k.ins.size()), out_off(k.outs.size());
    for (size_t i = 0; i < k.ins.size(); i++) in_off[i] = offset_of(k.ins[i].subs);
    for (size_t i = 0; i < k.outs.size(); i++) out_off[i] = offset_of(k.outs[i].dst.subs);
    std::vector<std::string> names;
    emit_loads(o, k, vec, in_acc, in_off, names, "      ");
    emit_ssa(o, k, vec, names, in_acc, "      ");
    for (size_t i = 0; i < k.outs.size(); i++) {
        std::string p = "a.out[" + std::to_string(i) + "]";
        std::string v = "v" + std::to_string(k.outs[i].ssa);
        if (vec == 1)
            o << "      " << p << "[" << out_off[i] << "] = " << v << "_0;\n";
        else if (out_acc[i].mode == Access::VEC4)
            o << "      *reinterpret_cast<float4*>(" << p << " + (" << out_off[i] << ")) = make_float4(" << v << "_0, " << v
              << "_1, " << v << "_2, " << v << "_3);\n";
        else
            for (int l = 0; l < 4; l++)
                o << "      " << p << "[(" << out_off[i] << ") + " << l * out_acc[i].lane_stride << "] = " << v << "_" << l << ";\n";
    }
    o << "  }\n}\n";
    finish(k, o.str(), "adb_elw");
}

// Element-wise pass that also sums some of its values.  The flat index space is walked as [P, Q]
// (i = p * Q + q): a block covers 8 rows (one per warp) by 32 * vec columns per iteration and a chunk of rows
// (blockIdx.y) in total.  Sums over q (axis 0): warp-shuffle tree, one partial per row and column tile.  Sums over
// p (axis 1): per-thread accumulators over the rows of the chunk, combined across the 8 warps in shared memory
// in a fixed order, one partial per column and row chunk.  The partials are added by a small reduce step.
void gen_elw_red(KernelSpec& k) {
    std::vector<const Operand*> ops;
    for (auto& i : k.ins) ops.push_back(&i);
    for (auto& o : k.outs) ops.push_back(&o.dst);
    k.wide_index = needs_wide(k.n, ops);
    const char* idx_t = k.wide_index ? "long long" : "unsigned int";
    const int vec = elw_vec_impl(k);
    k.vec = vec;
    k.threads = 256;
    const int64_t P = k.p2, Q = k.q2;
    const int64_t W = 32 * vec;
    const int64_t tiles_q = (Q + W - 1) / W;

    std::vector<Access> in_acc(k.ins.size()), out_acc(k.outs.size());
    for (size_t i = 0; i < k.ins.size(); i++) in_acc[i] = classify(k.ins[i].subs, k.ins[i].offset, vec, false);
    for (size_t i = 0; i < k.outs.size(); i++) out_acc[i] = classify(k.outs[i].dst.subs, k.outs[i].dst.offset, vec, true);
    bool any_col = false;
    for (auto& r : k.reds) any_col = any_col || r.axis == 1;

    std::ostringstream o;
    o << helpers() << "struct Args { const float* in[" << std::max<size_t>(1, k.ins.size()) << "]; float* out["
      << k.outs.size() + k.reds.size() << "]; long long n; };\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
    if (any_col) o << "  __shared__ float sm[8][" << W << "];\n";
    o << "  const unsigned int lane = threadIdx.x & 31u, wrp = threadIdx.x >> 5;\n";
    o << "  const " << idx_t << " c = ((" << idx_t << ")blockIdx.x * 32u + lane) * " << vec << "u;\n";
    o << "  const bool cok = c < " << Q << ";\n";
    o << "  const " << idx_t << " p_beg = (" << idx_t << ")blockIdx.y * " << k.row_chunk << ";\n";
    o << "  const " << idx_t << " p_end = p_beg + " << k.row_chunk << " < " << P << " ? p_beg + " << k.row_chunk << " : " << P << ";\n";
    for (size_t r = 0; r < k.reds.size(); r++)
        if (k.reds[r].axis == 1)
            for (int l = 0; l < vec; l++) o << "  float ca" << r << "_" << l << " = 0.0f;\n";
    o << "  for (" << idx_t << " pb = p_beg; pb < p_end; pb += 8) {\n";
    o << "    const " << idx_t << " p = pb + wrp;\n";
    for (size_t r = 0; r < k.reds.size(); r++)
        if (k.reds[r].axis == 0) o << "    float rs" << r << " = 0.0f;\n";
    o << "    if (cok && p < p_end) {\n";
    o << "      const " << idx_t << " i = p * " << Q << " + c;\n";
    std::vector<std::pair<std::vector<Sub>, std::string>> seen;
    auto offset_of = [&](const std::vector<Sub>& subs) {
        for (auto& s : seen)
            if (s.first == subs) return s.second;
        std::ostringstream pre;
        std::string tag = std::to_string(seen.size());
        std::string e = offset_expr(subs, "i", pre, tag, idx_t);
        o << pre.str();
        std::string var = "o" + tag;
        o << "      const " << idx_t << " " << var << " = " << e << ";\n";
        seen.push_back({subs, var});
        return var;
    };
    std::vector<std::string> in_off(k.ins.size()), out_off(k.outs.size());
    for (size_t i = 0; i < k.ins.size(); i++) in_off[i] = offset_of(k.ins[i].subs);
    for (size_t i = 0; i < k.outs.size(); i++) out_off[i] = offset_of(k.outs[i].dst.subs);
    std::vector<std::string> names;
    emit_loads(o, k, vec, in_acc, in_off, names, "      ");
    emit_ssa(o, k, vec, names, in_acc, "      ");
    for (size_t i = 0; i < k.outs.size(); i++) {
        std::string p = "a.out[" + std::to_string(i) + "]";
        std::string v = "v" + std::to_string(k.outs[i].ssa);
        if (vec == 1)
            o << "      " << p << "[" << out_off[i] << "] = " << v << "_0;\n";
        else if (out_acc[i].mode == Access::VEC4)
            o << "      *reinterpret_cast<float4*>(" << p << " + (" << out_off[i] << ")) = make_float4(" << v << "_0, " << v
              << "_1, " << v << "_2, " << v << "_3);\n";
        else
            for (int l = 0; l < 4; l++)
                o << "      " << p << "[(" << out_off[i] << ") + " << l * out_acc[i].lane_stride << "] = " << v << "_" << l << ";\n";
    }
    for (size_t r = 0; r < k.reds.size(); r++) {
        std::string v = "v" + std::to_string(k.reds[r].ssa);
        if (k.reds[r].axis == 1) {
            for (int l = 0; l < vec; l++) o << "      ca" << r << "_" << l << " = __fadd_rn(ca" << r << "_" << l << ", " << v << "_" << l << ");\n";
        } else if (vec == 4) {
            o << "      rs" << r << " = __fadd_rn(__fadd_rn(" << v << "_0, " << v << "_1), __fadd_rn(" << v << "_2, " << v << "_3));\n";
        } else {
            o << "      rs" << r << " = " << v << "_0;\n";
        }
    }
    o << "    }\n";
    for (size_t r = 0; r < k.reds.size(); r++) {
        if (k.reds[r].axis != 0) continue;
        std::string q = "a.out[" + std::to_string(k.outs.size() + r) + "]";
        o << "    for (int s = 16; s > 0; s >>= 1) rs" << r << " = __fadd_rn(rs" << r << ", __shfl_xor_sync(0xffffffffu, rs" << r << ", s));\n";
        o << "    if (lane == 0 && p < p_end) " << q << "[(size_t)p * " << tiles_q << " + blockIdx.x] = rs" << r << ";\n";
    }
    o << "  }\n";
    for (size_t r = 0; r < k.reds.size(); r++) {
        if (k.reds[r].axis != 1) continue;
        std::string q = "a.out[" + std::to_string(k.outs.size() + r) + "]";
        for (int l = 0; l < vec; l++) o << "  sm[wrp][lane * " << vec << " + " << l << "] = ca" << r << "_" << l << ";\n";
        o << "  __syncthreads();\n";
        o << "  if (wrp == 0 && cok) {\n";
        for (int l = 0; l < vec; l++) {
            o << "    float t" << l << " = sm[0][lane * " << vec << " + " << l << "];\n";
            o << "    for (int w = 1; w < 8; w++) t" << l << " = __fadd_rn(t" << l << ", sm[w][lane * " << vec << " + " << l << "]);\n";
        }
        o << "    float* dst = " << q << " + (size_t)blockIdx.y * " << Q << " + c;\n";
        if (vec == 4) o << "    *reinterpret_cast<float4*>(dst) = make_float4(t0, t1, t2, t3);\n";
        else o << "    dst[0] = t0;\n";
        o << "  }\n";
        o << "  __syncthreads();\n";
    }
    o << "}\n";
    finish(k, o.str(), "adb_elwsum");
}

// Row reductions and the element-wise work that depends on them in one kernel: one block (rows longer than 2048
// elements) or one warp (shorter rows) walks one row of the [P, Q] space at a time.  Phase k loops over the row, reduces its value across the block (warp shuffles, then
// eight partials in shared memory combined in a fixed order) and leaves the result in a register every thread
// holds; later phases and the final store loop read the row again (it was just read by the same block, so it comes
// from L1 / L2, not from HBM) and use those registers.
int64_t footprint(const Operand& o);

void gen_rows(KernelSpec& k) {
    std::vector<const Operand*> ops;
    for (auto& i : k.ins) ops.push_back(&i);
    for (auto& o : k.outs) ops.push_back(&o.dst);
    k.wide_index = needs_wide(k.n, ops);
    const char* idx_t = k.wide_index ? "long long" : "unsigned int";
    const int64_t P = k.p2, Q = k.q2;
    int vec = 4;
    if (Q % 4) vec = 1;
    for (auto& i : k.ins)
        if (!lanes_ok(i.subs)) vec = 1;
    for (auto& o : k.outs)
        if (!lanes_ok(o.dst.subs) || o.dst.subs.empty() || o.dst.subs.back().stride == 0) vec = 1;
    k.vec = vec;
    // threads per row: a warp for short rows (eight rows per block, shuffles only, eight times as many bytes in
    // flight per SM), the whole block for long ones
    const int TPR = Q <= 2048 ? 32 : 256;
    const int RPB = 256 / TPR;
    k.threads = TPR;
    std::vector<Access> in_acc(k.ins.size()), out_acc(k.outs.size());
    for (size_t i = 0; i < k.ins.size(); i++) in_acc[i] = classify(k.ins[i].subs, k.ins[i].offset, vec, false);
    for (size_t i = 0; i < k.outs.size(); i++) out_acc[i] = classify(k.outs[i].dst.subs, k.outs[i].dst.offset, vec, true);

    // which SSA values (and loads) a set of roots needs
    auto slice = [&](const std::vector<int>& roots, std::vector<char>& need, std::vector<char>& need_in) {
        need.assign(k.ssa.size(), 0);
        need_in.assign(k.ins.size(), 0);
        for (int r : roots) need[size_t(r)] = 1;
        for (size_t i = k.ssa.size(); i-- > 0;) {
            if (!need[i]) continue;
            const Ssa& s = k.ssa[i];
            if (s.kind == Ssa::OP) {
                need[size_t(s.a)] = 1;
                if (s.b >= 0) need[size_t(s.b)] = 1;
            } else if (s.kind == Ssa::LOAD) need_in[size_t(s.operand)] = 1;
        }
    };

    // Operands that cover the whole [P, Q] space are read by every phase; when a thread's share of a row is small
    // they are loaded into registers once per row (fully unrolled loops) instead of coming back from L1 / L2.
    const int64_t NIT = (Q + int64_t(TPR) * vec - 1) / (int64_t(TPR) * vec);   // loop trips per row and thread
    std::vector<char> cached(k.ins.size(), 0);
    {
        int64_t n_full = 0;
        for (size_t i = 0; i < k.ins.size(); i++)
            if ((in_acc[i].mode == Access::VEC4 || (vec == 1 && !k.ins[i].subs.empty() && k.ins[i].subs.back().stride == 1)) &&
                footprint(k.ins[i]) == P * Q)
                n_full++;
        if (n_full > 0 && NIT * vec * n_full <= 64 && NIT <= 16)
            for (size_t i = 0; i < k.ins.size(); i++)
                cached[i] = (in_acc[i].mode == Access::VEC4 || (vec == 1 && !k.ins[i].subs.empty() && k.ins[i].subs.back().stride == 1)) &&
                            footprint(k.ins[i]) == P * Q;
    }
    bool any_cached = false;
    for (char c : cached) any_cached = any_cached || c;

    std::ostringstream o;
    o << helpers() << "struct Args { const float* in[" << std::max<size_t>(1, k.ins.size()) << "]; float* out["
      << k.outs.size() + k.phases.size() << "]; long long n; };\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
    if (TPR == 256) o << "  __shared__ float sm[8];\n";
    o << "  const unsigned int lane = threadIdx.x & 31u, wrp = threadIdx.x >> 5;\n";
    if (TPR == 256)
        o << "  for (" << idx_t << " p = blockIdx.x; p < " << P << "; p += gridDim.x) {\n";
    else
        o << "  for (" << idx_t << " p = (" << idx_t << ")blockIdx.x * " << RPB << "u + wrp; p < " << P << "; p += ("
          << idx_t << ")gridDim.x * " << RPB << "u) {\n";
    if (any_cached) {
        for (size_t i = 0; i < k.ins.size(); i++)
            if (cached[i]) o << "    " << (vec == 4 ? "float4" : "float") << " c" << i << "[" << NIT << "];\n";
        o << "#pragma unroll\n    for (int t = 0; t < " << NIT << "; t++) {\n";
        o << "      const " << idx_t << " q = (" << (TPR == 256 ? "threadIdx.x" : "lane") << " + (unsigned int)t * " << TPR << "u) * " << vec << "u;\n";
        o << "      if (q >= " << Q << ") continue;\n";
        o << "      const " << idx_t << " i = p * " << Q << " + q;\n";
        for (size_t i = 0; i < k.ins.size(); i++) {
            if (!cached[i]) continue;
            std::ostringstream pre;
            std::string e = offset_expr(k.ins[i].subs, "i", pre, "c" + std::to_string(i), idx_t);
            o << pre.str();
            if (vec == 4) o << "      c" << i << "[t] = *reinterpret_cast<const float4*>(a.in[" << i << "] + (" << e << "));\n";
            else o << "      c" << i << "[t] = a.in[" << i << "][" << e << "];\n";
        }
        o << "    }\n";
    }
    auto body_prefix = [&](const std::vector<char>& need_in, std::vector<std::string>& in_off, std::vector<std::string>& out_off,
                           bool with_outs) {
        if (any_cached) {
            o << "#pragma unroll\n    for (int t = 0; t < " << NIT << "; t++) {\n";
            o << "      const " << idx_t << " q = (" << (TPR == 256 ? "threadIdx.x" : "lane") << " + (unsigned int)t * " << TPR << "u) * " << vec << "u;\n";
            o << "      if (q >= " << Q << ") continue;\n";
        } else {
            o << "    for (" << idx_t << " q = " << (TPR == 256 ? "threadIdx.x" : "lane") << " * " << vec << "u; q < " << Q << "; q += "
              << TPR * vec << "u) {\n";
        }
        o << "      const " << idx_t << " i = p * " << Q << " + q;\n";
        std::vector<std::pair<std::vector<Sub>, std::string>> seen;
        auto offset_of = [&](const std::vector<Sub>& subs) {
            for (auto& s : seen)
                if (s.first == subs) return s.second;
            std::ostringstream pre;
            std::string tag = std::to_string(seen.size());
            std::string e = offset_expr(subs, "i", pre, tag, idx_t);
            o << pre.str();
            std::string var = "o" + tag;
            o << "      const " << idx_t << " " << var << " = " << e << ";\n";
            seen.push_back({subs, var});
            return var;
        };
        in_off.assign(k.ins.size(), "0");
        for (size_t i = 0; i < k.ins.size(); i++)
            if (need_in[i] && !cached[i]) in_off[i] = offset_of(k.ins[i].subs);
        out_off.assign(k.outs.size(), "0");
        if (with_outs)
            for (size_t i = 0; i < k.outs.size(); i++) out_off[i] = offset_of(k.outs[i].dst.subs);
    };
    for (size_t ph = 0; ph < k.phases.size(); ph++) {
        const auto& phs = k.phases[ph];
        const char* ident = phs.red_op ? "__int_as_float(0xff800000)" : "0.0f";
        auto comb = [&](const std::string& x, const std::string& y) {
            return (phs.red_op ? "fmaxf(" : "__fadd_rn(") + x + ", " + y + ")";
        };
        std::vector<char> need, need_in;
        slice({phs.ssa}, need, need_in);
        o << "    float red" << ph << ";\n    {\n";
        for (int l = 0; l < vec; l++) o << "    float acc" << l << " = " << ident << ";\n";
        std::vector<std::string> in_off, out_off, names;
        body_prefix(need_in, in_off, out_off, false);
        emit_loads(o, k, vec, in_acc, in_off, names, "      ", &need_in, &cached);
        emit_ssa(o, k, vec, names, in_acc, "      ", &need);
        for (int l = 0; l < vec; l++)
            o << "      acc" << l << " = " << comb("acc" + std::to_string(l), "v" + std::to_string(phs.ssa) + "_" + std::to_string(l)) << ";\n";
        o << "    }\n";
        if (vec == 4) o << "    float s = " << comb(comb("acc0", "acc1"), comb("acc2", "acc3")) << ";\n";
        else o << "    float s = acc0;\n";
        o << "    for (int m = 16; m > 0; m >>= 1) s = " << comb("s", "__shfl_xor_sync(0xffffffffu, s, m)") << ";\n";
        if (TPR == 256) {
            o << "    __syncthreads();\n";   // the previous phase's readers of sm are done
            o << "    if (lane == 0u) sm[wrp] = s;\n";
            o << "    __syncthreads();\n";
            o << "    s = sm[0];\n";
            o << "    for (int w = 1; w < 8; w++) s = " << comb("s", "sm[w]") << ";\n";
        }
        o << "    red" << ph << " = s;\n";
        o << "    if (" << (TPR == 256 ? "threadIdx.x" : "lane") << " == 0u) a.out[" << k.outs.size() + ph << "][p] = s;\n";
        o << "    }\n";
    }
    if (!k.outs.empty()) {
        std::vector<int> roots;
        for (auto& out : k.outs) roots.push_back(out.ssa);
        std::vector<char> need, need_in;
        slice(roots, need, need_in);
        std::vector<std::string> in_off, out_off, names;
        body_prefix(need_in, in_off, out_off, true);
        emit_loads(o, k, vec, in_acc, in_off, names, "      ", &need_in, &cached);
        emit_ssa(o, k, vec, names, in_acc, "      ", &need);
        for (size_t i = 0; i < k.outs.size(); i++) {
            std::string pp = "a.out[" + std::to_string(i) + "]";
            std::string v = "v" + std::to_string(k.outs[i].ssa);
            if (vec == 1)
                o << "      " << pp << "[" << out_off[i] << "] = " << v << "_0;\n";
            else if (out_acc[i].mode == Access::VEC4)
                o << "      *reinterpret_cast<float4*>(" << pp << " + (" << out_off[i] << ")) = make_float4(" << v << "_0, " << v
                  << "_1, " << v << "_2, " << v << "_3);\n";
            else
                for (int l = 0; l < 4; l++)
                    o << "      " << pp << "[(" << out_off[i] << ") + " << l * out_acc[i].lane_stride << "] = " << v << "_" << l << ";\n";
        }
        o << "    }\n";
    }
    o << "  }\n}\n";
    finish(k, o.str(), "adb_rows");
}

// -------------------------------------------------------------------------------- reduce
int64_t pow2_floor(int64_t v) {
    int64_t p = 1;
    while (p * 2 <= v) p *= 2;
    return p;
}

int64_t footprint(const Operand& o) {
    int64_t n = 1;
    for (auto& s : o.subs) if (s.stride) n *= s.size;
    for (auto& s : o.xsubs) if (s.stride) n *= s.size;
    return n;
}

void gen_reduce(KernelSpec& k) {
    std::vector<const Operand*> ops;
    for (auto& i : k.ins) ops.push_back(&i);
    ops.push_back(&k.outs[0].dst);
    k.wide_index = needs_wide(std::max(k.n, k.r) * std::max<int64_t>(1, k.split), ops) || k.n * k.r >= (int64_t(1) << 31);
    const char* idx_t = k.wide_index ? "long long" : "unsigned int";
    const int64_t R = k.r, S = k.split;
    const int64_t chunk = k.chunk > 0 ? k.chunk : (R + S - 1) / S;  // summed elements per partial
    std::ostringstream o;
    // how two partial results combine and what an empty partial is: sum (round-to-nearest adds, 0) or maximum
    // (fmaxf: a NaN operand is ignored, -inf)
    o << helpers()
      << (k.red_op ? "#define ADB_IDENT __int_as_float(0xff800000)\n"
                     "__device__ __forceinline__ float adb_comb(float a, float b) { return fmaxf(a, b); }\n"
                   : "#define ADB_IDENT 0.0f\n"
                     "__device__ __forceinline__ float adb_comb(float a, float b) { return __fadd_rn(a, b); }\n")
      << "struct Args { const float* in[" << std::max<size_t>(1, k.ins.size()) << "]; float* out[1]; long long n; };\n";

    if (k.mode == 0) {
        // lanes along the summed axis: TPR threads cooperate on one row, 256/TPR rows per block
        int vec = k.vec;
        const int TPR = k.threads;  // threads per row (power of two <= 256)
        const int RPB = 256 / TPR;
        std::vector<Access> acc(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) acc[i] = classify(k.ins[i].subs, k.ins[i].offset, vec, false);
        if (vec == 4)
            for (size_t i = 0; i < k.ins.size(); i++)
                if (acc[i].mode == Access::VEC4)
                    for (auto& s : k.ins[i].xsubs)
                        if (s.stride % 4) { acc[i].mode = Access::GATHER; acc[i].lane_stride = 1; }
        o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
        if (TPR > 32) o << "  __shared__ float sm[8];\n";
        o << "  const unsigned int lane = threadIdx.x % " << TPR << "u, rib = threadIdx.x / " << TPR << "u;\n";
        o << "  const " << idx_t << " V = (" << idx_t << ")a.n;\n";
        o << "  const " << idx_t << " ybeg = (" << idx_t << ")blockIdx.y * " << chunk << ";\n";
        o << "  const " << idx_t << " yend = ybeg + " << chunk << " < " << R << " ? ybeg + " << chunk << " : " << R << ";\n";
        o << "  for (" << idx_t << " xb = (" << idx_t << ")blockIdx.x * " << RPB << "u; xb < V; xb += (" << idx_t << ")gridDim.x * " << RPB << "u) {\n";
        o << "    const " << idx_t << " x = xb + rib;\n";
        o << "    const bool valid = x < V;\n";
        o << "    float acc0 = ADB_IDENT, acc1 = ADB_IDENT, acc2 = ADB_IDENT, acc3 = ADB_IDENT;\n";
        o << "    if (valid) {\n";
        std::vector<std::pair<std::vector<Sub>, std::string>> seenx, seeny;
        std::vector<std::string> xo(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) {
            bool found = false;
            for (auto& s : seenx)
                if (s.first == k.ins[i].xsubs) { xo[i] = s.second; found = true; }
            if (found) continue;
            std::ostringstream pre;
            std::string tag = "x" + std::to_string(seenx.size());
            std::string e = offset_expr(k.ins[i].xsubs, "x", pre, tag, idx_t);
            o << pre.str();
            o << "      const " << idx_t << " o" << tag << " = " << e << ";\n";
            xo[i] = "o" + tag;
            seenx.push_back({k.ins[i].xsubs, xo[i]});
        }
        o << "#pragma unroll 4\n";
        o << "      for (" << idx_t << " y = ybeg + lane * " << vec << "u; y < yend; y += " << TPR * vec << "u) {\n";
        std::vector<std::string> off(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) {
            std::string yo;
            for (auto& s : seeny)
                if (s.first == k.ins[i].subs) yo = s.second;
            if (yo.empty()) {
                std::ostringstream pre;
                std::string tag = "y" + std::to_string(seeny.size());
                std::string e = offset_expr(k.ins[i].subs, "y", pre, tag, idx_t);
                o << pre.str();
                o << "      const " << idx_t << " o" << tag << " = " << e << ";\n";
                yo = "o" + tag;
                seeny.push_back({k.ins[i].subs, yo});
            }
            off[i] = xo[i] + " + " + yo;
        }
        std::vector<std::string> names;
        emit_loads(o, k, vec, acc, off, names, "        ");
        emit_ssa(o, k, vec, names, acc, "        ");
        for (int l = 0; l < vec; l++)
            o << "        acc" << l << " = adb_comb(acc" << l << ", v" << k.outs[0].ssa << "_" << l << ");\n";
        o << "      }\n    }\n";
        o << "    float s = adb_comb(adb_comb(acc0, acc1), adb_comb(acc2, acc3));\n";
        for (int m = std::min(TPR, 32) / 2; m >= 1; m /= 2)
            o << "    s = adb_comb(s, __shfl_xor_sync(0xffffffffu, s, " << m << "));\n";
        if (TPR > 32) {
            const int wpr = TPR / 32;
            o << "    __syncthreads();\n";
            o << "    if ((threadIdx.x & 31u) == 0u) sm[threadIdx.x >> 5] = s;\n";
            o << "    __syncthreads();\n";
            o << "    if (lane == 0u) { s = sm[rib * " << wpr << "u];";
            for (int w = 1; w < wpr; w++) o << " s = adb_comb(s, sm[rib * " << wpr << "u + " << w << "u]);";
            o << " }\n";
        }
        {
            std::ostringstream pre;
            std::string e = offset_expr(k.outs[0].dst.xsubs, "x", pre, "out", idx_t);
            o << "    if (valid && lane == 0u) {\n" << pre.str();
            o << "      a.out[0][(" << e << ")" << (S > 1 ? " * " + std::to_string(S) + " + blockIdx.y" : "") << "] = s;\n    }\n";
        }
        o << "  }\n}\n";
    } else {
        // lanes along the kept axis (a column sum): 32 x-lanes by 8 y-groups per block, each thread
        // walks down its column(s); the 8 partials meet in shared memory
        int vec = k.vec;
        std::vector<Access> acc(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) {
            acc[i] = classify(k.ins[i].xsubs, k.ins[i].offset, vec, false);
            if (vec == 4 && acc[i].mode == Access::VEC4)
                for (auto& s : k.ins[i].subs)
                    if (s.stride % 4) { acc[i].mode = Access::GATHER; acc[i].lane_stride = 1; }
        }
        o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
        o << "  __shared__ float sm[8][" << 32 * vec << " + 1];\n";
        o << "  const unsigned int tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;\n";
        o << "  const " << idx_t << " V = (" << idx_t << ")a.n;\n";
        o << "  const " << idx_t << " x = ((" << idx_t << ")blockIdx.x * 32u + tx) * " << vec << "u;\n";
        o << "  const " << idx_t << " ybeg = (" << idx_t << ")blockIdx.y * " << chunk << ";\n";
        o << "  const " << idx_t << " yend = ybeg + " << chunk << " < " << R << " ? ybeg + " << chunk << " : " << R << ";\n";
        o << "  float acc0 = ADB_IDENT, acc1 = ADB_IDENT, acc2 = ADB_IDENT, acc3 = ADB_IDENT;\n";
        o << "  if (x < V) {\n";
        std::vector<std::pair<std::vector<Sub>, std::string>> seenx, seeny;
        std::vector<std::string> xo(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) {
            bool found = false;
            for (auto& s : seenx)
                if (s.first == k.ins[i].xsubs) { xo[i] = s.second; found = true; }
            if (found) continue;
            std::ostringstream pre;
            std::string tag = "x" + std::to_string(seenx.size());
            std::string e = offset_expr(k.ins[i].xsubs, "x", pre, tag, idx_t);
            o << pre.str();
            o << "      const " << idx_t << " o" << tag << " = " << e << ";\n";
            xo[i] = "o" + tag;
            seenx.push_back({k.ins[i].xsubs, xo[i]});
        }
        o << "#pragma unroll 4\n";
        o << "    for (" << idx_t << " y = ybeg + ty; y < yend; y += 8u) {\n";
        std::vector<std::string> off(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) {
            std::string yo;
            for (auto& s : seeny)
                if (s.first == k.ins[i].subs) yo = s.second;
            if (yo.empty()) {
                std::ostringstream pre;
                std::string tag = "y" + std::to_string(seeny.size());
                std::string e = offset_expr(k.ins[i].subs, "y", pre, tag, idx_t);
                o << pre.str();
                o << "      const " << idx_t << " o" << tag << " = " << e << ";\n";
                yo = "o" + tag;
                seeny.push_back({k.ins[i].subs, yo});
            }
            off[i] = xo[i] + " + " + yo;
        }
        std::vector<std::string> names;
        emit_loads(o, k, vec, acc, off, names, "      ");
        emit_ssa(o, k, vec, names, acc, "      ");
        for (int l = 0; l < vec; l++)
            o << "      acc" << l << " = adb_comb(acc" << l << ", v" << k.outs[0].ssa << "_" << l << ");\n";
        o << "    }\n  }\n";
        for (int l = 0; l < vec; l++) o << "  sm[ty][tx * " << vec << " + " << l << "] = acc" << l << ";\n";
        o << "  __syncthreads();\n";
        o << "  if (ty == 0u && x < V) {\n";
        {
            std::ostringstream pre;
            std::string e = offset_expr(k.outs[0].dst.xsubs, "x", pre, "out", idx_t);
            o << pre.str();
            o << "    const " << idx_t << " oo = (" << e << ")" << (S > 1 ? " + (" + std::string(idx_t) + ")blockIdx.y * V" : "") << ";\n";
        }
        int64_t out_stride = k.outs[0].dst.xsubs.empty() ? 0 : k.outs[0].dst.xsubs.back().stride;
        for (int l = 0; l < vec; l++) {
            o << "    { float s = sm[0][tx * " << vec << " + " << l << "];";
            for (int t = 1; t < 8; t++) o << " s = adb_comb(s, sm[" << t << "][tx * " << vec << " + " << l << "]);";
            o << " a.out[0][oo + " << l * out_stride << "] = s; }\n";
        }
        o << "  }\n}\n";
    }
    finish(k, o.str(), k.red_op ? (k.mode ? "adb_colmax" : "adb_rowmax") : (k.mode ? "adb_colsum" : "adb_rowsum"));
}

}  // namespace

// Chooses the thread mapping of a reduce kernel (row / column lanes, vector width, threads per row,
// split factor).  Called while lowering because a split needs a scratch buffer and a second pass.
void plan_reduce(KernelSpec& k, int sm_count) {
    const int64_t V = k.n, R = k.r;
    // the operand that moves the most bytes decides which axis the lanes follow
    const Operand* big = nullptr;
    int64_t best = -1;
    for (auto& in : k.ins) {
        int64_t f = footprint(in);
        if (f > best) { best = f; big = &in; }
    }
    k.mode = 0;
    if (big) {
        bool y_unit = !big->subs.empty() && big->subs.back().stride == 1;
        bool x_unit = !big->xsubs.empty() && big->xsubs.back().stride == 1;
        if (!y_unit && x_unit) k.mode = 1;
    }
    if (k.mode == 0) {
        int vec = R % 4 == 0 ? 4 : 1;
        for (auto& in : k.ins)
            if (!lanes_ok(in.subs)) vec = 1;
        k.vec = vec;
        int64_t per_row = std::max<int64_t>(1, R / vec);
        // up to a warp per row needs no shared memory and no block barrier; only very long rows get a block
        int64_t tpr = per_row >= 4096 ? 256 : std::min<int64_t>(32, pow2_floor(std::max<int64_t>(1, per_row / 2)));
        k.threads = int(tpr);
        int64_t blocks = (V + (256 / tpr) - 1) / (256 / tpr);
        k.split = 1;
        // few long rows: split each row so that every SM has work
        if (blocks < sm_count && R >= 16384) {
            int64_t want = (2 * sm_count + blocks - 1) / blocks;
            int64_t max_split = std::max<int64_t>(1, R / 4096);
            k.split = std::max<int64_t>(1, std::min(want, max_split));
            // keep chunks a multiple of the vector width
            int64_t chunk = (R + k.split - 1) / k.split;
            chunk = (chunk + 255) / 256 * 256;
            k.split = (R + chunk - 1) / chunk;
        }
        k.chunk = (R + k.split - 1) / k.split;
        if (k.split > 1) k.chunk = (k.chunk + 255) / 256 * 256;
    } else {
        int vec = V % 4 == 0 ? 4 : 1;
        for (auto& in : k.ins)
            if (!lanes_ok(in.xsubs)) vec = 1;
        if (!lanes_ok(k.outs[0].dst.xsubs)) vec = 1;
        k.vec = vec;
        k.threads = 256;
        int64_t bx = (V + 32 * vec - 1) / (32 * vec);
        k.split = 1;
        if (bx < 2 * sm_count && R >= 512) {
            int64_t want = (2 * sm_count + bx - 1) / bx;
            k.split = std::max<int64_t>(1, std::min(want, R / 256));
        }
        k.chunk = (R + k.split - 1) / k.split;
        k.split = (R + k.chunk - 1) / k.chunk;
    }
}

int elw_vec(const KernelSpec& k) { return elw_vec_impl(k); }

bool elw_uses_tile(const KernelSpec& k) {
    KernelSpec probe = k;
    return gen_transpose(probe);
}

namespace {

void replace_all(std::string& s, const std::string& from, const std::string& to) {
    for (size_t p = 0; (p = s.find(from, p)) != std::string::npos; p += to.size()) s.replace(p, from.size(), to);
}

// One launch for several independent kernels: every member's source becomes a device function that takes its block
// index and block count as arguments, and the entry point hands each range of blockIdx.x to one member.  The
// argument block is the members' argument blocks one after another, then the first block index of each member.
void gen_group(Plan& plan, KernelSpec& g) {
    static const std::string sig_head = "extern \"C\" __global__ void __launch_bounds__(256) ";
    static const std::string sig_tail = "(const __grid_constant__ Args a) {";
    std::ostringstream o;
    o << helpers();
    const std::string help = helpers();
    for (size_t m = 0; m < g.members.size(); m++) {
        const KernelSpec& k = plan.kernels[size_t(g.members[m])];
        const std::string tag = std::to_string(m);
        std::string src = k.source;
        if (!help.empty() && src.compare(0, help.size(), help) == 0) src.erase(0, help.size());
        const size_t h = src.find(sig_head), t = src.find(sig_tail);
        if (h == std::string::npos || t == std::string::npos || t < h) { g.source.clear(); g.entry.clear(); return; }
        src.replace(h, t + sig_tail.size() - h,
                    "__device__ void adb_member" + tag + "(const Args" + tag + "& a, const unsigned int adb_bid, const unsigned int adb_nb) {");
        replace_all(src, "struct Args ", "struct Args" + tag + " ");
        replace_all(src, "ADB_IDENT", "ADB_IDENT" + tag);
        replace_all(src, "adb_comb", "adb_comb" + tag);
        replace_all(src, "blockIdx.x", "adb_bid");
        replace_all(src, "gridDim.x", "adb_nb");
        replace_all(src, "blockIdx.y", "0u");
        replace_all(src, "gridDim.y", "1u");
        o << src;
    }
    const size_t n = g.members.size();
    o << "struct Args {";
    for (size_t m = 0; m < n; m++) o << " Args" << m << " a" << m << ";";
    o << " unsigned int start[" << n + 1 << "]; };\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) @ENTRY@(const __grid_constant__ Args a) {\n";
    o << "  const unsigned int b = blockIdx.x;\n";
    for (size_t m = 0; m < n; m++)
        o << "  " << (m ? "else " : "") << "if (b < a.start[" << m + 1 << "]) adb_member" << m << "(a.a" << m << ", b - a.start[" << m
          << "], a.start[" << m + 1 << "] - a.start[" << m << "]);\n";
    o << "}\n";
    finish(g, o.str(), "adb_group");
}

}  // namespace

void generate_kernels(Plan& plan) {
    g_exact_div = plan.exact_div;
    for (auto& k : plan.kernels) {
        if (!k.source.empty() || k.dead || k.type == KernelSpec::GROUP) continue;
        if (k.type == KernelSpec::ELW) gen_elw(k);
        else if (k.type == KernelSpec::ROWS) gen_rows(k);
        else gen_reduce(k);
    }
    for (auto& k : plan.kernels)
        if (k.type == KernelSpec::GROUP && k.source.empty() && !k.dead) gen_group(plan, k);
}

}  // namespace adb
