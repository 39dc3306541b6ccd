// Executes a lowered plan on the CPU, step by step, with the memory layout the GPU executor uses (one arena,
// buffers at their planned offsets, partial-sum buffers in the layout the generated kernels write).  Test
// infrastructure only: it lets the lowering and all of its fusion passes be checked numerically against the CPU
// oracle without a GPU, on thousands of programs, under the sanitizers.  The arena starts out as NaN, so a buffer
// that is read before it is written, or that shares arena space with one that is still alive, shows up in the
// results.
#pragma once
#include <cmath>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string>
#include <vector>

#include "adb_lower.hpp"

namespace adbtest {

using namespace adb;

struct PlanInterp {
    int world = 1;   // ranks simulated as identical copies (ALLREDUCE multiplies by it)
    const Plan& plan;
    std::vector<float> arena;
    bool exited = false;
    long long while_iterations = 0;

    explicit PlanInterp(const Plan& p) : plan(p) {
        arena.assign(size_t(p.arena_bytes / 4) + 64, std::numeric_limits<float>::quiet_NaN());
    }

    float* ptr(int buf, int64_t off = 0) {
        const BufferInfo& b = plan.bufs[size_t(buf)];
        if (b.external) return reinterpret_cast<float*>(uintptr_t(plan.payloads[size_t(b.payload)].addr)) + off;
        if (b.arena_off < 0) throw std::runtime_error("buffer '" + b.name + "' has no storage");
        if (b.arena_off / 4 + off + 0 > int64_t(arena.size())) throw std::runtime_error("buffer '" + b.name + "' outside the arena");
        return arena.data() + b.arena_off / 4 + off;
    }
    // offset of index r through a digit list (outermost digit takes what is left)
    static int64_t offset(const std::vector<Sub>& subs, int64_t r) {
        int64_t off = 0;
        for (size_t t = subs.size(); t-- > 1;) {
            off += (r % subs[t].size) * subs[t].stride;
            r /= subs[t].size;
        }
        if (!subs.empty()) off += r * subs[0].stride;
        return off;
    }
    static float apply(EOp op, float a, float b) {
        switch (op) {
        case E_ADD: return a + b;
        case E_MUL: return a * b;
        case E_EXP2: return exp2f(a);
        case E_LOG2: return log2f(a);
        case E_SIN: return sinf(a);
        case E_RECIP: return 1.0f / a;
        case E_SQRT: return sqrtf(fabsf(a));
        case E_EQZ: return a == 0.0f ? 1.0f : 0.0f;
        case E_GTZ: return a > 0.0f ? 1.0f : 0.0f;
        case E_LTZ: return a < 0.0f ? 1.0f : 0.0f;
        }
        return 0.f;
    }
    // evaluates the SSA of `k` for one element; `in_off[i]` is the element offset of operand i
    void eval(const KernelSpec& k, const std::vector<float*>& in, const std::vector<int64_t>& in_off, const std::vector<float>& red,
              std::vector<float>& v) {
        v.resize(k.ssa.size());
        for (size_t i = 0; i < k.ssa.size(); i++) {
            const Ssa& s = k.ssa[i];
            volatile float r;   // (volatile: keep every operation a separately rounded fp32 operation)
            if (s.kind == Ssa::LOAD) r = in[size_t(s.operand)][in_off[size_t(s.operand)]];
            else if (s.kind == Ssa::CONST) r = s.c;
            else if (s.kind == Ssa::RED) r = red[size_t(s.operand)];
            else r = apply(s.op, v[size_t(s.a)], s.b >= 0 ? v[size_t(s.b)] : 0.f);
            v[i] = r;
        }
    }
    static float combine(int red_op, float a, float b) { return red_op ? fmaxf(a, b) : a + b; }
    static float identity(int red_op) { return red_op ? -std::numeric_limits<float>::infinity() : 0.f; }

    void run_kernel(const KernelSpec& k) {
        std::vector<float*> in(k.ins.size());
        for (size_t i = 0; i < k.ins.size(); i++) in[i] = ptr(k.ins[i].buf, k.ins[i].offset);
        std::vector<int64_t> in_off(k.ins.size());
        std::vector<float> v, none;
        if (k.type == KernelSpec::ELW) {
            std::vector<float*> out(k.outs.size());
            for (size_t i = 0; i < k.outs.size(); i++) out[i] = ptr(k.outs[i].dst.buf, k.outs[i].dst.offset);
            // side sums: partial buffers in the layout of the generated kernel
            const int64_t P = k.p2, Q = k.q2, W = 32 * k.vec;
            const int64_t tiles_q = k.reds.empty() ? 0 : (Q + W - 1) / W;
            std::vector<float*> rout(k.reds.size());
            for (size_t r = 0; r < k.reds.size(); r++) {
                rout[r] = ptr(k.reds[r].dst.buf, k.reds[r].dst.offset);
                const int64_t n = k.reds[r].axis == 0 ? P * tiles_q : ((P + k.row_chunk - 1) / k.row_chunk) * Q;
                for (int64_t t = 0; t < n; t++) rout[r][t] = 0.f;
            }
            // GPU threads load their 4 elements before they store them: evaluate in groups of `vec`
            const int64_t step = std::max(1, k.vec);
            std::vector<std::vector<float>> group{static_cast<size_t>(step)};
            for (int64_t i0 = 0; i0 < k.n; i0 += step) {
                const int64_t cnt = std::min<int64_t>(step, k.n - i0);
                for (int64_t g = 0; g < cnt; g++) {
                    for (size_t t = 0; t < k.ins.size(); t++) in_off[t] = offset(k.ins[t].subs, i0 + g);
                    eval(k, in, in_off, none, group[size_t(g)]);
                }
                for (int64_t g = 0; g < cnt; g++) {
                    const int64_t i = i0 + g;
                    for (size_t t = 0; t < k.outs.size(); t++) out[t][offset(k.outs[t].dst.subs, i)] = group[size_t(g)][size_t(k.outs[t].ssa)];
                    for (size_t r = 0; r < k.reds.size(); r++) {
                        const int64_t p = i / Q, q = i % Q;
                        const float x = group[size_t(g)][size_t(k.reds[r].ssa)];
                        if (k.reds[r].axis == 0) rout[r][p * tiles_q + q / W] += x;
                        else rout[r][(p / k.row_chunk) * Q + q] += x;
                    }
                }
            }
        } else if (k.type == KernelSpec::ROWS) {
            const int64_t P = k.p2, Q = k.q2;
            std::vector<float*> out(k.outs.size()), pout(k.phases.size());
            for (size_t i = 0; i < k.outs.size(); i++) out[i] = ptr(k.outs[i].dst.buf, k.outs[i].dst.offset);
            for (size_t i = 0; i < k.phases.size(); i++) pout[i] = ptr(k.phases[i].dst.buf, k.phases[i].dst.offset);
            std::vector<float> red(k.phases.size(), 0.f);
            for (int64_t p = 0; p < P; p++) {
                for (size_t ph = 0; ph < k.phases.size(); ph++) {
                    float acc = identity(k.phases[ph].red_op);
                    for (int64_t q = 0; q < Q; q++) {
                        for (size_t t = 0; t < k.ins.size(); t++) in_off[t] = offset(k.ins[t].subs, p * Q + q);
                        eval(k, in, in_off, red, v);
                        acc = combine(k.phases[ph].red_op, acc, v[size_t(k.phases[ph].ssa)]);
                    }
                    red[ph] = acc;
                    pout[ph][p] = acc;
                }
                std::vector<std::vector<float>> row{static_cast<size_t>(Q)};
                for (int64_t q = 0; q < Q && !k.outs.empty(); q++) {
                    for (size_t t = 0; t < k.ins.size(); t++) in_off[t] = offset(k.ins[t].subs, p * Q + q);
                    eval(k, in, in_off, red, row[size_t(q)]);
                }
                for (int64_t q = 0; q < Q && !k.outs.empty(); q++)
                    for (size_t t = 0; t < k.outs.size(); t++) out[t][offset(k.outs[t].dst.subs, p * Q + q)] = row[size_t(q)][size_t(k.outs[t].ssa)];
            }
        } else {
            // REDUCE: out[x] = comb_y summand(x, y), in `split` partials when the kernel is the first pass of two
            const int64_t V = k.n, R = k.r, S = std::max<int64_t>(1, k.split);
            const int64_t chunk = k.chunk > 0 ? k.chunk : (R + S - 1) / S;
            float* out = ptr(k.outs[0].dst.buf, k.outs[0].dst.offset);
            for (int64_t x = 0; x < V; x++) {
                const int64_t xo = offset(k.outs[0].dst.xsubs, x);
                for (int64_t part = 0; part < S; part++) {
                    const int64_t ybeg = part * chunk, yend = std::min(ybeg + chunk, R);
                    float acc = identity(k.red_op);
                    for (int64_t y = ybeg; y < yend; y++) {
                        for (size_t t = 0; t < k.ins.size(); t++) in_off[t] = offset(k.ins[t].xsubs, x) + offset(k.ins[t].subs, y);
                        eval(k, in, in_off, none, v);
                        acc = combine(k.red_op, acc, v[size_t(k.outs[0].ssa)]);
                    }
                    if (S == 1) out[xo] = acc;
                    else if (k.mode == 0) out[xo * S + part] = acc;
                    else out[xo + part * V] = acc;
                }
            }
        }
    }

    void run_step(const Step& s) {
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE: {
            const KernelSpec& k = plan.kernels[size_t(s.kernel)];
            // a group's members are independent of one another: any order gives the same memory
            if (k.type == KernelSpec::GROUP) for (size_t m = k.members.size(); m-- > 0;) run_kernel(plan.kernels[size_t(k.members[m])]);
            else run_kernel(k);
            break;
        }
        case Step::GEMM: {
            const auto& g = s.gemm;
          for (int64_t slice = 0; slice < g.batch; slice++) {
            const float* A = ptr(g.a, g.a_off) + slice * g.a_bs;
            const float* B = ptr(g.b, g.b_off) + slice * g.b_bs;
            float* C = ptr(g.c, g.c_off) + slice * g.c_bs;
            // C is written in place, element by element; a plan whose product lands in one of its own operands shows
            // up as a wrong result here too.  A plain product zeroes C first, as the split-k path of the GPU kernel does.
            if (!(g.epi == Step::Gemm::EPI_SCALE && g.accumulate))
                for (int64_t i = 0; i < g.M * g.N; i++) C[i] = 0.f;
            float* out = g.out >= 0 ? ptr(g.out, g.out_off) + slice * g.c_bs : nullptr;
            const float* colvec = g.colvec >= 0 ? ptr(g.colvec, g.colvec_off) : nullptr;
            for (int64_t m = 0; m < g.M; m++)
                for (int64_t n = 0; n < g.N; n++) {
                    double acc = 0;
                    for (int64_t kk = 0; kk < g.K; kk++) acc += double(A[m * g.a_rs + kk * g.a_cs]) * double(B[kk * g.b_rs + n * g.b_cs]);
                    volatile float v = float(acc);
                    if (g.epi == Step::Gemm::EPI_SCALE) {
                        for (auto& op : g.ops) v = v * op.c;
                        C[m * g.N + n] = g.accumulate ? C[m * g.N + n] + v : v;
                    } else if (g.epi == Step::Gemm::EPI_CHAIN) {
                        if (g.store_raw) C[m * g.N + n] = v;
                        volatile float saved = v;
                        for (auto& op : g.ops) {
                            if (op.operand == 4) { saved = v; continue; }
                            const float o = op.operand == 1 ? op.c : op.operand == 2 ? colvec[n] : op.operand == 3 ? float(saved) : 0.f;
                            v = apply(op.op, v, o);
                        }
                        out[m * g.N + n] = v;
                    } else
                        C[m * g.N + n] = v;
                }
          }
            break;
        }
        case Step::UPLOAD: {
            const PayloadSlot& p = plan.payloads[size_t(s.payload)];
            if (p.kind == PAYLOAD_DEVICE) throw std::runtime_error("device payloads cannot be interpreted on the host");
            std::memcpy(ptr(s.buf), reinterpret_cast<const void*>(uintptr_t(p.addr)), size_t(s.nelem) * 4);
            break;
        }
        case Step::ALLREDUCE: {
            // one rank: the sum over ranks is the value itself; several ranks that all hold the same data (the only
            // multi-rank case this interpreter runs): the sum is `world` times the value, over the whole range the
            // step covers (a bucket's alignment padding included, as on the device)
            if (world > 1) {
                float* p = ptr(s.buf, s.off);
                for (int64_t i = 0; i < s.nelem; i++) p[i] *= float(world);
            }
            break;
        }
        case Step::WHILE:
            while (!exited && *ptr(s.cond_buf, s.cond_off) != 0.0f) {
                run_block(*s.body);
                if (++while_iterations > 100000) throw std::runtime_error("loop does not terminate");
            }
            break;
        case Step::IF: {
            bool taken = false;
            for (auto& br : s.branches)
                if (*ptr(br.cond_buf, br.cond_off) == 1.0f) {
                    run_block(*br.body);
                    taken = true;
                    break;
                }
            if (!taken && s.else_body) run_block(*s.else_body);
            break;
        }
        case Step::EXIT: exited = true; break;
        }
    }
    void run_block(const StepBlock& blk) {
        for (auto& s : blk.steps) {
            if (exited) return;
            run_step(s);
        }
    }
    void run() { run_block(plan.main); }
};

}  // namespace adbtest
