// Host-side half of the backend (wire-format parser, data-parallel rewrite, lowering, CUDA source generation)
// as a stand-alone program, so that it can be built with AddressSanitizer + UndefinedBehaviorSanitizer and fed
// serialised programs from files.  No CUDA involved: the sources compiled in are plain C++.
//
//   hostcheck <flags> <world> <shard_batch> <blob files ...>
//
// flags: bit 0 no fusion, bit 1 fold small sums, bit 2 correctly rounded division, bit 3 also execute every plan on
// the CPU (plan_interp.hpp) and write the kept tensors to <blob file>.out, bit 4 keep element-wise kernels out of the
// dot products' epilogues.
// Malformed blobs must be rejected with an exception (counted), never crash.  Every plan that does come out is
// checked against the invariants below (step order, buffer lifetimes, arena placement).
#include <algorithm>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iterator>
#include <string>
#include <vector>

#include "adb_ir.hpp"
#include "adb_lower.hpp"
#include "adb_shard.hpp"
#include "plan_interp.hpp"

// Invariants every plan must satisfy, whatever passes rewrote its step list:
//   1. step positions increase in execution order (nested blocks lie between their parent and its successor);
//   2. a buffer is alive at every step that touches it (external and whole-program buffers always are);
//   3. buffers that are alive at the same time do not overlap in the arena;
//   5. a dot product never writes into one of its own operands;
//   7. a collective over several buffers finds them side by side in the arena, in order, and covers exactly their span;
//   6. the kernels that share one launch are independent: none writes a buffer that another reads or writes.
// Returns an empty string or a description of the first violation.
static void step_buffers(const adb::Plan& plan, const adb::Step& s, std::vector<int>& bufs) {
    using adb::Step;
    bufs.clear();
    switch (s.kind) {
    case Step::ELW: case Step::REDUCE:
        adb::kernel_rw(plan, s.kernel, bufs, bufs);
        break;
    case Step::GEMM:
        bufs = {s.gemm.a, s.gemm.b, s.gemm.c};
        if (s.gemm.out >= 0) bufs.push_back(s.gemm.out);
        if (s.gemm.colvec >= 0) bufs.push_back(s.gemm.colvec);
        break;
    case Step::UPLOAD: case Step::ALLREDUCE:
        bufs = {s.buf};
        bufs.insert(bufs.end(), s.more_bufs.begin(), s.more_bufs.end());
        break;
    case Step::WHILE: bufs = {s.cond_buf}; break;
    case Step::IF: for (auto& br : s.branches) bufs.push_back(br.cond_buf); break;
    default: break;
    }
}

static std::string check_block(const adb::Plan& plan, const adb::StepBlock& blk, int& last_pos) {
    std::vector<int> bufs;
    for (auto& s : blk.steps) {
        if (s.pos <= last_pos) return "step position " + std::to_string(s.pos) + " does not follow " + std::to_string(last_pos);
        last_pos = s.pos;
        if ((s.kind == adb::Step::ELW || s.kind == adb::Step::REDUCE) && plan.kernels[size_t(s.kernel)].dead)
            return "step at " + std::to_string(s.pos) + " runs a kernel that was marked dead";
        if ((s.kind == adb::Step::ELW || s.kind == adb::Step::REDUCE) && plan.kernels[size_t(s.kernel)].type == adb::KernelSpec::GROUP) {
            const auto& g = plan.kernels[size_t(s.kernel)];
            for (size_t x = 0; x < g.members.size(); x++)
                for (size_t y = 0; y < g.members.size(); y++) {
                    if (x == y) continue;
                    std::vector<int> rx, wx, ry, wy;
                    adb::kernel_rw(plan, g.members[x], rx, wx);
                    adb::kernel_rw(plan, g.members[y], ry, wy);
                    for (int w : wx) {
                        for (int r : ry) if (w == r) return "grouped launch at " + std::to_string(s.pos) + ": a member reads '" + plan.bufs[size_t(w)].name + "' that another member writes";
                        for (int r : wy) if (w == r) return "grouped launch at " + std::to_string(s.pos) + ": two members write '" + plan.bufs[size_t(w)].name + "'";
                    }
                }
        }
        if (s.kind == adb::Step::ALLREDUCE && !s.more_bufs.empty()) {
            int64_t at = plan.bufs[size_t(s.buf)].arena_off;
            std::vector<int> all = {s.buf};
            all.insert(all.end(), s.more_bufs.begin(), s.more_bufs.end());
            int64_t end = at;
            for (size_t i = 0; i < all.size(); i++) {
                const adb::BufferInfo& bi = plan.bufs[size_t(all[i])];
                if (bi.external || bi.arena_off != at) return "collective at " + std::to_string(s.pos) + ": '" + bi.name + "' is not where the bucket expects it";
                end = at + bi.numel * 4;
                at += ((bi.numel * 4 + 255) / 256) * 256;
            }
            if (s.off != 0 || s.nelem * 4 != end - plan.bufs[size_t(s.buf)].arena_off)
                return "collective at " + std::to_string(s.pos) + " does not cover its bucket";
        }
        if (s.kind == adb::Step::GEMM && (s.gemm.c == s.gemm.a || s.gemm.c == s.gemm.b || (s.gemm.out >= 0 && (s.gemm.out == s.gemm.a || s.gemm.out == s.gemm.b))))
            return "dot product at " + std::to_string(s.pos) + " writes into one of its operands";
        step_buffers(plan, s, bufs);
        for (int b : bufs) {
            if (b < 0 || size_t(b) >= plan.bufs.size()) return "step at " + std::to_string(s.pos) + " names buffer " + std::to_string(b);
            const adb::BufferInfo& bi = plan.bufs[size_t(b)];
            if (bi.external || bi.persistent) continue;
            if (!(bi.first <= s.pos && s.pos <= bi.last))
                return "buffer '" + bi.name + "' [" + std::to_string(bi.first) + "," + std::to_string(bi.last) + "] is touched at " + std::to_string(s.pos);
            if (bi.arena_off < 0 && bi.numel > 0) return "buffer '" + bi.name + "' has no place in the arena";
        }
        std::string e;
        if (s.body && !(e = check_block(plan, *s.body, last_pos)).empty()) return e;
        for (auto& br : s.branches)
            if (!(e = check_block(plan, *br.body, last_pos)).empty()) return e;
        if (s.else_body && !(e = check_block(plan, *s.else_body, last_pos)).empty()) return e;
    }
    return "";
}

// every buffer touched in `blk` (nested blocks included) and the position range of the block
static void collect(const adb::Plan& plan, const adb::StepBlock& blk, std::vector<int>& touched, int& lo, int& hi) {
    std::vector<int> bufs;
    for (auto& s : blk.steps) {
        lo = std::min(lo, s.pos);
        hi = std::max(hi, s.pos);
        step_buffers(plan, s, bufs);
        touched.insert(touched.end(), bufs.begin(), bufs.end());
        if (s.body) collect(plan, *s.body, touched, lo, hi);
        for (auto& br : s.branches) collect(plan, *br.body, touched, lo, hi);
        if (s.else_body) collect(plan, *s.else_body, touched, lo, hi);
    }
}

//   4. a buffer that a loop body shares with code outside the loop stays alive for the whole loop
static std::string check_loops(const adb::Plan& plan, const adb::StepBlock& blk) {
    for (size_t si = 0; si < blk.steps.size(); si++) {
        const adb::Step& s = blk.steps[si];
        std::string e;
        if (s.kind == adb::Step::WHILE && s.body) {
            std::vector<int> touched;
            int lo = INT_MAX, hi = -1;
            collect(plan, *s.body, touched, lo, hi);
            // positions that belong to the loop: behind the While step, in front of its successor (steps that a
            // pass moved or removed may have left earlier positions of the body in a buffer's lifetime)
            const int span_lo = s.pos, span_hi = si + 1 < blk.steps.size() ? blk.steps[si + 1].pos : INT_MAX;
            for (int b : touched) {
                const adb::BufferInfo& bi = plan.bufs[size_t(b)];
                if (bi.external || bi.persistent || hi < 0) continue;
                const bool outside = bi.first <= span_lo || bi.last >= span_hi;
                if (outside && !(bi.first <= lo && bi.last >= hi))
                    return "buffer '" + bi.name + "' [" + std::to_string(bi.first) + "," + std::to_string(bi.last) +
                           "] is shared with a loop spanning [" + std::to_string(lo) + "," + std::to_string(hi) + "] but dies inside it";
            }
            if (!(e = check_loops(plan, *s.body)).empty()) return e;
        }
        for (auto& br : s.branches)
            if (!(e = check_loops(plan, *br.body)).empty()) return e;
        if (s.else_body && !(e = check_loops(plan, *s.else_body)).empty()) return e;
    }
    return "";
}

static std::string check_plan(const adb::Plan& plan) {
    int last = -1;
    std::string e = check_block(plan, plan.main, last);
    if (!e.empty()) return e;
    if (!(e = check_loops(plan, plan.main)).empty()) return e;
    struct Live { int64_t lo, hi; long long first, last; const adb::BufferInfo* b; };
    std::vector<Live> live;
    for (auto& b : plan.bufs) {
        if (b.external || b.numel <= 0 || (!b.persistent && b.last < 0)) continue;
        if (b.arena_off < 0) return "buffer '" + b.name + "' is used but not placed";
        if (b.arena_off % 256) return "buffer '" + b.name + "' is not 256-byte aligned";
        if (b.arena_off + b.numel * 4 > plan.arena_bytes) return "buffer '" + b.name + "' ends beyond the arena";
        live.push_back({b.arena_off, b.arena_off + b.numel * 4, b.persistent ? LLONG_MIN : (long long)b.first,
                        b.persistent ? LLONG_MAX : (long long)b.last, &b});
    }
    for (size_t i = 0; i < live.size(); i++)
        for (size_t j = i + 1; j < live.size(); j++) {
            const bool time = !(live[i].last < live[j].first || live[j].last < live[i].first);
            const bool space = live[i].lo < live[j].hi && live[j].lo < live[i].hi;
            if (time && space) return "buffers '" + live[i].b->name + "' and '" + live[j].b->name + "' are alive together and overlap in the arena";
        }
    return "";
}

int main(int argc, char** argv) {
    if (argc < 5) return 2;
    const unsigned flags = unsigned(std::atoi(argv[1]));
    const int world = std::atoi(argv[2]);
    const long long batch = std::atoll(argv[3]);
    size_t kernels = 0, rejected = 0, fused = 0, executed = 0;
    for (int f = 4; f < argc; f++) {
        std::ifstream in(argv[f], std::ios::binary);
        std::vector<uint8_t> blob((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        for (int rank = 0; rank < world; rank++) {
            try {
                adb::Program prog = adb::parse_program(blob.data(), blob.size());
                adb::LowerOptions opt;
                opt.no_fusion = flags & 1;
                opt.fuse_small_sums = flags & 2;
                opt.exact_div = flags & 4;
                opt.no_dot_epilogue = flags & 16;
                opt.no_grouping = flags & 32;
                opt.no_tiny_dot = flags & 128;
                opt.bucket_collectives = world > 1 && !(flags & 64);
                opt.rank = rank;
                opt.world = world;
                if (world > 1 && batch) adb::shard_program(prog, rank, world, batch);
                adb::Plan plan;
                adb::lower_program(prog, plan, opt);
                adb::generate_kernels(plan);
                for (auto& k : plan.kernels) {
                    kernels += !k.dead;
                    fused += k.reds.size() + (k.type == adb::KernelSpec::ROWS ? 1 : 0);
                }
                std::string listing = adb::dump_plan(plan, true);
                if (listing.empty()) return 3;
                // several ranks are only interpreted when nothing is sharded (batch 0): every rank then holds the same
                // data and an all-reduce is a multiplication by the number of ranks
                if ((flags & 8) && (world == 1 || (batch == 0 && rank == 0))) {
                    adbtest::PlanInterp run(plan);
                    run.world = world;
                    run.run();
                    std::ofstream res(std::string(argv[f]) + ".out", std::ios::binary);
                    for (auto& r : plan.results) {
                        const uint32_t len = uint32_t(r.id.size()), nd = uint32_t(r.shape.size());
                        res.write(reinterpret_cast<const char*>(&len), 4);
                        res.write(r.id.data(), len);
                        res.write(reinterpret_cast<const char*>(&nd), 4);
                        uint64_t n = 1;
                        for (auto d : r.shape) {
                            const uint64_t dd = uint64_t(d);
                            res.write(reinterpret_cast<const char*>(&dd), 8);
                            n *= dd;
                        }
                        const uint8_t defined = r.buf >= 0;
                        res.write(reinterpret_cast<const char*>(&defined), 1);
                        if (defined) res.write(reinterpret_cast<const char*>(run.ptr(r.buf, r.off)), std::streamsize(n * 4));
                    }
                    executed++;
                }
                std::string bad = check_plan(plan);
                if (!bad.empty()) {
                    std::fprintf(stderr, "plan invariant violated in %s (rank %d): %s\n%s\n", argv[f], rank, bad.c_str(),
                                 adb::dump_plan(plan, false).c_str());
                    return 4;
                }
            } catch (const std::exception& e) {
                rejected++;
                if (argc == 5) std::printf("rejected: %s\n", e.what());
            }
        }
    }
    std::printf("files=%d kernels=%zu fused_sums=%zu rejected=%zu executed=%zu\n", argc - 4, kernels, fused, rejected, executed);
    return 0;
}
