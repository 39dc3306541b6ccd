// Runtime behind the C-ABI: JIT of the generated kernels, device arena, executor.
//
// Replaces the reference's OpenCL host runtime: `OpenCL::execute` / `proc_exec` / `exec`
// (src/devices/opencl/device.rs:62-164) and `OpenCLContext` (src/devices/opencl/context.rs:19-106).
// Differences by design: one arena laid out from buffer lifetimes instead of a buffer per id; no
// per-kernel wait (one stream, one synchronisation at the end); loop bodies are captured once into
// CUDA graphs and replayed, the host only reads the 4-byte condition between replays; compiled
// plans and kernels are cached across `execute` calls instead of being rebuilt every time
// (device.rs:63-65 builds a fresh context per call).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <nvrtc.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstddef>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/adb200.h"
#include "adb_gemm.hpp"
#include "adb_lower.hpp"
#include "adb_shard.hpp"

namespace adb {

// ------------------------------------------------------------------------------------------ JIT
struct CompiledKernel {
    std::vector<char> cubin;
    cudaLibrary_t lib = nullptr;
    cudaKernel_t fn = nullptr;
};

static bool nvrtc_compile(const std::string& src, const std::string& entry, std::vector<char>& cubin, std::string& log) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, src.c_str(), (entry + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS) {
        log = "nvrtcCreateProgram failed";
        return false;
    }
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device", "--fmad=false", "-lineinfo"};
    nvrtcResult rc = nvrtcCompileProgram(prog, int(sizeof(opts) / sizeof(opts[0])), opts);
    if (rc != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        log.resize(n);
        if (n) nvrtcGetProgramLog(prog, &log[0]);
        log = std::string("NVRTC: ") + nvrtcGetErrorString(rc) + "\n" + log;
        nvrtcDestroyProgram(&prog);
        return false;
    }
    size_t n = 0;
    nvrtcGetCUBINSize(prog, &n);
    cubin.resize(n);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    return true;
}

// ------------------------------------------------------------------------------------------ NCCL (loaded lazily)
struct NcclApi {
    void* handle = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    // libnccl is opened on first use so that single-GPU runs (and hosts without it) never need it; when
    // the caller's process already holds a libnccl.so.2 (torch.distributed), that copy is the one bound.
    bool load(std::string& err) {
        if (handle) return true;
        handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!handle) { err = std::string("cannot load libnccl.so.2: ") + dlerror(); return false; }
        GetUniqueId = (decltype(GetUniqueId))dlsym(handle, "ncclGetUniqueId");
        CommInitRank = (decltype(CommInitRank))dlsym(handle, "ncclCommInitRank");
        AllReduce = (decltype(AllReduce))dlsym(handle, "ncclAllReduce");
        CommDestroy = (decltype(CommDestroy))dlsym(handle, "ncclCommDestroy");
        GetErrorString = (decltype(GetErrorString))dlsym(handle, "ncclGetErrorString");
        if (!GetUniqueId || !CommInitRank || !AllReduce || !CommDestroy) { err = "libnccl.so.2 lacks expected symbols"; return false; }
        return true;
    }
};
static NcclApi g_nccl;

// ------------------------------------------------------------------------------------------ device
struct GraphSeg {
    size_t begin = 0, end = 0;       // [begin, end) steps of the block
    cudaGraphExec_t exec = nullptr;  // null: run the steps one by one
    uint64_t launches = 0, gemms = 0, tc = 0;
};

// Double-buffered staging for a host payload that a loop body uploads every iteration: the copy for
// the next iteration runs on the copy stream while the current iteration computes.
struct Prefetch {
    void* stage[2] = {nullptr, nullptr};
    cudaEvent_t ready[2] = {nullptr, nullptr};  // H2D into stage[b] finished
    cudaEvent_t freed[2] = {nullptr, nullptr};  // the compute stream has consumed stage[b]
    bool freed_valid[2] = {false, false};
    size_t bytes = 0;
};

// Where a step of a straight-line range runs and what it has to wait for.  Collectives and the
// element-wise kernel that produces their operand run on the communication stream so that they overlap
// with the dot products that follow them in program order.
struct StepSched {
    bool on_comm = false;
    int wait_main = -1;   // (comm step) index of the last earlier main-stream step touching one of its buffers
    int wait_comm = -1;   // (main step) index of the last earlier comm-stream step touching one of its buffers
    bool beside_comm = false;  // (main step) a collective launched earlier in the range may still be running
    bool record_after = false;
    cudaEvent_t done = nullptr;
};
struct RangeSched {
    std::vector<StepSched> steps;
    bool any_comm = false;
    cudaEvent_t fork = nullptr;
};

struct CompiledPlan {
    Plan plan;
    std::map<const Step*, Prefetch> prefetch;
    std::map<std::pair<const StepBlock*, size_t>, RangeSched> sched;  // keyed by (block, first step of the range)
    std::vector<int> kernel_slot;  // plan kernel -> device kernel cache slot
    std::map<const StepBlock*, std::vector<GraphSeg>> graphs;
    uint64_t graph_epoch = 0;      // arena generation + external addresses the graphs were captured with
    uint64_t runs = 0;             // completed executions of this plan
    bool top_level_graphs = false; // straight-line top-level code is replayed as graphs (addresses were stable)
    double lower_ms = 0;
    std::vector<uint8_t> structure;  // the program without payload addresses: compared on every cache hit
    uint64_t last_used = 0;
};

}  // namespace adb

using namespace adb;

struct adb_device {
    int ordinal = 0;
    int rank = 0, world = 1;
    uint32_t flags = 0;
    uint64_t shard_batch = 0;
    std::vector<std::string> shard_ids;  // optional: the CreateMat ids that hold the batch
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;  // host->device prefetch of in-loop payloads
    cudaStream_t comm_stream = nullptr;  // collectives (and the small kernels that feed them), high priority
    static constexpr int SIDE_LANES = 3;
    cudaStream_t lane_stream[SIDE_LANES] = {};  // kernels that do not depend on one another, while a graph is captured
    std::string err;
    // kernels compiled so far, by entry name
    std::unordered_map<std::string, int> kernel_index;
    std::vector<CompiledKernel> kernels;
    // plans by structural key
    std::unordered_map<uint64_t, std::unique_ptr<CompiledPlan>> plans;
    CompiledPlan* last = nullptr;
    // arena
    char* arena = nullptr;
    size_t arena_cap = 0;
    uint64_t arena_gen = 1;
    uint64_t use_counter = 0;      // orders plans by last use (cache eviction)
    // condition read-back
    float* cond_host = nullptr;
    // results of the last execute
    struct HostResult {
        std::string id;
        std::vector<uint64_t> dims;
        float* host = nullptr;      // pinned, cached across calls
        size_t host_cap = 0;
        const float* dev = nullptr;
        size_t n = 0;
        bool valid = false;
        bool fetched = false;
    };
    std::vector<HostResult> results;
    std::vector<std::pair<float*, size_t>> pinned_pool;
    float* result_block = nullptr;   // pinned; holds the kept tensors of plans whose results sit side by side in the arena
    size_t result_block_cap = 0;
    adb_stats stats{};
    ncclComm_t nccl_comm = nullptr;
    GemmContext gemm;
    bool exit_requested = false;
    struct ProfRec { int kind; int kernel; cudaEvent_t e0, e1; double work; };  // kind: Step::Kind
    std::vector<ProfRec> prof;
    std::vector<cudaEvent_t> ev_pool;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> upload_events;
};

namespace {

struct CudaFail {
    std::string msg;
};

void ck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw CudaFail{std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")"};
}

uint64_t fnv_bytes(const void* p, size_t n, uint64_t h = 1469598103934665603ull) {
    const unsigned char* c = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; i++) { h ^= c[i]; h *= 1099511628211ull; }
    return h;
}

// hash of everything in the program except payload addresses and payload data
uint64_t structure_key(Program& prog, uint32_t flags, int rank, int world, uint64_t shard_batch, std::vector<uint8_t>& structure) {
    struct Saved { Cmd* c; uint64_t payload; uint8_t kind; };
    std::vector<Saved> saved;
    std::function<void(Block&)> strip = [&](Block& b) {
        for (auto& c : b.cmds) {
            if (c.op == OP_CREATE_MAT) {
                saved.push_back({&c, c.payload, c.payload_kind});
                c.payload = 0;
                // inline payloads would be appended by the serialiser; hash them as pointers instead
                if (c.payload_kind == PAYLOAD_INLINE) c.payload_kind = PAYLOAD_HOST;
            } else if (c.op == OP_WHILE) strip(*c.block);
            else if (c.op == OP_IF) {
                for (auto& cb : c.conds) strip(*cb.second);
                if (c.else_block) strip(*c.else_block);
            }
        }
    };
    strip(prog.main);
    std::vector<uint8_t> bytes = serialize_program(prog);
    for (auto& s : saved) { s.c->payload = s.payload; s.c->payload_kind = s.kind; }
    // the device-vs-host distinction changes the plan (resident payloads are read in place)
    for (auto& s : saved) bytes.push_back(s.kind == PAYLOAD_DEVICE ? 1 : 0);
    uint64_t extra[4] = {flags, uint64_t(rank), uint64_t(world), shard_batch};
    const uint8_t* e = reinterpret_cast<const uint8_t*>(extra);
    bytes.insert(bytes.end(), e, e + sizeof extra);
    structure.swap(bytes);
    return fnv_bytes(structure.data(), structure.size());
}

void collect_payload_cmds(Block& b, std::vector<Cmd*>& out, const std::vector<char>* live) {
    (void)live;
    for (auto& c : b.cmds) {
        if (c.op == OP_CREATE_MAT) out.push_back(&c);
        else if (c.op == OP_WHILE) collect_payload_cmds(*c.block, out, live);
        else if (c.op == OP_IF) {
            for (auto& cb : c.conds) collect_payload_cmds(*cb.second, out, live);
            if (c.else_block) collect_payload_cmds(*c.else_block, out, live);
        }
    }
}

bool payload_uniform(const float* p, int64_t n, float v) {
    uint32_t want;
    std::memcpy(&want, &v, 4);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(p);
    for (int64_t i = 0; i < n; i++)
        if (u[i] != want) return false;
    return n > 0;
}

static_assert(GEMM_CHUNK_K == DOT_CHUNK_K, "the lowering and the dot kernels must agree on the accumulation chunk");

class Executor {
  public:
    Executor(adb_device* d, CompiledPlan* cp) : d_(d), cp_(cp), plan_(cp->plan) { cur_stream_ = d->stream; }

    float* buf_ptr(int buf, int64_t elem_off = 0) {
        const BufferInfo& b = plan_.bufs[buf];
        if (b.external) return reinterpret_cast<float*>(uintptr_t(plan_.payloads[b.payload].addr)) + elem_off;
        if (b.arena_off < 0) throw CudaFail{"internal: buffer '" + b.name + "' has no storage"};
        return reinterpret_cast<float*>(d_->arena + b.arena_off) + elem_off;
    }

    // argument block and grid of one generated kernel
    void kernel_launch_shape(const KernelSpec& k, std::vector<uint64_t>& args, dim3& grid) {
        // Args { const float* in[max(1,NI)]; float* out[NO + sums]; long long n; }
        args.clear();
        size_t ni = std::max<size_t>(1, k.ins.size());
        const size_t no = k.outs.size() + k.reds.size();
        args.resize(ni + no + 1, 0);
        for (size_t i = 0; i < k.ins.size(); i++) args[i] = uint64_t(uintptr_t(buf_ptr(k.ins[i].buf, k.ins[i].offset)));
        for (size_t i = 0; i < k.outs.size(); i++)
            args[ni + i] = uint64_t(uintptr_t(buf_ptr(k.outs[i].dst.buf, k.outs[i].dst.offset)));
        for (size_t i = 0; i < k.reds.size(); i++)
            args[ni + k.outs.size() + i] = uint64_t(uintptr_t(buf_ptr(k.reds[i].dst.buf, k.reds[i].dst.offset)));
        args[ni + no] = uint64_t(k.n);
        grid = dim3(1, 1, 1);
        const int64_t cap = int64_t(d_->sm_count) * 16;
        if (k.type == KernelSpec::ROWS) {
            // one block per row at a time; phase results follow the outputs in the argument block
            args.assign(ni + k.outs.size() + k.phases.size() + 1, 0);
            for (size_t i = 0; i < k.ins.size(); i++) args[i] = uint64_t(uintptr_t(buf_ptr(k.ins[i].buf, k.ins[i].offset)));
            for (size_t i = 0; i < k.outs.size(); i++)
                args[ni + i] = uint64_t(uintptr_t(buf_ptr(k.outs[i].dst.buf, k.outs[i].dst.offset)));
            for (size_t i = 0; i < k.phases.size(); i++)
                args[ni + k.outs.size() + i] = uint64_t(uintptr_t(buf_ptr(k.phases[i].dst.buf, k.phases[i].dst.offset)));
            args[ni + k.outs.size() + k.phases.size()] = uint64_t(k.p2);
            const int64_t rows_per_block = 256 / std::max(1, k.threads);   // one warp or one block per row
            grid.x = unsigned(std::max<int64_t>(1, std::min<int64_t>((k.p2 + rows_per_block - 1) / rows_per_block, int64_t(d_->sm_count) * 8)));
        } else if (k.type == KernelSpec::ELW && !k.reds.empty()) {
            // element-wise pass with side sums: 2-d launch over [p2, q2]
            grid.x = unsigned((k.q2 + 32 * k.vec - 1) / (32 * k.vec));
            grid.y = unsigned((k.p2 + k.row_chunk - 1) / k.row_chunk);
        } else if (k.type == KernelSpec::ELW && k.tr_tiles > 0) {
            grid.x = unsigned(std::max<int64_t>(1, std::min<int64_t>(k.tr_tiles, cap * 4)));
        } else if (k.type == KernelSpec::ELW) {
            int64_t nv = k.n / k.vec;
            grid.x = unsigned(std::max<int64_t>(1, std::min<int64_t>((nv + 255) / 256, cap)));
        } else if (k.mode == 0) {
            int64_t rpb = 256 / k.threads;
            grid.x = unsigned(std::max<int64_t>(1, std::min<int64_t>((k.n + rpb - 1) / rpb, cap)));
            grid.y = unsigned(k.split);
        } else {
            grid.x = unsigned(std::max<int64_t>(1, (k.n + 32 * k.vec - 1) / (32 * k.vec)));
            grid.y = unsigned(k.split);
        }
    }

    void launch_kernel(const KernelSpec& k, int slot) {
        std::vector<uint64_t> args;
        dim3 grid(1, 1, 1), block(256, 1, 1);
        if (k.type == KernelSpec::GROUP) {
            // the members' argument blocks one after another, then the first block index of every member
            std::vector<uint64_t> one;
            std::vector<uint32_t> start = {0};
            for (int m : k.members) {
                dim3 g;
                kernel_launch_shape(plan_.kernels[size_t(m)], one, g);
                if (g.y != 1 || g.z != 1) throw CudaFail{"internal: grouped kernel with a 2-d grid"};
                args.insert(args.end(), one.begin(), one.end());
                start.push_back(start.back() + g.x);
            }
            if (start.size() & 1) start.push_back(0);
            for (size_t i = 0; i < start.size(); i += 2) args.push_back(uint64_t(start[i]) | (uint64_t(start[i + 1]) << 32));
            grid.x = start[k.members.size()];
        } else {
            kernel_launch_shape(k, args, grid);
        }
        void* params[1] = {args.data()};
        ck(cudaLaunchKernel((const void*)d_->kernels[slot].fn, grid, block, params, 0, cur_stream_), k.entry.c_str());
        launches_++;
    }


    static double operand_bytes(const Operand& o) {
        double n = 1;
        for (auto& s : o.subs) if (s.stride) n *= double(s.size);
        for (auto& s : o.xsubs) if (s.stride) n *= double(s.size);
        return 4.0 * n;
    }
    // bytes a kernel has to move: every distinct operand once
    double kernel_bytes(const KernelSpec& k) const {
        double b = 0;
        for (int m : k.members) b += kernel_bytes(plan_.kernels[size_t(m)]);
        for (auto& in : k.ins) b += operand_bytes(in);
        for (auto& o : k.outs) b += k.type == KernelSpec::REDUCE ? 4.0 * double(k.n) * double(k.split) : operand_bytes(o.dst);
        for (auto& r : k.reds) b += operand_bytes(r.dst);
        b += 4.0 * double(k.phases.size()) * double(k.p2);
        return b;
    }

    void run_step(const Step& s) {
        const bool prof = (d_->flags & ADB_FLAG_PROFILE) && !capturing_ &&
                          (s.kind == Step::ELW || s.kind == Step::REDUCE || s.kind == Step::GEMM || s.kind == Step::ALLREDUCE);
        if (!prof) { run_step_impl(s); return; }
        adb_device::ProfRec r;
        r.kind = int(s.kind);
        r.kernel = s.kernel;
        r.e0 = event();
        r.e1 = event();
        r.work = s.kind == Step::GEMM ? 2.0 * double(s.gemm.M) * double(s.gemm.N) * double(s.gemm.K) * double(s.gemm.batch)
               : s.kind == Step::ALLREDUCE ? 4.0 * double(s.nelem)
               : kernel_bytes(plan_.kernels[s.kernel]);
        ck(cudaEventRecord(r.e0, cur_stream_), "event");
        run_step_impl(s);
        ck(cudaEventRecord(r.e1, cur_stream_), "event");
        d_->prof.push_back(r);
    }

    void run_step_impl(const Step& s) {
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE:
            launch_kernel(plan_.kernels[s.kernel], cp_->kernel_slot[s.kernel]);
            break;
        case Step::GEMM: {
            const auto& g = s.gemm;
            GemmArgs a;
            a.A = buf_ptr(g.a, g.a_off); a.B = buf_ptr(g.b, g.b_off); a.C = buf_ptr(g.c, g.c_off);
            a.M = g.M; a.N = g.N; a.K = g.K;
            a.a_rs = g.a_rs; a.a_cs = g.a_cs; a.b_rs = g.b_rs; a.b_cs = g.b_cs;
            a.batch = g.batch; a.a_bs = g.a_bs; a.b_bs = g.b_bs; a.c_bs = g.c_bs;
            a.force_simt = (d_->flags & ADB_FLAG_SIMT_DOT) != 0;
            a.no_pair = (d_->flags & ADB_FLAG_SINGLE_SM_DOT) != 0;
            a.no_k_split = (d_->flags & ADB_FLAG_DETERMINISTIC) != 0;
            a.short_chunks = (d_->flags & ADB_FLAG_SHORT_DOT_CHUNKS) != 0;
            a.reserve_sms = gemm_reserve_;
            if (g.epi != Step::Gemm::EPI_NONE) {
                a.epi.mode = int(g.epi);
                a.epi.accumulate = g.accumulate ? 1 : 0;
                a.epi.store_raw = g.store_raw ? 1 : 0;
                a.epi.exact_div = plan_.exact_div ? 1 : 0;
                a.epi.n_ops = int(g.ops.size());
                if (a.epi.n_ops > GEMM_EPI_MAX_OPS) throw CudaFail{"internal: dot-product epilogue too long"};
                for (int i = 0; i < a.epi.n_ops; i++) {
                    a.epi.op[i] = (unsigned char)g.ops[size_t(i)].op;
                    a.epi.operand[i] = g.ops[size_t(i)].operand;
                    a.epi.c[i] = g.ops[size_t(i)].c;
                }
                a.epi.out = g.out >= 0 ? buf_ptr(g.out, g.out_off) : nullptr;
                a.epi.colvec = g.colvec >= 0 ? buf_ptr(g.colvec, g.colvec_off) : nullptr;
            }
            std::string e;
            const unsigned long long tc0 = d_->gemm.tc_total;
            int n = gemm_launch(d_->gemm, a, cur_stream_, e);
            if (n < 0) throw CudaFail{"gemm: " + e};
            launches_ += uint64_t(n);
            gemms_++;
            tc_ += d_->gemm.tc_total - tc0;
            break;
        }
        case Step::UPLOAD: {
            const PayloadSlot& p = plan_.payloads[s.payload];
            auto pf = cp_->prefetch.find(&s);
            if (pf != cp_->prefetch.end() && loop_depth_ > 0) {
                // the batch for this iteration was copied ahead of time; start the copy for the next one
                Prefetch& f = pf->second;
                const int b = int(loop_iter_ & 1);
                const void* src = reinterpret_cast<const void*>(uintptr_t(p.addr));
                ck(cudaStreamWaitEvent(d_->stream, f.ready[b], 0), "wait prefetch");
                ck(cudaMemcpyAsync(buf_ptr(s.buf), f.stage[b], f.bytes, cudaMemcpyDeviceToDevice, d_->stream), "upload (staged)");
                ck(cudaEventRecord(f.freed[b], d_->stream), "event");
                f.freed_valid[b] = true;
                if (f.freed_valid[b ^ 1]) ck(cudaStreamWaitEvent(d_->copy_stream, f.freed[b ^ 1], 0), "wait stage free");
                ck(cudaMemcpyAsync(f.stage[b ^ 1], src, f.bytes, cudaMemcpyHostToDevice, d_->copy_stream), "prefetch (host)");
                ck(cudaEventRecord(f.ready[b ^ 1], d_->copy_stream), "event");
                d_->stats.h2d_bytes += f.bytes;
            } else if (p.kind == PAYLOAD_DEVICE) {
                ck(cudaMemcpyAsync(buf_ptr(s.buf), reinterpret_cast<const void*>(uintptr_t(p.addr)), size_t(s.nelem) * 4,
                                   cudaMemcpyDeviceToDevice, d_->stream), "upload (device)");
            } else {
                // host -> device copies on the compute stream are timed apart from the kernels (never inside a
                // stream capture: host payloads are not capturable)
                cudaEvent_t e0 = event(), e1 = event();
                ck(cudaEventRecord(e0, d_->stream), "event");
                ck(cudaMemcpyAsync(buf_ptr(s.buf), reinterpret_cast<const void*>(uintptr_t(p.addr)), size_t(s.nelem) * 4,
                                   cudaMemcpyHostToDevice, d_->stream), "upload (host)");
                ck(cudaEventRecord(e1, d_->stream), "event");
                d_->upload_events.push_back({e0, e1});
                d_->stats.h2d_bytes += uint64_t(s.nelem) * 4;
            }
            break;
        }
        case Step::ALLREDUCE: {
            if (d_->world > 1) {
                float* p = buf_ptr(s.buf, s.off);
                ncclResult_t rc = g_nccl.AllReduce(p, p, size_t(s.nelem), ncclFloat32, ncclSum, d_->nccl_comm, cur_stream_);
                if (rc != ncclSuccess) throw CudaFail{std::string("ncclAllReduce: ") + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "error")};
                launches_++;
            }
            break;
        }
        default: break;
        }
    }

    // Pinned host payloads (>= 1 MiB) that the body of an outermost loop uploads on every iteration get
    // two staging buffers; the first copy is issued here, before the first iteration.
    std::vector<Prefetch*> start_prefetch(const StepBlock& body) {
        std::vector<Prefetch*> active;
        for (auto& st : body.steps) {
            if (st.kind != Step::UPLOAD) continue;
            const PayloadSlot& p = plan_.payloads[st.payload];
            const size_t bytes = size_t(st.nelem) * 4;
            if (p.kind == PAYLOAD_DEVICE || bytes < (size_t(1) << 20)) continue;
            cudaPointerAttributes attr;
            if (cudaPointerGetAttributes(&attr, reinterpret_cast<const void*>(uintptr_t(p.addr))) != cudaSuccess ||
                attr.type != cudaMemoryTypeHost) {
                cudaGetLastError();
                cp_->prefetch.erase(&st);  // pageable memory cannot be copied asynchronously
                continue;
            }
            Prefetch& f = cp_->prefetch[&st];
            if (f.bytes != bytes) {
                for (int b = 0; b < 2; b++) {
                    if (f.stage[b]) cudaFree(f.stage[b]);
                    f.stage[b] = nullptr;
                    if (cudaMalloc(&f.stage[b], bytes) != cudaSuccess) {
                        cudaGetLastError();
                        if (b == 1) cudaFree(f.stage[0]);
                        cp_->prefetch.erase(&st);
                        goto next;
                    }
                    if (!f.ready[b]) ck(cudaEventCreateWithFlags(&f.ready[b], cudaEventDisableTiming), "event create");
                    if (!f.freed[b]) ck(cudaEventCreateWithFlags(&f.freed[b], cudaEventDisableTiming), "event create");
                }
                f.bytes = bytes;
            }
            {
                // copies of an earlier execute may still own the staging buffers: order behind the compute stream
                cudaEvent_t here = event();
                ck(cudaEventRecord(here, d_->stream), "event");
                ck(cudaStreamWaitEvent(d_->copy_stream, here, 0), "order copy stream");
                f.freed_valid[0] = f.freed_valid[1] = false;
                ck(cudaMemcpyAsync(f.stage[0], reinterpret_cast<const void*>(uintptr_t(p.addr)), bytes, cudaMemcpyHostToDevice,
                                   d_->copy_stream), "prefetch (host)");
                ck(cudaEventRecord(f.ready[0], d_->copy_stream), "event");
                d_->stats.h2d_bytes += bytes;
                active.push_back(&f);
            }
        next:;
        }
        return active;
    }

    float read_cond(int buf, int64_t off) {
        ck(cudaMemcpyAsync(d_->cond_host, buf_ptr(buf, off), 4, cudaMemcpyDeviceToHost, d_->stream), "condition read-back");
        ck(cudaStreamSynchronize(d_->stream), "condition sync");
        d_->stats.d2h_bytes += 4;
        return *d_->cond_host;
    }

    void step_buffers(const Step& s, std::vector<int>& bufs) const {
        bufs.clear();
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE:
            kernel_rw(plan_, s.kernel, bufs, bufs);
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
        default: break;
        }
    }

    RangeSched& schedule(const StepBlock& blk, size_t begin, size_t end) {
        auto key = std::make_pair(&blk, begin);
        auto it = cp_->sched.find(key);
        if (it != cp_->sched.end() && it->second.steps.size() == end - begin) return it->second;
        RangeSched rs;
        rs.steps.resize(end - begin);
        // dependencies are tracked on memory ranges, not buffer ids: buffers with disjoint lifetimes share
        // arena space, and a step that runs early on the other stream must not touch memory that steps
        // before it in program order still use (nor the other way round)
        struct Touch { uintptr_t lo, hi; int idx; };
        std::vector<Touch> main_touch, comm_touch;
        std::vector<int> bufs;
        auto range_of = [&](int b) {
            const BufferInfo& bi = plan_.bufs[size_t(b)];
            uintptr_t lo = reinterpret_cast<uintptr_t>(buf_ptr(b));
            return std::make_pair(lo, lo + uintptr_t(bi.numel) * 4);
        };
        for (size_t t = begin; t < end; t++) {
            const Step& s = blk.steps[t];
            StepSched& sc = rs.steps[t - begin];
            if (d_->world > 1 && (d_->flags & ADB_FLAG_COMM_STREAM)) {
                if (s.kind == Step::ALLREDUCE) sc.on_comm = true;
                // the small kernel that writes the operand of the collective right before it
                if (s.kind == Step::ELW && t + 1 < end && blk.steps[t + 1].kind == Step::ALLREDUCE) {
                    const KernelSpec& k = plan_.kernels[s.kernel];
                    if (k.outs.size() == 1 && k.outs[0].dst.buf == blk.steps[t + 1].buf) sc.on_comm = true;
                }
            }
            step_buffers(s, bufs);
            for (int b : bufs) {
                auto r = range_of(b);
                for (auto& o : (sc.on_comm ? main_touch : comm_touch))
                    if (o.lo < r.second && r.first < o.hi) {
                        if (sc.on_comm) sc.wait_main = std::max(sc.wait_main, o.idx);
                        else sc.wait_comm = std::max(sc.wait_comm, o.idx);
                    }
            }
            for (int b : bufs) {
                auto r = range_of(b);
                (sc.on_comm ? comm_touch : main_touch).push_back({r.first, r.second, int(t - begin)});
            }
            if (sc.on_comm) {
                rs.any_comm = true;
                if (sc.wait_main >= 0) rs.steps[size_t(sc.wait_main)].record_after = true;
            }
        }
        // which compute-stream steps run while a collective may still be in flight (the communication stream
        // completes in order: once the compute stream has waited for comm step k, all comm steps <= k are done)
        {
            int latest_comm = -1, waited = -1;
            for (size_t t = 0; t < rs.steps.size(); t++) {
                StepSched& sc = rs.steps[t];
                if (sc.on_comm) {
                    if (blk.steps[begin + t].kind == Step::ALLREDUCE) latest_comm = int(t);
                } else {
                    waited = std::max(waited, sc.wait_comm);
                    sc.beside_comm = latest_comm > waited;
                }
            }
        }
        for (auto& sc : rs.steps)
            if (sc.on_comm || sc.record_after) ck(cudaEventCreateWithFlags(&sc.done, cudaEventDisableTiming), "event create");
        if (rs.any_comm) ck(cudaEventCreateWithFlags(&rs.fork, cudaEventDisableTiming), "event create");
        return cp_->sched[key] = std::move(rs);
    }

    // runs steps [begin, end) of a block: main-stream steps in order, collectives forked onto the
    // communication stream and joined again before the range ends
    void run_range(const StepBlock& blk, size_t begin, size_t end) {
        RangeSched& rs = schedule(blk, begin, end);
        if (!rs.any_comm) {
            if (capturing_ && !(d_->flags & ADB_FLAG_SERIAL_GRAPHS) && end - begin >= 3) { run_range_lanes(blk, begin, end); return; }
            for (size_t t = begin; t < end; t++) run_step(blk.steps[t]);
            return;
        }
        ck(cudaEventRecord(rs.fork, d_->stream), "fork");
        ck(cudaStreamWaitEvent(d_->comm_stream, rs.fork, 0), "fork");
        int last_comm = -1;
        for (size_t t = begin; t < end; t++) {
            StepSched& sc = rs.steps[t - begin];
            if (sc.on_comm) {
                if (sc.wait_main >= 0) ck(cudaStreamWaitEvent(d_->comm_stream, rs.steps[size_t(sc.wait_main)].done, 0), "comm waits");
                cur_stream_ = d_->comm_stream;
                run_step(blk.steps[t]);
                cur_stream_ = d_->stream;
                ck(cudaEventRecord(sc.done, d_->comm_stream), "event");
                last_comm = int(t - begin);
            } else {
                if (sc.wait_comm >= 0) ck(cudaStreamWaitEvent(d_->stream, rs.steps[size_t(sc.wait_comm)].done, 0), "main waits");
                // a dot product that runs beside a collective leaves it a few SMs: its persistent CTAs would
                // otherwise hold every SM until they finish and the collective could not start
                gemm_reserve_ = sc.beside_comm ? COMM_SMS : 0;
                run_step(blk.steps[t]);
                gemm_reserve_ = 0;
                if (sc.record_after) ck(cudaEventRecord(sc.done, d_->stream), "event");
            }
        }
        if (last_comm >= 0) ck(cudaStreamWaitEvent(d_->stream, rs.steps[size_t(last_comm)].done, 0), "join");
    }

    // While a graph is captured, generated kernels that do not depend on one another are issued on different streams, so
    // the graph holds their true dependencies and the GPU may run them side by side (a gradient that is a constant
    // fill beside the reductions that feed the next layer; the many small kernels of a small network).  Dependencies
    // are taken on the memory ranges each kernel reads and writes.  Dot products, collectives and copies stay on the
    // main stream and everything issued before them is joined first: a dot product fills every SM by itself.
    struct LaneAccess { uintptr_t lo, hi; bool write; };
    void lane_accesses(const Step& s, std::vector<LaneAccess>& acc) {
        acc.clear();
        std::vector<int> rd, wr;
        kernel_rw(plan_, s.kernel, rd, wr);
        auto add = [&](int b, bool w) {
            uintptr_t lo = reinterpret_cast<uintptr_t>(buf_ptr(b));
            acc.push_back({lo, lo + uintptr_t(plan_.bufs[size_t(b)].numel) * 4, w});
        };
        for (int b : rd) add(b, false);
        for (int b : wr) add(b, true);
    }
    static bool lane_conflict(const std::vector<LaneAccess>& a, const std::vector<LaneAccess>& b) {
        for (auto& x : a)
            for (auto& y : b)
                if ((x.write || y.write) && x.lo < y.hi && y.lo < x.hi) return true;
        return false;
    }
    void run_range_lanes(const StepBlock& blk, size_t begin, size_t end) {
        constexpr int L = adb_device::SIDE_LANES + 1;
        cudaStream_t lane[L];
        lane[0] = d_->stream;
        for (int l = 1; l < L; l++) {
            if (!d_->lane_stream[l - 1]) ck(cudaStreamCreateWithFlags(&d_->lane_stream[l - 1], cudaStreamNonBlocking), "cudaStreamCreate");
            lane[l] = d_->lane_stream[l - 1];
        }
        // events only carry the dependencies into the captured graph; they are destroyed when the capture has ended
        auto record = [&](cudaStream_t st) {
            cudaEvent_t e;
            ck(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event create");
            lane_events_.push_back(e);
            ck(cudaEventRecord(e, st), "event");
            return e;
        };
        struct Issued { int lane; cudaEvent_t done; std::vector<LaneAccess> acc; };
        std::vector<Issued> issued;          // kernels since the last join
        int lane_last[L];                    // index into `issued` of the last kernel on each lane, -1 = none since the join
        bool forked[L];
        cudaEvent_t fork = nullptr;          // recorded on the main stream at the last join
        auto reset = [&]() {
            issued.clear();
            for (int l = 0; l < L; l++) { lane_last[l] = -1; forked[l] = l == 0; }
            fork = nullptr;
        };
        auto join = [&]() {
            for (int l = 1; l < L; l++)
                if (lane_last[l] >= 0) ck(cudaStreamWaitEvent(lane[0], issued[size_t(lane_last[l])].done, 0), "join");
            reset();
        };
        reset();
        std::vector<LaneAccess> acc;
        std::vector<char> dep;
        for (size_t t = begin; t < end; t++) {
            const Step& s = blk.steps[t];
            if (s.kind != Step::ELW && s.kind != Step::REDUCE) {
                join();
                run_step(s);
                continue;
            }
            if (!fork) fork = record(lane[0]);
            lane_accesses(s, acc);
            dep.assign(issued.size(), 0);
            for (size_t i = 0; i < issued.size(); i++) dep[i] = lane_conflict(acc, issued[i].acc) ? 1 : 0;
            // the lane whose last kernel this one waits for anyway (the latest such kernel), else an idle lane
            int pick = -1;
            for (int l = 0; l < L; l++)
                if (lane_last[l] >= 0 && dep[size_t(lane_last[l])] && (pick < 0 || lane_last[l] > lane_last[pick])) pick = l;
            if (pick < 0)
                for (int l = 0; l < L && pick < 0; l++)
                    if (lane_last[l] < 0) pick = l;
            if (pick < 0) {
                pick = 0;
                for (int l = 1; l < L; l++)
                    if (lane_last[l] < lane_last[pick]) pick = l;
            }
            if (!forked[pick]) {
                ck(cudaStreamWaitEvent(lane[pick], fork, 0), "fork");
                forked[pick] = true;
            }
            for (int l = 0; l < L; l++) {
                if (l == pick) continue;
                int latest = -1;
                for (size_t i = 0; i < issued.size(); i++)
                    if (dep[i] && issued[i].lane == l) latest = int(i);
                if (latest >= 0) ck(cudaStreamWaitEvent(lane[pick], issued[size_t(latest)].done, 0), "lane waits");
            }
            cur_stream_ = lane[pick];
            try {
                run_step(s);
            } catch (...) {
                cur_stream_ = d_->stream;
                throw;
            }
            cur_stream_ = d_->stream;
            Issued rec;
            rec.lane = pick;
            rec.done = record(lane[pick]);
            rec.acc = acc;
            issued.push_back(std::move(rec));
            lane_last[pick] = int(issued.size()) - 1;
        }
        join();
    }

    static bool capturable(const Step& s, const Plan& plan) {
        switch (s.kind) {
        case Step::ELW: case Step::REDUCE: case Step::GEMM: case Step::ALLREDUCE: return true;
        case Step::UPLOAD: return plan.payloads[s.payload].kind == PAYLOAD_DEVICE;
        default: return false;
        }
    }

    // straight-line runs of a loop body are captured once and replayed
    std::vector<GraphSeg>& segments(const StepBlock& blk) {
        auto it = cp_->graphs.find(&blk);
        if (it != cp_->graphs.end()) return it->second;
        std::vector<GraphSeg> segs;
        size_t i = 0;
        while (i < blk.steps.size()) {
            size_t j = i;
            while (j < blk.steps.size() && capturable(blk.steps[j], plan_)) j++;
            if (j - i >= 2 && !(d_->flags & (ADB_FLAG_NO_GRAPHS | ADB_FLAG_PROFILE))) {
                GraphSeg g;
                g.begin = i;
                g.end = j;
                uint64_t l0 = launches_, g0 = gemms_, t0 = tc_;
                cudaGraph_t graph = nullptr;
                ck(cudaStreamBeginCapture(d_->stream, cudaStreamCaptureModeThreadLocal), "begin capture");
                capturing_ = true;
                try {
                    run_range(blk, i, j);
                } catch (...) {
                    capturing_ = false;
                    cudaStreamEndCapture(d_->stream, &graph);
                    if (graph) cudaGraphDestroy(graph);
                    drop_lane_events();
                    throw;
                }
                capturing_ = false;
                cudaError_t end_rc = cudaStreamEndCapture(d_->stream, &graph);
                drop_lane_events();
                ck(end_rc, "end capture");
                g.launches = launches_ - l0;
                g.gemms = gemms_ - g0;
                g.tc = tc_ - t0;
                launches_ = l0;
                gemms_ = g0;
                tc_ = t0;
                ck(cudaGraphInstantiate(&g.exec, graph, 0), "graph instantiate");
                cudaGraphDestroy(graph);
                segs.push_back(g);
                i = j;
            } else {
                GraphSeg g;
                g.begin = i;
                g.end = std::max(j, i + 1);
                segs.push_back(g);
                i = g.end;
            }
        }
        return cp_->graphs.emplace(&blk, std::move(segs)).first->second;
    }

    void run_block(const StepBlock& blk, bool in_loop) {
        // loop bodies always replay graphs; straight-line top-level code does so once a cached plan is
        // executed again with unchanged buffer addresses (otherwise capture would cost more than it saves)
        if (in_loop || cp_->top_level_graphs) {
            auto& segs = segments(blk);
            for (auto& g : segs) {
                if (g.exec) {
                    ck(cudaGraphLaunch(g.exec, d_->stream), "graph launch");
                    launches_ += g.launches;
                    gemms_ += g.gemms;
                    tc_ += g.tc;
                    d_->stats.graph_replays++;
                } else {
                    run_plain(blk, g.begin, g.end, in_loop);
                    if (d_->exit_requested) return;
                }
            }
            return;
        }
        run_plain(blk, 0, blk.steps.size(), false);
    }

    // steps launched one by one: maximal runs of kernels / collectives go through run_range (so that
    // collectives overlap), everything else (control flow, host uploads) is handled on its own
    void run_plain(const StepBlock& blk, size_t begin, size_t end, bool in_loop) {
        size_t t = begin;
        while (t < end) {
            size_t u = t;
            while (u < end && capturable(blk.steps[u], plan_)) u++;
            if (u > t) { run_range(blk, t, u); t = u; continue; }
            run_one(blk.steps[t], in_loop);
            if (d_->exit_requested) return;
            t++;
        }
    }

    void run_one(const Step& s, bool in_loop) {
        switch (s.kind) {
        case Step::WHILE: {
            // `while (cond[0] != 0.0)`: src/devices/opencl/device.rs:132-137
            if (read_cond(s.cond_buf, s.cond_off) == 0.0f) break;
            std::vector<Prefetch*> active;
            if (loop_depth_ == 0) active = start_prefetch(*s.body);
            const uint64_t saved_iter = loop_iter_;
            loop_depth_++;
            loop_iter_ = 0;
            do {
                run_block(*s.body, true);
                d_->stats.while_iterations++;
                loop_iter_++;
                if (d_->exit_requested) break;
            } while (read_cond(s.cond_buf, s.cond_off) != 0.0f);
            loop_depth_--;
            // the copy issued for the iteration that never came must land before its buffers are reused
            for (auto* f : active) ck(cudaStreamWaitEvent(d_->stream, f->ready[loop_iter_ & 1], 0), "drain prefetch");
            loop_iter_ = saved_iter;
            break;
        }
        case Step::IF: {
            // first condition equal to 1.0 wins, else the else-block: src/devices/opencl/device.rs:118-131
            bool taken = false;
            for (auto& br : s.branches) {
                if (read_cond(br.cond_buf, br.cond_off) == 1.0f) {
                    run_block(*br.body, in_loop);
                    taken = true;
                    break;
                }
            }
            if (!taken && s.else_body) run_block(*s.else_body, in_loop);
            break;
        }
        case Step::EXIT: d_->exit_requested = true; break;
        default: run_step(s); break;
        }
    }

    cudaEvent_t event() {
        cudaEvent_t e;
        if (!d_->ev_pool.empty()) {
            e = d_->ev_pool.back();
            d_->ev_pool.pop_back();
        } else
            ck(cudaEventCreate(&e), "event create");
        used_events_.push_back(e);
        return e;
    }
    void release_events() {
        for (auto e : used_events_) d_->ev_pool.push_back(e);
        used_events_.clear();
    }

    static constexpr int COMM_SMS = 8;   // SMs left to NCCL while a collective overlaps dot products
    int gemm_reserve_ = 0;
    uint64_t launches_ = 0, gemms_ = 0, tc_ = 0;
    bool capturing_ = false;
    std::vector<cudaEvent_t> lane_events_;   // dependency events of the capture in progress
    void drop_lane_events() {
        for (auto e : lane_events_) cudaEventDestroy(e);
        lane_events_.clear();
    }
    int loop_depth_ = 0;
    uint64_t loop_iter_ = 0;
    cudaStream_t cur_stream_ = nullptr;

  private:
    adb_device* d_;
    CompiledPlan* cp_;
    Plan& plan_;
    std::vector<cudaEvent_t> used_events_;
};

void destroy_prefetch(CompiledPlan& cp) {
    for (auto& kv : cp.prefetch)
        for (int b = 0; b < 2; b++) {
            if (kv.second.stage[b]) cudaFree(kv.second.stage[b]);
            if (kv.second.ready[b]) cudaEventDestroy(kv.second.ready[b]);
            if (kv.second.freed[b]) cudaEventDestroy(kv.second.freed[b]);
        }
    cp.prefetch.clear();
}

void destroy_sched(CompiledPlan& cp) {
    for (auto& kv : cp.sched) {
        for (auto& sc : kv.second.steps)
            if (sc.done) cudaEventDestroy(sc.done);
        if (kv.second.fork) cudaEventDestroy(kv.second.fork);
    }
    cp.sched.clear();
}

void destroy_graphs(CompiledPlan& cp) {
    for (auto& kv : cp.graphs)
        for (auto& g : kv.second)
            if (g.exec) cudaGraphExecDestroy(g.exec);
    cp.graphs.clear();
}

int ensure_kernel(adb_device* d, KernelSpec& k) {
    auto it = d->kernel_index.find(k.entry);
    if (it != d->kernel_index.end()) return it->second;
    CompiledKernel ck_;
    std::string log;
    if (!nvrtc_compile(k.source, k.entry, ck_.cubin, log)) throw CudaFail{"JIT of " + k.entry + " failed: " + log + "\n" + k.source};
    ck(cudaLibraryLoadData(&ck_.lib, ck_.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0), "cudaLibraryLoadData");
    ck(cudaLibraryGetKernel(&ck_.fn, ck_.lib, k.entry.c_str()), "cudaLibraryGetKernel");
    d->stats.jit_compiles++;
    d->kernels.push_back(std::move(ck_));
    int slot = int(d->kernels.size()) - 1;
    d->kernel_index[k.entry] = slot;
    return slot;
}

float* pinned_alloc(adb_device* d, size_t bytes, size_t& cap) {
    for (size_t i = 0; i < d->pinned_pool.size(); i++)
        if (d->pinned_pool[i].second >= bytes) {
            auto p = d->pinned_pool[i];
            d->pinned_pool.erase(d->pinned_pool.begin() + long(i));
            cap = p.second;
            return p.first;
        }
    float* p = nullptr;
    size_t want = std::max<size_t>(bytes, 4096);
    ck(cudaMallocHost(&p, want), "cudaMallocHost");
    cap = want;
    return p;
}

adb_status do_execute(adb_device* d, const uint8_t* blob, size_t nbytes) {
    auto t_begin = std::chrono::steady_clock::now();
    Program prog = parse_program(blob, nbytes);
    d->stats = adb_stats{};
    d->stats.ir_commands = prog.n_cmds;
    if (d->world > 1 && d->shard_batch) shard_program(prog, d->rank, d->world, int64_t(d->shard_batch), &d->shard_ids);
    std::vector<uint8_t> structure;
    uint64_t key = structure_key(prog, d->flags, d->rank, d->world, d->shard_batch, structure);

    std::vector<Cmd*> mats;
    collect_payload_cmds(prog.main, mats, nullptr);

    CompiledPlan* cp = nullptr;
    auto it = d->plans.find(key);
    if (it != d->plans.end()) {
        cp = it->second.get();
        // equal hashes are not proof of equal programs; and a cached plan may have folded a constant-filled payload,
        // which must still hold
        bool ok = cp->structure == structure && cp->plan.payloads.size() <= mats.size();
        if (ok) {
            // payload slots are recorded in program order together with the command index
            for (size_t s = 0; s < cp->plan.payloads.size() && ok; s++) {
                PayloadSlot& ps = cp->plan.payloads[s];
                if (ps.cmd_index < 0 || size_t(ps.cmd_index) >= mats.size()) { ok = false; break; }
                Cmd* c = mats[size_t(ps.cmd_index)];
                if (int64_t(c->count) != ps.count) { ok = false; break; }
                if (ps.assumed_const) {
                    if (c->payload_kind == PAYLOAD_DEVICE ||
                        !payload_uniform(reinterpret_cast<const float*>(uintptr_t(c->payload)), ps.count, ps.const_val))
                        ok = false;
                } else {
                    ps.kind = c->payload_kind;
                    ps.addr = c->payload;
                }
            }
        }
        if (!ok) {
            destroy_graphs(*cp);
            destroy_prefetch(*cp);
            destroy_sched(*cp);
            d->plans.erase(it);
            cp = nullptr;
        }
    }
    if (!cp) {
        auto t0 = std::chrono::steady_clock::now();
        auto fresh = std::make_unique<CompiledPlan>();
        LowerOptions opt;
        opt.no_fusion = (d->flags & ADB_FLAG_NO_FUSION) != 0;
        opt.exact_div = (d->flags & ADB_FLAG_EXACT_DIV) != 0;
        opt.fuse_small_sums = (d->flags & ADB_FLAG_FUSE_SMALL_SUMS) != 0;
        opt.no_grouping = (d->flags & ADB_FLAG_NO_GROUPING) != 0;
        opt.no_tiny_dot = (d->flags & ADB_FLAG_NO_TINY_DOT) != 0;
        opt.bucket_collectives = d->world > 1 && !(d->flags & (ADB_FLAG_COMM_STREAM | ADB_FLAG_NO_BUCKETS));
        opt.rank = d->rank;
        opt.world = d->world;
        opt.sm_count = d->sm_count;
        lower_program(prog, fresh->plan, opt);
        generate_kernels(fresh->plan);
        fresh->kernel_slot.resize(fresh->plan.kernels.size());
        for (size_t i = 0; i < fresh->plan.kernels.size(); i++)
            fresh->kernel_slot[i] = (fresh->plan.kernels[i].dead || fresh->plan.kernels[i].grouped) ? -1 : ensure_kernel(d, fresh->plan.kernels[i]);
        fresh->plan.key = key;
        fresh->lower_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        d->stats.lower_ms = fresh->lower_ms;
        fresh->structure = std::move(structure);
        cp = fresh.get();
        // bounded cache: a process that keeps producing new programs drops the plan it used longest ago
        if (d->plans.size() >= 256) {
            auto old = d->plans.begin();
            for (auto p = d->plans.begin(); p != d->plans.end(); ++p)
                if (p->second->last_used < old->second->last_used) old = p;
            destroy_graphs(*old->second);
            destroy_prefetch(*old->second);
            destroy_sched(*old->second);
            d->plans.erase(old);
        }
        d->plans[key] = std::move(fresh);
    }
    d->last = cp;
    cp->last_used = ++d->use_counter;
    Plan& plan = cp->plan;
    d->stats.plan_steps = uint64_t(plan.n_steps);
    d->stats.arena_bytes = uint64_t(plan.arena_bytes);

    // arena
    if (size_t(plan.arena_bytes) > d->arena_cap) {
        if (d->arena) ck(cudaFree(d->arena), "cudaFree(arena)");
        d->arena = nullptr;
        size_t want = size_t(plan.arena_bytes) + (size_t(1) << 20);
        cudaError_t e = cudaMalloc(&d->arena, want);
        if (e != cudaSuccess) {
            d->arena_cap = 0;
            cudaGetLastError();
            d->err = "arena of " + std::to_string(want) + " bytes does not fit in device memory";
            return ADB_ERR_OOM;
        }
        d->arena_cap = want;
        d->arena_gen++;
    }
    // graphs hold raw addresses: rebuild them when the arena or a resident payload moved
    uint64_t epoch = d->arena_gen;
    for (auto& b : plan.bufs)
        if (b.external) epoch = fnv_bytes(&plan.payloads[b.payload].addr, 8, epoch);
    for (auto& p : plan.payloads)
        if (p.kind == PAYLOAD_DEVICE) epoch = fnv_bytes(&p.addr, 8, epoch);
    // top-level code is only worth capturing when the same addresses come back run after run
    cp->top_level_graphs = cp->runs > 0 && cp->graph_epoch == epoch;
    if (cp->graph_epoch != epoch) {
        destroy_graphs(*cp);
        cp->graph_epoch = epoch;
    }

    Executor ex(d, cp);
    struct EventGuard {   // events go back to the pool however this function is left
        Executor& e;
        ~EventGuard() { e.release_events(); }
    } event_guard{ex};
    d->exit_requested = false;
    d->upload_events.clear();
    d->prof.clear();
    cudaEvent_t ev0 = ex.event(), ev1 = ex.event(), ev2 = ex.event();
    ck(cudaEventRecord(ev0, d->stream), "event record");
    ex.run_block(plan.main, false);
    ck(cudaEventRecord(ev1, d->stream), "event record");

    // read-back of dep-list ids (src/devices/opencl/device.rs:82-87)
    for (auto& r : d->results) {
        if (r.host && r.host_cap) d->pinned_pool.push_back({r.host, r.host_cap});
    }
    d->results.clear();
    // small kept tensors sit side by side at the start of the arena: one copy brings all of them back
    float* block = nullptr;
    if (plan.results_bytes > 0) {
        if (d->result_block_cap < size_t(plan.results_bytes)) {
            if (d->result_block) cudaFreeHost(d->result_block);
            d->result_block = nullptr;
            ck(cudaMallocHost(&d->result_block, size_t(plan.results_bytes)), "cudaMallocHost");
            d->result_block_cap = size_t(plan.results_bytes);
        }
        block = d->result_block;
        ck(cudaMemcpyAsync(block, d->arena, size_t(plan.results_bytes), cudaMemcpyDeviceToHost, d->stream), "read-back");
        d->stats.d2h_bytes += uint64_t(plan.results_bytes);
    }
    for (auto& ri : plan.results) {
        adb_device::HostResult hr;
        hr.id = ri.id;
        if (ri.buf >= 0) {
            hr.valid = true;
            for (auto x : ri.shape) hr.dims.push_back(uint64_t(x));
            hr.n = size_t(numel(ri.shape));
            hr.dev = ex.buf_ptr(ri.buf, ri.off);
            const BufferInfo& bi = plan.bufs[size_t(ri.buf)];
            if (block && !bi.external && bi.arena_off >= 0 && bi.arena_off + (ri.off + int64_t(hr.n)) * 4 <= plan.results_bytes) {
                hr.host = block + bi.arena_off / 4 + ri.off;   // inside the shared block: not returned to the pool
                hr.host_cap = 0;
            } else {
                hr.host = pinned_alloc(d, hr.n * 4, hr.host_cap);
                if (hr.n) ck(cudaMemcpyAsync(hr.host, hr.dev, hr.n * 4, cudaMemcpyDeviceToHost, d->stream), "read-back");
                d->stats.d2h_bytes += hr.n * 4;
            }
            hr.fetched = true;
        }
        d->results.push_back(std::move(hr));
    }
    ck(cudaEventRecord(ev2, d->stream), "event record");
    ck(cudaStreamSynchronize(d->stream), "synchronize");
    d->gemm.tc_launches = ex.tc_;  // graph replays launch the kernel without passing through gemm_launch
    if (int gs = gemm_check_status(d->gemm, d->stream)) {
        d->err = "tensor-core dot product gave up on a bounded wait (code " + std::to_string(gs) + "); results are invalid";
        return ADB_ERR_CUDA;
    }
    float ms_run = 0, ms_rb = 0;
    ck(cudaEventElapsedTime(&ms_run, ev0, ev1), "elapsed time");
    ck(cudaEventElapsedTime(&ms_rb, ev1, ev2), "elapsed time");
    double up = 0;
    for (auto& pr : d->upload_events) {
        float m = 0;
        ck(cudaEventElapsedTime(&m, pr.first, pr.second), "elapsed time");
        up += m;
    }
    d->stats.upload_ms = up;
    d->stats.device_ms = std::max(0.0, double(ms_run) - up);
    d->stats.readback_ms = ms_rb;
    cp->runs++;
    d->stats.kernel_launches = ex.launches_;
    d->stats.gemm_launches = ex.gemms_;
    d->stats.tc_gemm_launches = ex.tc_;
    if (!d->prof.empty()) {
        std::map<int, std::pair<double, std::pair<double, uint64_t>>> per_kernel;  // kernel -> (ms, (bytes, launches))
        for (auto& r : d->prof) {
            float m = 0;
            ck(cudaEventElapsedTime(&m, r.e0, r.e1), "elapsed time");
            switch (r.kind) {
            case Step::ELW: d->stats.elw_ms += m; d->stats.elw_bytes += r.work; d->stats.elw_launches++; break;
            case Step::REDUCE: d->stats.reduce_ms += m; d->stats.reduce_bytes += r.work; d->stats.reduce_launches++; break;
            case Step::GEMM: d->stats.gemm_ms += m; d->stats.gemm_flops += r.work; break;
            case Step::ALLREDUCE: d->stats.collective_ms += m; d->stats.collective_bytes += r.work; d->stats.collective_launches++; break;
            default: break;
            }
            if (r.kind == Step::ELW || r.kind == Step::REDUCE) {
                auto& pk = per_kernel[r.kernel];
                pk.first += m;
                pk.second.first += r.work;
                pk.second.second++;
            }
        }
        for (auto& kv : per_kernel)
            if (kv.second.first > d->stats.top_ms) {
                d->stats.top_ms = kv.second.first;
                d->stats.top_bytes = kv.second.second.first;
                d->stats.top_launches = kv.second.second.second;
                std::snprintf(d->stats.top_name, sizeof d->stats.top_name, "%s", plan.kernels[size_t(kv.first)].entry.c_str());
            }
        d->prof.clear();
    }
    (void)t_begin;
    return ADB_OK;
}

}  // namespace

// ============================================================================================ C-ABI
extern "C" {

const char* adb_version(void) { return "adb200 0.1 (sm_100a)"; }

// the optional tail of adb_config (older callers pass a shorter struct)
static std::vector<std::string> config_shard_ids(const adb_config* cfg) {
    std::vector<std::string> ids;
    if (!cfg || cfg->struct_size < offsetof(adb_config, n_shard_ids) + sizeof(uint32_t)) return ids;
    if (!cfg->shard_ids) return ids;
    for (uint32_t i = 0; i < cfg->n_shard_ids; i++)
        if (cfg->shard_ids[i]) ids.emplace_back(cfg->shard_ids[i]);
    return ids;
}

void adb_destroy(adb_device* d);

adb_status adb_create(const adb_config* cfg, adb_device** out) {
    if (!out) return ADB_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return ADB_ERR_NO_DEVICE;
    }
    auto d = std::make_unique<adb_device>();
    if (cfg) {
        d->ordinal = cfg->device_ordinal;
        d->rank = cfg->rank;
        d->world = cfg->world_size > 0 ? cfg->world_size : 1;
        d->flags = cfg->flags;
        d->shard_batch = cfg->shard_batch;
        d->shard_ids = config_shard_ids(cfg);
    }
    if (d->ordinal < 0 || d->ordinal >= count) return ADB_ERR_INVALID;
    // every failure past this point goes through adb_destroy, which releases whatever was created so far
    auto give_up = [&](adb_status st) {
        adb_destroy(d.release());
        return st;
    };
    try {
        ck(cudaSetDevice(d->ordinal), "cudaSetDevice");
        cudaDeviceProp prop;
        ck(cudaGetDeviceProperties(&prop, d->ordinal), "cudaGetDeviceProperties");
        d->sm_count = prop.multiProcessorCount;
        if (prop.major < 10) {
            // the generated kernels and the tcgen05 GEMM are sm_100a only; no fallback path exists
            return give_up(ADB_ERR_UNSUPPORTED);
        }
        ck(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking), "cudaStreamCreate");
        ck(cudaStreamCreateWithFlags(&d->copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        {
            int lo = 0, hi = 0;
            ck(cudaDeviceGetStreamPriorityRange(&lo, &hi), "priority range");
            ck(cudaStreamCreateWithPriority(&d->comm_stream, cudaStreamNonBlocking, hi), "cudaStreamCreate");
        }
        ck(cudaMallocHost(&d->cond_host, 64), "cudaMallocHost");
        std::string gerr;
        if (!gemm_init(d->gemm, d->sm_count, gerr)) throw CudaFail{gerr};
        if (d->world > 1) {
            if (!cfg->nccl_unique_id) return give_up(ADB_ERR_INVALID);
            std::string nerr;
            if (!g_nccl.load(nerr)) return give_up(ADB_ERR_NCCL);
            ncclUniqueId uid;
            static_assert(sizeof(uid) == 128, "ncclUniqueId is 128 bytes");
            std::memcpy(&uid, cfg->nccl_unique_id, 128);
            // collectives that overlap dot products get 8 SMs (Executor::COMM_SMS): keep NCCL's kernels that small
            if (d->flags & ADB_FLAG_COMM_STREAM) setenv("NCCL_MAX_CTAS", "8", 0);
            if (g_nccl.CommInitRank(&d->nccl_comm, d->world, uid, d->rank) != ncclSuccess) {
                d->nccl_comm = nullptr;
                return give_up(ADB_ERR_NCCL);
            }
        }
    } catch (CudaFail& f) {
        std::fprintf(stderr, "adb_create: %s\n", f.msg.c_str());
        return give_up(ADB_ERR_CUDA);
    }
    *out = d.release();
    return ADB_OK;
}

void adb_destroy(adb_device* d) {
    if (!d) return;
    cudaSetDevice(d->ordinal);
    if (d->stream) cudaStreamSynchronize(d->stream);
    if (d->copy_stream) cudaStreamSynchronize(d->copy_stream);
    if (d->comm_stream) cudaStreamSynchronize(d->comm_stream);
    for (auto& ls : d->lane_stream) if (ls) cudaStreamSynchronize(ls);
    for (auto& kv : d->plans) { destroy_graphs(*kv.second); destroy_prefetch(*kv.second); destroy_sched(*kv.second); }
    d->plans.clear();
    for (auto& k : d->kernels)
        if (k.lib) cudaLibraryUnload(k.lib);
    for (auto& r : d->results)
        if (r.host && r.host_cap) cudaFreeHost(r.host);
    if (d->result_block) cudaFreeHost(d->result_block);
    for (auto& p : d->pinned_pool) cudaFreeHost(p.first);
    for (auto e : d->ev_pool) cudaEventDestroy(e);
    gemm_destroy(d->gemm);
    if (d->nccl_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(d->nccl_comm);
    if (d->arena) cudaFree(d->arena);
    if (d->cond_host) cudaFreeHost(d->cond_host);
    if (d->copy_stream) cudaStreamDestroy(d->copy_stream);
    if (d->comm_stream) cudaStreamDestroy(d->comm_stream);
    for (auto& ls : d->lane_stream) if (ls) cudaStreamDestroy(ls);
    if (d->stream) cudaStreamDestroy(d->stream);
    delete d;
}

adb_status adb_execute(adb_device* d, const uint8_t* blob, size_t nbytes) {
    if (!d || !blob) return ADB_ERR_INVALID;
    d->err.clear();
    try {
        if (cudaSetDevice(d->ordinal) != cudaSuccess) { d->err = "cudaSetDevice failed"; return ADB_ERR_CUDA; }
        cudaGetLastError();  // an error left behind by the caller's own CUDA calls is not ours to report
        return do_execute(d, blob, nbytes);
    } catch (IrError& e) {
        d->err = std::string("invalid program: ") + e.what();
        return ADB_ERR_INVALID;
    } catch (LowerError& e) {
        d->err = std::string("cannot lower program: ") + e.what();
        return ADB_ERR_INVALID;
    } catch (CudaFail& f) {
        d->err = f.msg;
        // leave the stream usable for the next call
        cudaStreamSynchronize(d->stream);
        cudaGetLastError();
        return ADB_ERR_CUDA;
    } catch (std::exception& e) {
        d->err = e.what();
        return ADB_ERR_INVALID;
    }
}

adb_status adb_get_tensor(adb_device* d, const char* id, const float** data, const uint64_t** dims, uint32_t* ndim) {
    if (!d || !id) return ADB_ERR_INVALID;
    for (auto& r : d->results)
        if (r.id == id) {
            if (!r.valid) return ADB_NONE;
            if (data) *data = r.host;
            if (dims) *dims = r.dims.data();
            if (ndim) *ndim = uint32_t(r.dims.size());
            return ADB_OK;
        }
    return ADB_NONE;
}

adb_status adb_get_tensor_device(adb_device* d, const char* id, const float** dptr, const uint64_t** dims, uint32_t* ndim) {
    if (!d || !id) return ADB_ERR_INVALID;
    for (auto& r : d->results)
        if (r.id == id) {
            if (!r.valid) return ADB_NONE;
            if (dptr) *dptr = r.dev;
            if (dims) *dims = r.dims.data();
            if (ndim) *ndim = uint32_t(r.dims.size());
            return ADB_OK;
        }
    return ADB_NONE;
}

void adb_dot_prod_shape(const uint64_t a[2], const uint64_t b[2], uint64_t out[2]) {
    out[0] = a[0];
    out[1] = b[1];
}

const char* adb_last_error(adb_device* d) { return d ? d->err.c_str() : "null device"; }

adb_status adb_get_stats(adb_device* d, adb_stats* out) {
    if (!d || !out) return ADB_ERR_INVALID;
    *out = d->stats;
    return ADB_OK;
}

size_t adb_dump_plan(adb_device* d, char* buf, size_t cap) {
    if (!d || !d->last) return 0;
    std::string s = dump_plan(d->last->plan, false);
    if (buf && cap) {
        size_t n = std::min(cap - 1, s.size());
        std::memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return s.size() + 1;
}

static void set_err(char* err, size_t cap, const std::string& s) {
    if (err && cap) {
        size_t n = std::min(cap - 1, s.size());
        std::memcpy(err, s.data(), n);
        err[n] = 0;
    }
}

adb_status adb_lower_check(const uint8_t* blob, size_t nbytes, const adb_config* cfg, int with_source, char* buf,
                           size_t cap, size_t* needed, char* err, size_t err_cap) {
    try {
        Program prog = parse_program(blob, nbytes);
        LowerOptions opt;
        if (cfg) {
            opt.no_fusion = (cfg->flags & ADB_FLAG_NO_FUSION) != 0;
            opt.exact_div = (cfg->flags & ADB_FLAG_EXACT_DIV) != 0;
            opt.fuse_small_sums = (cfg->flags & ADB_FLAG_FUSE_SMALL_SUMS) != 0;
            opt.no_grouping = (cfg->flags & ADB_FLAG_NO_GROUPING) != 0;
            opt.no_tiny_dot = (cfg->flags & ADB_FLAG_NO_TINY_DOT) != 0;
            opt.bucket_collectives = cfg->world_size > 1 && !(cfg->flags & (ADB_FLAG_COMM_STREAM | ADB_FLAG_NO_BUCKETS));
            opt.rank = cfg->rank;
            opt.world = cfg->world_size > 0 ? cfg->world_size : 1;
            std::vector<std::string> ids = config_shard_ids(cfg);
            if (opt.world > 1 && cfg->shard_batch) shard_program(prog, opt.rank, opt.world, int64_t(cfg->shard_batch), &ids);
        }
        Plan plan;
        lower_program(prog, plan, opt);
        generate_kernels(plan);
        std::unordered_map<std::string, bool> done;
        for (auto& k : plan.kernels) {
            if (k.dead || k.grouped || done.count(k.entry)) continue;
            done[k.entry] = true;
            std::vector<char> cubin;
            std::string log;
            if (!nvrtc_compile(k.source, k.entry, cubin, log)) {
                set_err(err, err_cap, "JIT of " + k.entry + " failed: " + log + "\n" + k.source);
                return ADB_ERR_CUDA;
            }
        }
        std::string s = dump_plan(plan, with_source != 0);
        if (needed) *needed = s.size() + 1;
        if (buf && cap) {
            size_t n = std::min(cap - 1, s.size());
            std::memcpy(buf, s.data(), n);
            buf[n] = 0;
        }
        return ADB_OK;
    } catch (std::exception& e) {
        set_err(err, err_cap, e.what());
        return ADB_ERR_INVALID;
    }
}

adb_status adb_shard_ir(const uint8_t* blob, size_t nbytes, const adb_config* cfg, uint8_t* out, size_t cap, size_t* needed,
                        char* err, size_t err_cap) {
    try {
        if (!cfg) throw IrError("data-parallel rewrite: no configuration");
        Program prog = parse_program(blob, nbytes);
        std::vector<std::string> ids = config_shard_ids(cfg);
        shard_program(prog, cfg->rank, cfg->world_size, int64_t(cfg->shard_batch), &ids);
        std::vector<uint8_t> bytes = serialize_program(prog);
        if (needed) *needed = bytes.size();
        if (out && cap >= bytes.size()) std::memcpy(out, bytes.data(), bytes.size());
        return ADB_OK;
    } catch (std::exception& e) {
        set_err(err, err_cap, e.what());
        return ADB_ERR_INVALID;
    }
}

adb_status adb_inject_dot_status(adb_device* d, int code) {
    if (!d || !d->gemm.status) return ADB_ERR_INVALID;
    if (cudaSetDevice(d->ordinal) != cudaSuccess) return ADB_ERR_CUDA;
    if (cudaMemcpyAsync(d->gemm.status, &code, sizeof(int), cudaMemcpyHostToDevice, d->stream) != cudaSuccess) return ADB_ERR_CUDA;
    return cudaStreamSynchronize(d->stream) == cudaSuccess ? ADB_OK : ADB_ERR_CUDA;
}

adb_status adb_nccl_unique_id(void* out128) {
    std::string e;
    if (!out128) return ADB_ERR_INVALID;
    if (!g_nccl.load(e)) return ADB_ERR_NCCL;
    ncclUniqueId uid;
    if (g_nccl.GetUniqueId(&uid) != ncclSuccess) return ADB_ERR_NCCL;
    std::memcpy(out128, &uid, 128);
    return ADB_OK;
}

}  // extern "C"
