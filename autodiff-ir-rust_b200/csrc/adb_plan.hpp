// The lowered program: what the reference calls a `KernelProcedure` (src/kernel/kernel_decl.rs:81-189),
// re-designed for this backend.  Instead of thirteen `Kernels` variants holding `Expression` index
// trees, a plan is a tree of steps over three kernel kinds:
//   ELW     one fused element-wise kernel: straight-line SSA over strided loads, one pass, any number
//           of outputs (covers Unary / Binary / Movement / ElwExpr of the reference)
//   REDUCE  row sum with the producing expression fused in front (Reduce / ReduceElwExpr)
//   GEMM    C = A.B on strided 2-d operands (DotProd)
// plus uploads, collectives and host-driven control flow (While / If / EX).
#pragma once
#include <climits>
#include <memory>
#include <string>
#include <vector>

#include "adb_node.hpp"

namespace adb {

struct BufferInfo {
    int64_t numel = 0;
    bool external = false;   // caller-owned device memory used in place (never written)
    int payload = -1;        // external: index of the payload slot holding the address
    bool persistent = false; // live for the whole program (ids that cross blocks, results)
    int first = INT_MAX, last = -1;
    int64_t arena_off = -1;  // byte offset in the arena
    std::string name;
};

// one strided access of a kernel: flat digits (outer -> inner) over the kernel's index space
struct Operand {
    int buf = -1;
    int64_t offset = 0;          // elements; applied by the host to the pointer at launch
    std::vector<Sub> subs;       // ELW: digits over the linear index; REDUCE: digits over y (the summed axis)
    std::vector<Sub> xsubs;      // REDUCE: digits over x (the kept axis)
    bool same_access(const Operand& o) const {
        return buf == o.buf && offset == o.offset && subs == o.subs && xsubs == o.xsubs;
    }
};

struct Ssa {
    enum Kind : uint8_t { LOAD, CONST, OP, RED } kind = CONST;
    int operand = -1;  // LOAD: index into ins; RED (ROWS kernels): index of the row reduction whose result this is
    float c = 0.f;     // CONST
    EOp op = E_ADD;    // OP
    int a = -1, b = -1;
};

struct KernelSpec {
    // ROWS: several reductions along the rows of a [p2, q2] space and the element-wise work that uses their
    // results, one block per row at a time (a normalisation layer in one pass over its input)
    // GROUP: several independent kernels of the other types launched as one grid (each member takes a range of
    // block indices); `members` are indices into Plan::kernels
    enum Type { ELW, REDUCE, ROWS, GROUP } type = ELW;
    std::vector<int> members;
    bool grouped = false;   // runs only as a member of a GROUP kernel: source is generated, no module of its own
    int64_t n = 0;  // ELW: elements; REDUCE: rows kept (V)
    int64_t r = 0;  // REDUCE: elements summed per row (R)
    int red_op = 0; // REDUCE: 0 = sum, 1 = maximum (fmaxf)
    std::vector<Operand> ins;
    std::vector<Ssa> ssa;
    struct Out {
        int ssa;
        Operand dst;
    };
    std::vector<Out> outs;  // REDUCE: one entry; `ssa` is the summand, dst is indexed by x
    // ELW only: sums computed in the same pass.  The index space is then walked as [p2, q2] (i = p * q2 + q) by
    // blocks of 8 rows x 32*vec columns; axis 0 = sum over q (one partial per row and column tile, dst holds
    // [p2][tiles_q]), axis 1 = sum over p (one partial per column and row chunk, dst holds [chunks_p][q2]).
    // A small REDUCE step after the kernel adds the partials up.
    struct Red {
        int ssa = -1;
        int axis = 0;
        Operand dst;  // scratch buffer of the partial sums (contiguous)
    };
    std::vector<Red> reds;
    // ROWS only: the row reductions in the order they are computed; phase k may use the results of phases < k
    // (Ssa::RED).  Each result is also stored to its destination ([p2] values, contiguous).
    struct Phase {
        int red_op = 0;   // 0 sum, 1 maximum
        int ssa = -1;     // the value that is reduced
        Operand dst;
    };
    std::vector<Phase> phases;
    int64_t p2 = 0, q2 = 0;
    int64_t row_chunk = 0;  // rows per blockIdx.y (a multiple of 8)
    bool dead = false;      // no step refers to this kernel any more (its work moved into another kernel)
    // filled in by the code generator
    std::string source, entry;
    int vec = 1;            // elements per thread along the innermost digit
    int mode = 0;           // REDUCE: 0 = lanes along y (row), 1 = lanes along x (column)
    int threads = 256;
    int64_t split = 1;      // REDUCE: number of partial sums per row (two-pass when > 1)
    int64_t chunk = 0;      // REDUCE: summed elements per partial (a multiple of the vector width)
    int jit = -1;           // index into the module cache
    int jit2 = -1;          // REDUCE: second-pass kernel
    int scratch = -1;       // REDUCE two-pass: buffer holding the partial sums
    bool wide_index = false;
    int64_t tr_tiles = 0;   // ELW generated as a shared-memory tiled axis swap: number of 64 x 64 tiles (one block each, grid-stride)
};

struct StepBlock;

// k elements the dot kernels accumulate in tensor memory before the partial sum is added into C with a rounded fp32 add
constexpr int64_t DOT_CHUNK_K = 1024;

struct Step {
    enum Kind { ELW, REDUCE, GEMM, UPLOAD, ALLREDUCE, WHILE, IF, EXIT } kind = EXIT;
    int pos = 0;
    int kernel = -1;
    // GEMM: C[M,N] = A[M,K] . B[K,N], strides in elements
    struct Gemm {
        int a = -1, b = -1, c = -1;
        int64_t M = 0, N = 0, K = 0;
        int64_t a_off = 0, b_off = 0, c_off = 0;
        int64_t a_rs = 0, a_cs = 0, b_rs = 0, b_cs = 0;
        // batched product (BatchDot): `batch` independent products, operand / result slices this many elements apart
        int64_t batch = 1, a_bs = 0, b_bs = 0, c_bs = 0;
        // Element-wise work on the product, done while the accumulator is still in registers (the reference's
        // `DPElwExpr`, src/kernel/fusion/dp_elw.rs:13-150 / src/devices/opencl/kernels/fuse_dp_elw.rs:48-67): a
        // chain  v = acc; v = op_i(v, operand_i)  whose operands are constants, one vector indexed by the column
        // (a bias broadcast over the rows) or a value saved earlier in the chain.
        //   EPI_SCALE  every op is a multiplication by a constant: the chain commutes with the summation over k, so
        //              it is applied to every partial product.  With `accumulate` the scaled product is ADDED to what
        //              C already holds (`W += -lr * (x^T . g)`: the gradient never exists in memory,
        //              src/kernel/alloc/alloc_temp_opt.rs:37-122).
        //   EPI_CHAIN  any chain, applied once to the finished sum; the result goes to `out` (row-major [M,N]); the
        //              plain product is still written to C when `store_raw` (something else reads it).  With
        //              store_raw off, C and out are the same buffer.
        enum EpiMode : uint8_t { EPI_NONE = 0, EPI_SCALE = 1, EPI_CHAIN = 2 };
        struct EpiOp {
            EOp op = E_ADD;
            uint8_t operand = 0;   // 0 none (unary), 1 constant, 2 column vector, 3 saved value; 4 = "save the running value"
            float c = 0.f;
        };
        EpiMode epi = EPI_NONE;
        bool accumulate = false;
        bool store_raw = true;
        int out = -1;              // EPI_CHAIN: destination of the chain
        int64_t out_off = 0;
        int colvec = -1;           // the column-indexed vector (N elements, contiguous)
        int64_t colvec_off = 0;
        std::vector<EpiOp> ops;
    } gemm;
    // UPLOAD: payload slot -> buffer; ALLREDUCE: buffer range
    // (a bucketed ALLREDUCE covers `buf` and `more_bufs`, which the arena keeps side by side in that order: one
    // collective over [start of buf, end of the last member))
    std::vector<int> more_bufs;
    int buf = -1;
    int payload = -1;
    int64_t off = 0, nelem = 0;
    // control flow: conditions are single floats living at (buf, off)
    int cond_buf = -1;
    int64_t cond_off = 0;
    std::unique_ptr<StepBlock> body;  // WHILE
    struct Branch {
        int cond_buf;
        int64_t cond_off;
        std::unique_ptr<StepBlock> body;
    };
    std::vector<Branch> branches;  // IF
    std::unique_ptr<StepBlock> else_body;
};

struct StepBlock {
    std::vector<Step> steps;
};

struct PayloadSlot {
    uint8_t kind = 0;   // PayloadKind
    uint64_t addr = 0;  // host or device address, rebound on every execute
    int64_t count = 0;  // elements
    int cmd_index = -1; // which CreateMat of the program (in program order) feeds this slot
    bool assumed_const = false;  // the plan folded this payload to a constant because every element was equal
    float const_val = 0.f;
};

struct ResultInfo {
    std::string id;
    Shape shape;
    int buf = -1;      // -1: the id was never defined
    int64_t off = 0;
};

struct Plan {
    std::vector<BufferInfo> bufs;
    std::vector<KernelSpec> kernels;
    StepBlock main;
    std::vector<PayloadSlot> payloads;
    std::vector<ResultInfo> results;
    int64_t arena_bytes = 0;
    std::vector<std::vector<int>> packs;   // buffers that must lie side by side in the arena, in this order
    int64_t results_bytes = 0;   // > 0: the kept tensors' buffers are the first `results_bytes` of the arena (one read-back copy)
    int n_steps = 0;
    size_t ir_commands = 0;
    uint64_t key = 0;
    bool exact_div = false;  // 1/x and sqrt correctly rounded instead of the <= 1 ulp hardware approximations
};

// buffers a kernel reads and writes (a GROUP: those of all its members); appended to rd / wr
inline void kernel_rw(const Plan& p, int kernel, std::vector<int>& rd, std::vector<int>& wr) {
    const KernelSpec& k = p.kernels[size_t(kernel)];
    if (k.type == KernelSpec::GROUP) {
        for (int m : k.members) kernel_rw(p, m, rd, wr);
        return;
    }
    for (auto& in : k.ins) rd.push_back(in.buf);
    for (auto& o : k.outs) wr.push_back(o.dst.buf);
    for (auto& r : k.reds) wr.push_back(r.dst.buf);
    for (auto& ph : k.phases) wr.push_back(ph.dst.buf);
}

struct LowerOptions {
    bool no_grouping = false;       // every kernel in a launch of its own
    bool no_tiny_dot = false;       // dot products of a few multiply-adds stay dot-product steps
    bool bucket_collectives = false;  // all-reduces of neighbouring gradients become one collective over adjacent buffers
    bool no_fusion = false;
    bool no_reduce_fusion = false;  // keep every Sum in a kernel of its own
    bool fuse_small_sums = false;   // fold sums into element-wise kernels of any size (the thresholds only exist for speed)
    bool no_dot_epilogue = false;   // keep element-wise kernels behind dot products apart from them
    bool exact_div = false;
    int64_t fuse_limit = 768;  // largest expression DAG fused into one kernel
    int rank = 0, world = 1;
    int sm_count = 148;        // B200: 148 SMs; reduce kernels split rows until every SM has work
};

std::string dump_plan(const Plan& plan, bool with_source);

}  // namespace adb
