#pragma once
#include <stdexcept>

#include "adb_ir.hpp"
#include "adb_plan.hpp"

namespace adb {

struct LowerError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// IR -> plan (buffers, fused kernels as SSA, control-flow tree, arena layout).  Throws LowerError.
void lower_program(Program& prog, Plan& plan, const LowerOptions& opt);

// Picks the thread mapping of a reduce kernel (lanes along the summed or the kept axis, vector
// width, split factor); needed while lowering because a split adds a scratch buffer and a second pass.
void plan_reduce(KernelSpec& k, int sm_count);

// Elements per thread an element-wise kernel will use (4 when every operand's innermost digit can hold
// four consecutive lanes, else 1); the lowering needs it to size the partial-sum buffers of fused sums.
int elw_vec(const KernelSpec& k);

// True when the code generator will emit this element-wise kernel as a shared-memory tiled axis swap.
bool elw_uses_tile(const KernelSpec& k);

// Fills KernelSpec::source / entry / launch shape for every kernel of the plan.
void generate_kernels(Plan& plan);

}  // namespace adb
