// Data-parallel rewrite of a program (no counterpart in the reference, which is single-device).
#pragma once
#include <string>
#include <vector>

#include "adb_ir.hpp"

namespace adb {

// Splits axis 0 of every CreateMat whose axis 0 has length `batch` across `world` ranks, follows the
// split through the program and inserts AllReduce commands where batch-partial sums meet
// replicated values.  Throws IrError when the program cannot be split this way.  With `only` (ids of the
// CreateMat tensors that hold the batch) every other CreateMat stays replicated whatever its shape.
void shard_program(Program& prog, int rank, int world, int64_t batch, const std::vector<std::string>* only = nullptr);

}  // namespace adb
