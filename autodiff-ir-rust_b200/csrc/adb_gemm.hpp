// Dot product C[M,N] = A[M,K] . B[K,N] on strided fp32 operands (the reference's `DotProd` kernel,
// src/devices/opencl/kernels/dotprod.rs:4-75: one work-item per output, scalar k loop).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

namespace adb {

// Element-wise work on the product while it is still in registers (see Step::Gemm in adb_plan.hpp): a chain
// v = acc; v = op_i(v, operand_i).  Passed to the kernels by value.
constexpr int GEMM_EPI_MAX_OPS = 12;
constexpr int GEMM_CHUNK_K = 1024;   // k elements of the shortest accumulation chunk of the tensor-core kernels (and the unit of k splits)
struct GemmEpilogue {
    int mode = 0;                 // 0 none, 1 scale (every partial product; optionally added to C), 2 chain on the finished sum
    int accumulate = 0;           // mode 1: C += scaled product instead of C = scaled product
    int store_raw = 1;            // mode 2: also write the plain product to C
    int exact_div = 0;            // 1/x and sqrt correctly rounded instead of the <= 1 ulp hardware forms
    int n_ops = 0;
    float* out = nullptr;         // mode 2: row-major [M,N] destination of the chain (may equal C when store_raw is 0)
    const float* colvec = nullptr;  // N values indexed by the column
    unsigned char op[GEMM_EPI_MAX_OPS] = {};       // EOp
    unsigned char operand[GEMM_EPI_MAX_OPS] = {};  // 0 none, 1 constant, 2 column vector, 3 saved value, 4 save the running value
    float c[GEMM_EPI_MAX_OPS] = {};
};

struct GemmArgs {
    const float* A = nullptr;
    const float* B = nullptr;
    float* C = nullptr;  // row-major [M,N], leading dimension N
    int64_t M = 0, N = 0, K = 0;
    int64_t a_rs = 0, a_cs = 0, b_rs = 0, b_cs = 0;  // element strides of A[m,k] and B[k,n]
    int64_t batch = 1, a_bs = 0, b_bs = 0, c_bs = 0; // batched product: slices this many elements apart
    bool force_simt = false;
    bool no_pair = false;  // keep the tensor-core kernel on one SM per tile
    bool short_chunks = false;  // accumulate 1024 k elements per chunk instead of 4096 (4x smaller truncation error, ~9 % slower)
    bool no_k_split = false;  // one owner per output tile: the order of the additions into C never depends on timing
    int reserve_sms = 0;   // leave this many SMs to a kernel running beside the product (a collective on another stream)
    GemmEpilogue epi;
};

struct GemmContext {
    int sm_count = 148;
    void* encode_tiled = nullptr;  // cuTensorMapEncodeTiled, fetched through the runtime (no libcuda link)
    bool tc_ready = false;
    int pair_clusters = 0;         // two-CTA clusters of the paired kernel that can be resident at once (0 = unavailable)
    int* status = nullptr;         // device word the tensor-core kernel sets when a bounded wait runs out
    int* status_host = nullptr;
    unsigned long long tc_launches = 0;  // tensor-core launches since the last status check
    unsigned long long tc_total = 0;     // tensor-core launches since the context was created
};

bool gemm_init(GemmContext& ctx, int sm_count, std::string& err);
void gemm_destroy(GemmContext& ctx);

// Enqueues the product on `stream`; returns the number of kernels launched, or -1 with `err` set.
int gemm_launch(GemmContext& ctx, const GemmArgs& a, cudaStream_t stream, std::string& err);

// Reads the status word of the tensor-core kernel (0 = fine; otherwise which bounded wait ran out).
// Synchronises `stream`.  Returns -1 when the status itself could not be read.
int gemm_check_status(GemmContext& ctx, cudaStream_t stream);

}  // namespace adb
