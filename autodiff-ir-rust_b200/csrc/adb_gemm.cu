// fp32 dot product C[M,N] = A[M,K] . B[K,N] for sm_100a.
//
// Two kernels:
//   adb_dot_tc    TMA-fed tcgen05.mma (kind::tf32) with the 3xTF32 split: every fp32 operand is cut
//                 into hi = tf32(a) and lo = tf32(a - hi), and hi.hi + hi.lo + lo.hi is accumulated in
//                 fp32 in tensor memory, which recovers fp32-level accuracy from tf32 multipliers.
//   adb_dot_simt  plain CUDA-core tiles for small or unaligned problems.
// The reference computes one output per work-item with a scalar k loop
// (src/devices/opencl/kernels/dotprod.rs:4-75); transposed operands arrive as index expressions there
// and as (row stride, column stride) pairs here, which map onto K-major / MN-major shared-memory
// descriptors, so `A^T` and `B^T` need no copy.
#include "adb_gemm.hpp"

#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace adb {

// ====================================================================================================
// Element-wise epilogue (the reference's fused dot-product + element-wise kernel,
// src/devices/opencl/kernels/fuse_dp_elw.rs:48-67: the chain runs on the accumulator before it is stored)
// ====================================================================================================
// Same arithmetic as the generated element-wise kernels: + and * are never contracted, 1/x and sqrt(|x|) are the
// <= 1 ulp special-function forms unless correctly rounded ones are asked for.
__device__ __forceinline__ float epi_rcp(float x) { float r; asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float epi_sqrt(float x) { float r; asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }

__device__ __forceinline__ float epi_apply(int op, float v, float o, int exact) {
    switch (op) {
    case 0: return __fadd_rn(v, o);
    case 1: return __fmul_rn(v, o);
    case 2: return exp2f(v);
    case 3: return log2f(v);
    case 4: return sinf(v);
    case 5: return exact ? __frcp_rn(v) : epi_rcp(v);
    case 6: return exact ? __fsqrt_rn(fabsf(v)) : epi_sqrt(fabsf(v));
    case 7: return v == 0.f ? 1.f : 0.f;
    case 8: return v > 0.f ? 1.f : 0.f;
    default: return v < 0.f ? 1.f : 0.f;
    }
}

// the chain on one value (CUDA-core kernel)
__device__ __forceinline__ float epi_chain1(const GemmEpilogue& e, float v, float cv) {
    float saved = v;
    for (int i = 0; i < e.n_ops; i++) {
        const int kind = e.operand[i];
        if (kind == 4) { saved = v; continue; }
        const float o = kind == 1 ? e.c[i] : kind == 2 ? cv : kind == 3 ? saved : 0.f;
        v = epi_apply(e.op[i], v, o, e.exact_div);
    }
    return v;
}

// the chain on 32 values held in registers; control flow depends only on the (warp-uniform) program
__device__ __forceinline__ void epi_chain32(const GemmEpilogue& e, float (&v)[32], const float (&cv)[32]) {
    float saved[32];
#pragma unroll
    for (int j = 0; j < 32; j++) saved[j] = v[j];
    for (int i = 0; i < e.n_ops; i++) {
        const int op = e.op[i], kind = e.operand[i], exact = e.exact_div;
        const float c = e.c[i];
        if (kind == 4) {
#pragma unroll
            for (int j = 0; j < 32; j++) saved[j] = v[j];
            continue;
        }
#define ADB_EPI_EACH(expr)                                                             \
    _Pragma("unroll") for (int j = 0; j < 32; j++) {                                   \
        const float o = kind == 1 ? c : kind == 2 ? cv[j] : kind == 3 ? saved[j] : 0.f; \
        (void)o;                                                                        \
        v[j] = (expr);                                                                  \
    }
        switch (op) {
        case 0: ADB_EPI_EACH(__fadd_rn(v[j], o)) break;
        case 1: ADB_EPI_EACH(__fmul_rn(v[j], o)) break;
        case 2: ADB_EPI_EACH(exp2f(v[j])) break;
        case 3: ADB_EPI_EACH(log2f(v[j])) break;
        case 4: ADB_EPI_EACH(sinf(v[j])) break;
        case 5: if (exact) { ADB_EPI_EACH(__frcp_rn(v[j])) } else { ADB_EPI_EACH(epi_rcp(v[j])) } break;
        case 6: if (exact) { ADB_EPI_EACH(__fsqrt_rn(fabsf(v[j]))) } else { ADB_EPI_EACH(epi_sqrt(fabsf(v[j]))) } break;
        case 7: ADB_EPI_EACH(v[j] == 0.f ? 1.f : 0.f) break;
        case 8: ADB_EPI_EACH(v[j] > 0.f ? 1.f : 0.f) break;
        default: ADB_EPI_EACH(v[j] < 0.f ? 1.f : 0.f) break;
        }
#undef ADB_EPI_EACH
    }
}

// ====================================================================================================
// CUDA-core path
// ====================================================================================================
// 64x64 tile per block, 4x4 outputs per thread, fp32 FMA with k ascending in every output element
// (the order of the reference kernel, dotprod.rs:31-41).  Handles any strides and sizes.
template <int BM, int BN, int BK>
__global__ void __launch_bounds__(256) adb_dot_simt(const float* __restrict__ A, const float* __restrict__ B,
                                                    float* __restrict__ C, long long M, long long N, long long K,
                                                    long long a_rs, long long a_cs, long long b_rs, long long b_cs,
                                                    long long a_bs, long long b_bs, long long c_bs, const GemmEpilogue epi) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    // batched product: one slice per blockIdx.z
    A += (long long)blockIdx.z * a_bs;
    B += (long long)blockIdx.z * b_bs;
    C += (long long)blockIdx.z * c_bs;
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    // loader mapping: walk the unit-stride axis of each operand with consecutive threads
    const bool a_k_fast = a_cs == 1;
    const bool b_n_fast = b_cs == 1;
    for (long long k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += 256) {
            int m, k;
            if (a_k_fast) { k = e % BK; m = e / BK; } else { m = e % BM; k = e / BM; }
            long long gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? A[gm * a_rs + gk * a_cs] : 0.f;
        }
        for (int e = tid; e < BN * BK; e += 256) {
            int n, k;
            if (b_n_fast) { n = e % BN; k = e / BN; } else { k = e % BK; n = e / BK; }
            long long gn = n0 + n, gk = k0 + k;
            Bs[k][n] = (gn < N && gk < K) ? B[gk * b_rs + gn * b_cs] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        long long gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            long long gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            const long long at = gm * N + gn;
            if (epi.mode == 1) {
                for (int t = 0; t < epi.n_ops; t++) v = __fmul_rn(v, epi.c[t]);
                C[at] = epi.accumulate ? __fadd_rn(C[at], v) : v;
            } else if (epi.mode == 2) {
                if (epi.store_raw) C[at] = v;
                epi.out[at] = epi_chain1(epi, v, epi.colvec ? epi.colvec[gn] : 0.f);
            } else
                C[at] = v;
        }
    }
}

// ====================================================================================================
// Tensor-core path
// ====================================================================================================
namespace tc {

constexpr int BM = 128;          // rows of C per tile (one tcgen05.mma M)
constexpr int BN = 256;          // columns of C per tile (one tcgen05.mma N)
constexpr int BK = 32;           // fp32 elements per k-block: 128 bytes = one 128B-swizzle span
constexpr int UMMA_K = 8;        // k elements of one kind::tf32 instruction (32 bytes)
constexpr int STAGES = 2;
// The tensor core adds each K=8 partial product into the fp32 accumulator with truncation, so the error of a
// long accumulation grows linearly with the number of instructions.  The k loop is therefore cut into chunks: each
// chunk accumulates into a fresh TMEM buffer and the epilogue warps add finished chunks into C with round-to-nearest
// fp32 adds (the C tile stays in L2 between chunks).  Measured on random normal operands, error relative to max|C|
// and speed at 8192^3: chunks of 1024 k elements 7.6e-6 / 226 TFLOP/s, 2048: 1.5e-5 / 232, 4096: 3.0e-5 / 243,
// 8192: 5.9e-5 / 246 -- the error follows the chunk length, not K, and every chunk costs a read-modify-write of the C
// tile at the L2 that competes with the operand feed.  Default: LONG_CHUNK_KB k-blocks (4096 elements; a third of the
// 1e-4 the products are held to); GemmArgs::short_chunks selects CHUNK_KB (1024 elements).  CHUNK_KB is also the
// unit in which a k axis is split over clusters.
constexpr int CHUNK_KB = 32;
constexpr int LONG_CHUNK_KB = 128;
static_assert(CHUNK_KB * BK == GEMM_CHUNK_K, "accumulation chunk");
constexpr int A_BYTES = BM * BK * 4;                  // 16 KiB
constexpr int B_BYTES = BN * BK * 4;                  // 32 KiB
constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);  // hi and lo copies of both operands: 96 KiB
constexpr int TMEM_COLS = 512;                        // two 128 x 256 fp32 accumulators
constexpr int NUM_THREADS = 320;                      // warp 0 TMA, warp 1 MMA, warps 2-5 split, warps 6-9 epilogue
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr uint32_t SPIN_LIMIT = 1u << 22;             // bounded waits: ~0.2-1 s, then the kernel gives up

enum Status { OK = 0, TIMEOUT_EMPTY = 1, TIMEOUT_RAW = 2, TIMEOUT_SPLIT = 3, TIMEOUT_ACC_EMPTY = 4, TIMEOUT_ACC_FULL = 5, TIMEOUT_DRAIN = 6 };

struct Params {
    float* C;
    int M, N, K;
    int tiles_m, tiles_n, k_blocks;
    int* status;
    // shared-memory descriptor geometry of the two operands (bytes)
    uint32_t a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;
    uint32_t a_layout, b_layout;  // descriptor swizzle mode: 2 = 128B (K-major), 1 = 128B with 32B atoms (MN-major tf32)
    // the k loop of every tile is cut into k_splits ranges of kb_per_split k-blocks that different CTAs (clusters) work
    // on when there are few tiles and K is long; all of them then add into a zeroed C
    int k_splits = 1, kb_per_split = 0;
    int chunk_kb = CHUNK_KB;   // k-blocks per accumulation chunk
    GemmEpilogue epi;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the block was told to stop or the limit ran out (then it also
// raises the block-wide stop flag and records `code` in the global status word).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* stop, int* status, int code) {
    for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*stop) return false;
        if (it > 64) __nanosleep(64);
    }
    *stop = 1;
    atomicCAS(status, 0, code);
    return false;
}

// All lanes of a warp wait (each observes the phase itself), then agree on the outcome so that the
// warp never diverges around .aligned instructions or __syncwarp().
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* stop, int* status, int code) {
    bool ok = mbar_wait(bar, parity, stop, status, code);
    return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// shared-memory matrix descriptor: start address, leading / stride byte offsets in 16-byte units, swizzle mode
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    d |= (uint64_t)layout << 61;
    return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrives once every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load_32cols(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// 32 consecutive floats of one row: plain stores, reductions performed at the L2, or loads that are ordered
// behind this thread's earlier reductions to the same addresses
__device__ __forceinline__ void row_store32(float* dst, const float (&v)[32], int n_valid, bool vec) {
    if (vec && n_valid == 32) {
        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int j = 0; j < 8; j++) d4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (j < n_valid) dst[j] = v[j];
    }
}
__device__ __forceinline__ void row_add32(float* dst, const float (&v)[32], int n_valid, bool vec) {
    if (vec && n_valid == 32) {
        // fire-and-forget fp32 adds performed at the L2 (round to nearest): no load latency in the epilogue and no
        // extra registers; same-thread same-address ordering keeps them behind the stores of the first chunk
#pragma unroll
        for (int j = 0; j < 8; j++)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                         "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (j < n_valid) atomicAdd(dst + j, v[j]);
    }
}
__device__ __forceinline__ void row_load32(const float* src, float (&v)[32], int n_valid, bool vec) {
    if (vec && n_valid == 32) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[4 * j]), "=f"(v[4 * j + 1]), "=f"(v[4 * j + 2]),
                         "=f"(v[4 * j + 3]) : "l"(src + 4 * j) : "memory");
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            v[j] = 0.f;
            if (j < n_valid) asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v[j]) : "l"(src + j) : "memory");
        }
    }
}

// One 32-column slice of one row of a finished accumulation chunk goes to memory.  `first`: the chunk opens the k
// range of its tile and nobody else works on the tile (it may overwrite C); `last`: it closes the range (the sum is
// complete once it is added).
__device__ __forceinline__ void epilogue_slice(const Params& p, int row, int col0, float (&v)[32], bool first, bool last, bool vec_c,
                                               bool vec_out) {
    if (row >= p.M || col0 >= p.N) return;
    const int n_valid = min(32, p.N - col0);
    float* crow = p.C + (size_t)row * p.N + col0;
    const GemmEpilogue& e = p.epi;
    if (e.mode == 1) {
        // scaling commutes with the summation over k: every partial product is scaled, then stored or added
        for (int t = 0; t < e.n_ops; t++) {
            const float c = e.c[t];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __fmul_rn(v[j], c);
        }
        if (first && !e.accumulate) row_store32(crow, v, n_valid, vec_c);
        else row_add32(crow, v, n_valid, vec_c);
        return;
    }
    if (e.mode == 2 && last) {
        if (!first) {
            // the earlier chunks of this tile were added to C by this very thread: read the running sum back (L2)
            float run[32];
            row_load32(crow, run, n_valid, vec_c);
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __fadd_rn(run[j], v[j]);
        }
        if (e.store_raw) row_store32(crow, v, n_valid, vec_c);
        float cv[32];
#pragma unroll
        for (int j = 0; j < 32; j++) cv[j] = (e.colvec && j < n_valid) ? __ldg(e.colvec + col0 + j) : 0.f;
        epi_chain32(e, v, cv);
        row_store32(e.out + (size_t)row * p.N + col0, v, n_valid, vec_out);
        return;
    }
    if (first) row_store32(crow, v, n_valid, vec_c);
    else row_add32(crow, v, n_valid, vec_c);
}

// A_MN / B_MN: the operand is contiguous along M (resp. N) in global memory instead of along K.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
adb_dot_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128B swizzle pattern
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    // per stage: [A hi][B hi][A lo][B lo]
    auto a_hi = [&](int s) { return base + s * STAGE_BYTES; };
    auto b_hi = [&](int s) { return base + s * STAGE_BYTES + A_BYTES; };
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    auto bar_raw = [&](int s) { return bars + 8u * s; };                    // TMA landed
    auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };       // hi/lo written
    auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };   // MMAs of the stage done
    auto bar_acc_full = [&](int a) { return bars + 8u * (3 * STAGES + a); };
    auto bar_acc_empty = [&](int a) { return bars + 8u * (3 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + STAGES * STAGE_BYTES + 8 * (3 * STAGES + 4));
    volatile int* stop = reinterpret_cast<volatile int*>(gen_base + STAGES * STAGE_BYTES + 8 * (3 * STAGES + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.tiles_m * p.tiles_n * p.k_splits;  // a unit of work is one k range of one tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_raw(s), 1);
            mbar_init(bar_split(s), 4);   // one arrival per split warp
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 4);  // one arrival per epilogue warp
        }
        *stop = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                const int tile = unit / p.k_splits;
                const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
                const int m0 = (tile / p.tiles_n) * BM, n0 = (tile % p.tiles_n) * BN;
                for (int kb = kb_begin; kb < kb_stop; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(bar_empty(s), ph ^ 1, stop, p.status, TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(bar_raw(s), A_BYTES + B_BYTES);
                    const int k0 = kb * BK;
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 32; c++) tma_load_2d(a_hi(s) + c * (BK * 128), &map_a, bar_raw(s), m0 + 32 * c, k0);
                    } else {
                        tma_load_2d(a_hi(s), &map_a, bar_raw(s), k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < BN / 32; c++) tma_load_2d(b_hi(s) + c * (BK * 128), &map_b, bar_raw(s), n0 + 32 * c, k0);
                    } else {
                        tma_load_2d(b_hi(s), &map_b, bar_raw(s), k0, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, tf32 x tf32, operand majorness, N, M
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major tiles: rows of 128 B, 8-row groups 1024 B apart (SBO), a k-step moves 32 B inside the
            // swizzle span.  MN-major tiles (tf32 allows only the 128B swizzle with 32-byte atoms there):
            // 32-element column chunks of BK rows x 128 B, chunks BK*128 B apart (LBO), 4-row groups 512 B
            // apart (SBO), a k-step moves 8 rows = 1024 B.
            const uint32_t a_lbo = p.a_lbo, a_sbo = p.a_sbo, a_kstep = p.a_kstep;
            const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
            uint32_t it = 0, chunk_no = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
                for (int kb0 = kb_begin; kb0 < kb_stop && ok; kb0 += p.chunk_kb, chunk_no++) {
                    const int acc = chunk_no & 1;
                    const uint32_t acc_ph = (chunk_no >> 1) & 1;
                    if (!mbar_wait(bar_acc_empty(acc), acc_ph ^ 1, stop, p.status, TIMEOUT_ACC_EMPTY)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int kb_end = min(kb0 + p.chunk_kb, kb_stop);
                    for (int kb = kb0; kb < kb_end; kb++, it++) {
                        const int s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!mbar_wait(bar_split(s), ph, stop, p.status, TIMEOUT_SPLIT)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < BK / UMMA_K; j++) {
                            const uint64_t ah = make_desc(a_hi(s) + j * a_kstep, a_lbo, a_sbo, p.a_layout);
                            const uint64_t bh = make_desc(b_hi(s) + j * b_kstep, b_lbo, b_sbo, p.b_layout);
                            const uint64_t al = make_desc(a_hi(s) + (A_BYTES + B_BYTES) + j * a_kstep, a_lbo, a_sbo, p.a_layout);
                            const uint64_t bl = make_desc(b_hi(s) + (A_BYTES + B_BYTES) + j * b_kstep, b_lbo, b_sbo, p.b_layout);
                            // small terms first, then the dominant one
                            umma_tf32(d_tmem, al, bh, idesc, ((kb - kb0) | j) != 0);
                            umma_tf32(d_tmem, ah, bl, idesc, 1);
                            umma_tf32(d_tmem, ah, bh, idesc, 1);
                        }
                        umma_commit(bar_empty(s));
                    }
                    if (ok) umma_commit(bar_acc_full(acc));
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ split: raw fp32 -> tf32 lo beside it
        const int t = threadIdx.x - 64;  // 0..127
        uint32_t it = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
            for (int kb = kb_begin; kb < kb_stop; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait_warp(bar_raw(s), ph, stop, p.status, TIMEOUT_RAW)) { ok = false; break; }
                // kind::tf32 reads the upper 19 bits of each fp32 word, so the raw tile already serves as
                // hi = trunc_tf32(x); only lo = x - hi (exact in fp32, truncated again by the MMA) is written.
                // Every byte less through shared memory counts: the MMAs' own operand reads take 3/4 of its bandwidth.
                const uint4* raw = reinterpret_cast<const uint4*>(gen_base + s * STAGE_BYTES);
                uint4* lo = reinterpret_cast<uint4*>(gen_base + s * STAGE_BYTES + A_BYTES + B_BYTES);
#pragma unroll 8
                for (int i = t; i < (A_BYTES + B_BYTES) / 16; i += 128) {
                    const uint4 v = raw[i];
                    uint4 l;
                    l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
                    l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
                    l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
                    l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
                    lo[i] = l;
                }
                // make the generic-proxy writes visible to the tensor core (async proxy) before signalling
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_split(s));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        uint32_t chunk_no = 0;
        bool ok = true;
        const bool vec_ok = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        const bool vec_out = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.epi.out) & 15) == 0);
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const int tile = unit / p.k_splits;
            const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
            const int m0 = (tile / p.tiles_n) * BM, n0 = (tile % p.tiles_n) * BN;
            const int row = m0 + q * 32 + lane;
            for (int kb0 = kb_begin; kb0 < kb_stop && ok; kb0 += p.chunk_kb, chunk_no++) {
                const int acc = chunk_no & 1;
                const uint32_t acc_ph = (chunk_no >> 1) & 1;
                // first chunk of the tile overwrites C, later ones add to it (split k ranges: C is zeroed, all add)
                const bool first = kb0 == 0 && p.k_splits == 1;
                const bool last = kb0 + p.chunk_kb >= p.k_blocks && p.k_splits == 1;   // the sum of the tile is complete after this chunk
                if (!mbar_wait_warp(bar_acc_full(acc), acc_ph, stop, p.status, TIMEOUT_ACC_FULL)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (p.epi.mode == 2 && last && !first) __threadfence();   // the running sum is read back below
#pragma unroll 1
                for (int c = 0; c < BN / 32; c++) {
                    float v[32];
                    tmem_load_32cols(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 32, v);
                    const int col0 = n0 + c * 32;
                    epilogue_slice(p, row, col0, v, first, last, vec_ok, vec_out);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty(acc));
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (*stop && threadIdx.x == 0) {
        // a role gave up: give bulk copies that may still be in flight a bounded time to land
        for (int i = 0; i < 256; i++) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ====================================================================================================
// Paired-CTA variant (cta_group::2)
// ====================================================================================================
// Two CTAs of a cluster (two SMs) work on one 256 x 256 tile of C.  Each CTA holds 128 rows of A, one half
// (128 columns) of the B tile and the 128 x 256 accumulator of its own rows in its own tensor memory; one
// thread of the leader CTA issues M = 256 instructions that run on both SMs and read each B half only once.
// Per SM and k-block that is 24 KiB of operand reads per pass instead of 36 and 32 KiB of raw tile instead
// of 48, which is what matters here: shared-memory bandwidth, not the tensor pipe, bounds the 3xTF32 loop.
//
// Hand-shakes (all waits bounded, as in the single-CTA kernel):
//   raw[s]        local   TMA of this CTA landed
//   split[s]      leader  8 arrivals: the four split warps of both CTAs wrote their lo tiles
//   empty[s]      both    the leader's MMAs that read stage s finished (one commit per CTA)
//   acc_full[a]   both    accumulator a holds a finished chunk (one commit per CTA)
//   acc_empty[a]  leader  8 arrivals: the epilogue warps of both CTAs drained accumulator a
namespace pair {

using namespace tc;

constexpr int BNH = BN / 2;                             // columns of the B tile held by one CTA
constexpr int PSTAGES = 3;
constexpr int BH_BYTES = BNH * BK * 4;                  // 16 KiB
constexpr int RAW_BYTES = A_BYTES + BH_BYTES;           // 32 KiB
constexpr int PSTAGE_BYTES = 2 * RAW_BYTES;             // raw + lo: 64 KiB
constexpr int PSMEM_BYTES = PSTAGES * PSTAGE_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier that threads of the other CTA arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* stop, int* status, int code) {
    for (uint32_t it = 0; it < SPIN_LIMIT; it++) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*stop) return false;
        if (it > 64) __nanosleep(64);
    }
    *stop = 1;
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// `cluster_addr` may name a barrier of either CTA of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
adb_dot_tc_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    // per stage: [A raw][B-half raw][A lo][B-half lo]
    auto a_raw = [&](int s) { return base + s * PSTAGE_BYTES; };
    auto b_raw = [&](int s) { return base + s * PSTAGE_BYTES + A_BYTES; };
    const uint32_t bars = base + PSTAGES * PSTAGE_BYTES;
    auto bar_raw = [&](int s) { return bars + 8u * s; };
    auto bar_split = [&](int s) { return bars + 8u * (PSTAGES + s); };
    auto bar_empty = [&](int s) { return bars + 8u * (2 * PSTAGES + s); };
    auto bar_acc_full = [&](int a) { return bars + 8u * (3 * PSTAGES + a); };
    auto bar_acc_empty = [&](int a) { return bars + 8u * (3 * PSTAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + PSTAGES * PSTAGE_BYTES + 8 * (3 * PSTAGES + 4));
    volatile int* stop = reinterpret_cast<volatile int*>(gen_base + PSTAGES * PSTAGE_BYTES + 8 * (3 * PSTAGES + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();       // 0 = leader
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    // a unit of work is one k range of one tile (tiles_m counts 256-row tiles here)
    const int total_units = p.tiles_m * p.tiles_n * p.k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; s++) {
            mbar_init(bar_raw(s), 1);
            mbar_init(bar_split(s), 8);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 8);
        }
        *stop = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised and its tensor memory is allocated
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs, own halves)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int unit = cluster_id; unit < total_units && ok; unit += num_clusters) {
                const int tile = unit / p.k_splits;
                const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
                const int m0 = (tile / p.tiles_n) * (2 * BM) + (int)rank * BM;
                const int n0 = (tile % p.tiles_n) * BN + (int)rank * BNH;
                for (int kb = kb_begin; kb < kb_stop; kb++, it++) {
                    const int s = it % PSTAGES;
                    const uint32_t ph = (it / PSTAGES) & 1;
                    if (!mbar_wait(bar_empty(s), ph ^ 1, stop, p.status, TIMEOUT_EMPTY)) { ok = false; break; }
                    mbar_expect_tx(bar_raw(s), RAW_BYTES);
                    const int k0 = kb * BK;
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 32; c++) tma_load_2d(a_raw(s) + c * (BK * 128), &map_a, bar_raw(s), m0 + 32 * c, k0);
                    } else {
                        tma_load_2d(a_raw(s), &map_a, bar_raw(s), k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < BNH / 32; c++) tma_load_2d(b_raw(s) + c * (BK * 128), &map_b, bar_raw(s), n0 + 32 * c, k0);
                    } else {
                        tma_load_2d(b_raw(s), &map_b, bar_raw(s), k0, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t a_lbo = p.a_lbo, a_sbo = p.a_sbo, a_kstep = p.a_kstep;
            const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
            uint32_t it = 0, chunk_no = 0;
            bool ok = true;
            for (int unit = cluster_id; unit < total_units && ok; unit += num_clusters) {
                const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
                for (int kb0 = kb_begin; kb0 < kb_stop && ok; kb0 += p.chunk_kb, chunk_no++) {
                    const int acc = chunk_no & 1;
                    const uint32_t acc_ph = (chunk_no >> 1) & 1;
                    if (!mbar_wait_cluster(bar_acc_empty(acc), acc_ph ^ 1, stop, p.status, TIMEOUT_ACC_EMPTY)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int kb_end = min(kb0 + p.chunk_kb, kb_stop);
                    for (int kb = kb0; kb < kb_end; kb++, it++) {
                        const int s = it % PSTAGES;
                        const uint32_t ph = (it / PSTAGES) & 1;
                        if (!mbar_wait_cluster(bar_split(s), ph, stop, p.status, TIMEOUT_SPLIT)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < BK / UMMA_K; j++) {
                            const uint64_t ah = make_desc(a_raw(s) + j * a_kstep, a_lbo, a_sbo, p.a_layout);
                            const uint64_t bh = make_desc(b_raw(s) + j * b_kstep, b_lbo, b_sbo, p.b_layout);
                            const uint64_t al = make_desc(a_raw(s) + RAW_BYTES + j * a_kstep, a_lbo, a_sbo, p.a_layout);
                            const uint64_t bl = make_desc(b_raw(s) + RAW_BYTES + j * b_kstep, b_lbo, b_sbo, p.b_layout);
                            umma_tf32_pair(d_tmem, al, bh, idesc, ((kb - kb0) | j) != 0);
                            umma_tf32_pair(d_tmem, ah, bl, idesc, 1);
                            umma_tf32_pair(d_tmem, ah, bh, idesc, 1);
                        }
                        umma_commit_pair(bar_empty(s));
                        umma_commit_pair(map_to_cta(bar_empty(s), 1));
                    }
                    if (ok) {
                        umma_commit_pair(bar_acc_full(acc));
                        umma_commit_pair(map_to_cta(bar_acc_full(acc), 1));
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ split: lo tiles beside the raw ones
        const int t = threadIdx.x - 64;
        uint32_t it = 0;
        bool ok = true;
        for (int unit = cluster_id; unit < total_units && ok; unit += num_clusters) {
            const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
            for (int kb = kb_begin; kb < kb_stop; kb++, it++) {
                const int s = it % PSTAGES;
                const uint32_t ph = (it / PSTAGES) & 1;
                if (!mbar_wait_warp(bar_raw(s), ph, stop, p.status, TIMEOUT_RAW)) { ok = false; break; }
                const uint4* raw = reinterpret_cast<const uint4*>(gen_base + s * PSTAGE_BYTES);
                uint4* lo = reinterpret_cast<uint4*>(gen_base + s * PSTAGE_BYTES + RAW_BYTES);
#pragma unroll 16
                for (int i = t; i < RAW_BYTES / 16; i += 128) {
                    const uint4 v = raw[i];
                    uint4 l;
                    l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
                    l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
                    l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
                    l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
                    lo[i] = l;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_split(s), 0));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: own rows, all 256 columns
        const int q = warp & 3;
        uint32_t chunk_no = 0;
        bool ok = true;
        const bool vec_ok = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        const bool vec_out = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.epi.out) & 15) == 0);
        for (int unit = cluster_id; unit < total_units && ok; unit += num_clusters) {
            const int tile = unit / p.k_splits;
            const int kb_begin = (unit % p.k_splits) * p.kb_per_split, kb_stop = min(kb_begin + p.kb_per_split, p.k_blocks);
            const int m0 = (tile / p.tiles_n) * (2 * BM) + (int)rank * BM, n0 = (tile % p.tiles_n) * BN;
            const int row = m0 + q * 32 + lane;
            for (int kb0 = kb_begin; kb0 < kb_stop && ok; kb0 += p.chunk_kb, chunk_no++) {
                const int acc = chunk_no & 1;
                const uint32_t acc_ph = (chunk_no >> 1) & 1;
                // the first chunk of a tile overwrites C, later ones add to it; with split k ranges nobody knows who
                // is first, so C was zeroed and everybody adds
                const bool first = kb0 == 0 && p.k_splits == 1;
                const bool last = kb0 + p.chunk_kb >= p.k_blocks && p.k_splits == 1;   // the sum of the tile is complete after this chunk
                if (!mbar_wait_warp(bar_acc_full(acc), acc_ph, stop, p.status, TIMEOUT_ACC_FULL)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (p.epi.mode == 2 && last && !first) __threadfence();   // the running sum is read back below
#pragma unroll 1
                for (int c = 0; c < BN / 32; c++) {
                    float v[32];
                    tmem_load_32cols(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 32, v);
                    const int col0 = n0 + c * 32;
                    epilogue_slice(p, row, col0, v, first, last, vec_ok, vec_out);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_acc_empty(acc), 0));
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (*stop && threadIdx.x == 0) {
        for (int i = 0; i < 256; i++) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // neither CTA may free tensor memory or leave while the other can still signal its barriers or while
    // instructions issued by the leader still read its shared memory
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pair

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-d fp32 tensor map: inner axis `inner` elements (unit stride), outer axis `outer` elements with
// `outer_stride` elements between rows; boxes are 32 inner elements (128 B, swizzled) by `box_outer` rows.
static bool encode(EncodeTiledFn fn, CUtensorMap* map, const float* ptr, long long inner, long long outer, long long outer_stride,
                   int box_outer, bool mn_major) {
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)outer_stride * 4};
    cuuint32_t box[2] = {32, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace tc

bool gemm_init(GemmContext& ctx, int sm_count, std::string& err) {
    ctx.sm_count = sm_count;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && fn &&
        q == cudaDriverEntryPointSuccess) {
        ctx.encode_tiled = fn;
    } else {
        cudaGetLastError();
        err = "cuTensorMapEncodeTiled is not available from this driver";
        return false;
    }
    if (cudaMalloc(&ctx.status, sizeof(int)) != cudaSuccess) { err = "cudaMalloc(status)"; return false; }
    cudaMemset(ctx.status, 0, sizeof(int));
    if (cudaMallocHost(&ctx.status_host, sizeof(int)) != cudaSuccess) { err = "cudaMallocHost(status)"; return false; }
    *ctx.status_host = 0;
    cudaError_t e = cudaSuccess;
    e = cudaFuncSetAttribute(tc::adb_dot_tc<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::adb_dot_tc<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::adb_dot_tc<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::adb_dot_tc<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
    if (e != cudaSuccess) { err = std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e); return false; }
    ctx.tc_ready = true;
    // paired-CTA variant: clusters of two CTAs; how many fit at once depends on how the SMs are grouped
    e = cudaFuncSetAttribute(tc::pair::adb_dot_tc_pair<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::pair::PSMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::pair::adb_dot_tc_pair<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::pair::PSMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::pair::adb_dot_tc_pair<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::pair::PSMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::pair::adb_dot_tc_pair<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::pair::PSMEM_BYTES);
    if (e == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sm_count & ~1));
        cfg.blockDim = dim3(tc::NUM_THREADS);
        cfg.dynamicSmemBytes = tc::pair::PSMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, tc::pair::adb_dot_tc_pair<false, false>, &cfg);
        if (e == cudaSuccess && clusters > 0) ctx.pair_clusters = clusters;
    }
    if (e != cudaSuccess) cudaGetLastError();  // the single-CTA kernel remains available
    return true;
}

void gemm_destroy(GemmContext& ctx) {
    if (ctx.status) cudaFree(ctx.status);
    if (ctx.status_host) cudaFreeHost(ctx.status_host);
    ctx.status = nullptr;
    ctx.status_host = nullptr;
}

// An operand can be fed by TMA when one axis has unit stride, the other a stride that is a multiple
// of 16 bytes, and the base is 16-byte aligned.
static bool tma_ok(const float* p, long long unit_len, long long other_stride) {
    (void)unit_len;
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && other_stride % 4 == 0 && other_stride > 0;
}

// Few tiles, or a last wave that leaves most SMs (pairs) idle, and a long k loop: cut k into ranges that different
// workers accumulate.  Ranges are whole 1024-element accumulation chunks; the partial products meet in a zeroed C through
// the adds the epilogue performs anyway.  The split is chosen by a small cost model: waves of units times the k-blocks
// of one unit, plus what the extra passes over C cost; it must beat the unsplit launch by 8 % to be taken.
static bool plan_k_split(tc::Params& p, long long tiles, int workers, const GemmArgs& a, cudaStream_t stream, std::string& err) {
    using namespace tc;
    p.k_splits = 1;
    p.kb_per_split = p.k_blocks;
    // a chain that runs on the finished sum needs one owner per tile
    if (a.epi.mode == 2 || a.no_k_split) return true;
    if (p.k_blocks < 2 * CHUNK_KB || workers <= 0) return true;
    auto cost = [&](long long per, long long splits) {
        const long long units = tiles * splits, waves = (units + workers - 1) / workers;
        // every extra range adds one more read-modify-write of its C tile at the L2 (~2 k-blocks of time) and the launch
        // gains a memset
        return double(waves) * double(per) + (splits > 1 ? 2.0 * double(splits) + 8.0 : 0.0);
    };
    const double base = cost(p.k_blocks, 1);
    double best = base;
    long long best_per = p.k_blocks;
    const long long max_splits = std::min<long long>(p.k_blocks / CHUNK_KB, 64);
    for (long long want = 2; want <= max_splits; want++) {
        long long per = (p.k_blocks + want - 1) / want;
        per = (per + CHUNK_KB - 1) / CHUNK_KB * CHUNK_KB;
        const long long splits = (p.k_blocks + per - 1) / per;
        if (splits < 2) continue;
        const double c = cost(per, splits);
        if (c < best) { best = c; best_per = per; }
    }
    if (best > 0.92 * base) return true;
    p.kb_per_split = (int)best_per;
    p.k_splits = (int)((p.k_blocks + best_per - 1) / best_per);
    // (a product that is added to what C holds must not clear it: every range adds anyway)
    if (p.k_splits > 1 && !(a.epi.mode == 1 && a.epi.accumulate) &&
        cudaMemsetAsync(a.C, 0, size_t(a.M) * size_t(a.N) * sizeof(float), stream) != cudaSuccess) {
        err = "cudaMemsetAsync(C)";
        return false;
    }
    return true;
}

static int gemm_launch_one(GemmContext& ctx, const GemmArgs& a, cudaStream_t stream, std::string& err);

int gemm_launch(GemmContext& ctx, const GemmArgs& a, cudaStream_t stream, std::string& err) {
    if (a.batch <= 1) return gemm_launch_one(ctx, a, stream, err);
    if (a.M <= 0 || a.N <= 0) return 0;
    // Batched product.  Slices that are big enough for the tensor-core kernel to pay (and few enough to launch one by
    // one) run as separate launches; everything else -- the many small products of attention heads -- is one launch of
    // the CUDA-core kernel with the slice index in blockIdx.z.
    const bool big = double(a.M) * double(a.N) * double(a.K) >= double(1 << 24) && a.batch <= 64 && !a.force_simt;
    if (big) {
        int n = 0;
        for (int64_t s = 0; s < a.batch; s++) {
            GemmArgs one = a;
            one.batch = 1;
            one.A = a.A + s * a.a_bs;
            one.B = a.B + s * a.b_bs;
            one.C = a.C + s * a.c_bs;
            if (one.epi.out) one.epi.out = a.epi.out + s * a.c_bs;
            const int r = gemm_launch_one(ctx, one, stream, err);
            if (r < 0) return r;
            n += r;
        }
        return n;
    }
    if (a.batch > 65535) { err = "batched dot product: more than 65535 slices"; return -1; }
    dim3 grid((unsigned)((a.N + 63) / 64), (unsigned)((a.M + 63) / 64), (unsigned)a.batch);
    if (grid.y > 65535) { err = "M too large for the SIMT dot kernel"; return -1; }
    adb_dot_simt<64, 64, 16><<<grid, 256, 0, stream>>>(a.A, a.B, a.C, a.M, a.N, a.K, a.a_rs, a.a_cs, a.b_rs, a.b_cs, a.a_bs, a.b_bs, a.c_bs, a.epi);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { err = cudaGetErrorString(e); return -1; }
    return 1;
}

static int gemm_launch_one(GemmContext& ctx, const GemmArgs& a, cudaStream_t stream, std::string& err) {
    if (a.M <= 0 || a.N <= 0) return 0;
    bool use_tc = ctx.tc_ready && !a.force_simt && a.K >= 8 && a.M >= 32 && a.N >= 32 &&
                  (double)a.M * (double)a.N * (double)a.K >= double(1 << 21) && a.M < (1ll << 31) && a.N < (1ll << 31) &&
                  a.K < (1ll << 31);
    bool a_k = a.a_cs == 1 && tma_ok(a.A, a.K, a.a_rs);    // K contiguous
    bool a_mn = a.a_rs == 1 && tma_ok(a.A, a.M, a.a_cs);   // M contiguous
    bool b_mn = a.b_cs == 1 && tma_ok(a.B, a.N, a.b_rs);   // N contiguous
    bool b_k = a.b_rs == 1 && tma_ok(a.B, a.K, a.b_cs);    // K contiguous
    if (use_tc && (a_k || a_mn) && (b_k || b_mn)) {
        using namespace tc;
        auto enc = reinterpret_cast<EncodeTiledFn>(ctx.encode_tiled);
        CUtensorMap ma, mb;
        const bool A_MN = !a_k, B_MN = !b_k;
        // two SMs per 256-row tile when there are at least two 128-row tiles to pair up
        const bool paired = ctx.pair_clusters > 0 && !a.no_pair && a.M > BM;
        bool ok = A_MN ? encode(enc, &ma, a.A, a.M, a.K, a.a_cs, BK, true) : encode(enc, &ma, a.A, a.K, a.M, a.a_rs, BM, false);
        ok = ok && (B_MN ? encode(enc, &mb, a.B, a.N, a.K, a.b_rs, BK, true)
                         : encode(enc, &mb, a.B, a.K, a.N, a.b_cs, paired ? pair::BNH : BN, false));
        if (ok) {
            Params p;
            p.epi = a.epi;
            p.C = a.C;
            p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
            p.tiles_m = (int)((a.M + BM - 1) / BM);
            p.tiles_n = (int)((a.N + BN - 1) / BN);
            p.k_blocks = (int)((a.K + BK - 1) / BK);
            p.chunk_kb = a.short_chunks ? CHUNK_KB : LONG_CHUNK_KB;
            p.status = ctx.status;
            p.a_lbo = A_MN ? BK * 128 : 16; p.a_sbo = A_MN ? 512 : 1024; p.a_kstep = A_MN ? 1024 : UMMA_K * 4; p.a_layout = A_MN ? 1 : 2;
            p.b_lbo = B_MN ? BK * 128 : 16; p.b_sbo = B_MN ? 512 : 1024; p.b_kstep = B_MN ? 1024 : UMMA_K * 4; p.b_layout = B_MN ? 1 : 2;
            if (paired) {
                p.tiles_m = (int)((a.M + 2 * BM - 1) / (2 * BM));
                const long long tiles = (long long)p.tiles_m * p.tiles_n;
                if (!plan_k_split(p, tiles, ctx.pair_clusters, a, stream, err)) return -1;
                long long clusters = tiles * p.k_splits;
                const int usable = std::max(1, ctx.pair_clusters - (a.reserve_sms + 1) / 2);
                if (clusters > usable) clusters = usable;
                const int grid = int(2 * clusters);
                using namespace pair;
                if (A_MN && B_MN) adb_dot_tc_pair<true, true><<<grid, NUM_THREADS, PSMEM_BYTES, stream>>>(ma, mb, p);
                else if (A_MN) adb_dot_tc_pair<true, false><<<grid, NUM_THREADS, PSMEM_BYTES, stream>>>(ma, mb, p);
                else if (B_MN) adb_dot_tc_pair<false, true><<<grid, NUM_THREADS, PSMEM_BYTES, stream>>>(ma, mb, p);
                else adb_dot_tc_pair<false, false><<<grid, NUM_THREADS, PSMEM_BYTES, stream>>>(ma, mb, p);
                cudaError_t e = cudaGetLastError();
                if (e != cudaSuccess) { err = std::string("adb_dot_tc_pair launch: ") + cudaGetErrorString(e); return -1; }
                ctx.tc_launches++;
                ctx.tc_total++;
                return 1;
            }
            if (!plan_k_split(p, (long long)p.tiles_m * p.tiles_n, ctx.sm_count, a, stream, err)) return -1;
            long long units = (long long)p.tiles_m * p.tiles_n * p.k_splits;
            const int usable_sms = std::max(1, ctx.sm_count - a.reserve_sms);
            const int grid = int(units > usable_sms ? usable_sms : units);
            if (A_MN && B_MN) adb_dot_tc<true, true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
            else if (A_MN) adb_dot_tc<true, false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
            else if (B_MN) adb_dot_tc<false, true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
            else adb_dot_tc<false, false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) { err = std::string("adb_dot_tc launch: ") + cudaGetErrorString(e); return -1; }
            ctx.tc_launches++;
            ctx.tc_total++;
            return 1;
        }
        // descriptor could not be encoded (odd strides): fall through to the CUDA-core kernel
    }
    dim3 grid((unsigned)((a.N + 63) / 64), (unsigned)((a.M + 63) / 64));
    if (grid.y > 65535) { err = "M too large for the SIMT dot kernel"; return -1; }
    adb_dot_simt<64, 64, 16><<<grid, 256, 0, stream>>>(a.A, a.B, a.C, a.M, a.N, a.K, a.a_rs, a.a_cs, a.b_rs, a.b_cs, 0, 0, 0, a.epi);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { err = cudaGetErrorString(e); return -1; }
    return 1;
}

int gemm_check_status(GemmContext& ctx, cudaStream_t stream) {
    if (!ctx.status || ctx.tc_launches == 0) return 0;
    if (cudaMemcpyAsync(ctx.status_host, ctx.status, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
    int s = *ctx.status_host;
    if (s != 0) cudaMemsetAsync(ctx.status, 0, sizeof(int), stream);
    ctx.tc_launches = 0;
    return s;
}

}  // namespace adb
