// fp32 dot product kernels.
#include "adb_gemm.hpp"

namespace adb {

// Plain CUDA-core path: 64x64 tile per block, 4x4 outputs per thread, fp32 FMA with k ascending in
// every output element (the order of the reference kernel, src/devices/opencl/kernels/dotprod.rs:31-41).
// Handles any strides and sizes; used for small or unaligned problems.
template <int BM, int BN, int BK>
__global__ void __launch_bounds__(256) adb_dot_simt(const float* __restrict__ A, const float* __restrict__ B,
                                                    float* __restrict__ C, long long M, long long N, long long K,
                                                    long long a_rs, long long a_cs, long long b_rs, long long b_cs) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    // loader mapping: pick the thread->element assignment that walks the unit-stride axis of each operand
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
            if (gn < N) C[gm * N + gn] = acc[i][j];
        }
    }
}

bool gemm_init(GemmContext& ctx, int sm_count, std::string& err) {
    ctx.sm_count = sm_count;
    (void)err;
    return true;
}

void gemm_destroy(GemmContext& ctx) { (void)ctx; }

int gemm_launch(GemmContext& ctx, const GemmArgs& a, cudaStream_t stream, std::string& err) {
    (void)ctx;
    if (a.M <= 0 || a.N <= 0) return 0;
    dim3 grid((unsigned)((a.N + 63) / 64), (unsigned)((a.M + 63) / 64));
    if (grid.y > 65535) { err = "M too large for the SIMT dot kernel"; return -1; }
    adb_dot_simt<64, 64, 16><<<grid, 256, 0, stream>>>(a.A, a.B, a.C, a.M, a.N, a.K, a.a_rs, a.a_cs, a.b_rs, a.b_cs);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { err = cudaGetErrorString(e); return -1; }
    return 1;
}

}  // namespace adb
