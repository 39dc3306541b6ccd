// Row sums for callers that must not allocate device memory.
//
// Some callers of this library run where cudaMalloc is off limits: inside a host callback or a
// latency-critical loop where an allocation would synchronise the device, in a process whose memory
// is fully handed to another pool, or while a stream capture is open.  The regular path
// (adb_execute) plans an arena and may grow it; this entry point instead keeps the scratch memory of
// the two-pass row sum in a fixed file-scope device array, so calling it allocates nothing: no
// cudaMalloc / cudaFree, no allocating library routine.
//
// Limits and rules (also stated in include/adb200.h):
//   * the scratch array holds ADB_NOALLOC_MAX_PARTIALS floats (4 MiB); every GPU that loads the
//     library carries it until the process exits.  A call needs rows * split partial sums and is
//     refused with ADB_ERR_INVALID when even split == 1 does not fit (rows > ADB_NOALLOC_MAX_PARTIALS).
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current) and remembers it; make that first call before any stream capture begins.
//   * all calls share the one array.  Every partial a call reads was written by the same call, so
//     nothing has to be cleared between calls, but two calls that overlap on the GPU (different
//     streams, no ordering between them) race on it.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "../../include/adb200.h"

namespace {

constexpr unsigned long long kMaxPartials = ADB_NOALLOC_MAX_PARTIALS;

// In host code this name is only a handle for the symbol APIs, never a usable device address.
static __device__ __align__(256) float g_row_sum_scratch[kMaxPartials];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};  // per device: address of g_row_sum_scratch on that device

// pass 1: block (x = row, y = part) sums elements [part*chunk, min(len, (part+1)*chunk)) of its row
__global__ void __launch_bounds__(256) adb_noalloc_rowsum_partial(const float* __restrict__ in, float* __restrict__ partial,
                                                                  unsigned long long rows, unsigned long long len,
                                                                  unsigned long long chunk, unsigned int split) {
    __shared__ float warp_sums[8];
    const unsigned int part = blockIdx.y;
    for (unsigned long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const unsigned long long beg = (unsigned long long)part * chunk;
        unsigned long long end = beg + chunk;
        if (end > len) end = len;
        const float* p = in + row * len;
        float s = 0.0f;
        for (unsigned long long i = beg + threadIdx.x; i < end; i += 256) s = __fadd_rn(s, p[i]);
        for (int m = 16; m >= 1; m >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, m));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = warp_sums[0];
            for (int w = 1; w < 8; w++) t = __fadd_rn(t, warp_sums[w]);
            partial[row * split + part] = t;
        }
    }
}

// pass 2: one thread per row adds that row's partials in order
__global__ void __launch_bounds__(256) adb_noalloc_rowsum_final(const float* __restrict__ partial, float* __restrict__ out,
                                                                unsigned long long rows, unsigned int split) {
    for (unsigned long long row = (unsigned long long)blockIdx.x * 256 + threadIdx.x; row < rows;
         row += (unsigned long long)gridDim.x * 256) {
        const float* p = partial + row * split;
        float t = p[0];
        for (unsigned int k = 1; k < split; k++) t = __fadd_rn(t, p[k]);
        out[row] = t;
    }
}

void set_err(char* err, size_t cap, const char* msg) {
    if (err && cap) std::snprintf(err, cap, "%s", msg);
}

}  // namespace

extern "C" adb_status adb_row_sum_noalloc(const float* d_in, float* d_out, uint64_t rows, uint64_t len, void* stream,
                                          char* err, size_t err_cap) {
    if (err && err_cap) err[0] = 0;
    if (!d_in || !d_out) { set_err(err, err_cap, "null device pointer"); return ADB_ERR_INVALID; }
    if (rows == 0) return ADB_OK;
    if (rows > kMaxPartials) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "adb_row_sum_noalloc: %llu rows exceed the fixed scratch of %llu partial sums",
                      (unsigned long long)rows, kMaxPartials);
        set_err(err, err_cap, msg);
        return ADB_ERR_INVALID;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        set_err(err, err_cap, "no current CUDA device");
        return ADB_ERR_NO_DEVICE;
    }
    if (!g_scratch_addr[dev]) {
        // one-time set-up for this device: translate the symbol into its device address
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_row_sum_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_err(err, err_cap, "cudaGetSymbolAddress failed for the scratch array");
            return ADB_ERR_CUDA;
        }
        g_scratch_addr[dev] = p;
    }
    float* scratch = g_scratch_addr[dev];
    // split long rows so that a few rows still fill the GPU, within the fixed scratch
    uint64_t split = 1;
    if (len > 8192) {
        split = (len + 8191) / 8192;
        if (split > 64) split = 64;
        if (rows * split > kMaxPartials) split = kMaxPartials / rows;
        if (split < 1) split = 1;
    }
    const uint64_t chunk = len == 0 ? 1 : (len + split - 1) / split;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 g1((unsigned)(rows < 65535 ? rows : 65535), (unsigned)split);
    adb_noalloc_rowsum_partial<<<g1, 256, 0, s>>>(d_in, scratch, rows, len, chunk, (unsigned)split);
    unsigned g2 = (unsigned)((rows + 255) / 256 < 4096 ? (rows + 255) / 256 : 4096);
    adb_noalloc_rowsum_final<<<g2, 256, 0, s>>>(scratch, d_out, rows, (unsigned)split);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_err(err, err_cap, cudaGetErrorString(e));
        return ADB_ERR_CUDA;
    }
    return ADB_OK;
}
