/*
 * adb200 — C-ABI of the B200 execution backend for the autodiff-ir `Device` boundary.
 *
 * Every entry point is plain C (pointers and sizes only).  The library is what a
 * `impl Device for B200` in the reference crate would bind through FFI; each function
 * names the reference interface it replaces (paths are relative to the reference tree).
 *
 * Threading: one caller thread per handle; `adb_execute` is synchronous on return
 * (the reference serialises all calls behind one global mutex, src/core/ir.rs:121).
 * Errors: status codes, never abort, never a device trap (the reference panics,
 * src/devices/opencl/context.rs:31,58,75,99).
 */
#ifndef ADB200_H
#define ADB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct adb_device adb_device;

typedef enum adb_status {
    ADB_OK = 0,
    ADB_NONE = 1,            /* get_tensor: id was not kept (ValueData::none(), src/core/value_data.rs:27-34) */
    ADB_ERR_INVALID = 2,     /* malformed blob / IR that cannot be lowered */
    ADB_ERR_CUDA = 3,        /* a CUDA / NVRTC call failed; see adb_last_error */
    ADB_ERR_UNSUPPORTED = 4,
    ADB_ERR_OOM = 5,
    ADB_ERR_NCCL = 6,
    ADB_ERR_NO_DEVICE = 7    /* no CUDA device: the backend has no CPU fallback */
} adb_status;

/* ---- wire format of the program handed to adb_execute -------------------------------
 * Little-endian.  `id` operands are u32 indices into the id string table.
 *
 *   u32 magic = 0x52494441 ('ADIR'), u32 version = 1, u32 flags = 0, u32 n_ids
 *   n_ids x { u16 len, len bytes }                       id strings (src/ir/base.rs:17-31)
 *   u32 n_dep, n_dep x u32                                dep list  (src/core/dependency.rs:4-33)
 *   procedure := u32 n_cmds, n_cmds x command            (struct IRProcedure, src/core/ir.rs:109-112)
 *   command   := u8 opcode, operands:                    (enum IRCmds, src/core/ir.rs:8-105)
 *      1 CreateMat      res, u8 nd, nd x u64 dim, u8 kind, u64 where, u64 n
 *                       kind 0: `where` = byte offset of n f32 inside the blob
 *                       kind 1: `where` = host address of n f32 (borrowed during the call)
 *                       kind 2: `where` = device address of n f32 resident in HBM (borrowed)
 *      2 CreateConstant res, f32 value, u8 nd, nd x u64 dim
 *      3 ElwMultiply a b res      4 ElwAdd a b res
 *      5 ElwMultiplyEq s o        6 ElwAddEq s o
 *      7 EqualZero a res          8 MoreZero a res         9 LessZero a res
 *     10 Sum a res               11 DotProduct a b res
 *     12 View a res, u8 nd, nd x u64            13 Index a res, u64 index, u32 dim
 *     14 Concat a b res, u32 dim                15 Permute a res, u8 n, n x u32
 *     16 Broadcast a res, u32 dim, u64 r        17 Contigious a res
 *     18 Exp2  19 Log2  20 Sin  21 Recip  22 Sqrt   (a res)
 *     23 While cond, procedure
 *     24 If u32 n, n x { cond, procedure }, u8 has_else, [procedure]
 *     25 EX                      26 Heading u16 len, bytes
 *     27 AllReduce id   (extension, no reference counterpart: in-place sum over all ranks)
 *     28 Max a, res     (extension: row maximum of a 2-d tensor, same shape contract as Sum; the reference's kernel
 *                        layer names ReduceOp::Max, src/kernel/kernel_decl.rs:77, but no IR command reaches it)
 */
#define ADB_IR_MAGIC 0x52494441u
#define ADB_IR_VERSION 1u

typedef struct adb_config {
    uint32_t struct_size;      /* sizeof(adb_config) */
    int32_t device_ordinal;    /* CUDA device to run on */
    int32_t rank;              /* data-parallel rank, 0 when world_size == 1 */
    int32_t world_size;        /* number of data-parallel ranks (one process per GPU) */
    const void *nccl_unique_id;/* 128 bytes from adb_nccl_unique_id on rank 0; NULL when world_size == 1 */
    uint32_t flags;            /* ADB_FLAG_* */
    uint64_t shard_batch;      /* world_size > 1: CreateMat tensors whose dim 0 equals this are split by rank */
    /* Optional (read only when struct_size covers them): the ids of the CreateMat tensors that hold the batch.  When
     * given, only these are split; otherwise every CreateMat whose dim 0 equals shard_batch is, which cannot tell a
     * batch tensor from a parameter that happens to have as many rows. */
    const char *const *shard_ids;
    uint32_t n_shard_ids;
} adb_config;

#define ADB_FLAG_NO_GRAPHS 1u         /* launch loop bodies kernel by kernel instead of replaying CUDA graphs */
#define ADB_FLAG_NO_FUSION 2u         /* one kernel per IR command (debug aid, like the reference's unfused path) */
#define ADB_FLAG_SIMT_DOT 4u          /* force the plain fp32 dot kernel instead of the tcgen05 3xTF32 kernels */
#define ADB_FLAG_PROFILE 8u           /* CUDA events around every kernel (fills the per-kind times of adb_stats);
                                         loop bodies are then launched kernel by kernel, not as graphs */
#define ADB_FLAG_COMM_STREAM 16u      /* issue collectives on a second, high-priority stream (ordered by events on the
                                         memory they touch) beside the remaining dot products, which then leave 8 SMs
                                         free; off by default: measured 1.5-3 % slower on 2 and on 8 GPUs (the dot
                                         products lose more than the all-reduce time that is hidden) */
#define ADB_FLAG_SINGLE_SM_DOT 32u    /* keep the tcgen05 dot kernel on one SM per 128 x 256 tile instead of pairing two
                                         SMs (cta_group::2) on a 256 x 256 tile */
#define ADB_FLAG_EXACT_DIV 64u        /* Recip and Sqrt correctly rounded (bit-identical to IEEE 1.0f/x and sqrtf) instead
                                         of the special-function-unit forms (<= 1 ulp); costs ~10 issue slots per use */
#define ADB_FLAG_FUSE_SMALL_SUMS 128u /* fold sums into neighbouring element-wise kernels whatever their size (by default
                                         only above 2^18 elements and 128 columns, where it pays); lets small tests reach
                                         that path */
#define ADB_FLAG_NO_GROUPING 256u     /* every generated kernel in a launch of its own (by default independent kernels
                                         that follow one another share one grid) */
#define ADB_FLAG_DETERMINISTIC 512u    /* dot products never split the k axis across clusters: by default a product with few
                                         output tiles and a long k axis is cut into k ranges whose partial sums meet in C
                                         through red.global.add, in an order that depends on timing (results then differ
                                         in the last bits from run to run); with this flag every run gives the same bits */
#define ADB_FLAG_SERIAL_GRAPHS 1024u   /* captured graphs keep the kernels in one chain (by default generated kernels that do not
                                         depend on one another are captured on different streams and may run side by side) */
#define ADB_FLAG_NO_BUCKETS 2048u      /* every all-reduce of the data-parallel rewrite as a collective of its own (by default
                                         the gradients that are reduced next to one another share one collective) */
#define ADB_FLAG_NO_TINY_DOT 4096u     /* dot products of a few multiply-adds (K <= 8, M*N*K <= 256) stay dot-product steps
                                         instead of becoming element-wise sums of products (lets small tests reach the dot
                                         kernels) */
#define ADB_FLAG_SHORT_DOT_CHUNKS 8192u /* the tensor-core dot kernels add their accumulator into C every 1024 k elements instead
                                         of every 4096: the tensor core truncates when it accumulates, so the error
                                         relative to max|C| drops from 3e-5 to 8e-6 (the contract is 1e-4), at ~9 % of the
                                         dot products' speed */

/* Replaces OpenCL::new (src/devices/opencl/device.rs:41-58) + autodiff::set_device's device slot
 * (src/core/autodiff.rs:82-97).  Fails with ADB_ERR_NO_DEVICE when no GPU is present. */
adb_status adb_create(const adb_config *cfg, adb_device **out);
void adb_destroy(adb_device *dev);

/* Replaces `Device::execute` (src/core/ir.rs:128; OpenCL: src/devices/opencl/device.rs:62-88) together
 * with the `to_kernel` lowering that feeds it (src/kernel/to_kernel.rs:34-107): lowers the procedure to
 * fused kernels, runs it (If / While blocks included, src/devices/opencl/device.rs:107-146), and makes
 * every dep-list id readable through adb_get_tensor.  The blob and the memory it points to are borrowed
 * for the duration of the call. */
adb_status adb_execute(adb_device *dev, const uint8_t *blob, size_t nbytes);

/* Replaces `Device::get_tensor` (src/core/ir.rs:131; OpenCL: src/devices/opencl/device.rs:90-102).
 * On ADB_OK, *data / *dims point to handle-owned host memory valid until the next adb_execute or
 * adb_destroy.  ADB_NONE when the id is not in the dep list of the last program. */
adb_status adb_get_tensor(adb_device *dev, const char *id, const float **data,
                          const uint64_t **dims, uint32_t *ndim);

/* Like adb_get_tensor but leaves the data in HBM: *dptr is the device address of the id's buffer
 * (valid until the next adb_execute).  No reference counterpart (the reference always copies back). */
adb_status adb_get_tensor_device(adb_device *dev, const char *id, const float **dptr,
                                 const uint64_t **dims, uint32_t *ndim);

/* Replaces the defaulted `Device::dot_prod_shape` (src/core/ir.rs:140-142): result is [a[0], b[1]]. */
void adb_dot_prod_shape(const uint64_t a[2], const uint64_t b[2], uint64_t out[2]);

/* `Device::ir_callback` (src/core/ir.rs:135) needs no entry point: this backend asks for no IR rewrite. */

const char *adb_last_error(adb_device *dev);

/* Counters of the last adb_execute (the reference only prints a wall-clock time,
 * src/devices/opencl/device.rs:78-80). */
typedef struct adb_stats {
    double device_ms;          /* CUDA-event time of the compute region (first kernel .. last kernel) */
    double upload_ms;          /* host->device copies of CreateMat payloads before / between kernels */
    double readback_ms;        /* device->host copies of dep-list tensors */
    double lower_ms;           /* host time spent lowering + JIT-compiling (0 when the plan was cached) */
    uint64_t h2d_bytes;
    uint64_t d2h_bytes;
    uint64_t kernel_launches;  /* kernels of this library launched (graph replays count their kernel nodes) */
    uint64_t graph_replays;
    uint64_t gemm_launches;
    uint64_t jit_compiles;
    uint64_t arena_bytes;
    uint64_t while_iterations;
    uint64_t ir_commands;
    uint64_t plan_steps;
    /* filled when ADB_FLAG_PROFILE is set: device time, launches and algorithmic work per kernel kind.
     * Bytes are the bytes a kernel must move (each operand once, 4 B per element); flops are 2*M*N*K. */
    double elw_ms, reduce_ms, gemm_ms, collective_ms;
    uint64_t elw_launches, reduce_launches, collective_launches;
    double elw_bytes, reduce_bytes, gemm_flops, collective_bytes;
    /* the single generated kernel with the largest total time */
    double top_ms, top_bytes;
    uint64_t top_launches;
    char top_name[64];
    uint64_t tc_gemm_launches; /* dot products of this execute that ran on the tcgen05 3xTF32 kernel */
} adb_stats;
adb_status adb_get_stats(adb_device *dev, adb_stats *out);

/* Text listing of the lowered program of the last adb_execute (kernels, their fused expressions,
 * buffers): the counterpart of the reference's side-by-side kernel/IR print
 * (src/core/ir.rs:190-192, src/kernel/helper/debug.rs:149-217).  Returns the number of bytes needed. */
size_t adb_dump_plan(adb_device *dev, char *buf, size_t cap);

/* Host-only entry points (work without a GPU; used by the CPU test-suite). */

/* Lowers a blob and JIT-compiles every generated kernel for sm_100a without running anything.
 * Writes the plan listing (and, with `with_source`, the generated CUDA) into buf. */
adb_status adb_lower_check(const uint8_t *blob, size_t nbytes, const adb_config *cfg, int with_source,
                           char *buf, size_t cap, size_t *needed, char *err, size_t err_cap);

/* Data-parallel rewrite used when world_size > 1 (no reference counterpart; the reference is
 * single-device): splits dim 0 of CreateMat tensors whose dim 0 == cfg->shard_batch (or exactly those named in
 * cfg->shard_ids) across cfg->world_size ranks and inserts AllReduce commands where batch-partial values meet
 * replicated ones.  Writes rank cfg->rank's blob into out (cap bytes); *needed receives its size. */
adb_status adb_shard_ir(const uint8_t *blob, size_t nbytes, const adb_config *cfg, uint8_t *out, size_t cap,
                        size_t *needed, char *err, size_t err_cap);

/* Diagnostic (no reference counterpart): writes `code` into the status word through which the tensor-core dot
 * kernels report a bounded wait that ran out.  The next adb_execute that launches such a kernel then fails with
 * ADB_ERR_CUDA exactly as it would after a real time-out (and clears the word), which lets the host side of that
 * error path be tested without a kernel that actually waits for something that never comes. */
adb_status adb_inject_dot_status(adb_device *dev, int code);

/* 128-byte NCCL unique id for adb_config.nccl_unique_id (rank 0 creates, the caller broadcasts it). */
adb_status adb_nccl_unique_id(void *out128);

/* No counterpart in the reference.  Row sums (out[r] = sum of in[r*len .. r*len+len)) of a row-major
 * f32 matrix resident in HBM, for callers that cannot allocate device memory at the point of the call
 * (host callbacks, code running while a capture is open, processes whose memory belongs to another
 * pool): the scratch of the two-pass sum lives in a fixed device array inside the library, so the call
 * performs no cudaMalloc / cudaFree and uses no allocating routine.
 *   - limit: rows <= ADB_NOALLOC_MAX_PARTIALS (the array holds that many floats, 4 MiB, on every GPU
 *     that loads the library, until exit); larger inputs return ADB_ERR_INVALID with a message in err.
 *   - the first call on a device resolves the array's address and should happen before any stream
 *     capture starts.
 *   - all calls share the array: calls that overlap on the GPU race; calls ordered on one stream are safe
 *     and need no clearing in between (each call only reads partial sums it wrote itself).
 * d_in / d_out are device pointers, `stream` a cudaStream_t (NULL = default stream); the call is
 * asynchronous with respect to the host. */
#define ADB_NOALLOC_MAX_PARTIALS (1u << 20)
adb_status adb_row_sum_noalloc(const float *d_in, float *d_out, uint64_t rows, uint64_t len, void *stream,
                               char *err, size_t err_cap);

const char *adb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ADB200_H */
