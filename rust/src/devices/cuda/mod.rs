//! `impl Device for B200`: the reference's `Device` trait (`src/core/ir.rs:126-143`) over the C-ABI of the B200
//! backend (`include/adb200.h`, `libadb200.so`).  Fills the empty slot `src/devices/cuda/mod.rs:1-17`.
//!
//! NOT COMPILED HERE (no Rust toolchain in the environment this backend was built in).  To use: copy this directory
//! over `src/devices/cuda/` of the reference, add `pub mod cuda; pub use cuda::B200;` to `src/devices/mod.rs`, and link
//! `libadb200.so` (`cargo:rustc-link-lib=dylib=adb200` + its directory in `cargo:rustc-link-search`).
//!
//! The backend lowers the IR itself, so the `KernelProcedure` / `KernelTracker` that `Device::execute` receives are
//! ignored; the IR is captured in `ir_callback`, which `autodiff::execute()` calls right before the IR optimiser and
//! `execute` (`src/core/autodiff.rs:108-114`, `src/core/ir.rs:167-198`).
use std::cell::RefCell;
use std::ffi::{c_char, c_void, CStr, CString};
use std::sync::Arc;

use crate::core::ret_dep_list;
use crate::kernel_decl::KernelProcedure;
use crate::trackers::KernelTracker;
use crate::{Device, IRBase, IRProcedure, ValueData};

pub mod wire;

#[repr(C)]
struct AdbConfig {
    struct_size: u32,
    device_ordinal: i32,
    rank: i32,
    world_size: i32,
    nccl_unique_id: *const c_void,
    flags: u32,
    shard_batch: u64,
    shard_ids: *const *const c_char,
    n_shard_ids: u32,
}

#[link(name = "adb200")]
extern "C" {
    fn adb_create(cfg: *const AdbConfig, out: *mut *mut c_void) -> i32;
    fn adb_destroy(dev: *mut c_void);
    fn adb_execute(dev: *mut c_void, blob: *const u8, n: usize) -> i32;
    fn adb_get_tensor(dev: *mut c_void, id: *const c_char, data: *mut *const f32, dims: *mut *const u64, ndim: *mut u32) -> i32;
    fn adb_last_error(dev: *mut c_void) -> *const c_char;
    fn adb_nccl_unique_id(out128: *mut c_void) -> i32;
}

/// Payloads larger than this travel by address instead of being copied into the blob.
const INLINE_LIMIT: usize = 1 << 16;

/// `adb_config.flags` (include/adb200.h); 0 is the fast path, the rest are switches for debugging, tests and callers
/// with special needs.
pub mod flags {
    pub const NO_GRAPHS: u32 = 1;
    pub const NO_FUSION: u32 = 2;
    pub const SIMT_DOT: u32 = 4;
    pub const PROFILE: u32 = 8;
    pub const COMM_STREAM: u32 = 16;
    pub const SINGLE_SM_DOT: u32 = 32;
    pub const EXACT_DIV: u32 = 64;
    pub const FUSE_SMALL_SUMS: u32 = 128;
    pub const NO_GROUPING: u32 = 256;
    /// dot products never split their k axis over clusters: the same bits on every run
    pub const DETERMINISTIC: u32 = 512;
    pub const SERIAL_GRAPHS: u32 = 1024;
    pub const NO_BUCKETS: u32 = 2048;
    pub const NO_TINY_DOT: u32 = 4096;
    /// accumulate 1024 instead of 4096 k elements per chunk in the dot kernels: 8e-6 instead of 3e-5 of max|C|, 9 % slower
    pub const SHORT_DOT_CHUNKS: u32 = 8192;
}

pub struct B200 {
    h: *mut c_void,
    /// the program captured by `ir_callback`; it owns the `CreateMat` vectors the blob points into
    pending: RefCell<Option<(IRProcedure, Vec<u8>)>>,
}
// the reference keeps its device in a global `Mutex<Option<Box<dyn Device + Send + Sync>>>` and serialises all calls
unsafe impl Send for B200 {}
unsafe impl Sync for B200 {}

impl B200 {
    /// One GPU, no data parallelism.
    pub fn new(ordinal: i32) -> B200 { B200::with_config(ordinal, 0, 1, None, 0, 0) }

    /// One process per GPU: `rank` of `world_size`, the 128-byte NCCL id made on rank 0 (`B200::nccl_unique_id`) and
    /// broadcast by the caller, `shard_batch` = the global batch size (axis 0 of the tensors to split).
    pub fn with_config(ordinal: i32, rank: i32, world_size: i32, nccl_id: Option<&[u8; 128]>, flags: u32, shard_batch: u64) -> B200 {
        let cfg = AdbConfig {
            struct_size: std::mem::size_of::<AdbConfig>() as u32,
            device_ordinal: ordinal,
            rank,
            world_size,
            nccl_unique_id: nccl_id.map_or(std::ptr::null(), |b| b.as_ptr() as *const c_void),
            flags,
            shard_batch,
            shard_ids: std::ptr::null(),
            n_shard_ids: 0,
        };
        let mut h = std::ptr::null_mut();
        let rc = unsafe { adb_create(&cfg, &mut h) };
        assert!(rc == 0, "adb_create failed with status {rc} (a B200 is required; the backend has no CPU path)");
        B200 { h, pending: RefCell::new(None) }
    }

    pub fn nccl_unique_id() -> [u8; 128] {
        let mut id = [0u8; 128];
        let rc = unsafe { adb_nccl_unique_id(id.as_mut_ptr() as *mut c_void) };
        assert!(rc == 0, "adb_nccl_unique_id failed with status {rc}");
        id
    }
}

impl Device for B200 {
    /// The IR as traced, before the reference's optimiser and lowering touch it.
    fn ir_callback(&self, cmds: &mut IRBase) {
        let proc = cmds.proc.clone(); // cheap: CreateMat contents are Arc<Vec<f32>>
        let blob = wire::serialize(&proc, &ret_dep_list(), wire::Payloads::HostPointersAbove(INLINE_LIMIT));
        *self.pending.borrow_mut() = Some((proc, blob));
    }

    fn execute(&mut self, _proc: KernelProcedure, _tracker: KernelTracker) {
        let (_keep_alive, blob) = self.pending.borrow_mut().take().expect("ir_callback runs before execute");
        let rc = unsafe { adb_execute(self.h, blob.as_ptr(), blob.len()) };
        if rc != 0 {
            let msg = unsafe { CStr::from_ptr(adb_last_error(self.h)) }.to_string_lossy().into_owned();
            panic!("adb_execute failed with status {rc}: {msg}"); // the reference's devices panic as well (src/devices/opencl/context.rs:31)
        }
    }

    fn get_tensor(&self, id: &String) -> ValueData {
        let cid = CString::new(id.as_str()).expect("ids contain no NUL");
        let (mut data, mut dims, mut nd) = (std::ptr::null::<f32>(), std::ptr::null::<u64>(), 0u32);
        match unsafe { adb_get_tensor(self.h, cid.as_ptr(), &mut data, &mut dims, &mut nd) } {
            0 => unsafe {
                let dim: Vec<usize> = std::slice::from_raw_parts(dims, nd as usize).iter().map(|&d| d as usize).collect();
                let n: usize = dim.iter().product();
                ValueData { dim, data: Arc::new(std::slice::from_raw_parts(data, n).to_vec()), id: id.clone(), is_none: false }
            },
            _ => ValueData::none(), // the id is not in the dep list (src/core/value_data.rs:6-11)
        }
    }
    // dot_prod_shape: the trait's default ([a[0], b[last]], row-major) is what the backend produces
}

impl Drop for B200 {
    fn drop(&mut self) { unsafe { adb_destroy(self.h) } }
}
