//! Rust bindings of the CUDA batch-distance bridge (libann_cuda, sm_100a).
//!
//! Takes the place of `rust_lib/src/metal_ffi.rs` in the reference: the three
//! `diskann_metal_*` symbols keep their names and signatures
//! (src/include/metal_diskann_bridge.h:8-23), so `disk_provider.rs` and
//! `provider.rs` call `metal_batch_distances` / `metal_multi_batch_distances`
//! exactly as before.  New here: a device-resident table handle, so the search
//! loops can pass row ids instead of gathering rows on the host
//! (disk_provider.rs:420-424, 592-600).
//!
//! This file is source only in this repository: there is no Rust toolchain in the
//! build image.  The same calls are exercised from Python (ctypes) and C++.

use std::os::raw::{c_char, c_int, c_uint, c_void};
use std::sync::atomic::{AtomicI32, Ordering};

#[repr(C)]
pub struct DiskannCudaTable {
    _private: [u8; 0],
}

extern "C" {
    fn diskann_metal_available() -> c_int;
    fn diskann_metal_batch_distances(
        query: *const f32,
        candidates: *const f32,
        n: c_int,
        dim: c_int,
        metric: c_int,
        out_distances: *mut f32,
    ) -> c_int;
    fn diskann_metal_multi_batch_distances(
        queries: *const f32,
        candidates: *const f32,
        query_map: *const c_uint,
        total_n: c_int,
        nq: c_int,
        dim: c_int,
        metric: c_int,
        out_distances: *mut f32,
    ) -> c_int;

    fn diskann_cuda_last_error() -> *const c_char;
    fn diskann_cuda_register_table(
        device: c_int,
        host_rows: *const f32,
        num: usize,
        dim: c_int,
        out: *mut *mut DiskannCudaTable,
    ) -> c_int;
    fn diskann_cuda_register_sq8(
        device: c_int,
        codes: *const u8,
        mins: *const f32,
        scale: *const f32,
        num: usize,
        dim: c_int,
        out: *mut *mut DiskannCudaTable,
    ) -> c_int;
    fn diskann_cuda_unregister(table: *mut DiskannCudaTable) -> c_int;
    fn diskann_cuda_batch_distances_by_id(
        table: *const DiskannCudaTable,
        queries: *const f32,
        nq: c_int,
        ids: *const u32,
        query_map: *const u32,
        total_n: c_int,
        metric: c_int,
        out_distances: *mut f32,
    ) -> c_int;
    #[allow(dead_code)]
    fn diskann_cuda_batch_distances_by_id_device(
        table: *const DiskannCudaTable,
        queries: *const f32,
        nq: c_int,
        ids: *const u32,
        query_map: *const u32,
        total_n: c_int,
        metric: c_int,
        out_distances: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    #[allow(dead_code)]
    fn diskann_cuda_batch_distances_by_id_device_multi(
        table: *const DiskannCudaTable,
        batches: *const DiskannCudaBatch,
        nbatches: c_int,
        metric: c_int,
        stream: *mut c_void,
    ) -> c_int;
}

/// `struct diskann_cuda_index_info`: header and segment offsets of a serialized index.
#[repr(C)]
#[derive(Default, Debug, Clone)]
#[allow(dead_code)]
pub struct DiskannCudaIndexInfo {
    pub num_vectors: u32,
    pub dimension: u32,
    pub max_degree: u32,
    pub num_entry_points: u32,
    pub build_complexity: u32,
    pub metric: u32,
    pub entry_points_offset: u64,
    pub vectors_offset: u64,
    pub adjacency_offset: u64,
    pub standard_size: u64,
    pub has_sq8: c_int,
    pub sq8_min_offset: u64,
    pub sq8_scale_offset: u64,
    pub sq8_codes_offset: u64,
    pub sq8_codes_size: u64,
}

extern "C" {
    /// Registers the vector segment (and the SQ8 trailer, if present) of the bytes written by
    /// `InMemoryIndex::serialize_to_bytes` / `file_format::write_index` as device tables.
    #[allow(dead_code)]
    fn diskann_cuda_load_index(
        device: c_int,
        image: *const u8,
        len: usize,
        info: *mut DiskannCudaIndexInfo,
        vectors: *mut *mut DiskannCudaTable,
        sq8: *mut *mut DiskannCudaTable,
    ) -> c_int;
}

/// `struct diskann_cuda_batch`: one batch of a multi-batch launch, device pointers.
#[repr(C)]
#[allow(dead_code)]
pub struct DiskannCudaBatch {
    pub queries: *const f32,
    pub ids: *const u32,
    pub query_map: *const u32,
    pub out_distances: *mut f32,
    pub nq: c_int,
    pub total_n: c_int,
}

/// -1 = not probed yet, 0 = no usable GPU, 1 = available.
static GPU_STATUS: AtomicI32 = AtomicI32::new(-1);

/// Smallest `n * dim` worth a launch plus two PCIe copies in the iterative search
/// loops.  The Metal bridge needs 131072 because a command buffer costs
/// 100-450 us; a CUDA launch with small pageable copies costs ~20-30 us.
pub const MIN_GPU_WORK: usize = 65536;

/// Threshold for one-shot callers (`vector_distances()`).
pub const MIN_GPU_WORK_ONESHOT: usize = 32768;

/// Cached availability probe.  The name is kept so callers need no change.
pub fn is_metal_available() -> bool {
    let s = GPU_STATUS.load(Ordering::Relaxed);
    if s >= 0 {
        return s == 1;
    }
    let a = unsafe { diskann_metal_available() };
    GPU_STATUS.store(a, Ordering::Relaxed);
    a == 1
}

/// One query against `n` gathered rows.  `true` means `out[..n]` holds the
/// distances; `false` means the caller must use its CPU loop (batch too small,
/// no GPU, or the call failed).
pub fn metal_batch_distances(
    query: &[f32],
    candidates: &[f32],
    n: usize,
    dim: usize,
    metric: u8,
    out: &mut [f32],
) -> bool {
    if n == 0 || dim == 0 {
        return true;
    }
    if n * dim < MIN_GPU_WORK || !is_metal_available() {
        return false;
    }
    debug_assert_eq!(candidates.len(), n * dim);
    debug_assert!(out.len() >= n);
    let rc = unsafe {
        diskann_metal_batch_distances(
            query.as_ptr(),
            candidates.as_ptr(),
            n as c_int,
            dim as c_int,
            metric as c_int,
            out.as_mut_ptr(),
        )
    };
    rc == 0
}

/// Lock-step batch: row `i` is scored against `queries[query_map[i]]`.  The
/// caller decides whether the batch is large enough.
pub fn metal_multi_batch_distances(
    queries: &[f32],
    candidates: &[f32],
    query_map: &[u32],
    total_n: usize,
    nq: usize,
    dim: usize,
    metric: u8,
    out: &mut [f32],
) -> bool {
    if total_n == 0 || nq == 0 || dim == 0 {
        return true;
    }
    if !is_metal_available() {
        return false;
    }
    debug_assert_eq!(queries.len(), nq * dim);
    debug_assert_eq!(candidates.len(), total_n * dim);
    debug_assert_eq!(query_map.len(), total_n);
    debug_assert!(out.len() >= total_n);
    let rc = unsafe {
        diskann_metal_multi_batch_distances(
            queries.as_ptr(),
            candidates.as_ptr(),
            query_map.as_ptr(),
            total_n as c_int,
            nq as c_int,
            dim as c_int,
            metric as c_int,
            out.as_mut_ptr(),
        )
    };
    rc == 0
}

/// A vector table kept in GPU memory and scored by row id.
pub struct DeviceTable {
    handle: *mut DiskannCudaTable,
    pub num: usize,
    pub dim: usize,
}

// The C side takes a private stream and staging buffers per call.
unsafe impl Send for DeviceTable {}
unsafe impl Sync for DeviceTable {}

impl DeviceTable {
    /// Uploads the fp32 table of a provider (`num * dim` floats, row-major).
    pub fn from_rows(device: i32, rows: &[f32], num: usize, dim: usize) -> Option<Self> {
        if !is_metal_available() || rows.len() != num * dim {
            return None;
        }
        let mut h: *mut DiskannCudaTable = std::ptr::null_mut();
        let rc = unsafe { diskann_cuda_register_table(device, rows.as_ptr(), num, dim as c_int, &mut h) };
        if rc == 0 { Some(DeviceTable { handle: h, num, dim }) } else { None }
    }

    /// Uploads an SQ8 table: codes plus `SQ8Params` min / scale (provider.rs:25-38).
    pub fn from_sq8(device: i32, codes: &[u8], mins: &[f32], scale: &[f32], num: usize, dim: usize) -> Option<Self> {
        if !is_metal_available() || codes.len() != num * dim || mins.len() != dim || scale.len() != dim {
            return None;
        }
        let mut h: *mut DiskannCudaTable = std::ptr::null_mut();
        let rc = unsafe {
            diskann_cuda_register_sq8(device, codes.as_ptr(), mins.as_ptr(), scale.as_ptr(), num, dim as c_int, &mut h)
        };
        if rc == 0 { Some(DeviceTable { handle: h, num, dim }) } else { None }
    }

    /// `out[i] = distance(queries[query_map[i]], row ids[i])`; `false` -> CPU loop.
    pub fn batch_distances_by_id(
        &self,
        queries: &[f32],
        nq: usize,
        ids: &[u32],
        query_map: &[u32],
        metric: u8,
        out: &mut [f32],
    ) -> bool {
        if ids.is_empty() {
            return true;
        }
        debug_assert_eq!(queries.len(), nq * self.dim);
        debug_assert_eq!(ids.len(), query_map.len());
        debug_assert!(out.len() >= ids.len());
        let rc = unsafe {
            diskann_cuda_batch_distances_by_id(
                self.handle,
                queries.as_ptr(),
                nq as c_int,
                ids.as_ptr(),
                query_map.as_ptr(),
                ids.len() as c_int,
                metric as c_int,
                out.as_mut_ptr(),
            )
        };
        rc == 0
    }

    /// Text of the calling thread's last failure.
    pub fn last_error() -> String {
        unsafe { std::ffi::CStr::from_ptr(diskann_cuda_last_error()).to_string_lossy().into_owned() }
    }
}

impl Drop for DeviceTable {
    fn drop(&mut self) {
        unsafe {
            diskann_cuda_unregister(self.handle);
        }
    }
}
