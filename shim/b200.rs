// zyx/src/backend/b200.rs — the Rust side of the B200 backend: binds libzyxb.so (include/zyxb.h) behind zyx's
// enum-dispatched backend interface (zyx/src/backend/mod.rs: MemoryPool 542-803, Device 806-1028).
//
// NOT COMPILED: the image this repository is built in has no Rust toolchain.  The file is written against zyx 0.16
// (backend/cblas.rs is the structural model: an AOT-only device that adds Node::Kernel alternatives in match_graph and
// runs them in launch).  What *is* machine-checked: every #[repr(C)] struct below is parsed by tests/test_abi_loads.py and its
// field offsets are compared with offsetof() of the C header and with the ctypes mirror the parity tests use; the
// matcher (vendor_b200.rs) is a port of zyx_b200/csrc/host/matcher.hpp, which tests/test_matcher.py drives through the C ABI.
//
// Wiring in backend/mod.rs (one arm per method, as for every other backend):
//   mod b200;                                     Config { .., pub b200: b200::B200Config }   (mod.rs:391-414)
//   Event::B200(b200::B200Event)                  MemoryPool::B200(b200::B200MemoryPool)     Device::B200(b200::B200Device)
//   initialize_backends: b200::initialize_device(&config.b200, memory_pools, devices, debug_dev)   (mod.rs:263-331)
//   Device::aot_only: Device::B200(_) => true     (mod.rs:892-894)

use std::collections::BTreeSet;
use std::ffi::{CStr, c_char, c_void};
use std::sync::Arc;

use libloading::Library;
use nanoserde::DeJson;

use super::{BackendError, DTypeCapability, Device, DeviceId, DeviceInfo, DeviceProgramId, ErrorStatus, Event, MemoryPool, PoolBufferId, PoolId,
            ProgramId};
use crate::{
    DType,
    dtype::Constant,
    graph::{ClassId, Graph, Node, NodeData},
    kernel::Kernel,
    shape::Dim,
    slab::Slab,
    Set,
};

// ------------------------------------------------------------------------------------------------------------------
// C structs, field for field as in include/zyxb.h
// ------------------------------------------------------------------------------------------------------------------
#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct ZyxbEvent { pub id: u64 }

#[repr(C)] #[derive(Clone, Copy)]
pub struct ZyxbConfig { pub n_device_ids: i32, pub device_ids: [i32; 16], pub debug: i32, pub round_nearest: i32 }

#[repr(C)] #[derive(Clone, Copy)]
pub struct ZyxbDevinfo { pub compute_flops: u64, pub max_global_work_dims: [u64; 3], pub max_local_threads: u32,
                         pub max_local_work_dims: [u32; 3], pub preferred_vector_size: u32, pub local_mem_size: u64,
                         pub max_register_bytes: u64, pub tensor_cores: i32, pub warp_size: u32, pub dtype_capability: [u32; 13],
                         pub has_native_exp2: i32, pub sm_count: u32, pub total_mem_bytes: u64, pub cc_major: i32, pub cc_minor: i32,
                         pub name: [c_char; 128] }

#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct ZyxbRowreduceDesc { pub op: i32, pub dtype: i32, pub rows: u64, pub cols: u64, pub eps: f32, pub correction: i32,
                               pub has_weight: i32, pub has_bias: i32, pub scale: f32, pub causal: i32, pub period: u64 }

#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct ZyxbGemmDesc { pub dtype: i32, pub m: u64, pub n: u64, pub k: u64, pub batch: u64, pub trans_a: i32, pub trans_b: i32,
                          pub stride_a: i64, pub stride_b: i64, pub stride_c: i64, pub epilogue: i32, pub store_preact: i32,
                          pub alpha: f32, pub lda: u64, pub ldb: u64, pub ldc: u64, pub batch_inner: u64, pub stride_a_inner: i64,
                          pub stride_b_inner: i64, pub stride_c_inner: i64, pub tri: i32 }

#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct ZyxbEltwiseDesc { pub op: i32, pub dtype: i32, pub dtype_out: i32, pub numel: u64, pub cols: u64, pub p0: f32 }

#[repr(C)] #[derive(Clone, Copy)]
pub struct ZyxbOptimDesc { pub algo: i32, pub dtype: i32, pub n_tensors: i32, pub numel: *const u64, pub lr: f32, pub weight_decay: f32,
                           pub momentum: f32, pub dampening: f32, pub nesterov: i32, pub maximize: i32, pub beta1: f32, pub beta2: f32,
                           pub eps: f32, pub grad_scale: f32, pub standard: i32 }

#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct ZyxbAttentionDesc { pub dtype: i32, pub batch: u64, pub heads: u64, pub seq: u64, pub head_dim: u64, pub ld: u64,
                               pub scale: f32, pub causal: i32 }

#[repr(C)] #[derive(Clone, Copy, Default)]
pub struct ZyxbConvDesc { pub dtype: i32, pub n: u64, pub c: u64, pub h: u64, pub w: u64, pub o: u64, pub kh: u64, pub kw: u64,
                          pub stride_h: u32, pub stride_w: u32, pub dil_h: u32, pub dil_w: u32, pub pad_top: u32, pub pad_bottom: u32,
                          pub pad_left: u32, pub pad_right: u32, pub has_bias: i32, pub channels_last: i32, pub flip_filter: i32 }

#[repr(C)] #[derive(Clone, Copy)]
pub union ZyxbDescUnion { pub rowreduce: ZyxbRowreduceDesc, pub gemm: ZyxbGemmDesc, pub eltwise: ZyxbEltwiseDesc, pub optim: ZyxbOptimDesc,
                          pub attention: ZyxbAttentionDesc, pub conv: ZyxbConvDesc }

#[repr(C)] #[derive(Clone, Copy)]
pub struct ZyxbKernelDesc { pub kind: i32, pub u: ZyxbDescUnion }

pub const ZYXB_KIND_ROWREDUCE: i32 = 1;
pub const ZYXB_KIND_GEMM: i32 = 2;
pub const ZYXB_KIND_ELTWISE: i32 = 3;
pub const ZYXB_KIND_OPTIM: i32 = 4;
pub const ZYXB_KIND_ATTENTION: i32 = 5;
pub const ZYXB_KIND_ATTENTION_BWD: i32 = 6;
pub const ZYXB_KIND_CONV: i32 = 7;
pub const ZYXB_KIND_CONV_WGRAD: i32 = 8;
pub const ZYXB_KIND_CONV_DGRAD: i32 = 9;

// ------------------------------------------------------------------------------------------------------------------
// The entry points, resolved once (as CUDAMemoryPool / CblasDevice resolve theirs with libloading)
// ------------------------------------------------------------------------------------------------------------------
type Ctx = *mut c_void;
pub(super) struct Api {
    _lib: Library,
    init: unsafe extern "C" fn(*const ZyxbConfig, *mut Ctx) -> i32,
    shutdown: unsafe extern "C" fn(Ctx) -> i32,
    last_error: unsafe extern "C" fn(Ctx) -> *const c_char,
    device_count: unsafe extern "C" fn(Ctx, *mut i32) -> i32,
    device_info: unsafe extern "C" fn(Ctx, i32, *mut ZyxbDevinfo) -> i32,
    free_compute: unsafe extern "C" fn(Ctx, i32, *mut u64) -> i32,
    free_bytes: unsafe extern "C" fn(Ctx, i32, *mut u64) -> i32,
    alloc: unsafe extern "C" fn(Ctx, i32, u64, *mut u32, *mut ZyxbEvent) -> i32,
    free: unsafe extern "C" fn(Ctx, i32, u32, *const ZyxbEvent, i32) -> i32,
    h2d: unsafe extern "C" fn(Ctx, i32, *const c_void, u64, u32, u64, *const ZyxbEvent, i32, *mut ZyxbEvent) -> i32,
    d2h: unsafe extern "C" fn(Ctx, i32, u32, u64, *mut c_void, u64, *const ZyxbEvent, i32) -> i32,
    d2d: unsafe extern "C" fn(Ctx, i32, u32, u64, i32, u32, u64, u64, *const ZyxbEvent, i32, *mut ZyxbEvent) -> i32,
    buffer_bytes: unsafe extern "C" fn(Ctx, i32, u32, *mut u64) -> i32,
    buffer_view: unsafe extern "C" fn(Ctx, i32, u32, u64, u64, *mut u32) -> i32,
    sync: unsafe extern "C" fn(Ctx, i32, *const ZyxbEvent, i32) -> i32,
    release_events: unsafe extern "C" fn(Ctx, i32, *const ZyxbEvent, i32) -> i32,
    store_variable: unsafe extern "C" fn(Ctx, i32, i32, *const c_void, *mut u32) -> i32,
    get_variable: unsafe extern "C" fn(Ctx, i32, u32, *mut i32, *mut c_void) -> i32,
    program_create: unsafe extern "C" fn(Ctx, i32, *const ZyxbKernelDesc, *mut u32) -> i32,
    launch: unsafe extern "C" fn(Ctx, i32, u32, *const u32, i32, *const ZyxbEvent, i32, *mut ZyxbEvent) -> i32,
    program_release: unsafe extern "C" fn(Ctx, i32, u32) -> i32,
    program_set_step: unsafe extern "C" fn(Ctx, i32, u32, u64) -> i32,
}

impl Api {
    fn load(path: &str) -> Result<Api, BackendError> {
        let lib = unsafe { Library::new(path) }?;       // From<libloading::Error> for BackendError (mod.rs:257-261): DyLibNotFound
        macro_rules! sym { ($name:literal) => { *unsafe { lib.get($name) }? } }
        Ok(Api {
            init: sym!(b"zyxb_init\0"), shutdown: sym!(b"zyxb_shutdown\0"), last_error: sym!(b"zyxb_last_error\0"),
            device_count: sym!(b"zyxb_device_count\0"), device_info: sym!(b"zyxb_device_info\0"), free_compute: sym!(b"zyxb_free_compute\0"),
            free_bytes: sym!(b"zyxb_free_bytes\0"), alloc: sym!(b"zyxb_alloc\0"), free: sym!(b"zyxb_free\0"), h2d: sym!(b"zyxb_h2d\0"),
            d2h: sym!(b"zyxb_d2h\0"), d2d: sym!(b"zyxb_d2d\0"), buffer_bytes: sym!(b"zyxb_buffer_bytes\0"), buffer_view: sym!(b"zyxb_buffer_view\0"), sync: sym!(b"zyxb_sync\0"),
            release_events: sym!(b"zyxb_release_events\0"), store_variable: sym!(b"zyxb_store_variable\0"),
            get_variable: sym!(b"zyxb_get_variable\0"), program_create: sym!(b"zyxb_program_create\0"), launch: sym!(b"zyxb_launch\0"),
            program_release: sym!(b"zyxb_program_release\0"), program_set_step: sym!(b"zyxb_program_set_step\0"),
            _lib: lib,
        })
    }
}

/// One libzyxb context shared by every pool and device of the process.
struct Shared { api: Api, ctx: Ctx }
unsafe impl Send for Shared {}
unsafe impl Sync for Shared {}
impl Drop for Shared {
    fn drop(&mut self) { unsafe { (self.api.shutdown)(self.ctx) }; }
}

/// Status codes are 1 + the ordinal of ErrorStatus (error.rs:127-153).
fn check(sh: &Shared, status: i32) -> Result<(), BackendError> {
    const STATUSES: [ErrorStatus; 13] = [
        ErrorStatus::DyLibNotFound, ErrorStatus::Initialization, ErrorStatus::Deinitialization, ErrorStatus::DeviceEnumeration,
        ErrorStatus::DeviceQuery, ErrorStatus::MemoryAllocation, ErrorStatus::MemoryDeallocation, ErrorStatus::MemoryCopyH2P,
        ErrorStatus::MemoryCopyP2H, ErrorStatus::IncorrectKernelArg, ErrorStatus::KernelCompilation, ErrorStatus::KernelLaunch,
        ErrorStatus::KernelSync,
    ];
    if status == 0 {
        return Ok(());
    }
    let text = unsafe { CStr::from_ptr((sh.api.last_error)(sh.ctx)) }.to_string_lossy().into_owned();
    let status = STATUSES.get((status - 1) as usize).copied().unwrap_or(ErrorStatus::KernelLaunch);
    Err(BackendError { status, context: text.into() })
}

// ------------------------------------------------------------------------------------------------------------------
// Config, events
// ------------------------------------------------------------------------------------------------------------------
/// `"b200": {"enabled": true, "device_ids": [0, 1], "library": "/path/to/libzyxb.so", "round_nearest": false}` in config.json
#[derive(DeJson, Debug, Default)]
pub struct B200Config {
    pub enabled: bool,
    /// None: every visible B200 (CUDAConfig::device_ids has the same meaning, cuda.rs:142-148)
    pub device_ids: Option<Vec<i32>>,
    pub library: Option<String>,
    /// false (default): bf16 / f16 stores truncate like the C backend (codegen/c.rs:475-496)
    pub round_nearest: bool,
}

/// An event handle of the library; id 0 is "already complete".
#[derive(Debug, Clone, Copy)]
pub struct B200Event(pub ZyxbEvent);

fn raw_events(events: Vec<Event>) -> Vec<ZyxbEvent> {
    // events are moved into the callee, which consumes them (mod.rs:658-662); foreign events cannot reach this pool
    events.into_iter().filter_map(|e| if let Event::B200(B200Event(ev)) = e { (ev.id != 0).then_some(ev) } else { None }).collect()
}
fn ptr_len(evs: &[ZyxbEvent]) -> (*const ZyxbEvent, i32) {
    if evs.is_empty() { (std::ptr::null(), 0) } else { (evs.as_ptr(), evs.len() as i32) }
}

// ------------------------------------------------------------------------------------------------------------------
// Memory pool (one per GPU)
// ------------------------------------------------------------------------------------------------------------------
pub struct B200MemoryPool { sh: Arc<Shared>, dev: i32 }

impl std::fmt::Debug for B200MemoryPool {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "B200MemoryPool(dev {})", self.dev) }
}

impl B200MemoryPool {
    pub fn deinitialize(&mut self) {}     // the context goes with the last Arc<Shared>

    pub fn free_bytes(&self) -> Dim {
        let mut bytes = 0u64;
        unsafe { (self.sh.api.free_bytes)(self.sh.ctx, self.dev, &mut bytes) };
        bytes
    }

    /// `bytes` already includes the caller's slack (mod.rs:627).
    pub fn allocate(&mut self, bytes: Dim) -> Result<(PoolBufferId, Event), BackendError> {
        let (mut id, mut ev) = (0u32, ZyxbEvent::default());
        check(&self.sh, unsafe { (self.sh.api.alloc)(self.sh.ctx, self.dev, bytes, &mut id, &mut ev) })?;
        Ok((PoolBufferId::from(id as usize), Event::B200(B200Event(ev))))
    }

    pub fn deallocate(&mut self, buffer_id: PoolBufferId, event_wait_list: Vec<Event>) {
        let evs = raw_events(event_wait_list);
        let (p, n) = ptr_len(&evs);
        let _ = check(&self.sh, unsafe { (self.sh.api.free)(self.sh.ctx, self.dev, usize::from(buffer_id) as u32, p, n) });
    }

    /// Asynchronous: `src` must stay valid until the returned event has been synced (the rule at runtime.rs:1-16).
    pub fn host_to_pool(&mut self, src: &[u8], dst: PoolBufferId, event_wait_list: Vec<Event>) -> Result<Event, BackendError> {
        let evs = raw_events(event_wait_list);
        let (p, n) = ptr_len(&evs);
        let mut out = ZyxbEvent::default();
        check(&self.sh, unsafe {
            (self.sh.api.h2d)(self.sh.ctx, self.dev, src.as_ptr().cast(), src.len() as u64, usize::from(dst) as u32, 0, p, n, &mut out)
        })?;
        Ok(Event::B200(B200Event(out)))
    }

    /// Blocking.
    pub fn pool_to_host(&mut self, src: PoolBufferId, dst: &mut [u8], event_wait_list: Vec<Event>) -> Result<(), BackendError> {
        let evs = raw_events(event_wait_list);
        let (p, n) = ptr_len(&evs);
        check(&self.sh, unsafe {
            (self.sh.api.d2h)(self.sh.ctx, self.dev, usize::from(src) as u32, 0, dst.as_mut_ptr().cast(), dst.len() as u64, p, n)
        })
    }

    pub fn pool_to_pool(&mut self, src_pool: &mut MemoryPool, src: PoolBufferId, dst: PoolBufferId, event_wait_list: Vec<Event>)
        -> Result<Event, BackendError> {
        let evs = raw_events(event_wait_list);
        let (p, n) = ptr_len(&evs);
        match src_pool {
            MemoryPool::B200(sp) => {
                let mut bytes = 0u64;
                check(&self.sh, unsafe { (self.sh.api.buffer_bytes)(self.sh.ctx, sp.dev, usize::from(src) as u32, &mut bytes) })?;
                let mut out = ZyxbEvent::default();
                check(&self.sh, unsafe {
                    (self.sh.api.d2d)(self.sh.ctx, sp.dev, usize::from(src) as u32, 0, self.dev, usize::from(dst) as u32, 0, bytes, p, n, &mut out)
                })?;
                Ok(Event::B200(B200Event(out)))
            }
            other => {
                // through the host, like the other backends' cross-pool copies
                let mut bytes = 0u64;
                check(&self.sh, unsafe { (self.sh.api.buffer_bytes)(self.sh.ctx, self.dev, usize::from(dst) as u32, &mut bytes) })?;
                let mut staging = vec![0u8; bytes as usize];
                other.pool_to_host(src, &mut staging, Vec::new())?;
                let ev = self.host_to_pool(&staging, dst, Vec::new())?;
                self.sync_events(vec![ev])?;        // staging dies here
                Ok(Event::B200(B200Event(ZyxbEvent::default())))
            }
        }
    }

    pub fn sync_events(&mut self, events: Vec<Event>) -> Result<(), BackendError> {
        let evs = raw_events(events);
        let (p, n) = ptr_len(&evs);
        check(&self.sh, unsafe { (self.sh.api.sync)(self.sh.ctx, self.dev, p, n) })
    }

    pub fn release_events(&mut self, events: Vec<Event>) {
        let evs = raw_events(events);
        let (p, n) = ptr_len(&evs);
        unsafe { (self.sh.api.release_events)(self.sh.ctx, self.dev, p, n) };
    }

    /// Scalars passed by value (mod.rs:597-621).
    pub fn store_variable(&mut self, scalar: Constant) -> PoolBufferId {
        let (dtype, bytes): (DType, [u8; 8]) = constant_le_bytes(scalar);
        let mut id = 0u32;
        unsafe { (self.sh.api.store_variable)(self.sh.ctx, self.dev, dtype as i32, bytes.as_ptr().cast(), &mut id) };
        PoolBufferId::from(id as usize)
    }

    pub fn get_variable(&mut self, buffer_id: PoolBufferId) -> Option<Constant> {
        let (mut dtype, mut bytes) = (0i32, [0u8; 8]);
        let st = unsafe { (self.sh.api.get_variable)(self.sh.ctx, self.dev, usize::from(buffer_id) as u32, &mut dtype, bytes.as_mut_ptr().cast()) };
        (st == 0).then(|| constant_from_le_bytes(dtype, bytes))
    }
}

fn constant_le_bytes(c: Constant) -> (DType, [u8; 8]) {
    let mut b = [0u8; 8];
    let dt = match c {
        Constant::BF16(x) => { b[..2].copy_from_slice(&x); DType::BF16 }
        Constant::F16(x) => { b[..2].copy_from_slice(&x); DType::F16 }
        Constant::F32(x) => { b[..4].copy_from_slice(&x); DType::F32 }
        Constant::F64(x) => { b.copy_from_slice(&x); DType::F64 }
        Constant::U8(x) => { b[0] = x; DType::U8 }
        Constant::U16(x) => { b[..2].copy_from_slice(&x.to_le_bytes()); DType::U16 }
        Constant::U32(x) => { b[..4].copy_from_slice(&x.to_le_bytes()); DType::U32 }
        Constant::U64(x) => { b.copy_from_slice(&x); DType::U64 }
        Constant::I8(x) => { b[0] = x as u8; DType::I8 }
        Constant::I16(x) => { b[..2].copy_from_slice(&x.to_le_bytes()); DType::I16 }
        Constant::I32(x) => { b[..4].copy_from_slice(&x.to_le_bytes()); DType::I32 }
        Constant::I64(x) => { b.copy_from_slice(&x); DType::I64 }
        Constant::Bool(x) => { b[0] = x as u8; DType::Bool }
    };
    (dt, b)
}

fn constant_from_le_bytes(dtype: i32, b: [u8; 8]) -> Constant {
    // the order of DType (dtype.rs:18-32) is the order of the ZYXB_* dtype codes
    match dtype {
        0 => Constant::BF16([b[0], b[1]]), 1 => Constant::F16([b[0], b[1]]), 2 => Constant::F32([b[0], b[1], b[2], b[3]]), 3 => Constant::F64(b),
        4 => Constant::U8(b[0]), 5 => Constant::U16(u16::from_le_bytes([b[0], b[1]])), 6 => Constant::U32(u32::from_le_bytes([b[0], b[1], b[2], b[3]])),
        7 => Constant::U64(b), 8 => Constant::I8(b[0] as i8), 9 => Constant::I16(i16::from_le_bytes([b[0], b[1]])),
        10 => Constant::I32(i32::from_le_bytes([b[0], b[1], b[2], b[3]])), 11 => Constant::I64(b), _ => Constant::Bool(b[0] != 0),
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Device
// ------------------------------------------------------------------------------------------------------------------
pub struct B200Device {
    sh: Arc<Shared>,
    dev: i32,
    device_info: DeviceInfo,
    device_id: DeviceId,
    memory_pool_id: PoolId,
    programs: Slab<DeviceProgramId, ProgramEntry>,
}

/// What the device keeps per program beside the library's handle.
#[derive(Clone, Default)]
struct ProgramEntry {
    handle: u32,
    /// buffers the device itself appends to every launch: the fused attention program writes its log-sum-exp
    /// [batch*heads, seq] f32 behind the output, and the graph has no class for it
    scratch: Vec<u32>,
    /// an optimizer program updates its tensors where they lie, while the graph hands the launch fresh buffers for p', m', v'
    /// (args = loads ++ stores) and still owns the old values: the launch copies p, m, v into the stores first and runs the
    /// program on the copies
    in_place: Option<InPlace>,
    /// (argument index, byte offset): arguments that are slices of their buffer (q of a fused q/k/v projection); the launch
    /// passes a view of the buffer from that byte on
    slices: Vec<(usize, u64)>,
}
#[derive(Clone, Copy)]
struct InPlace {
    tensors: usize,
    /// state tensors per parameter: 0 plain SGD, 1 SGD with momentum (the buffer), 2 Adam / AdamW (m, v)
    states: usize,
    /// false on a first step: the loads are p.., g.. only and the program writes the state without reading it
    reads_state: bool,
}

impl std::fmt::Debug for B200Device {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "B200Device(dev {})", self.dev) }
}

pub(super) fn initialize_device(
    config: &B200Config,
    memory_pools: &mut Slab<PoolId, MemoryPool>,
    devices: &mut Slab<DeviceId, Device>,
    debug_dev: bool,
) -> Result<(), BackendError> {
    if !config.enabled {
        if debug_dev {
            println!("[b200] configured out");
        }
        return Ok(());
    }
    let api = Api::load(config.library.as_deref().unwrap_or("libzyxb.so"))?;
    let mut c = ZyxbConfig { n_device_ids: 0, device_ids: [0; 16], debug: debug_dev as i32, round_nearest: config.round_nearest as i32 };
    if let Some(ids) = &config.device_ids {
        c.n_device_ids = ids.len().min(16) as i32;
        c.device_ids[..c.n_device_ids as usize].copy_from_slice(&ids[..c.n_device_ids as usize]);
    }
    let mut ctx: Ctx = std::ptr::null_mut();
    let st = unsafe { (api.init)(&c, &mut ctx) };
    if st != 0 {
        // no CPU fallback: without a compute-capability-10 device the backend reports DeviceEnumeration and zyx skips it (mod.rs:289-293)
        let text = unsafe { CStr::from_ptr((api.last_error)(std::ptr::null_mut())) }.to_string_lossy().into_owned();
        return Err(BackendError { status: ErrorStatus::DeviceEnumeration, context: text.into() });
    }
    let sh = Arc::new(Shared { api, ctx });
    let mut n = 0i32;
    check(&sh, unsafe { (sh.api.device_count)(sh.ctx, &mut n) })?;
    for dev in 0..n {
        let mut info: ZyxbDevinfo = unsafe { std::mem::zeroed() };
        check(&sh, unsafe { (sh.api.device_info)(sh.ctx, dev, &mut info) })?;
        let memory_pool_id = memory_pools.push(MemoryPool::B200(B200MemoryPool { sh: sh.clone(), dev }));
        let mut dtype_capability = [DTypeCapability::none(); DType::N_DTYPES];
        for (slot, bits) in dtype_capability.iter_mut().zip(info.dtype_capability) {
            *slot = DTypeCapability::from_bits(bits);
        }
        let device_id = devices.push(Device::B200(B200Device {
            sh: sh.clone(),
            dev,
            device_info: DeviceInfo {
                compute: u128::from(info.compute_flops),
                max_global_work_dims: info.max_global_work_dims.to_vec(),
                max_local_threads: info.max_local_threads as Dim,
                max_local_work_dims: info.max_local_work_dims.iter().map(|&d| Dim::from(d)).collect(),
                preferred_vector_size: info.preferred_vector_size as u8,
                local_mem_size: info.local_mem_size,
                max_register_bytes: info.max_register_bytes,
                tensor_cores: info.tensor_cores != 0,
                warp_size: info.warp_size as u8,
                dtype_capability,
                has_native_exp2: info.has_native_exp2 != 0,
                supported_vec_lens: vec![2, 4, 8],
            },
            device_id: DeviceId::NULL,
            memory_pool_id,
            programs: Slab::new(),
        }));
        if let Device::B200(d) = &mut devices[device_id] {
            d.device_id = device_id;      // Node::Kernel carries ProgramId { device, program } (cblas.rs:168-177)
        }
        if debug_dev {
            let name = unsafe { CStr::from_ptr(info.name.as_ptr()) }.to_string_lossy();
            println!("[b200] device {dev}: {name}, {} SMs, {} MiB", info.sm_count, info.total_mem_bytes >> 20);
        }
    }
    Ok(())
}

impl B200Device {
    pub fn deinitialize(&mut self) {}
    pub const fn info(&self) -> &DeviceInfo { &self.device_info }
    pub const fn memory_pool_id(&self) -> PoolId { self.memory_pool_id }
    pub const fn aot_only(&self) -> bool { true }

    pub fn free_compute(&self) -> u128 {
        let mut flops = 0u64;
        unsafe { (self.sh.api.free_compute)(self.sh.ctx, self.dev, &mut flops) };
        u128::from(flops)
    }

    /// Programs come from descriptors, never from zyx IR (as CblasDevice::compile, cblas.rs:203-208).
    pub fn compile(&mut self, _kernel: &Kernel, _debug_asm: bool) -> Result<DeviceProgramId, BackendError> {
        Err(BackendError { status: ErrorStatus::KernelCompilation, context: "b200 device runs descriptor programs only (aot_only)".into() })
    }

    pub fn release(&mut self, program_id: DeviceProgramId) {
        let ProgramEntry { handle, scratch, .. } = self.programs[program_id].clone();
        unsafe { (self.sh.api.program_release)(self.sh.ctx, self.dev, handle) };
        for buffer in scratch {
            unsafe { (self.sh.api.free)(self.sh.ctx, self.dev, buffer, std::ptr::null(), 0) };
        }
        self.programs.remove(program_id);
    }

    /// The e-graph hook (mod.rs:952-961).  `graph.match_b200` (vendor_b200.rs) recognises the subgraphs; each becomes a program
    /// and a Node::Kernel alternative in every class it produces, `time: 1` so that extraction prefers it (cblas.rs:213-238).
    pub fn match_graph(&mut self, graph: &mut Graph, outputs: &BTreeSet<ClassId>) {
        let order = graph.topo_sort_classes_without_kernels(&Set::default(), outputs, None);
        for m in graph.match_b200(&order, outputs) {
            let mut desc = m.desc;
            if desc.kind == ZYXB_KIND_OPTIM {
                unsafe { desc.u.optim.numel = m.numel.as_ptr() };      // copied by the library at program creation
            }
            let mut handle = 0u32;
            let st = unsafe { (self.sh.api.program_create)(self.sh.ctx, self.dev, &desc, &mut handle) };
            if st != 0 {
                continue;       // a shape the library refuses stays with whatever else can produce the class
            }
            if m.optim_step > 0 {
                // an optimizer program's own counter says whether state is read and which bias correction applies
                unsafe { (self.sh.api.program_set_step)(self.sh.ctx, self.dev, handle, m.optim_step - 1) };
            }
            let mut entry = ProgramEntry { handle, ..Default::default() };
            if desc.kind == ZYXB_KIND_OPTIM {
                let tensors = unsafe { desc.u.optim.n_tensors } as usize;
                let states = m.outputs.len() / tensors - 1;
                entry.in_place = Some(InPlace { tensors, states, reads_state: m.inputs.len() > 2 * tensors });
            }
            if desc.kind == ZYXB_KIND_GEMM {
                let es: u64 = if unsafe { desc.u.gemm.dtype } == DType::F32 as i32 || unsafe { desc.u.gemm.dtype } == DType::I32 as i32 { 4 } else { 2 };
                entry.slices = m.input_offsets.iter().enumerate().filter(|&(_, &o)| o != 0).map(|(i, &o)| (i, o * es)).collect();
            }
            if desc.kind == ZYXB_KIND_ATTENTION {
                let a = unsafe { desc.u.attention };
                let (mut lse, mut ev) = (0u32, ZyxbEvent::default());
                if unsafe { (self.sh.api.alloc)(self.sh.ctx, self.dev, a.batch * a.heads * a.seq * 4, &mut lse, &mut ev) } != 0 {
                    unsafe { (self.sh.api.program_release)(self.sh.ctx, self.dev, handle) };
                    continue;
                }
                entry.scratch.push(lse);
            }
            let program = self.programs.push(entry);
            let nid = graph.nodes.push(NodeData {
                node: Node::Kernel {
                    inputs: m.inputs.clone().into_boxed_slice(),
                    outputs: m.outputs.clone().into_boxed_slice(),
                    program_id: ProgramId { device: self.device_id, program },
                    time: 1,
                },
                class_of: m.outputs[0],
            });
            for &out in &m.outputs {
                graph.classes[out].nodes.push(nid);
            }
        }
    }

    /// args = loads then stores (mod.rs:974, runtime.rs:2285-2291).
    pub fn launch(&mut self, program_id: DeviceProgramId, memory_pool: &mut B200MemoryPool, args: &[PoolBufferId], event_wait_list: Vec<Event>)
        -> Result<Event, BackendError> {
        let _ = memory_pool;        // buffer ids are the library's own handles
        let evs = raw_events(event_wait_list);
        let (p, n) = ptr_len(&evs);
        let entry = self.programs[program_id].clone();
        let mut ids: Vec<u32> = args.iter().map(|&a| usize::from(a) as u32).chain(entry.scratch.iter().copied()).collect();
        let (mut p, mut n) = (p, n);
        let mut views = Vec::new();
        for &(arg, byte_offset) in &entry.slices {
            let (mut bytes, mut view) = (0u64, 0u32);
            check(&self.sh, unsafe { (self.sh.api.buffer_bytes)(self.sh.ctx, self.dev, ids[arg], &mut bytes) })?;
            check(&self.sh, unsafe { (self.sh.api.buffer_view)(self.sh.ctx, self.dev, ids[arg], byte_offset, bytes - byte_offset, &mut view) })?;
            ids[arg] = view;
            views.push(view);
        }
        if let Some(InPlace { tensors: t, states, reads_state }) = entry.in_place {
            // loads p.., g.. [, state0.., state1..]; stores (p', state0', state1') per tensor.  The copies and the launch run in
            // order on the device's compute stream; the first copy takes the wait list.
            let loads = t * (2 + if reads_state { states } else { 0 });
            let store = |i: usize, s: usize| ids[loads + i * (1 + states) + s];
            let mut copies = Vec::new();
            for i in 0..t {
                copies.push((ids[i], store(i, 0)));
                if reads_state { for s in 0..states { copies.push((ids[(2 + s) * t + i], store(i, 1 + s))); } }
            }
            for (src, dst) in copies {
                let (mut bytes, mut ev) = (0u64, ZyxbEvent::default());
                check(&self.sh, unsafe { (self.sh.api.buffer_bytes)(self.sh.ctx, self.dev, src, &mut bytes) })?;
                check(&self.sh, unsafe { (self.sh.api.d2d)(self.sh.ctx, self.dev, src, 0, self.dev, dst, 0, bytes, p, n, &mut ev) })?;
                unsafe { (self.sh.api.release_events)(self.sh.ctx, self.dev, &ev, 1) };
                (p, n) = (std::ptr::null(), 0);
            }
            // what the program takes: p'.., g.., state0'.., state1'..
            ids = (0..t).map(|i| store(i, 0)).chain(ids[t..2 * t].iter().copied())
                .chain((0..states).flat_map(|s| (0..t).map(move |i| (i, s))).map(|(i, s)| store(i, 1 + s))).collect();
        }
        let mut out = ZyxbEvent::default();
        let launched = check(&self.sh, unsafe {
            (self.sh.api.launch)(self.sh.ctx, self.dev, entry.handle, ids.as_ptr(), ids.len() as i32, p, n, &mut out)
        });
        for view in views {             // a view is a name for a range of its parent: releasing it frees nothing
            unsafe { (self.sh.api.free)(self.sh.ctx, self.dev, view, std::ptr::null(), 0) };
        }
        launched?;
        Ok(Event::B200(B200Event(out)))
    }
}
