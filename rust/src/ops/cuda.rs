//! `ops::cuda` -- the B200 (sm_100a) backend of the reference's MoE dispatch layer.
//!
//! Same function names, argument meaning and error behaviour as the Metal wrappers it stands beside
//! (`mv_id::mul_mv_id` src/ops/mv_id.rs:37, `mv_id::mul_mv` :54, `mm_id::mul_mm_id` src/ops/mm_id.rs:16,
//! `mm_id::prepare_map0` :27, `mm_id::mul_mm_id_shared` :32, `mm_id::supported` :48, `combine::combine`
//! src/ops/combine.rs:16, `silu_mul::silu_mul` src/ops/silu_mul.rs:14), over the C ABI of `lmoe.h`; plus the
//! fused runner `CudaFusedExperts`, an `ExpertFfn` (src/moe.rs:19-21) that `MoeBlock` (src/moe.rs:28-79) can
//! hold in place of `FusedExperts`, and `CudaMoeBlock`, the whole block in one call.
//!
//! Every op is asynchronous on the device's stream, returns a fresh device tensor and reports shape or dtype
//! mismatches as `Err` before anything is launched, like the reference's ops.  There is no CPU fallback.
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain, no candle source there): it
//! is the text a maintainer adds as `src/ops/cuda.rs`, with `pub mod cuda;` in `src/ops/mod.rs` and the
//! `build.rs` that sits beside this tree.  The candle calls are written against candle-core 0.11's CUDA
//! backend (`CudaStorage::as_cuda_slice`, cudarc `DevicePtr`); adjust to the pinned revision.
#![allow(clippy::too_many_arguments)]

use std::ffi::{c_void, CStr};
use std::os::raw::c_char;
use std::sync::Arc;

use anyhow::{bail, ensure, Context, Result};
use candle_core::cuda_backend::cudarc::driver::{CudaSlice, DevicePtr};
use candle_core::cuda_backend::CudaDevice;
use candle_core::quantized::GgmlDType;
use candle_core::{DType, Device, Storage, Tensor};

// ------------------------------------------------------------------------------------------ FFI
#[repr(C)]
pub struct LmoeExpertStack {
    _private: [u8; 0],
}
#[repr(C)]
pub struct LmoeLayer {
    _private: [u8; 0],
}

pub const LMOE_Q4_K: i32 = 12;
pub const LMOE_Q6_K: i32 = 14;

extern "C" {
    fn lmoe_last_error() -> *const c_char;
    fn lmoe_mm_id_min_seq() -> i64;
    fn lmoe_expert_stack_wrap(dtype: i32, n_expert: i64, n_out: i64, k: i64, device_base: *const c_void, nbytes: usize,
                              base_off: usize, out: *mut *mut LmoeExpertStack) -> i32;
    fn lmoe_expert_stack_destroy(stack: *mut LmoeExpertStack);
    fn lmoe_route_workspace_bytes(t: i64, n_expert: i64) -> usize;
    fn lmoe_route(router: *const f32, bias: *const f32, x: *const f32, t: i64, hidden: i64, n_expert: i64, top_k: i64,
                  scale: f32, norm: i32, ids_out: *mut u32, weights_out: *mut f32, workspace: *mut c_void,
                  workspace_bytes: usize, stream: *mut c_void) -> i32;
    fn lmoe_mul_mv_id(stack: *const LmoeExpertStack, x: *const f32, t: i64, x_per_row: i64, k: i64, ids: *const u32,
                      t_ids: i64, top_k: i64, out: *mut f32, stream: *mut c_void) -> i32;
    fn lmoe_mul_mv(weight: *const c_void, dtype: i32, n_out: i64, k: i64, x: *const f32, t: i64, out: *mut f32,
                   stream: *mut c_void) -> i32;
    fn lmoe_map0_scratch_bytes(n_expert: i64, t: i64) -> usize;
    fn lmoe_prepare_map0(ids: *const u32, t: i64, top_k: i64, n_expert: i64, scratch: *mut c_void, scratch_bytes: usize,
                         stream: *mut c_void) -> i32;
    fn lmoe_mm_id_supported(dtype: i32, top_k: i64) -> i32;
    fn lmoe_mm_id_workspace_bytes(stack: *const LmoeExpertStack, t: i64, top_k: i64, x_per_row: i64) -> usize;
    fn lmoe_mul_mm_id_shared(stack: *const LmoeExpertStack, x: *const f32, t: i64, x_per_row: i64, k: i64, ids: *const u32,
                             t_ids: i64, top_k: i64, map0_scratch: *const c_void, map_n_expert: i64, map_t: i64,
                             map_top_k: i64, out: *mut f32, workspace: *mut c_void, workspace_bytes: usize,
                             stream: *mut c_void) -> i32;
    fn lmoe_mul_mm_id(stack: *const LmoeExpertStack, x: *const f32, t: i64, x_per_row: i64, k: i64, ids: *const u32,
                      t_ids: i64, top_k: i64, out: *mut f32, workspace: *mut c_void, workspace_bytes: usize,
                      stream: *mut c_void) -> i32;
    fn lmoe_silu_mul(gate: *const f32, up: *const f32, n: i64, out: *mut f32, stream: *mut c_void) -> i32;
    fn lmoe_combine(down: *const f32, col_l2: *const f32, weights: *const f32, seq: i64, top_k: i64, n_out: i64,
                    out: *mut f32, stream: *mut c_void) -> i32;
    fn lmoe_layer_create(hidden: i64, expert_ff: i64, n_expert: i64, top_k: i64, scale: f32, norm: i32, router: *const f32,
                         bias: *const f32, gate: *const LmoeExpertStack, up: *const LmoeExpertStack,
                         down: *const LmoeExpertStack, shared_gate: *const LmoeExpertStack,
                         shared_up: *const LmoeExpertStack, shared_down: *const LmoeExpertStack,
                         out: *mut *mut LmoeLayer) -> i32;
    fn lmoe_layer_destroy(layer: *mut LmoeLayer);
    fn lmoe_layer_workspace_bytes(layer: *const LmoeLayer, max_tokens: i64) -> usize;
    fn lmoe_moe_forward_decode(layer: *const LmoeLayer, x: *const f32, t: i64, out: *mut f32, ids_out: *mut u32,
                               weights_out: *mut f32, workspace: *mut c_void, workspace_bytes: usize,
                               stream: *mut c_void) -> i32;
    fn lmoe_moe_forward_prefill(layer: *const LmoeLayer, x: *const f32, t: i64, out: *mut f32, ids_out: *mut u32,
                                weights_out: *mut f32, workspace: *mut c_void, workspace_bytes: usize,
                                stream: *mut c_void) -> i32;
    fn lmoe_experts_workspace_bytes(layer: *const LmoeLayer, max_tokens: i64) -> usize;
    fn lmoe_experts_forward(layer: *const LmoeLayer, x: *const f32, ids: *const u32, weights: *const f32, t: i64,
                            add_shared: i32, out: *mut f32, workspace: *mut c_void, workspace_bytes: usize,
                            stream: *mut c_void) -> i32;
}

/// Status code of the C ABI -> `anyhow::Error` carrying the library's message, like the `anyhow` strings of
/// src/ops/dispatch.rs:812-847.
fn check(status: i32) -> Result<()> {
    if status == 0 {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(lmoe_last_error()) }.to_string_lossy().into_owned();
    bail!("lmoe status {status}: {msg}")
}

// ----------------------------------------------------------------------------- tensor plumbing
/// Device pointer of a contiguous CUDA tensor of element type `T` (offset applied), with the guard that keeps
/// the storage borrowed while the pointer is in use.
fn dev_ptr<T: candle_core::cuda_backend::CudaDType + candle_core::WithDType>(
    t: &Tensor,
    what: &str,
) -> Result<(u64, impl Drop + '_)> {
    ensure!(t.is_contiguous(), "{what} must be contiguous");
    let (storage, layout) = t.storage_and_layout();
    let ptr = match &*storage {
        Storage::Cuda(cs) => {
            let slice: &CudaSlice<T> = cs.as_cuda_slice::<T>()?;
            *slice.device_ptr() + (layout.start_offset() * std::mem::size_of::<T>()) as u64
        }
        _ => bail!("{what} must be on a CUDA device"),
    };
    Ok((ptr, storage))
}

fn cuda_dev(t: &Tensor) -> Result<CudaDevice> {
    match t.device() {
        Device::Cuda(d) => Ok(d.clone()),
        _ => bail!("tensor is not on a CUDA device; the fused MoE path requires CUDA"),
    }
}

/// The stream every op of this module is enqueued on: the device's own, so ordering against candle's
/// kernels needs no extra synchronisation (the counterpart of the shared command encoder,
/// src/ops/dispatch.rs:891-917).
fn stream_of(dev: &CudaDevice) -> *mut c_void {
    dev.cuda_stream().cu_stream() as *mut c_void
}

fn scratch(dev: &CudaDevice, bytes: usize) -> Result<CudaSlice<u8>> {
    Ok(unsafe { dev.alloc::<u8>(bytes.max(16)) }?)
}

fn ggml_dtype_id(dt: GgmlDType) -> Result<i32> {
    match dt {
        GgmlDType::Q4K => Ok(LMOE_Q4_K),
        GgmlDType::Q6K => Ok(LMOE_Q6_K),
        other => bail!("fused MoE kernels not instantiated for dtype {other:?}"),
    }
}

// ------------------------------------------------------------------------------- ExpertStack
/// Device-resident stacked experts for the CUDA kernels: the raw GGUF super-blocks, `[n_expert, n_out, k/256]`,
/// byte-identical to the file (src/gguf.rs:247-276).  `Weights::expert_stack` builds one per stack by uploading
/// the tensor's bytes once (`CudaDevice::htod_copy`) and keeps it in the reference's `ExpertStack` next to the
/// Metal `buffer` field.
pub struct CudaExpertStack {
    handle: *mut LmoeExpertStack,
    /// owns the bytes the handle points into
    pub bytes: Arc<CudaSlice<u8>>,
    pub base_off: usize,
    pub dtype: GgmlDType,
    pub n_expert: usize,
    pub n_out: usize,
    pub k: usize,
}
unsafe impl Send for CudaExpertStack {}
unsafe impl Sync for CudaExpertStack {}

impl CudaExpertStack {
    pub fn new(bytes: Arc<CudaSlice<u8>>, base_off: usize, dtype: GgmlDType, n_expert: usize, n_out: usize, k: usize) -> Result<Self> {
        let type_size = match dtype {
            GgmlDType::Q4K => 144,
            GgmlDType::Q6K => 210,
            other => bail!("unsupported expert dtype {other:?}"),
        };
        ensure!(k % 256 == 0, "expert stack k ({k}) is not a multiple of the block size 256");
        let nbytes = n_expert * n_out * (k / 256) * type_size;
        let mut handle = std::ptr::null_mut();
        check(unsafe {
            lmoe_expert_stack_wrap(ggml_dtype_id(dtype)?, n_expert as i64, n_out as i64, k as i64,
                                   *bytes.device_ptr() as *const c_void, nbytes, base_off, &mut handle)
        })?;
        Ok(Self { handle, bytes, base_off, dtype, n_expert, n_out, k })
    }
    pub fn handle(&self) -> *const LmoeExpertStack {
        self.handle
    }
}
impl Drop for CudaExpertStack {
    fn drop(&mut self) {
        unsafe { lmoe_expert_stack_destroy(self.handle) }
    }
}

// -------------------------------------------------------------------------------- the ops
/// Shapes of an indexed matmul call, validated like `run_inner` (src/ops/dispatch.rs:812-847).
fn id_shapes(stack: &CudaExpertStack, x: &Tensor, ids: &Tensor) -> Result<(usize, usize, usize, usize)> {
    let (t, x_per_row, k) = x.dims3().context("x must be rank-3 [t, x_per_row, k]")?;
    let (t_ids, top_k) = ids.dims2().context("ids must be rank-2 [t, top_k]")?;
    ensure!(x.dtype() == DType::F32, "x must be f32, got {:?}", x.dtype());
    ensure!(ids.dtype() == DType::U32, "ids must be u32, got {:?}", ids.dtype());
    ensure!(k == stack.k, "x k ({k}) does not match expert stack k ({})", stack.k);
    ensure!(t_ids == t, "ids t ({t_ids}) does not match x t ({t})");
    ensure!(x_per_row == 1 || x_per_row == top_k, "x_per_row ({x_per_row}) must be 1 (shared row) or top_k ({top_k}) (per-slot row)");
    Ok((t, x_per_row, k, top_k))
}

/// `ops::mul_mv_id` (src/ops/mv_id.rs:37): x `[t, x_per_row, k]` f32, ids `[t, top_k]` u32 -> `[t, top_k, n_out]` f32.
pub fn mul_mv_id(stack: &CudaExpertStack, x: &Tensor, ids: &Tensor) -> Result<Tensor> {
    let (t, xpr, k, top_k) = id_shapes(stack, x, ids)?;
    let dev = cuda_dev(x)?;
    let out = Tensor::zeros((t, top_k, stack.n_out), DType::F32, x.device())?;
    {
        let (xp, _gx) = dev_ptr::<f32>(x, "x")?;
        let (ip, _gi) = dev_ptr::<u32>(ids, "ids")?;
        let (op, _go) = dev_ptr::<f32>(&out, "out")?;
        check(unsafe {
            lmoe_mul_mv_id(stack.handle(), xp as *const f32, t as i64, xpr as i64, k as i64, ip as *const u32, t as i64,
                           top_k as i64, op as *mut f32, stream_of(&dev))
        })?;
    }
    Ok(out)
}

/// `ops::mul_mv` (src/ops/mv_id.rs:54): plain quantized mat-vec, weight = raw `[n_out, k/256]` super-blocks.
pub fn mul_mv(weight: &CudaSlice<u8>, dtype: GgmlDType, n_out: usize, k: usize, x: &Tensor) -> Result<Tensor> {
    let (t, kx) = x.dims2().context("x must be rank-2 [t, k]")?;
    ensure!(kx == k, "x k ({kx}) does not match weight k ({k})");
    let dev = cuda_dev(x)?;
    let out = Tensor::zeros((t, n_out), DType::F32, x.device())?;
    {
        let (xp, _gx) = dev_ptr::<f32>(x, "x")?;
        let (op, _go) = dev_ptr::<f32>(&out, "out")?;
        check(unsafe {
            lmoe_mul_mv(*weight.device_ptr() as *const c_void, ggml_dtype_id(dtype)?, n_out as i64, k as i64, xp as *const f32,
                        t as i64, op as *mut f32, stream_of(&dev))
        })?;
    }
    Ok(out)
}

/// `Map0Scratch` (src/ops/dispatch.rs:752-757): the per-expert token-slot map plus the geometry it was laid out for.
pub struct Map0Scratch {
    pub buffer: CudaSlice<u8>,
    pub n_expert: usize,
    pub t: usize,
    pub top_k: usize,
}

/// `mm_id::prepare_map0` (src/ops/mm_id.rs:27).
pub fn prepare_map0(n_expert: usize, ids: &Tensor) -> Result<Map0Scratch> {
    let (t, top_k) = ids.dims2().context("ids must be rank-2 [t, top_k]")?;
    ensure!(ids.dtype() == DType::U32, "ids must be u32, got {:?}", ids.dtype());
    let dev = cuda_dev(ids)?;
    let bytes = unsafe { lmoe_map0_scratch_bytes(n_expert as i64, t as i64) };
    let buffer = scratch(&dev, bytes)?;
    {
        let (ip, _gi) = dev_ptr::<u32>(ids, "ids")?;
        check(unsafe {
            lmoe_prepare_map0(ip as *const u32, t as i64, top_k as i64, n_expert as i64, *buffer.device_ptr() as *mut c_void, bytes,
                              stream_of(&dev))
        })?;
    }
    Ok(Map0Scratch { buffer, n_expert, t, top_k })
}

/// `mm_id::supported` (src/ops/mm_id.rs:48): the CUDA build has one variant (f16 operand tiles, f32 accumulation).
pub fn supported(dt: GgmlDType, top_k: usize) -> bool {
    ggml_dtype_id(dt).map(|id| unsafe { lmoe_mm_id_supported(id, top_k as i64) } != 0).unwrap_or(false)
}

/// `mm_id::mul_mm_id_shared` (src/ops/mm_id.rs:32): one projection against a shared map0 scratch.
pub fn mul_mm_id_shared(stack: &CudaExpertStack, x: &Tensor, ids: &Tensor, scratch_map: &Map0Scratch) -> Result<Tensor> {
    let (t, xpr, k, top_k) = id_shapes(stack, x, ids)?;
    let dev = cuda_dev(x)?;
    let ws_bytes = unsafe { lmoe_mm_id_workspace_bytes(stack.handle(), t as i64, top_k as i64, xpr as i64) };
    let ws = scratch(&dev, ws_bytes)?;
    let out = Tensor::zeros((t, top_k, stack.n_out), DType::F32, x.device())?;
    {
        let (xp, _gx) = dev_ptr::<f32>(x, "x")?;
        let (ip, _gi) = dev_ptr::<u32>(ids, "ids")?;
        let (op, _go) = dev_ptr::<f32>(&out, "out")?;
        check(unsafe {
            lmoe_mul_mm_id_shared(stack.handle(), xp as *const f32, t as i64, xpr as i64, k as i64, ip as *const u32, t as i64,
                                  top_k as i64, *scratch_map.buffer.device_ptr() as *const c_void, scratch_map.n_expert as i64,
                                  scratch_map.t as i64, scratch_map.top_k as i64, op as *mut f32,
                                  *ws.device_ptr() as *mut c_void, ws_bytes, stream_of(&dev))
        })?;
    }
    Ok(out)
}

/// `ops::mul_mm_id` (src/ops/mm_id.rs:16): self-contained (runs its own map0 pass).
pub fn mul_mm_id(stack: &CudaExpertStack, x: &Tensor, ids: &Tensor) -> Result<Tensor> {
    let (t, xpr, k, top_k) = id_shapes(stack, x, ids)?;
    let dev = cuda_dev(x)?;
    let ws_bytes = unsafe {
        lmoe_mm_id_workspace_bytes(stack.handle(), t as i64, top_k as i64, xpr as i64) + lmoe_map0_scratch_bytes(stack.n_expert as i64, t as i64)
    };
    let ws = scratch(&dev, ws_bytes)?;
    let out = Tensor::zeros((t, top_k, stack.n_out), DType::F32, x.device())?;
    {
        let (xp, _gx) = dev_ptr::<f32>(x, "x")?;
        let (ip, _gi) = dev_ptr::<u32>(ids, "ids")?;
        let (op, _go) = dev_ptr::<f32>(&out, "out")?;
        check(unsafe {
            lmoe_mul_mm_id(stack.handle(), xp as *const f32, t as i64, xpr as i64, k as i64, ip as *const u32, t as i64, top_k as i64,
                           op as *mut f32, *ws.device_ptr() as *mut c_void, ws_bytes, stream_of(&dev))
        })?;
    }
    Ok(out)
}

/// `ops::silu_mul` (src/ops/silu_mul.rs:14): `(g / (1 + exp(-g))) * u`, same shape, f32.
pub fn silu_mul(gate: &Tensor, up: &Tensor) -> Result<Tensor> {
    ensure!(gate.shape() == up.shape(), "silu_mul: gate {:?} and up {:?} differ in shape", gate.shape(), up.shape());
    ensure!(gate.dtype() == DType::F32 && up.dtype() == DType::F32, "silu_mul: f32 only");
    let dev = cuda_dev(gate)?;
    let out = Tensor::zeros(gate.shape(), DType::F32, gate.device())?;
    {
        let (gp, _g1) = dev_ptr::<f32>(gate, "gate")?;
        let (up_, _g2) = dev_ptr::<f32>(up, "up")?;
        let (op, _g3) = dev_ptr::<f32>(&out, "out")?;
        check(unsafe { lmoe_silu_mul(gp as *const f32, up_ as *const f32, gate.elem_count() as i64, op as *mut f32, stream_of(&dev)) })?;
    }
    Ok(out)
}

/// `ops::combine` (src/ops/combine.rs:16): `out[s, c] = sum_k down[s, k, c] * (col_l2[s, k] * 2^-15) * w[s, k]`.
pub fn combine(down: &Tensor, col_l2: Option<&Tensor>, weights: &Tensor) -> Result<Tensor> {
    let (seq, top_k, n_out) = down.dims3().context("down must be rank-3 [seq, top_k, n_out]")?;
    ensure!(weights.dims2()? == (seq, top_k), "combine: weights must be [seq, top_k]");
    let dev = cuda_dev(down)?;
    let out = Tensor::zeros((seq, n_out), DType::F32, down.device())?;
    {
        let (dp, _g1) = dev_ptr::<f32>(down, "down")?;
        let (wp, _g2) = dev_ptr::<f32>(weights, "weights")?;
        let (op, _g3) = dev_ptr::<f32>(&out, "out")?;
        let l2 = match col_l2 {
            Some(c) => Some(dev_ptr::<f32>(c, "col_l2")?),
            None => None,
        };
        let lp = l2.as_ref().map(|(p, _)| *p as *const f32).unwrap_or(std::ptr::null());
        check(unsafe {
            lmoe_combine(dp as *const f32, lp, wp as *const f32, seq as i64, top_k as i64, n_out as i64, op as *mut f32, stream_of(&dev))
        })?;
    }
    Ok(out)
}

// ------------------------------------------------------------------- the fused runner / block
/// Token count from which the fused entries use the grouped GEMM (`ops::mm_id_min_seq`, src/ops/mod.rs:38;
/// on B200 the default is 65, the reference's `LAGUNA_MM_ID_MIN_SEQ` / `LAGUNA_NO_MM_ID` switches apply).
pub fn mm_id_min_seq() -> usize {
    unsafe { lmoe_mm_id_min_seq() }.clamp(1, i64::MAX) as usize
}

/// One MoE layer on the device: the handle the fused entries take.  Borrows router / bias / stacks; they are
/// kept alive by the fields below.
pub struct CudaLayer {
    handle: *mut LmoeLayer,
    hidden: usize,
    top_k: usize,
    _router: Tensor,
    _bias: Option<Tensor>,
    _stacks: Vec<Arc<CudaExpertStack>>,
}
unsafe impl Send for CudaLayer {}

impl CudaLayer {
    /// router `[n_expert, hidden]` f32 (the GGUF `ffn_gate_inp` orientation, NOT the transposed copy of
    /// src/moe.rs:43), bias `[n_expert]` or None, stacks as `FusedExperts::new` / `SharedExpert::new` load them.
    pub fn new(hidden: usize, expert_ff: usize, n_expert: usize, top_k: usize, scale: f32, norm: bool, router: Tensor,
               bias: Option<Tensor>, gate: Arc<CudaExpertStack>, up: Arc<CudaExpertStack>, down: Arc<CudaExpertStack>,
               shared: Option<[Arc<CudaExpertStack>; 3]>) -> Result<Self> {
        let mut handle = std::ptr::null_mut();
        {
            let (rp, _g1) = dev_ptr::<f32>(&router, "router")?;
            let b = match &bias {
                Some(b) => Some(dev_ptr::<f32>(b, "exp_probs_b")?),
                None => None,
            };
            let bp = b.as_ref().map(|(p, _)| *p as *const f32).unwrap_or(std::ptr::null());
            let (sg, su, sd) = match &shared {
                Some([g, u, d]) => (g.handle(), u.handle(), d.handle()),
                None => (std::ptr::null(), std::ptr::null(), std::ptr::null()),
            };
            check(unsafe {
                lmoe_layer_create(hidden as i64, expert_ff as i64, n_expert as i64, top_k as i64, scale, norm as i32, rp as *const f32, bp,
                                  gate.handle(), up.handle(), down.handle(), sg, su, sd, &mut handle)
            })?;
        }
        let mut stacks = vec![gate, up, down];
        if let Some(s) = shared {
            stacks.extend(s);
        }
        Ok(Self { handle, hidden, top_k, _router: router, _bias: bias, _stacks: stacks })
    }
}
impl Drop for CudaLayer {
    fn drop(&mut self) {
        unsafe { lmoe_layer_destroy(self.handle) }
    }
}

/// `ExpertFfn` over the fused kernels: what `MoeBlock::experts` holds when the model is built with
/// `ExpertRunner::Fused` on a CUDA device (src/moe.rs:46-54).  `MoeBlock::forward` (src/moe.rs:73-78) is
/// unchanged: it routes, calls `forward(x, ids, weights)` and adds the shared expert.
pub struct CudaFusedExperts {
    pub layer: Arc<CudaLayer>,
}

impl crate::moe::ExpertFfn for CudaFusedExperts {
    fn forward(&self, x: &Tensor, ids: &Tensor, weights: &Tensor) -> Result<Tensor> {
        let (seq, hidden) = x.dims2()?;
        ensure!(hidden == self.layer.hidden, "x hidden ({hidden}) does not match the layer's ({})", self.layer.hidden);
        ensure!(ids.dims2()? == (seq, self.layer.top_k) && weights.dims2()? == (seq, self.layer.top_k),
                "ids / weights must be [seq, top_k = {}]", self.layer.top_k);
        let x = x.to_dtype(DType::F32)?.contiguous()?;
        let weights = weights.to_dtype(DType::F32)?.contiguous()?;
        let dev = cuda_dev(&x)?;
        let ws_bytes = unsafe { lmoe_experts_workspace_bytes(self.layer.handle, seq as i64) };
        let ws = scratch(&dev, ws_bytes)?;
        let out = Tensor::zeros((seq, hidden), DType::F32, x.device())?;
        {
            let (xp, _g1) = dev_ptr::<f32>(&x, "x")?;
            let (ip, _g2) = dev_ptr::<u32>(ids, "ids")?;
            let (wp, _g3) = dev_ptr::<f32>(&weights, "weights")?;
            let (op, _g4) = dev_ptr::<f32>(&out, "out")?;
            check(unsafe {
                lmoe_experts_forward(self.layer.handle, xp as *const f32, ip as *const u32, wp as *const f32, seq as i64, 0,
                                     op as *mut f32, *ws.device_ptr() as *mut c_void, ws_bytes, stream_of(&dev))
            })?;
        }
        Ok(out)
    }
}

/// The whole block in one call (route + routed experts + shared expert): `MoeBlock::forward`, src/moe.rs:73-78.
/// Decode batches (< `mm_id_min_seq()` tokens) run one cooperative kernel per 64 tokens; longer inputs the
/// grouped-GEMM path.  Returns the output and, when asked, the routing decision (`MoeBlock::route`, src/moe.rs:62-71).
pub struct CudaMoeBlock {
    pub layer: Arc<CudaLayer>,
}

impl CudaMoeBlock {
    pub fn forward(&self, x_normed: &Tensor) -> Result<Tensor> {
        let (seq, hidden) = x_normed.dims2()?;
        let x = x_normed.to_dtype(DType::F32)?.contiguous()?;
        let dev = cuda_dev(&x)?;
        let ws_bytes = unsafe { lmoe_layer_workspace_bytes(self.layer.handle, seq as i64) };
        let ws = scratch(&dev, ws_bytes)?;
        let out = Tensor::zeros((seq, hidden), DType::F32, x.device())?;
        {
            let (xp, _g1) = dev_ptr::<f32>(&x, "x")?;
            let (op, _g2) = dev_ptr::<f32>(&out, "out")?;
            let f = if seq >= mm_id_min_seq() { lmoe_moe_forward_prefill } else { lmoe_moe_forward_decode };
            check(unsafe {
                f(self.layer.handle, xp as *const f32, seq as i64, op as *mut f32, std::ptr::null_mut(), std::ptr::null_mut(),
                  *ws.device_ptr() as *mut c_void, ws_bytes, stream_of(&dev))
            })?;
        }
        Ok(out)
    }
}

/// `MoeBlock::route` on the device (src/moe.rs:62-71, 84-119): ids `[seq, top_k]` u32, weights `[seq, top_k]` f32.
pub fn route(router: &Tensor, bias: Option<&Tensor>, x_normed: &Tensor, top_k: usize, scale: f32, norm: bool) -> Result<(Tensor, Tensor)> {
    let (seq, hidden) = x_normed.dims2()?;
    let (n_expert, h2) = router.dims2()?;
    ensure!(h2 == hidden, "router is [n_expert, {h2}], x is [seq, {hidden}]");
    let dev = cuda_dev(x_normed)?;
    let ids = Tensor::zeros((seq, top_k), DType::U32, x_normed.device())?;
    let w = Tensor::zeros((seq, top_k), DType::F32, x_normed.device())?;
    let ws_bytes = unsafe { lmoe_route_workspace_bytes(seq as i64, n_expert as i64) };
    let ws = scratch(&dev, ws_bytes)?;
    {
        let (rp, _g1) = dev_ptr::<f32>(router, "router")?;
        let (xp, _g2) = dev_ptr::<f32>(x_normed, "x")?;
        let (ip, _g3) = dev_ptr::<u32>(&ids, "ids")?;
        let (wp, _g4) = dev_ptr::<f32>(&w, "weights")?;
        let b = match bias {
            Some(b) => Some(dev_ptr::<f32>(b, "exp_probs_b")?),
            None => None,
        };
        let bp = b.as_ref().map(|(p, _)| *p as *const f32).unwrap_or(std::ptr::null());
        check(unsafe {
            lmoe_route(rp as *const f32, bp, xp as *const f32, seq as i64, hidden as i64, n_expert as i64, top_k as i64, scale,
                       norm as i32, ip as *mut u32, wp as *mut f32, *ws.device_ptr() as *mut c_void, ws_bytes, stream_of(&dev))
        })?;
    }
    Ok((ids, w))
}
