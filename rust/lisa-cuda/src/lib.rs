//! Safe wrappers over `lisa-cuda-sys` with the signatures `lisa-engine` dispatches through, so that the
//! crate drops in behind `lisa_mlx::ops::{quantized_matmul, gather_qmm, dequantize, quantize}` and
//! `lisa_mlx::models::deepseek41::{packed_matvec, expert_matvec}` for the quantized-weight matmul path.
//!
//! Not compiled in this repository (the build image has no Rust toolchain); the C header is the source of
//! truth.  `Array` here is the minimum the path needs of the reference's `ops::array::Array` (device buffer +
//! shape + dtype, contiguous, offset applied): an engine that keeps its own array type implements `DeviceArray`
//! for it instead of using this one.  The callee allocates outputs from the engine's pool, as the reference
//! does (`buffer_for_gpu_write`); the library itself never allocates.
use std::ffi::CStr;
use std::os::raw::{c_int, c_void};

use lisa_cuda_sys as sys;

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Dtype {
    Bfloat16,
    Float16,
    Float32,
    Uint32,
    Uint8,
    Int32,
}

impl Dtype {
    fn code(self) -> Result<c_int> {
        match self {
            Dtype::Bfloat16 => Ok(sys::LISA_BF16),
            Dtype::Float16 => Ok(sys::LISA_F16),
            Dtype::Float32 => Ok(sys::LISA_F32),
            other => Err(Error::Msg(format!("unsupported compute dtype {other:?}"))),
        }
    }
    pub fn size_of(self) -> usize {
        match self {
            Dtype::Bfloat16 | Dtype::Float16 => 2,
            Dtype::Float32 | Dtype::Uint32 | Dtype::Int32 => 4,
            Dtype::Uint8 => 1,
        }
    }
}

/// Mirrors `lisa_mlx::error::Error::Msg`: unsupported modes are refused before anything is enqueued.
#[derive(Debug)]
pub enum Error {
    Msg(String),
}
pub type Result<T> = std::result::Result<T, Error>;

fn check(rc: c_int) -> Result<()> {
    if rc == sys::LISA_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(sys::lisa_cuda_last_error_string()) }.to_string_lossy().into_owned();
    Err(Error::Msg(msg))
}

/// What the wrappers need from an engine's array type.
pub trait DeviceArray: Sized {
    fn device_ptr(&self) -> *const c_void;
    fn shape(&self) -> &[i64];
    fn dtype(&self) -> Dtype;
    /// A contiguous array of `shape` and `dtype` from the engine's buffer pool.
    fn alloc(shape: &[i64], dtype: Dtype) -> Result<Self>;
    fn device_ptr_mut(&mut self) -> *mut c_void;
}

/// The stream every call is ordered on (`cudaStream_t`); the reference's `Stream::thread_local_or_default()`.
#[derive(Clone, Copy)]
pub struct Stream(pub *mut c_void);

fn rows_of(shape: &[i64]) -> i64 {
    shape[..shape.len() - 1].iter().product()
}

/// `ops::quantized_matmul(x, w, scales, biases, transpose, group_size, bits)`,
/// crates/lisa-mlx/src/ops/array_ops.rs:378-493.
pub fn quantized_matmul<A: DeviceArray>(stream: Stream, x: &A, w: &A, scales: &A, biases: Option<&A>, transpose: bool,
                                        group_size: i32, bits: i32) -> Result<A> {
    let k = *x.shape().last().unwrap();
    let m = rows_of(x.shape());
    let n = w.shape()[0];
    let mut shape = x.shape().to_vec();
    *shape.last_mut().unwrap() = n;
    let mut y = A::alloc(&shape, x.dtype())?;
    check(unsafe {
        sys::lisa_cuda_quantized_matmul(stream.0, x.device_ptr(), m, k, w.device_ptr() as *const u32, scales.device_ptr(),
                                        biases.map_or(std::ptr::null(), |b| b.device_ptr()), n, transpose as c_int, group_size,
                                        bits, x.dtype().code()?, y.device_ptr_mut())
    })?;
    Ok(y)
}

/// `ops::quantized_matmul_serial_rows`, array_ops.rs:500-555: x `[rows, 1, K]`.
pub fn quantized_matmul_serial_rows<A: DeviceArray>(stream: Stream, x: &A, w: &A, scales: &A, biases: Option<&A>,
                                                    transpose: bool, group_size: i32, bits: i32) -> Result<A> {
    let k = *x.shape().last().unwrap();
    let rows = rows_of(x.shape());
    let n = w.shape()[0];
    let mut shape = x.shape().to_vec();
    *shape.last_mut().unwrap() = n;
    let mut y = A::alloc(&shape, x.dtype())?;
    check(unsafe {
        sys::lisa_cuda_quantized_matmul_serial_rows(stream.0, x.device_ptr(), rows, k, w.device_ptr() as *const u32,
                                                    scales.device_ptr(), biases.map_or(std::ptr::null(), |b| b.device_ptr()), n,
                                                    transpose as c_int, group_size, bits, x.dtype().code()?, y.device_ptr_mut())
    })?;
    Ok(y)
}

/// `ops::dequantize(w, scales, biases, group_size, bits)`, array_ops.rs:37-84: output dtype = scales dtype.
pub fn dequantize<A: DeviceArray>(stream: Stream, w: &A, scales: &A, biases: &A, group_size: i32, bits: i32) -> Result<A> {
    let kq = *w.shape().last().unwrap();
    let k = kq * 32 / bits as i64;
    let rows = rows_of(w.shape());
    let mut shape = w.shape().to_vec();
    *shape.last_mut().unwrap() = k;
    let mut out = A::alloc(&shape, scales.dtype())?;
    check(unsafe {
        sys::lisa_cuda_dequantize(stream.0, w.device_ptr() as *const u32, scales.device_ptr(), biases.device_ptr(), rows, k,
                                  group_size, bits, scales.dtype().code()?, out.device_ptr_mut())
    })?;
    Ok(out)
}

/// `ops::quantize(w, group_size, bits)`, array_ops.rs:218-290: `(wq, scales, biases)`.
pub fn quantize<A: DeviceArray>(stream: Stream, w: &A, group_size: Option<i32>, bits: Option<i32>) -> Result<(A, A, A)> {
    let (gs, bits) = (group_size.unwrap_or(64), bits.unwrap_or(4));
    let k = *w.shape().last().unwrap();
    let rows = rows_of(w.shape());
    let lead = &w.shape()[..w.shape().len() - 1];
    let with_last = |last: i64| lead.iter().copied().chain(std::iter::once(last)).collect::<Vec<_>>();
    let mut wq = A::alloc(&with_last(k * bits as i64 / 32), Dtype::Uint32)?;
    let mut sc = A::alloc(&with_last(k / gs as i64), w.dtype())?;
    let mut bi = A::alloc(&with_last(k / gs as i64), w.dtype())?;
    check(unsafe {
        sys::lisa_cuda_quantize(stream.0, w.device_ptr(), rows, k, gs, bits, w.dtype().code()?, wq.device_ptr_mut() as *mut u32,
                                sc.device_ptr_mut(), bi.device_ptr_mut())
    })?;
    Ok((wq, sc, bi))
}

/// `ops::gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, transpose, group_size, bits, sorted_indices)`,
/// array_ops.rs:561-642.  `workspace` comes from the engine's pool
/// (`lisa_cuda_gather_qmm_workspace_bytes(rows, experts)` bytes).
#[allow(clippy::too_many_arguments)]
pub fn gather_qmm<A: DeviceArray>(stream: Stream, x: &A, w: &A, scales: &A, biases: Option<&A>, lhs_indices: Option<&A>,
                                  rhs_indices: Option<&A>, transpose: bool, group_size: i32, bits: i32, sorted_indices: bool,
                                  workspace: &mut A) -> Result<A> {
    let k = *x.shape().last().unwrap();
    let rows = rows_of(x.shape());
    let experts = w.shape()[0];
    let n = w.shape()[w.shape().len() - 2];
    let mut shape = x.shape().to_vec();
    *shape.last_mut().unwrap() = n;
    let mut y = A::alloc(&shape, x.dtype())?;
    let ws_bytes = workspace.shape().iter().product::<i64>() as usize * workspace.dtype().size_of();
    check(unsafe {
        sys::lisa_cuda_gather_qmm(stream.0, x.device_ptr(), rows, k, w.device_ptr() as *const u32, scales.device_ptr(),
                                  biases.map_or(std::ptr::null(), |b| b.device_ptr()),
                                  lhs_indices.map_or(std::ptr::null(), |a| a.device_ptr() as *const i32),
                                  rhs_indices.map_or(std::ptr::null(), |a| a.device_ptr() as *const i32), experts, n,
                                  transpose as c_int, group_size, bits, sorted_indices as c_int, x.dtype().code()?,
                                  y.device_ptr_mut(), workspace.device_ptr_mut(), ws_bytes)
    })?;
    Ok(y)
}

/// `deepseek41::BlockFormat`, crates/lisa-mlx/src/models/deepseek41.rs:23-44 (the formats on this path).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum BlockFormat {
    Q2K,
    Q4K,
    Q5K,
}
impl BlockFormat {
    fn code(self) -> c_int {
        match self {
            BlockFormat::Q2K => sys::LISA_GGUF_Q2_K,
            BlockFormat::Q4K => sys::LISA_GGUF_Q4_K,
            BlockFormat::Q5K => sys::LISA_GGUF_Q5_K,
        }
    }
    pub fn block_bytes(self) -> i64 {
        match self {
            BlockFormat::Q2K => 84,
            BlockFormat::Q4K => 144,
            BlockFormat::Q5K => 176,
        }
    }
}

/// `deepseek41::packed_matvec(format, weights, input)`, deepseek41.rs:93-110: weights `Uint8 [rows, row_bytes]`,
/// input f32 `[tokens, K]` -> f32 `[tokens, rows]`.
pub fn packed_matvec<A: DeviceArray>(stream: Stream, format: BlockFormat, weights: &A, input: &A) -> Result<A> {
    let (rows, row_bytes) = (weights.shape()[0], weights.shape()[1]);
    let tokens = input.shape()[0];
    let mut y = A::alloc(&[tokens, rows], Dtype::Float32)?;
    check(unsafe {
        sys::lisa_cuda_gguf_packed_matvec(stream.0, format.code(), weights.device_ptr() as *const u8, rows, row_bytes,
                                          input.device_ptr() as *const f32, tokens, y.device_ptr_mut() as *mut f32)
    })?;
    Ok(y)
}

/// `deepseek41::expert_matvec(format, weights, input, ids)`, deepseek41.rs:204-283: weights `[E, rows, row_bytes]`,
/// input f32 `[tokens, slots, K]`, ids i32 `[tokens, top_k]` -> f32 `[tokens, top_k, rows]`.
pub fn expert_matvec<A: DeviceArray>(stream: Stream, format: BlockFormat, weights: &A, input: &A, ids: &A) -> Result<A> {
    let (experts, rows, row_bytes) = (weights.shape()[0], weights.shape()[1], weights.shape()[2]);
    let (tokens, top_k) = (ids.shape()[0], ids.shape()[1]);
    let slots = input.shape()[1];
    let mut y = A::alloc(&[tokens, top_k, rows], Dtype::Float32)?;
    check(unsafe {
        sys::lisa_cuda_gguf_expert_matvec(stream.0, format.code(), weights.device_ptr() as *const u8, experts, rows, row_bytes,
                                          input.device_ptr() as *const f32, tokens, slots, ids.device_ptr() as *const i32, top_k,
                                          y.device_ptr_mut() as *mut f32)
    })?;
    Ok(y)
}

/// `QuantizedEmbedding::forward`, crates/lisa-engine/src/core/quant.rs:449-455: ids i32 `[..]` -> `[.., K]`.
pub fn dequantize_rows<A: DeviceArray>(stream: Stream, w: &A, scales: &A, biases: &A, ids: &A, group_size: i32, bits: i32) -> Result<A> {
    let vocab = w.shape()[0];
    let k = *w.shape().last().unwrap() * 32 / bits as i64;
    let count: i64 = ids.shape().iter().product();
    let mut shape = ids.shape().to_vec();
    shape.push(k);
    let mut out = A::alloc(&shape, scales.dtype())?;
    check(unsafe {
        sys::lisa_cuda_dequantize_rows(stream.0, w.device_ptr() as *const u32, scales.device_ptr(), biases.device_ptr(),
                                       ids.device_ptr() as *const i32, count, vocab, k, group_size, bits, scales.dtype().code()?,
                                       out.device_ptr_mut())
    })?;
    Ok(out)
}

/// `affine_qmv_fast_addnorm` and its sibling form (crates/lisa-mlx/src/jit/matmul.rs:304-577): residual add +
/// RMSNorm + one to three linears on the normed rows.  Returns `(outputs, sum, normed)`; `write_norm = false` is
/// accepted for the decode shapes that run as one launch.
#[allow(clippy::too_many_arguments)]
pub fn quantized_matmul_addnorm<A: DeviceArray>(stream: Stream, x: &A, r: &A, norm_weight: &A, linears: &[(&A, &A, &A)], eps: f32,
                                                group_size: i32, bits: i32, write_norm: bool) -> Result<(Vec<A>, A, Option<A>)> {
    let k = *x.shape().last().unwrap();
    let m: i64 = x.shape().iter().product::<i64>() / k;
    let mut ys = Vec::with_capacity(linears.len());
    for (w, _, _) in linears {
        ys.push(A::alloc(&[m, w.shape()[0]], x.dtype())?);
    }
    let mut sum = A::alloc(&[m, k], x.dtype())?;
    let mut normed = if write_norm { Some(A::alloc(&[m, k], x.dtype())?) } else { None };
    let w: Vec<*const u32> = linears.iter().map(|l| l.0.device_ptr() as *const u32).collect();
    let s: Vec<*const c_void> = linears.iter().map(|l| l.1.device_ptr()).collect();
    let b: Vec<*const c_void> = linears.iter().map(|l| l.2.device_ptr()).collect();
    let n: Vec<i64> = linears.iter().map(|l| l.0.shape()[0]).collect();
    let y: Vec<*mut c_void> = ys.iter_mut().map(|a| a.device_ptr_mut()).collect();
    check(unsafe {
        sys::lisa_cuda_quantized_matmul_addnorm(stream.0, x.device_ptr(), r.device_ptr(), norm_weight.device_ptr(), eps, m, k,
                                                linears.len() as c_int, w.as_ptr(), s.as_ptr(), b.as_ptr(), n.as_ptr(), 1,
                                                group_size, bits, x.dtype().code()?, y.as_ptr(), sum.device_ptr_mut(),
                                                normed.as_mut().map_or(std::ptr::null_mut(), |a| a.device_ptr_mut()),
                                                sys::LISA_FLAG_PDL)
    })?;
    Ok((ys, sum, normed))
}

/// SwiGLU in front of a linear: `swiglu(gate, up) . dequant(w)^T` (the down projection of an MLP; rounding points of
/// crates/lisa-mlx/src/shaders/common/exact_header.metal:2-11).  Returns `(y, act)`; `write_act = false` is accepted
/// for the decode shapes that run as one launch.
#[allow(clippy::too_many_arguments)]
pub fn quantized_matmul_swiglu<A: DeviceArray>(stream: Stream, gate: &A, up: &A, w: &A, scales: &A, biases: &A, group_size: i32,
                                               bits: i32, write_act: bool) -> Result<(A, Option<A>)> {
    let k = *gate.shape().last().unwrap();
    let m: i64 = gate.shape().iter().product::<i64>() / k;
    let n = w.shape()[0];
    let mut y = A::alloc(&[m, n], gate.dtype())?;
    let mut act = if write_act { Some(A::alloc(&[m, k], gate.dtype())?) } else { None };
    check(unsafe {
        sys::lisa_cuda_quantized_matmul_swiglu(stream.0, gate.device_ptr(), up.device_ptr(), m, k, w.device_ptr() as *const u32,
                                               scales.device_ptr(), biases.device_ptr(), n, 1, group_size, bits,
                                               gate.dtype().code()?, y.device_ptr_mut(),
                                               act.as_mut().map_or(std::ptr::null_mut(), |a| a.device_ptr_mut()), sys::LISA_FLAG_PDL)
    })?;
    Ok((y, act))
}

/// `moe_decode::gate_up_act` (crates/lisa-mlx/src/models/qwen4/moe_decode.rs:136-184) without the shared
/// expert: `x [tokens, hidden]`, `idx [tokens, top_k]`, gate / up `(w [E, inter, hidden*bits/32], scales,
/// biases)` -> `act [tokens * top_k, inter]`; `xrow` maps slots to rows of `x` (default `slot / top_k`).
#[allow(clippy::too_many_arguments)]
pub fn gate_up_act<A: DeviceArray>(stream: Stream, wg: &A, sg: &A, bg: &A, wu: &A, su: &A, bu: &A, x: &A, idx: &A,
                                   xrow: Option<&A>, group_size: i32, bits: i32) -> Result<A> {
    let (experts, inter) = (wg.shape()[0], wg.shape()[1]);
    let hidden = *x.shape().last().unwrap();
    let top_k = *idx.shape().last().unwrap();
    let slots: i64 = idx.shape().iter().product();
    let mut act = A::alloc(&[slots, inter], x.dtype())?;
    check(unsafe {
        sys::lisa_cuda_moe_gate_up_act(stream.0, x.device_ptr(), idx.device_ptr() as *const i32,
                                       xrow.map_or(std::ptr::null(), |r| r.device_ptr() as *const i32), slots, top_k as c_int,
                                       experts, hidden, inter, wg.device_ptr() as *const u32, sg.device_ptr(), bg.device_ptr(),
                                       wu.device_ptr() as *const u32, su.device_ptr(), bu.device_ptr(), group_size, bits,
                                       x.dtype().code()?, act.device_ptr_mut())
    })?;
    Ok(act)
}

/// `moe_decode::down_combine` (moe_decode.rs:214-298) without the shared expert and its gate: `act [tokens *
/// top_k, inter]`, `idx` / `w [tokens, top_k]`, down `(w [E, hidden, inter*bits/32], scales, biases)` ->
/// `[tokens, hidden]`.
#[allow(clippy::too_many_arguments)]
pub fn down_combine<A: DeviceArray>(stream: Stream, wd: &A, sd: &A, bd: &A, act: &A, idx: &A, w: &A, group_size: i32,
                                    bits: i32) -> Result<A> {
    let (experts, hidden) = (wd.shape()[0], wd.shape()[1]);
    let inter = *act.shape().last().unwrap();
    let (tokens, top_k) = (idx.shape()[0], idx.shape()[1]);
    let mut out = A::alloc(&[tokens, hidden], act.dtype())?;
    check(unsafe {
        sys::lisa_cuda_moe_down_combine(stream.0, act.device_ptr(), idx.device_ptr() as *const i32,
                                        w.device_ptr() as *const f32, tokens, top_k as c_int, experts, inter, hidden,
                                        wd.device_ptr() as *const u32, sd.device_ptr(), bd.device_ptr(), group_size, bits,
                                        act.dtype().code()?, out.device_ptr_mut())
    })?;
    Ok(out)
}

/// `detect_group_size`, crates/lisa-engine/src/core/quant.rs:273-287.
pub fn detect_group_size(weight_cols: i32, scales_cols: i32, bits: i32) -> Option<i32> {
    match unsafe { sys::lisa_detect_group_size(weight_cols, scales_cols, bits) } {
        0 => None,
        g => Some(g),
    }
}

/// Non-zero once a kernel has given up on one of its bounded waits; `clear_device_status` resets it.
pub fn device_status() -> i32 {
    unsafe { sys::lisa_cuda_device_status() }
}
pub fn clear_device_status() -> Result<()> {
    check(unsafe { sys::lisa_cuda_clear_device_status() })
}
