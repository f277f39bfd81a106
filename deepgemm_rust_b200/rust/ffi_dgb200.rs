//! Rust binding of libdgb200.so (C ABI in include/dgb200.h) that keeps the host surface of
//! idrees2516/deepgemm-rust for the block-scaled FP8 / FP4 GEMM path: the same type and function
//! names, argument order and error type as deepgemm/src/ops_sm100.rs, deepgemm/src/ops.rs (the
//! f32-scale calls), deepgemm/src/device.rs (DgContext) and deepgemm/src/heuristics_sm100.rs.
//!
//! A maintainer drops this file into deepgemm/src/, adds `pub mod ffi_dgb200;` to lib.rs, links
//! `dgb200` (build.rs: `cargo:rustc-link-lib=dylib=dgb200` + the search path) and re-exports these
//! items in place of the bodies in ops_sm100.rs.  Device memory stays cudarc's (`CudaSlice`), like
//! in the crate; the library only sees raw device addresses.  Nothing here computes on the CPU.
//!
//! Source only: no Rust toolchain exists where this repository is built and tested, so the file
//! has not been compiled; the C ABI underneath is what the tests exercise (through ctypes).

#![allow(clippy::too_many_arguments)]

use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_void};
use std::sync::Arc;

use cudarc::driver::{CudaContext, CudaSlice, CudaStream, DevicePtr, DevicePtrMut};

use crate::types::{DgError, DgResult};

// ------------------------------------------------------------------------------------ raw C ABI
#[repr(C)]
pub struct RawCtx {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct RawLpOperand {
    pub data: *const c_void,
    pub sf: *const u32,
    pub rows: u32,
    pub k: u32,
    pub ld: u32,
    pub bits: u32,
    pub gran_k: u32,
    pub major_mn: u32,
    pub data_len: usize,
    pub sf_len: usize,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct RawOut {
    pub kind: c_int,
    pub buf: *mut c_void,
    pub ld: u32,
    pub sfd: *mut u32,
    pub buf_len: usize,
    pub sfd_len: usize,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct RawEpilogue {
    pub alpha: f32,
    pub has_alpha: c_int,
    pub accumulate: c_int,
    pub tc_util: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct RawDesc {
    pub gemm_type: u32,
    pub m: u32,
    pub n: u32,
    pub k: u32,
    pub num_groups: u32,
    pub expected_m: u32,
    pub a_bits: u32,
    pub b_bits: u32,
    pub gran_a: u32,
    pub gran_b: u32,
    pub cd_dtype: u32,
    pub num_sms: u32,
    pub major_a_mn: u32,
    pub major_b_mn: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Default, Debug)]
pub struct RawConfig {
    pub swap_ab: u32,
    pub block_m: u32,
    pub block_n: u32,
    pub block_k: u32,
    pub cluster_m: u32,
    pub cluster_n: u32,
    pub num_stages: u32,
    pub num_accum_stages: u32,
    pub smem_size: u32,
    pub num_tiles: u32,
    pub num_splits: u32,
}

pub const DG_STATIC_MAX_GROUPS: u32 = 4096;

#[link(name = "dgb200")]
extern "C" {
    pub fn dg_ctx_create(ordinal: c_int, out: *mut *mut RawCtx) -> c_int;
    pub fn dg_ctx_create_on_stream(ordinal: c_int, stream: *mut c_void, out: *mut *mut RawCtx) -> c_int;
    pub fn dg_ctx_destroy(ctx: *mut RawCtx) -> c_int;
    pub fn dg_ctx_sync(ctx: *mut RawCtx) -> c_int;
    pub fn dg_ctx_check_status(ctx: *mut RawCtx) -> c_int;
    pub fn dg_ctx_num_sms(ctx: *const RawCtx, out: *mut c_int) -> c_int;
    pub fn dg_ctx_stream(ctx: *const RawCtx) -> *mut c_void;
    pub fn dg_ctx_set_stream(ctx: *mut RawCtx, stream: *mut c_void) -> c_int;
    pub fn dg_last_error() -> *const c_char;

    pub fn dg_fp8_fp4_gemm(ctx: *mut RawCtx, a: *const RawLpOperand, b: *const RawLpOperand, out: *const RawOut, epi: *const RawEpilogue) -> c_int;
    pub fn dg_bf16_gemm(ctx: *mut RawCtx, a: *const u16, a_ld: u32, m: u32, b: *const u16, b_ld: u32, n: u32, k: u32, out: *const RawOut,
                        epi: *const RawEpilogue) -> c_int;
    pub fn dg_m_grouped_fp8_fp4_gemm_contiguous(ctx: *mut RawCtx, a: *const RawLpOperand, m_indices: *const i32, b: *const RawLpOperand,
                                                out: *const RawOut, num_groups: u32, epi: *const RawEpilogue) -> c_int;
    pub fn dg_m_grouped_fp8_fp4_gemm_contiguous_ends(ctx: *mut RawCtx, a: *const RawLpOperand, group_ends: *const u32, b: *const RawLpOperand,
                                                     out: *const RawOut, num_groups: u32, epi: *const RawEpilogue) -> c_int;
    pub fn dg_m_grouped_fp8_fp4_gemm_contiguous_static(device: c_int, stream: *mut c_void, a: *const RawLpOperand, m_indices: *const i32,
                                                       b: *const RawLpOperand, out: *const RawOut, num_groups: u32, epi: *const RawEpilogue) -> c_int;
    pub fn dg_static_check_status(device: c_int, stream: *mut c_void) -> c_int;
    pub fn dg_m_grouped_fp8_fp4_gemm_masked(ctx: *mut RawCtx, a: *const RawLpOperand, masked_m: *const i32, b: *const RawLpOperand,
                                            out: *const RawOut, num_groups: u32, expected_m: u32, epi: *const RawEpilogue) -> c_int;
    pub fn dg_fp8_fp4_bmm(ctx: *mut RawCtx, a: *const RawLpOperand, b: *const RawLpOperand, out: *const RawOut, num_groups: u32,
                          epi: *const RawEpilogue) -> c_int;

    pub fn dg_fp8_gemm_nt(ctx: *mut RawCtx, a: *const u8, a_ld: u32, a_sf_t: *const f32, b: *const u8, b_ld: u32, sfb: *const f32, m: u32, n: u32,
                          k: u32, out: *mut u16, out_ld: u32) -> c_int;
    pub fn dg_m_grouped_fp8_gemm_nt_contiguous(ctx: *mut RawCtx, a: *const u8, a_ld: u32, a_sf_t: *const f32, b: *const u8, b_ld: u32,
                                               sfb: *const f32, m_total: u32, n: u32, k: u32, out: *mut u16, out_ld: u32, m_indices: *const i32,
                                               num_groups: u32) -> c_int;
    pub fn dg_m_grouped_fp8_gemm_nt_masked(ctx: *mut RawCtx, a: *const u8, a_ld: u32, a_sf_t: *const f32, b: *const u8, b_ld: u32, sfb: *const f32,
                                           m_max: u32, n: u32, k: u32, out: *mut u16, out_ld: u32, masked_m: *const i32, num_groups: u32,
                                           expected_m: u32) -> c_int;
    pub fn dg_fp8_bmm_nt(ctx: *mut RawCtx, a: *const u8, a_ld: u32, a_sf_t: *const f32, b: *const u8, b_ld: u32, sfb: *const f32, m: u32, n: u32,
                         k: u32, out: *mut u16, out_ld: u32, num_groups: u32) -> c_int;

    pub fn dg_sf_packed_cols(k: u32, gran_k: u32) -> u32;
    pub fn dg_sf_aligned_rows(rows: u32) -> u32;
    pub fn dg_sf_words(rows: u32, k: u32, gran_k: u32, num_groups: u32) -> usize;

    pub fn dg_cast_bf16_to_fp8_sf(ctx: *mut RawCtx, src: *const u16, src_ld: u32, rows: u32, k: u32, gran_k: u32, num_groups: u32, dst: *mut u8,
                                  sf: *mut u32) -> c_int;
    pub fn dg_silu_mul_cast_fp8_sf(ctx: *mut RawCtx, gate_up: *const u16, src_ld: u32, rows: u32, n: u32, gran_k: u32, num_groups: u32,
                                   dst: *mut u8, sf: *mut u32, live_rows: *const u32) -> c_int;
    pub fn dg_cast_bf16_to_fp4_packed_sf(ctx: *mut RawCtx, src: *const u16, src_ld: u32, rows: u32, k: u32, num_groups: u32, sf_rule: c_int,
                                         dst: *mut u8, sf: *mut u32) -> c_int;
    pub fn dg_transform_sf(ctx: *mut RawCtx, sf: *const f32, mn: u32, sf_k: u32, num_batches: u32, dst: *mut f32) -> c_int;
    pub fn dg_transform_sf1d_packed_ue8m0(ctx: *mut RawCtx, src: *const f32, src_ld: u32, rows: u32, k: u32, gran_k: u32, num_groups: u32,
                                          dst: *mut u32) -> c_int;
    pub fn dg_transform_sf2d_packed_ue8m0(ctx: *mut RawCtx, src: *const f32, src_ld: u32, rows: u32, k: u32, num_groups: u32, dst: *mut u32) -> c_int;
    pub fn dg_transform_sf_t_packed_ue8m0(ctx: *mut RawCtx, src: *const f32, rows: u32, k: u32, gran_k: u32, num_groups: u32, dst: *mut u32) -> c_int;
    pub fn dg_group_ends_from_m_indices(ctx: *mut RawCtx, m_indices: *const i32, m: u32, num_groups: u32, group_ends: *mut u32) -> c_int;
    pub fn dg_unpack_fp4_raw(ctx: *mut RawCtx, src: *const u8, packed_len: usize, dst: *mut u8) -> c_int;

    pub fn dg_set_mk_alignment_for_contiguous_layout(value: u32) -> c_int;
    pub fn dg_get_mk_alignment_for_contiguous_layout() -> u32;
    pub fn dg_get_theoretical_mk_alignment_for_contiguous_layout(arch_major: u32) -> u32;
    pub fn dg_best_config(desc: *const RawDesc, out: *mut RawConfig) -> c_int;
}

/// Status code of the C ABI -> the crate's error type (types.rs:9-21).  A device-side wait that ran
/// out (code 4) has no variant of its own in the crate and is reported as a driver error.
fn check(rc: c_int) -> DgResult<()> {
    if rc == 0 {
        return Ok(());
    }
    let msg = unsafe {
        let p = dg_last_error();
        if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    };
    Err(match rc {
        2 => DgError::Shape(msg),
        3 => DgError::Unsupported(msg),
        4 => DgError::Driver(format!("device-side wait timed out: {msg}")),
        _ => DgError::Driver(msg),
    })
}

// ----------------------------------------------------------------------------------- DgContext
/// device.rs:40-56.  Same fields a caller of this path uses (`device`, `stream`), plus the library
/// handle; the JIT engine of the original has no counterpart (kernels are compiled ahead of time).
pub struct DgContext {
    pub device: Arc<CudaContext>,
    pub stream: Arc<CudaStream>,
    ordinal: usize,
    raw: *mut RawCtx,
}

unsafe impl Send for DgContext {}
unsafe impl Sync for DgContext {}

impl DgContext {
    /// device.rs:49
    pub fn new(ordinal: usize) -> DgResult<Self> {
        let device = CudaContext::new(ordinal).map_err(|e| DgError::Driver(format!("{e:?}")))?;
        let stream = device.default_stream();
        let mut raw: *mut RawCtx = std::ptr::null_mut();
        check(unsafe { dg_ctx_create_on_stream(ordinal as c_int, stream.cu_stream() as *mut c_void, &mut raw) })?;
        Ok(Self { device, stream, ordinal, raw })
    }

    /// device.rs:124
    pub fn num_sms(&self) -> u32 {
        let mut n: c_int = 0;
        unsafe { dg_ctx_num_sms(self.raw, &mut n) };
        n as u32
    }

    /// device.rs:129; also surfaces a kernel that gave up on a bounded wait.
    pub fn sync(&self) -> DgResult<()> {
        check(unsafe { dg_ctx_sync(self.raw) })
    }

    pub fn ordinal(&self) -> usize {
        self.ordinal
    }
}

impl Drop for DgContext {
    fn drop(&mut self) {
        unsafe { dg_ctx_destroy(self.raw) };
    }
}

// ------------------------------------------------------------------------------ operand / output
/// ops_sm100.rs:33-45
#[derive(Debug, Clone, Copy)]
pub struct LpOperand<'a> {
    pub data: &'a CudaSlice<u8>,
    pub sf: &'a CudaSlice<u32>,
    pub rows: u32,
    pub k: u32,
    pub ld: u32,
    pub bits: u32,
    pub gran_k: u32,
    pub major_mn: bool,
}

impl<'a> LpOperand<'a> {
    fn raw(&self, stream: &CudaStream) -> RawLpOperand {
        let (data, _g0) = self.data.device_ptr(stream);
        let (sf, _g1) = self.sf.device_ptr(stream);
        RawLpOperand {
            data: data as *const c_void,
            sf: sf as *const u32,
            rows: self.rows,
            k: self.k,
            ld: self.ld,
            bits: self.bits,
            gran_k: self.gran_k,
            major_mn: self.major_mn as u32,
            data_len: self.data.len(),
            sf_len: self.sf.len(),
        }
    }
}

/// ops_sm100.rs:95-110
pub enum Sm100Out<'a> {
    Bf16 { buf: &'a mut CudaSlice<u16>, ld: u32 },
    F32 { buf: &'a mut CudaSlice<f32>, ld: u32 },
    Fp8 { buf: &'a mut CudaSlice<u8>, ld: u32, sfd: &'a mut CudaSlice<u32> },
}

impl<'a> Sm100Out<'a> {
    // The reference passes `&Sm100Out` holding `&mut` buffers; the device address is all the library needs.
    fn raw(&self, stream: &CudaStream) -> RawOut {
        match self {
            Sm100Out::Bf16 { buf, ld } => {
                let (p, _g) = buf.device_ptr(stream);
                RawOut { kind: 0, buf: p as *mut c_void, ld: *ld, sfd: std::ptr::null_mut(), buf_len: buf.len(), sfd_len: 0 }
            }
            Sm100Out::F32 { buf, ld } => {
                let (p, _g) = buf.device_ptr(stream);
                RawOut { kind: 1, buf: p as *mut c_void, ld: *ld, sfd: std::ptr::null_mut(), buf_len: buf.len(), sfd_len: 0 }
            }
            Sm100Out::Fp8 { buf, ld, sfd } => {
                let (p, _g0) = buf.device_ptr(stream);
                let (s, _g1) = sfd.device_ptr(stream);
                RawOut { kind: 2, buf: p as *mut c_void, ld: *ld, sfd: s as *mut u32, buf_len: buf.len(), sfd_len: sfd.len() }
            }
        }
    }
}

/// ops_sm100.rs:114-131
#[derive(Debug, Clone, Copy)]
pub struct Sm100Epilogue {
    pub alpha: Option<f32>,
    pub accumulate: bool,
    pub tc_util: u32,
}

impl Default for Sm100Epilogue {
    fn default() -> Self {
        Self { alpha: None, accumulate: false, tc_util: 100 }
    }
}

impl Sm100Epilogue {
    fn raw(&self) -> RawEpilogue {
        RawEpilogue {
            alpha: self.alpha.unwrap_or(1.0),
            has_alpha: self.alpha.is_some() as c_int,
            accumulate: self.accumulate as c_int,
            tc_util: self.tc_util,
        }
    }
}

// ------------------------------------------------------------------------------------ the GEMMs
/// ops_sm100.rs:719
pub fn fp8_fp4_gemm_dev(ctx: &DgContext, a: &LpOperand, b: &LpOperand, out: &Sm100Out, epi: &Sm100Epilogue) -> DgResult<()> {
    let (ca, cb, co, ce) = (a.raw(&ctx.stream), b.raw(&ctx.stream), out.raw(&ctx.stream), epi.raw());
    check(unsafe { dg_fp8_fp4_gemm(ctx.raw, &ca, &cb, &co, &ce) })
}

/// ops_sm100.rs:759.  `b.rows = num_groups * n`, as the reference computes `n = b.rows / num_groups` (:778).
pub fn m_grouped_fp8_fp4_gemm_contiguous_dev(ctx: &DgContext, a: &LpOperand, m_indices: &CudaSlice<i32>, b: &LpOperand, out: &Sm100Out,
                                             num_groups: u32, epi: &Sm100Epilogue) -> DgResult<()> {
    let (ca, cb, co, ce) = (a.raw(&ctx.stream), b.raw(&ctx.stream), out.raw(&ctx.stream), epi.raw());
    let (idx, _g) = m_indices.device_ptr(&ctx.stream);
    check(unsafe { dg_m_grouped_fp8_fp4_gemm_contiguous(ctx.raw, &ca, idx as *const i32, &cb, &co, num_groups, &ce) })
}

/// ops_sm100.rs:815
pub fn m_grouped_fp8_fp4_gemm_masked_dev(ctx: &DgContext, a: &LpOperand, masked_m: &CudaSlice<i32>, b: &LpOperand, out: &Sm100Out,
                                         num_groups: u32, expected_m: u32, epi: &Sm100Epilogue) -> DgResult<()> {
    let (ca, cb, co, ce) = (a.raw(&ctx.stream), b.raw(&ctx.stream), out.raw(&ctx.stream), epi.raw());
    let (mm, _g) = masked_m.device_ptr(&ctx.stream);
    check(unsafe { dg_m_grouped_fp8_fp4_gemm_masked(ctx.raw, &ca, mm as *const i32, &cb, &co, num_groups, expected_m, &ce) })
}

/// ops_sm100.rs:864
pub fn fp8_fp4_bmm_dev(ctx: &DgContext, a: &LpOperand, b: &LpOperand, out: &Sm100Out, num_groups: u32, epi: &Sm100Epilogue) -> DgResult<()> {
    let (ca, cb, co, ce) = (a.raw(&ctx.stream), b.raw(&ctx.stream), out.raw(&ctx.stream), epi.raw());
    check(unsafe { dg_fp8_fp4_bmm(ctx.raw, &ca, &cb, &co, num_groups, &ce) })
}

/// ops_sm100.rs:893
pub fn bf16_gemm_dev(ctx: &DgContext, a: &CudaSlice<u16>, a_ld: u32, m: u32, b: &CudaSlice<u16>, b_ld: u32, n: u32, k: u32, out: &Sm100Out,
                     epi: &Sm100Epilogue) -> DgResult<()> {
    let (pa, _g0) = a.device_ptr(&ctx.stream);
    let (pb, _g1) = b.device_ptr(&ctx.stream);
    let (co, ce) = (out.raw(&ctx.stream), epi.raw());
    check(unsafe { dg_bf16_gemm(ctx.raw, pa as *const u16, a_ld, m, pb as *const u16, b_ld, n, k, &co, &ce) })
}

/// ops_sm100.rs:1693
pub fn fp4_gemm_packed_dev(ctx: &DgContext, a_data: &CudaSlice<u8>, a_sf: &CudaSlice<u32>, b_data: &CudaSlice<u8>, b_sf: &CudaSlice<u32>,
                           out: &mut CudaSlice<u16>, m: u32, n: u32, k: u32) -> DgResult<()> {
    let a = LpOperand { data: a_data, sf: a_sf, rows: m, k, ld: k, bits: 4, gran_k: 32, major_mn: false };
    let b = LpOperand { data: b_data, sf: b_sf, rows: n, k, ld: k, bits: 4, gran_k: 32, major_mn: false };
    fp8_fp4_gemm_dev(ctx, &a, &b, &Sm100Out::Bf16 { buf: out, ld: n }, &Sm100Epilogue::default())
}

/// ops_sm100.rs:1646: host bf16 in, host bf16 out (upload, quantise both operands, MXFP4 GEMM, download).
pub fn fp4_gemm_nt_native(ctx: &DgContext, a_bf16: &[u16], b_bf16: &[u16], m: u32, n: u32, k: u32) -> DgResult<Vec<u16>> {
    let drv = |e| DgError::Driver(format!("{e:?}"));
    let a_dev = ctx.stream.memcpy_stod(a_bf16).map_err(drv)?;
    let b_dev = ctx.stream.memcpy_stod(b_bf16).map_err(drv)?;
    let (a_data, a_sf) = cast_bf16_to_fp4_packed_sf_dev(ctx, &a_dev, k, m, k, 1)?;
    let (b_data, b_sf) = cast_bf16_to_fp4_packed_sf_dev(ctx, &b_dev, k, n, k, 1)?;
    let mut out = ctx.stream.alloc_zeros::<u16>(m as usize * n as usize).map_err(drv)?;
    fp4_gemm_packed_dev(ctx, &a_data, &a_sf, &b_data, &b_sf, &mut out, m, n, k)?;
    ctx.sync()?;
    ctx.stream.memcpy_dtov(&out).map_err(drv)
}

// ----------------------------------------------------------- the f32-scale calls of ops.rs
/// types.rs (Fp8Tensor): e4m3 bytes, K-major.
pub struct Fp8Tensor<'a> {
    pub data: &'a CudaSlice<u8>,
    pub rows: u32,
    pub k: u32,
    pub ld: u32,
}

/// ops.rs:328.  `a_sf_t` is the output of `transform_sf_dev` for a's (rows, k/128) f32 scales, `sfb` the
/// (n/128, k/128) tile scales; like the reference's bridge (ops_sm100.rs:1414-1605) only each scale's exponent is used.
pub fn fp8_gemm_nt_dev(ctx: &DgContext, a: &Fp8Tensor, a_sf_t: &CudaSlice<f32>, b: &Fp8Tensor, sfb: &CudaSlice<f32>, out: &mut CudaSlice<u16>,
                       out_ld: u32) -> DgResult<()> {
    let s = &ctx.stream;
    let ((pa, _a), (psa, _b), (pb, _c), (psb, _d), (po, _e)) =
        (a.data.device_ptr(s), a_sf_t.device_ptr(s), b.data.device_ptr(s), sfb.device_ptr(s), out.device_ptr_mut(s));
    check(unsafe {
        dg_fp8_gemm_nt(ctx.raw, pa as *const u8, a.ld, psa as *const f32, pb as *const u8, b.ld, psb as *const f32, a.rows, b.rows, a.k,
                       po as *mut u16, out_ld)
    })
}

/// ops.rs:422
pub fn m_grouped_fp8_gemm_nt_contiguous_dev(ctx: &DgContext, a: &Fp8Tensor, a_sf_t: &CudaSlice<f32>, b: &Fp8Tensor, sfb: &CudaSlice<f32>,
                                            out: &mut CudaSlice<u16>, out_ld: u32, m_indices: &CudaSlice<i32>, num_groups: u32) -> DgResult<()> {
    let s = &ctx.stream;
    let ((pa, _a), (psa, _b), (pb, _c), (psb, _d), (po, _e), (pi, _f)) =
        (a.data.device_ptr(s), a_sf_t.device_ptr(s), b.data.device_ptr(s), sfb.device_ptr(s), out.device_ptr_mut(s), m_indices.device_ptr(s));
    check(unsafe {
        dg_m_grouped_fp8_gemm_nt_contiguous(ctx.raw, pa as *const u8, a.ld, psa as *const f32, pb as *const u8, b.ld, psb as *const f32, a.rows,
                                            b.rows / num_groups.max(1), a.k, po as *mut u16, out_ld, pi as *const i32, num_groups)
    })
}

/// ops.rs:535
pub fn m_grouped_fp8_gemm_nt_masked_dev(ctx: &DgContext, a: &Fp8Tensor, a_sf_t: &CudaSlice<f32>, b: &Fp8Tensor, sfb: &CudaSlice<f32>,
                                        out: &mut CudaSlice<u16>, out_ld: u32, masked_m: &CudaSlice<i32>, num_groups: u32, m_max: u32,
                                        expected_m: u32) -> DgResult<()> {
    let s = &ctx.stream;
    let ((pa, _a), (psa, _b), (pb, _c), (psb, _d), (po, _e), (pm, _f)) =
        (a.data.device_ptr(s), a_sf_t.device_ptr(s), b.data.device_ptr(s), sfb.device_ptr(s), out.device_ptr_mut(s), masked_m.device_ptr(s));
    check(unsafe {
        dg_m_grouped_fp8_gemm_nt_masked(ctx.raw, pa as *const u8, a.ld, psa as *const f32, pb as *const u8, b.ld, psb as *const f32, m_max,
                                        b.rows / num_groups.max(1), a.k, po as *mut u16, out_ld, pm as *const i32, num_groups, expected_m)
    })
}

/// ops.rs:635
pub fn fp8_bmm_nt_dev(ctx: &DgContext, a: &Fp8Tensor, a_sf_t: &CudaSlice<f32>, b: &Fp8Tensor, sfb: &CudaSlice<f32>, out: &mut CudaSlice<u16>,
                      out_ld: u32, num_groups: u32, m: u32, n: u32) -> DgResult<()> {
    let s = &ctx.stream;
    let ((pa, _a), (psa, _b), (pb, _c), (psb, _d), (po, _e)) =
        (a.data.device_ptr(s), a_sf_t.device_ptr(s), b.data.device_ptr(s), sfb.device_ptr(s), out.device_ptr_mut(s));
    check(unsafe {
        dg_fp8_bmm_nt(ctx.raw, pa as *const u8, a.ld, psa as *const f32, pb as *const u8, b.ld, psb as *const f32, m, n, a.k, po as *mut u16, out_ld,
                      num_groups)
    })
}

// ------------------------------------------------------- scale-factor helpers and quantisers
/// ops_sm100.rs:1091
pub fn sf_packed_cols(k: u32, gran_k: u32) -> u32 {
    unsafe { dg_sf_packed_cols(k, gran_k) }
}

/// ops_sm100.rs:1096
pub fn sf_aligned_rows(rows: u32) -> u32 {
    unsafe { dg_sf_aligned_rows(rows) }
}

/// ops_sm100.rs:1107: zero-filled packed scale buffer.
pub fn alloc_sf(ctx: &DgContext, rows: u32, k: u32, gran_k: u32, num_groups: u32) -> DgResult<CudaSlice<u32>> {
    let words = unsafe { dg_sf_words(rows, k, gran_k, num_groups.max(1)) };
    ctx.stream.alloc_zeros::<u32>(words).map_err(|e| DgError::Driver(format!("{e:?}")))
}

/// ops_sm100.rs:1186
pub fn cast_bf16_to_fp8_sf_dev(ctx: &DgContext, src: &CudaSlice<u16>, src_ld: u32, rows: u32, k: u32, gran_k: u32, num_groups: u32)
                               -> DgResult<(CudaSlice<u8>, CudaSlice<u32>)> {
    let mut dst = unsafe { ctx.stream.alloc::<u8>(rows as usize * k as usize) }.map_err(|e| DgError::Driver(format!("{e:?}")))?;
    let mut sf = alloc_sf(ctx, rows, k, gran_k, num_groups)?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b), (pf, _c)) = (src.device_ptr(s), dst.device_ptr_mut(s), sf.device_ptr_mut(s));
        check(unsafe { dg_cast_bf16_to_fp8_sf(ctx.raw, ps as *const u16, src_ld, rows, k, gran_k, num_groups, pd as *mut u8, pf as *mut u32) })?;
    }
    Ok((dst, sf))
}

/// ops_sm100.rs:1135.  The scale rule is the one of the reference's CPU quantiser (reference.rs:273), the only
/// executable definition the crate has; `cast_bf16_to_fp4_packed_sf_with_rule_dev` exposes the range-fitting rule.
pub fn cast_bf16_to_fp4_packed_sf_dev(ctx: &DgContext, src: &CudaSlice<u16>, src_ld: u32, rows: u32, k: u32, num_groups: u32)
                                      -> DgResult<(CudaSlice<u8>, CudaSlice<u32>)> {
    cast_bf16_to_fp4_packed_sf_with_rule_dev(ctx, src, src_ld, rows, k, num_groups, 0)
}

pub fn cast_bf16_to_fp4_packed_sf_with_rule_dev(ctx: &DgContext, src: &CudaSlice<u16>, src_ld: u32, rows: u32, k: u32, num_groups: u32,
                                                sf_rule: i32) -> DgResult<(CudaSlice<u8>, CudaSlice<u32>)> {
    let mut dst = unsafe { ctx.stream.alloc::<u8>(rows as usize * k as usize / 2) }.map_err(|e| DgError::Driver(format!("{e:?}")))?;
    let mut sf = alloc_sf(ctx, rows, k, 32, num_groups)?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b), (pf, _c)) = (src.device_ptr(s), dst.device_ptr_mut(s), sf.device_ptr_mut(s));
        check(unsafe { dg_cast_bf16_to_fp4_packed_sf(ctx.raw, ps as *const u16, src_ld, rows, k, num_groups, sf_rule, pd as *mut u8, pf as *mut u32) })?;
    }
    Ok((dst, sf))
}

/// ops.rs:52
pub fn transform_sf_dev(ctx: &DgContext, sf: &CudaSlice<f32>, mn: u32, sf_k: u32, num_batches: u32) -> DgResult<CudaSlice<f32>> {
    let aligned = sf_aligned_rows(mn) as usize;
    let mut dst = ctx.stream.alloc_zeros::<f32>(num_batches as usize * sf_k as usize * aligned).map_err(|e| DgError::Driver(format!("{e:?}")))?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b)) = (sf.device_ptr(s), dst.device_ptr_mut(s));
        check(unsafe { dg_transform_sf(ctx.raw, ps as *const f32, mn, sf_k, num_batches, pd as *mut f32) })?;
    }
    Ok(dst)
}

/// ops_sm100.rs:1250
pub fn transform_sf1d_packed_ue8m0_dev(ctx: &DgContext, src: &CudaSlice<f32>, src_ld: u32, rows: u32, k: u32, gran_k: u32, num_groups: u32)
                                       -> DgResult<CudaSlice<u32>> {
    let mut dst = alloc_sf(ctx, rows, k, gran_k, num_groups)?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b)) = (src.device_ptr(s), dst.device_ptr_mut(s));
        check(unsafe { dg_transform_sf1d_packed_ue8m0(ctx.raw, ps as *const f32, src_ld, rows, k, gran_k, num_groups, pd as *mut u32) })?;
    }
    Ok(dst)
}

/// ops_sm100.rs:1294
pub fn transform_sf2d_packed_ue8m0_dev(ctx: &DgContext, src: &CudaSlice<f32>, src_ld: u32, rows: u32, k: u32, num_groups: u32)
                                       -> DgResult<CudaSlice<u32>> {
    let mut dst = alloc_sf(ctx, rows, k, 128, num_groups)?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b)) = (src.device_ptr(s), dst.device_ptr_mut(s));
        check(unsafe { dg_transform_sf2d_packed_ue8m0(ctx.raw, ps as *const f32, src_ld, rows, k, num_groups, pd as *mut u32) })?;
    }
    Ok(dst)
}

/// ops_sm100.rs:1372
pub fn transform_sf_t_packed_ue8m0_dev(ctx: &DgContext, src: &CudaSlice<f32>, rows: u32, k: u32, gran_k: u32, num_groups: u32)
                                       -> DgResult<CudaSlice<u32>> {
    let mut dst = alloc_sf(ctx, rows, k, gran_k, num_groups)?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b)) = (src.device_ptr(s), dst.device_ptr_mut(s));
        check(unsafe { dg_transform_sf_t_packed_ue8m0(ctx.raw, ps as *const f32, rows, k, gran_k, num_groups, pd as *mut u32) })?;
    }
    Ok(dst)
}

/// ops_sm100.rs:1338
pub fn unpack_fp4_raw_dev(ctx: &DgContext, src: &CudaSlice<u8>, packed_len: usize) -> DgResult<CudaSlice<u8>> {
    let mut dst = unsafe { ctx.stream.alloc::<u8>(packed_len * 2) }.map_err(|e| DgError::Driver(format!("{e:?}")))?;
    {
        let s = &ctx.stream;
        let ((ps, _a), (pd, _b)) = (src.device_ptr(s), dst.device_ptr_mut(s));
        check(unsafe { dg_unpack_fp4_raw(ctx.raw, ps as *const u8, packed_len, pd as *mut u8) })?;
    }
    Ok(dst)
}

/// ops_sm100.rs:1073 (run_psum_kernel): one past the last row of every group.
pub fn psum_from_m_indices_dev(ctx: &DgContext, m_indices: &CudaSlice<i32>, num_groups: u32) -> DgResult<CudaSlice<u32>> {
    let mut out = ctx.stream.alloc_zeros::<u32>(num_groups as usize).map_err(|e| DgError::Driver(format!("{e:?}")))?;
    {
        let s = &ctx.stream;
        let ((pi, _a), (po, _b)) = (m_indices.device_ptr(s), out.device_ptr_mut(s));
        check(unsafe { dg_group_ends_from_m_indices(ctx.raw, pi as *const i32, m_indices.len() as u32, num_groups, po as *mut u32) })?;
    }
    Ok(out)
}

// ------------------------------------------------------------------- knobs and heuristics
/// types.rs:195 (panics on a bad value like the original).
pub fn set_mk_alignment_for_contiguous_layout(value: u32) {
    assert!(unsafe { dg_set_mk_alignment_for_contiguous_layout(value) } == 0, "mk alignment must be a power of two in [16, 256], got {value}");
}

/// types.rs:204
pub fn get_mk_alignment_for_contiguous_layout() -> u32 {
    unsafe { dg_get_mk_alignment_for_contiguous_layout() }
}

/// types.rs:213
pub fn get_theoretical_mk_alignment_for_contiguous_layout(arch_major: u32) -> u32 {
    unsafe { dg_get_theoretical_mk_alignment_for_contiguous_layout(arch_major) }
}

/// heuristics_sm100.rs:61-87, the fields this build's tile choice reads.
#[derive(Debug, Clone, Copy)]
pub struct Sm100Desc {
    pub gemm_type: crate::types::GemmType,
    pub m: u32,
    pub n: u32,
    pub k: u32,
    pub num_groups: u32,
    pub expected_m: u32,
    pub a_bits: u32,
    pub b_bits: u32,
    pub gran_a: u32,
    pub gran_b: u32,
    pub cd_dtype: u32,
    pub num_sms: u32,
    pub major_a_mn: bool,
    pub major_b_mn: bool,
}

/// heuristics_sm100.rs:17-57, flattened: the same layout fields plus what this kernel adds (accumulator
/// stages, K ranges).
pub type Sm100Config = RawConfig;

/// heuristics_sm100.rs:455 (panics when nothing fits, like the original's assert).
pub fn best_config(desc: &Sm100Desc) -> Sm100Config {
    use crate::types::GemmType::*;
    let gemm_type = match desc.gemm_type {
        Normal => 0,
        MGroupedContiguous => 1,
        MGroupedMasked => 2,
        _ => 3,
    };
    let raw = RawDesc {
        gemm_type,
        m: desc.m,
        n: desc.n,
        k: desc.k,
        num_groups: desc.num_groups.max(1),
        expected_m: if desc.expected_m == 0 { desc.m } else { desc.expected_m },
        a_bits: desc.a_bits,
        b_bits: desc.b_bits,
        gran_a: desc.gran_a,
        gran_b: desc.gran_b,
        cd_dtype: desc.cd_dtype,
        num_sms: desc.num_sms,
        major_a_mn: desc.major_a_mn as u32,
        major_b_mn: desc.major_b_mn as u32,
    };
    let mut cfg = RawConfig::default();
    check(unsafe { dg_best_config(&raw, &mut cfg) }).expect("no SM100 layout candidate");
    cfg
}

// ------------------------------------------- the call that allocates nothing (no crate counterpart)
/// `m_grouped_fp8_fp4_gemm_contiguous_dev` for a host that may not allocate device memory while it runs:
/// no context, scratch inside the library, at most DG_STATIC_MAX_GROUPS groups, one stream per device.
pub fn m_grouped_fp8_fp4_gemm_contiguous_static_dev(device: usize, stream: &CudaStream, a: &LpOperand, m_indices: &CudaSlice<i32>,
                                                    b: &LpOperand, out: &Sm100Out, num_groups: u32, epi: &Sm100Epilogue) -> DgResult<()> {
    let (ca, cb, co, ce) = (a.raw(stream), b.raw(stream), out.raw(stream), epi.raw());
    let (idx, _g) = m_indices.device_ptr(stream);
    check(unsafe {
        dg_m_grouped_fp8_fp4_gemm_contiguous_static(device as c_int, stream.cu_stream() as *mut c_void, &ca, idx as *const i32, &cb, &co, num_groups, &ce)
    })
}

/// Waits for the stream and reports a kernel of the call above that gave up on a bounded wait.
pub fn static_check_status(device: usize, stream: &CudaStream) -> DgResult<()> {
    check(unsafe { dg_static_check_status(device as c_int, stream.cu_stream() as *mut c_void) })
}
