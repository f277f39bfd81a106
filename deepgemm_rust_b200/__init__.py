"""Host-side mirror of the reference crate's SM100 operator surface, over the C-ABI library.

Names, argument meaning and error behaviour follow deepgemm/src/ops_sm100.rs,
deepgemm/src/heuristics_sm100.rs, deepgemm/src/types.rs and deepgemm/src/device.rs of
idrees2516/deepgemm-rust.  Every compute call goes through libdgb200.so (hand-written sm_100a
kernels); torch is used only to own device memory and streams.  There is no CPU path: importing
works anywhere, but creating a DgContext needs a B200.
"""
import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("DGB200_LIBRARY") or os.path.join(_HERE, "libdgb200.so")  # override: an alternative build of the same ABI
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")


class DgError(RuntimeError):
    """deepgemm/src/types.rs:9-21 (DgError); .kind is one of Driver, Shape, Unsupported, Timeout."""

    KINDS = {1: "Driver", 2: "Shape", 3: "Unsupported", 4: "Timeout"}

    def __init__(self, code: int, message: str):
        self.code = code
        self.kind = self.KINDS.get(code, "Unknown")
        super().__init__(f"{self.kind}: {message}")


def _load():
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python deepgemm_rust_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    return C.CDLL(_LIB_PATH)


_lib = _load()


class _LpOperand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("sf", C.c_void_p), ("rows", C.c_uint32), ("k", C.c_uint32), ("ld", C.c_uint32),
                ("bits", C.c_uint32), ("gran_k", C.c_uint32), ("major_mn", C.c_uint32), ("data_len", C.c_size_t),
                ("sf_len", C.c_size_t)]


class _Out(C.Structure):
    _fields_ = [("kind", C.c_int), ("buf", C.c_void_p), ("ld", C.c_uint32), ("sfd", C.c_void_p), ("buf_len", C.c_size_t),
                ("sfd_len", C.c_size_t)]


class _Epilogue(C.Structure):
    _fields_ = [("alpha", C.c_float), ("has_alpha", C.c_int), ("accumulate", C.c_int), ("tc_util", C.c_uint32)]


class _Desc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("gemm_type", "m", "n", "k", "num_groups", "expected_m", "a_bits", "b_bits", "gran_a",
                                          "gran_b", "cd_dtype", "num_sms", "major_a_mn", "major_b_mn")]


class _Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("swap_ab", "block_m", "block_n", "block_k", "cluster_m", "cluster_n", "num_stages",
                                          "num_accum_stages", "smem_size", "num_tiles", "num_splits")]


def _proto(name, restype, *argtypes):
    f = getattr(_lib, name)
    f.restype = restype
    f.argtypes = list(argtypes)
    return f


_vp, _u32, _sz = C.c_void_p, C.c_uint32, C.c_size_t
_lib.dg_last_error.restype = C.c_char_p
_ctx_create = _proto("dg_ctx_create", C.c_int, C.c_int, C.POINTER(_vp))
_ctx_create_on_stream = _proto("dg_ctx_create_on_stream", C.c_int, C.c_int, _vp, C.POINTER(_vp))
_ctx_destroy = _proto("dg_ctx_destroy", C.c_int, _vp)
_ctx_sync = _proto("dg_ctx_sync", C.c_int, _vp)
_ctx_num_sms = _proto("dg_ctx_num_sms", C.c_int, _vp, C.POINTER(C.c_int))
_ctx_stream = _proto("dg_ctx_stream", _vp, _vp)
_ctx_set_stream = _proto("dg_ctx_set_stream", C.c_int, _vp, _vp)
_ctx_check_status = _proto("dg_ctx_check_status", C.c_int, _vp)
_gemm = _proto("dg_fp8_fp4_gemm", C.c_int, _vp, C.POINTER(_LpOperand), C.POINTER(_LpOperand), C.POINTER(_Out), C.POINTER(_Epilogue))
_gemm_contig = _proto("dg_m_grouped_fp8_fp4_gemm_contiguous", C.c_int, _vp, C.POINTER(_LpOperand), _vp, C.POINTER(_LpOperand),
                      C.POINTER(_Out), _u32, C.POINTER(_Epilogue))
_gemm_contig_ends = _proto("dg_m_grouped_fp8_fp4_gemm_contiguous_ends", C.c_int, _vp, C.POINTER(_LpOperand), _vp,
                           C.POINTER(_LpOperand), C.POINTER(_Out), _u32, C.POINTER(_Epilogue))
_gemm_contig_static = _proto("dg_m_grouped_fp8_fp4_gemm_contiguous_static", C.c_int, C.c_int, _vp, C.POINTER(_LpOperand), _vp,
                             C.POINTER(_LpOperand), C.POINTER(_Out), _u32, C.POINTER(_Epilogue))
_static_check_status = _proto("dg_static_check_status", C.c_int, C.c_int, _vp)
_bf16_gemm = _proto("dg_bf16_gemm", C.c_int, _vp, _vp, _u32, _u32, _vp, _u32, _u32, _u32, C.POINTER(_Out), C.POINTER(_Epilogue))
_gemm_masked = _proto("dg_m_grouped_fp8_fp4_gemm_masked", C.c_int, _vp, C.POINTER(_LpOperand), _vp, C.POINTER(_LpOperand),
                      C.POINTER(_Out), _u32, _u32, C.POINTER(_Epilogue))
_bmm = _proto("dg_fp8_fp4_bmm", C.c_int, _vp, C.POINTER(_LpOperand), C.POINTER(_LpOperand), C.POINTER(_Out), _u32, C.POINTER(_Epilogue))
_f32 = (_vp, _vp, _u32, _vp, _vp, _u32, _vp, _u32, _u32, _u32, _vp, _u32)
_gemm_nt = _proto("dg_fp8_gemm_nt", C.c_int, *_f32)
_gemm_nt_contig = _proto("dg_m_grouped_fp8_gemm_nt_contiguous", C.c_int, *_f32, _vp, _u32)
_gemm_nt_masked = _proto("dg_m_grouped_fp8_gemm_nt_masked", C.c_int, *_f32, _vp, _u32, _u32)
_bmm_nt = _proto("dg_fp8_bmm_nt", C.c_int, *_f32, _u32)
_sf_packed_cols = _proto("dg_sf_packed_cols", _u32, _u32, _u32)
_sf_aligned_rows = _proto("dg_sf_aligned_rows", _u32, _u32)
_sf_words = _proto("dg_sf_words", _sz, _u32, _u32, _u32, _u32)
_cast_fp8 = _proto("dg_cast_bf16_to_fp8_sf", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _vp)
_silu_cast = _proto("dg_silu_mul_cast_fp8_sf", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp)
_cast_fp4 = _proto("dg_cast_bf16_to_fp4_packed_sf", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, C.c_int, _vp, _vp)
_transform_sf = _proto("dg_transform_sf", C.c_int, _vp, _vp, _u32, _u32, _u32, _vp)
_tsf1d = _proto("dg_transform_sf1d_packed_ue8m0", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp)
_tsf2d = _proto("dg_transform_sf2d_packed_ue8m0", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _vp)
_tsft = _proto("dg_transform_sf_t_packed_ue8m0", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _vp)
_group_ends = _proto("dg_group_ends_from_m_indices", C.c_int, _vp, _vp, _u32, _u32, _vp)
_unpack_fp4 = _proto("dg_unpack_fp4_raw", C.c_int, _vp, _vp, _sz, _vp)
_gather_rows = _proto("dg_gather_rows", C.c_int, _vp, _vp, _sz, _vp, _u32, _u32, _vp, _sz)
_moe_pack = _proto("dg_moe_pack_rows", C.c_int, _vp, _vp, _u32, _vp, _u32, _u32, _vp, _u32, _vp, _sz)
_moe_unpack = _proto("dg_moe_unpack_rows", C.c_int, _vp, _vp, _sz, _u32, _u32, _vp, _u32, _vp, _vp, _u32)
_moe_combine = _proto("dg_moe_combine", C.c_int, _vp, _vp, _sz, _vp, _vp, _u32, _u32, _u32, _vp, _sz)
_peer_alloc = _proto("dg_peer_alloc", C.c_int, _vp, _sz, C.POINTER(_vp), C.c_char_p)
_peer_open = _proto("dg_peer_open", C.c_int, _vp, C.c_char_p, C.POINTER(_vp))
_peer_close = _proto("dg_peer_close", C.c_int, _vp, _vp)
_peer_free = _proto("dg_peer_free", C.c_int, _vp, _vp)
_ep_hist_words = _proto("dg_ep_block_hist_words", _sz, _u32, _u32)
_ep_count = _proto("dg_ep_count", C.c_int, _vp, _vp, _u32, _u32, _vp, _vp, _vp)
_ep_layout = _proto("dg_ep_layout", C.c_int, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp)
_ep_dispatch = _proto("dg_ep_dispatch", C.c_int, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _u32, _u32, _vp, _vp, _u32,
                      _u32, _u32, _vp, _u32)
_ep_combine = _proto("dg_ep_combine", C.c_int, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _sz, _u32, _vp, _sz, _u32)
_expire_wait = _proto("dg_debug_expire_wait", C.c_int, _vp, _u32)
_set_mk = _proto("dg_set_mk_alignment_for_contiguous_layout", C.c_int, _u32)
_get_mk = _proto("dg_get_mk_alignment_for_contiguous_layout", _u32)
_get_mk_theory = _proto("dg_get_theoretical_mk_alignment_for_contiguous_layout", _u32, _u32)
_best_config = _proto("dg_best_config", C.c_int, C.POINTER(_Desc), C.POINTER(_Config))

SF_RULE_REFERENCE_CPU = 0
SF_RULE_RANGE_FIT = 1


def _check(rc: int):
    if rc != 0:
        raise DgError(rc, (_lib.dg_last_error() or b"").decode())


class GemmType:
    """deepgemm/src/types.rs:27-38"""
    Normal = 0
    MGroupedContiguous = 1
    MGroupedMasked = 2
    Batched = 3


class DgContext:
    """deepgemm/src/device.rs:40-56: one device, one stream.  By default the context adopts the
    current torch stream of that device, so tensors produced by torch are ordered with the kernels."""

    def __init__(self, ordinal: int = 0, stream: Optional[int] = None, own_stream: bool = False):
        self._h = _vp()
        self.ordinal = ordinal
        if own_stream:
            _check(_ctx_create(ordinal, C.byref(self._h)))
        else:
            if stream is None:
                if not torch.cuda.is_available():
                    raise DgError(1, "no CUDA device available; this library has no CPU path")
                stream = torch.cuda.current_stream(ordinal).cuda_stream
            _check(_ctx_create_on_stream(ordinal, _vp(stream), C.byref(self._h)))

    @classmethod
    def new(cls, ordinal: int = 0) -> "DgContext":
        return cls(ordinal)

    def sync(self):
        """device.rs:129; raises DgError(Timeout) if a kernel gave up on a device-side wait."""
        _check(_ctx_sync(self._h))

    def num_sms(self) -> int:
        n = C.c_int()
        _check(_ctx_num_sms(self._h, C.byref(n)))
        return n.value

    @property
    def stream(self) -> int:
        return _ctx_stream(self._h) or 0

    def set_stream(self, cuda_stream: int):
        _check(_ctx_set_stream(self._h, _vp(cuda_stream)))

    def close(self):
        if self._h:
            _ctx_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class LpOperand:
    """ops_sm100.rs:33-45.  data: uint8 tensor; sf: int32 tensor holding the packed UE8M0 words."""
    data: torch.Tensor
    sf: torch.Tensor
    rows: int
    k: int
    ld: int
    bits: int = 8
    gran_k: int = 128
    major_mn: bool = False

    def _c(self) -> _LpOperand:
        return _LpOperand(self.data.data_ptr(), self.sf.data_ptr(), self.rows, self.k, self.ld, self.bits, self.gran_k,
                          1 if self.major_mn else 0, self.data.numel() * self.data.element_size(), self.sf.numel())


@dataclass
class Sm100Out:
    """ops_sm100.rs:95-110.  kind 0 = bf16, 1 = f32, 2 = e4m3 with per-row per-32-column UE8M0 scales,
    3 = the same for silu(gate) * up of a gate|up weight block (fused activation)."""
    kind: int
    buf: torch.Tensor
    ld: int
    sfd: Optional[torch.Tensor] = None

    @classmethod
    def Bf16(cls, buf, ld):
        return cls(0, buf, ld)

    @classmethod
    def F32(cls, buf, ld):
        return cls(1, buf, ld)

    @classmethod
    def Fp8(cls, buf, ld, sfd):
        return cls(2, buf, ld, sfd)

    @classmethod
    def SwiGluFp8(cls, buf, ld, sfd):
        """b holds n gate rows then n up rows per group; buf (rows, ld) receives e4m3(silu(gate) * up), sfd its per-32-column
        UE8M0 scale words: together the next GEMM's A operand with gran_k = 32."""
        return cls(3, buf, ld, sfd)

    def _c(self) -> _Out:
        return _Out(self.kind, self.buf.data_ptr(), self.ld, self.sfd.data_ptr() if self.sfd is not None else None,
                    self.buf.numel(), self.sfd.numel() if self.sfd is not None else 0)


@dataclass
class Sm100Epilogue:
    """ops_sm100.rs:114-131"""
    alpha: Optional[float] = None
    accumulate: bool = False
    tc_util: int = 100

    def _c(self) -> _Epilogue:
        return _Epilogue(self.alpha if self.alpha is not None else 1.0, 1 if self.alpha is not None else 0,
                         1 if self.accumulate else 0, self.tc_util)


def _epi(epi):
    return (epi or Sm100Epilogue())._c()


def fp8_fp4_gemm_dev(ctx: DgContext, a: LpOperand, b: LpOperand, out: Sm100Out, epi: Optional[Sm100Epilogue] = None):
    """ops_sm100.rs:719"""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_gemm(ctx._h, C.byref(ca), C.byref(cb), C.byref(co), C.byref(ce)))


def fp4_gemm_packed_dev(ctx, a_data: torch.Tensor, a_sf: torch.Tensor, b_data: torch.Tensor, b_sf: torch.Tensor, out: torch.Tensor,
                        m: int, n: int, k: int):
    """ops_sm100.rs:1693: MXFP4 GEMM over pre-quantised operands (packed e2m1 + per-32 UE8M0 words), bf16 output (m, n)."""
    fp8_fp4_gemm_dev(ctx, LpOperand(a_data, a_sf, m, k, k, 4, 32), LpOperand(b_data, b_sf, n, k, k, 4, 32), Sm100Out.Bf16(out, n))


def fp4_gemm_nt_native(ctx, a_bf16: torch.Tensor, b_bf16: torch.Tensor, m: int, n: int, k: int,
                       sf_rule: int = SF_RULE_REFERENCE_CPU) -> torch.Tensor:
    """ops_sm100.rs:1646: host bf16 tensors in, host bf16 result out: upload, quantise both operands to packed e2m1 +
    UE8M0 per 32, run the MXF4 kernel, download."""
    dev = torch.device(f"cuda:{ctx.ordinal}")
    a_dev, b_dev = a_bf16.reshape(m, k).to(dev), b_bf16.reshape(n, k).to(dev)
    a_data, a_sf = cast_bf16_to_fp4_packed_sf_dev(ctx, a_dev, k, m, k, 1, sf_rule)
    b_data, b_sf = cast_bf16_to_fp4_packed_sf_dev(ctx, b_dev, k, n, k, 1, sf_rule)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    fp4_gemm_packed_dev(ctx, a_data, a_sf, b_data, b_sf, out, m, n, k)
    ctx.sync()
    return out.cpu()


def bf16_gemm_dev(ctx, a: torch.Tensor, a_ld: int, m: int, b: torch.Tensor, b_ld: int, n: int, k: int, out, epi=None):
    """ops_sm100.rs:893: D[m,n] = A[m,k] . B[n,k]^T, bf16 K-major operands, f32 accumulation."""
    co, ce = out._c(), _epi(epi)
    _check(_bf16_gemm(ctx._h, _vp(a.data_ptr()), a_ld, m, _vp(b.data_ptr()), b_ld, n, k, C.byref(co), C.byref(ce)))


@dataclass
class Bf16Tensor:
    """deepgemm/src/types.rs (Bf16Tensor): a K-major bf16 matrix view."""
    data: torch.Tensor
    rows: int
    k: int
    ld: Optional[int] = None

    def __post_init__(self):
        if self.ld is None:
            self.ld = self.k


def bf16_gemm_nt_dev(ctx, a: "Bf16Tensor", b: "Bf16Tensor", out: torch.Tensor, out_ld: int):
    """deepgemm/src/ops.rs:769: bf16 output (m, out_ld)."""
    bf16_gemm_dev(ctx, a.data, a.ld, a.rows, b.data, b.ld, b.rows, a.k, Sm100Out.Bf16(out, out_ld))


def m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, m_indices: torch.Tensor, b, out, num_groups: int, epi=None):
    """ops_sm100.rs:759; b.rows = num_groups * n."""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_gemm_contig(ctx._h, C.byref(ca), _vp(m_indices.data_ptr()), C.byref(cb), C.byref(co), num_groups, C.byref(ce)))


def m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a, group_ends: torch.Tensor, b, out, num_groups: int, epi=None):
    """Same GEMM from a prebuilt group-end table (see psum_from_m_indices_dev)."""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_gemm_contig_ends(ctx._h, C.byref(ca), _vp(group_ends.data_ptr()), C.byref(cb), C.byref(co), num_groups, C.byref(ce)))


STATIC_MAX_GROUPS = 4096


def m_grouped_fp8_fp4_gemm_contiguous_static_dev(device: int, cuda_stream: int, a, m_indices: torch.Tensor, b, out, num_groups: int,
                                                 epi=None):
    """The contiguous grouped GEMM without a context and without any allocation (no reference
    counterpart): for hosts that may not call the device allocator while running.  Its scratch is an
    array inside the library, shared by all calls on a device (keep them on one stream), good for up
    to STATIC_MAX_GROUPS groups.  The first call on a device does a one-time address lookup and
    should come before any stream capture."""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_gemm_contig_static(device, _vp(cuda_stream), C.byref(ca), _vp(m_indices.data_ptr()), C.byref(cb), C.byref(co), num_groups,
                               C.byref(ce)))


def static_check_status(device: int, cuda_stream: int):
    """Waits for the stream, then raises DgError(Timeout) if a kernel of the allocation-free call gave up on a
    device-side wait (and clears that record); the counterpart of DgContext.sync() for calls made without a context."""
    _check(_static_check_status(device, _vp(cuda_stream)))


def m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, masked_m: torch.Tensor, b, out, num_groups: int, expected_m: int, epi=None):
    """ops_sm100.rs:815; a.rows = m_max, b.rows = num_groups * n."""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_gemm_masked(ctx._h, C.byref(ca), _vp(masked_m.data_ptr()), C.byref(cb), C.byref(co), num_groups, expected_m, C.byref(ce)))


def fp8_fp4_bmm_dev(ctx, a, b, out, num_groups: int, epi=None):
    """ops_sm100.rs:864; a.rows = m and b.rows = n per group."""
    ca, cb, co, ce = a._c(), b._c(), out._c(), _epi(epi)
    _check(_bmm(ctx._h, C.byref(ca), C.byref(cb), C.byref(co), num_groups, C.byref(ce)))


@dataclass
class Fp8Tensor:
    """deepgemm/src/types.rs (Fp8Tensor): e4m3 bytes (rows, ld), K-major."""
    data: torch.Tensor
    rows: int
    k: int
    ld: int


def _f32_args(ctx, a, a_sf_t, b, sfb, m, n, out, out_ld):
    return (ctx._h, _vp(a.data.data_ptr()), a.ld, _vp(a_sf_t.data_ptr()), _vp(b.data.data_ptr()), b.ld, _vp(sfb.data_ptr()), m, n, a.k,
            _vp(out.data_ptr()), out_ld)


def fp8_gemm_nt_dev(ctx, a: Fp8Tensor, a_sf_t: torch.Tensor, b: Fp8Tensor, sfb: torch.Tensor, out: torch.Tensor, out_ld: int):
    """deepgemm/src/ops.rs:328: f32 scales (a_sf_t from transform_sf_dev, sfb per 128x128 tile), bf16 out."""
    _check(_gemm_nt(*_f32_args(ctx, a, a_sf_t, b, sfb, a.rows, b.rows, out, out_ld)))


def m_grouped_fp8_gemm_nt_contiguous_dev(ctx, a, a_sf_t, b, sfb, out, out_ld, m_indices, num_groups: int):
    """deepgemm/src/ops.rs:422; b.rows = num_groups * n."""
    _check(_gemm_nt_contig(*_f32_args(ctx, a, a_sf_t, b, sfb, a.rows, b.rows // max(num_groups, 1), out, out_ld), _vp(m_indices.data_ptr()),
                           num_groups))


def m_grouped_fp8_gemm_nt_masked_dev(ctx, a, a_sf_t, b, sfb, out, out_ld, masked_m, num_groups: int, m_max: int, expected_m: int):
    """deepgemm/src/ops.rs:535; a is (num_groups, m_max, k), b.rows = num_groups * n."""
    _check(_gemm_nt_masked(*_f32_args(ctx, a, a_sf_t, b, sfb, m_max, b.rows // max(num_groups, 1), out, out_ld), _vp(masked_m.data_ptr()),
                           num_groups, expected_m))


def fp8_bmm_nt_dev(ctx, a, a_sf_t, b, sfb, out, out_ld, num_groups: int, m: int, n: int):
    """deepgemm/src/ops.rs:635; a is (num_groups, m, k), b is (num_groups, n, k)."""
    _check(_bmm_nt(*_f32_args(ctx, a, a_sf_t, b, sfb, m, n, out, out_ld), num_groups))


def sf_packed_cols(k: int, gran_k: int) -> int:
    """ops_sm100.rs:1091"""
    return _sf_packed_cols(k, gran_k)


def sf_aligned_rows(rows: int) -> int:
    """ops_sm100.rs:1096"""
    return _sf_aligned_rows(rows)


def alloc_sf(ctx: DgContext, rows: int, k: int, gran_k: int, num_groups: int = 1) -> torch.Tensor:
    """ops_sm100.rs:1107: zero-initialised packed scale buffer (int32 words)."""
    return torch.zeros(_sf_words(rows, k, gran_k, max(num_groups, 1)), dtype=torch.int32, device=f"cuda:{ctx.ordinal}")


def cast_bf16_to_fp8_sf_dev(ctx, src: torch.Tensor, src_ld: int, rows: int, k: int, gran_k: int, num_groups: int = 1
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """ops_sm100.rs:1186: bf16 -> (e4m3 bytes (rows, k), packed UE8M0 words)."""
    dst = torch.empty((rows, k), dtype=torch.uint8, device=src.device)
    sf = alloc_sf(ctx, rows, k, gran_k, num_groups)
    _check(_cast_fp8(ctx._h, _vp(src.data_ptr()), src_ld, rows, k, gran_k, num_groups, _vp(dst.data_ptr()), _vp(sf.data_ptr())))
    return dst, sf


def silu_mul_cast_fp8_sf_dev(ctx, gate_up: torch.Tensor, src_ld: int, rows: int, n: int, gran_k: int = 128, num_groups: int = 1,
                             live_rows: Optional[torch.Tensor] = None, out=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """moe.rs:273-296 (silu(gate) * up on a (rows, 2n) bf16 matrix) fused with the FP8 quantiser of the
    activation: returns (e4m3 bytes (rows, n), packed UE8M0 words) ready to be the next grouped GEMM's A.
    live_rows: optional device word (uint32/int32 tensor); rows from its value on are left unwritten.
    out: optional (bytes, scale words) tensors to write instead of new ones."""
    if out is not None:
        dst, sf = out
    else:
        dst = torch.empty((rows, n), dtype=torch.uint8, device=gate_up.device)
        sf = alloc_sf(ctx, rows, n, gran_k, num_groups)
    _check(_silu_cast(ctx._h, _vp(gate_up.data_ptr()), src_ld, rows, n, gran_k, num_groups, _vp(dst.data_ptr()), _vp(sf.data_ptr()),
                      _vp(live_rows.data_ptr()) if live_rows is not None else _vp()))
    return dst, sf


def cast_bf16_to_fp4_packed_sf_dev(ctx, src: torch.Tensor, src_ld: int, rows: int, k: int, num_groups: int = 1,
                                   sf_rule: int = SF_RULE_REFERENCE_CPU) -> Tuple[torch.Tensor, torch.Tensor]:
    """ops_sm100.rs:1135: bf16 -> (packed e2m1 (rows, k/2), packed per-32 UE8M0 words)."""
    dst = torch.empty((rows, k // 2), dtype=torch.uint8, device=src.device)
    sf = alloc_sf(ctx, rows, k, 32, num_groups)
    _check(_cast_fp4(ctx._h, _vp(src.data_ptr()), src_ld, rows, k, num_groups, sf_rule, _vp(dst.data_ptr()), _vp(sf.data_ptr())))
    return dst, sf


def transform_sf_dev(ctx, sf: torch.Tensor, mn: int, sf_k: int, num_batches: int = 1) -> torch.Tensor:
    """deepgemm/src/ops.rs:52: (batches, mn, sf_k) f32 -> (batches*sf_k, align4(mn)) f32."""
    dst = torch.empty((num_batches * sf_k, sf_aligned_rows(mn)), dtype=torch.float32, device=sf.device)
    _check(_transform_sf(ctx._h, _vp(sf.data_ptr()), mn, sf_k, num_batches, _vp(dst.data_ptr())))
    return dst


def transform_sf1d_packed_ue8m0_dev(ctx, src, src_ld, rows, k, gran_k, num_groups=1) -> torch.Tensor:
    """ops_sm100.rs:1250"""
    dst = alloc_sf(ctx, rows, k, gran_k, num_groups)
    _check(_tsf1d(ctx._h, _vp(src.data_ptr()), src_ld, rows, k, gran_k, num_groups, _vp(dst.data_ptr())))
    return dst


def transform_sf2d_packed_ue8m0_dev(ctx, src, src_ld, rows, k, num_groups=1) -> torch.Tensor:
    """ops_sm100.rs:1294"""
    dst = alloc_sf(ctx, rows, k, 128, num_groups)
    _check(_tsf2d(ctx._h, _vp(src.data_ptr()), src_ld, rows, k, num_groups, _vp(dst.data_ptr())))
    return dst


def transform_sf_t_packed_ue8m0_dev(ctx, src, rows, k, gran_k, num_groups=1) -> torch.Tensor:
    """ops_sm100.rs:1372"""
    dst = alloc_sf(ctx, rows, k, gran_k, num_groups)
    _check(_tsft(ctx._h, _vp(src.data_ptr()), rows, k, gran_k, num_groups, _vp(dst.data_ptr())))
    return dst


def psum_from_m_indices_dev(ctx, m_indices: torch.Tensor, num_groups: int) -> torch.Tensor:
    """ops_sm100.rs:1073: one-past-the-last row of every group (int32 words)."""
    out = torch.empty(num_groups, dtype=torch.int32, device=m_indices.device)
    _check(_group_ends(ctx._h, _vp(m_indices.data_ptr()), m_indices.numel(), num_groups, _vp(out.data_ptr())))
    return out


def unpack_fp4_raw_dev(ctx, src: torch.Tensor, packed_len: int) -> torch.Tensor:
    """ops_sm100.rs:1338"""
    dst = torch.empty(packed_len * 2, dtype=torch.uint8, device=src.device)
    _check(_unpack_fp4(ctx._h, _vp(src.data_ptr()), packed_len, _vp(dst.data_ptr())))
    return dst


def gather_rows_dev(ctx, src: torch.Tensor, idx: torch.Tensor, n_dst: int, dst: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dst row i = src row idx[i] for 2-D byte-addressable tensors (cuda/layout.rs:174 generalised); idx < 0 gives a zero row."""
    row_bytes = src.shape[1] * src.element_size()
    if dst is None:
        dst = torch.empty((n_dst, src.shape[1]), dtype=src.dtype, device=src.device)
    _check(_gather_rows(ctx._h, _vp(src.data_ptr()), src.stride(0) * src.element_size(), _vp(idx.data_ptr()), n_dst, row_bytes,
                        _vp(dst.data_ptr()), dst.stride(0) * dst.element_size()))
    return dst


def moe_pack_rows_dev(ctx, data: torch.Tensor, sf: torch.Tensor, rows: int, k: int, gran_k: int, idx: torch.Tensor, pitch: int) -> torch.Tensor:
    """All-to-all send rows: [k bytes of token idx[i] | its packed scale words | zero padding], `pitch` bytes each."""
    n = idx.numel()
    out = torch.empty((n, pitch), dtype=torch.uint8, device=data.device)
    _check(_moe_pack(ctx._h, _vp(data.data_ptr()), k, _vp(sf.data_ptr()), sf_aligned_rows(rows), sf_packed_cols(k, gran_k), _vp(idx.data_ptr()), n,
                     _vp(out.data_ptr()), pitch))
    return out


def moe_unpack_rows_dev(ctx, recv: torch.Tensor, k: int, gran_k: int, idx: torch.Tensor, n_dst: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Received rows -> (arena data (n_dst, k), packed scale words) with arena row i = received row idx[i] (-1: zero padding row)."""
    data = torch.empty((n_dst, k), dtype=torch.uint8, device=recv.device)
    cols, stride = sf_packed_cols(k, gran_k), sf_aligned_rows(n_dst)
    sf = torch.zeros(cols * stride, dtype=torch.int32, device=recv.device)
    _check(_moe_unpack(ctx._h, _vp(recv.data_ptr()), recv.stride(0), k, cols, _vp(idx.data_ptr()), n_dst, _vp(data.data_ptr()), _vp(sf.data_ptr()),
                       stride))
    return data, sf


def moe_combine_dev(ctx, rows: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out[t] = bf16(sum_j weights[t, j] * rows[pos[t, j]]) (cuda/layout.rs:192-216 as a gather-reduce)."""
    tokens, topk = pos.shape
    n = rows.shape[1]
    out = torch.empty((tokens, n), dtype=torch.bfloat16, device=rows.device)
    _check(_moe_combine(ctx._h, _vp(rows.data_ptr()), rows.stride(0), _vp(pos.data_ptr()), _vp(weights.data_ptr()), tokens, topk, n,
                        _vp(out.data_ptr()), out.stride(0)))
    return out


PEER_HANDLE_BYTES = 64


def peer_alloc(ctx, nbytes: int, export: bool = True) -> Tuple[int, bytes]:
    """A device buffer other processes on this node can map: (address, 64-byte handle to send them;
    empty when export is False, for a buffer nobody else will map)."""
    ptr, handle = _vp(), C.create_string_buffer(PEER_HANDLE_BYTES)
    _check(_peer_alloc(ctx._h, nbytes, C.byref(ptr), handle if export else None))
    return ptr.value, (handle.raw if export else b"")


def peer_open(ctx, handle: bytes) -> int:
    ptr = _vp()
    _check(_peer_open(ctx._h, C.create_string_buffer(bytes(handle), PEER_HANDLE_BYTES), C.byref(ptr)))
    return ptr.value


def peer_close(ctx, ptr: int):
    _check(_peer_close(ctx._h, _vp(ptr)))


def peer_free(ctx, ptr: int):
    _check(_peer_free(ctx._h, _vp(ptr)))


class _RawDeviceArray:
    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, ordinal: int) -> torch.Tensor:
    """A torch view of device memory this library allocated (no copy; the caller keeps the memory alive)."""
    if dtype == torch.bfloat16:     # the array interface has no bf16: view 16-bit words
        return torch.as_tensor(_RawDeviceArray(ptr, shape, "<i2"), device=f"cuda:{ordinal}").view(torch.bfloat16)
    typestr = {torch.uint8: "|u1", torch.int32: "<i4", torch.int64: "<i8", torch.float32: "<f4"}[dtype]
    return torch.as_tensor(_RawDeviceArray(ptr, shape, typestr), device=f"cuda:{ordinal}")


def ep_block_hist_words(pairs: int, num_experts: int) -> int:
    return _ep_hist_words(pairs, num_experts)


def ep_count_dev(ctx, expert_of_pair, pairs, num_experts, local_rank, block_hist, counts):
    _check(_ep_count(ctx._h, _vp(expert_of_pair.data_ptr()), pairs, num_experts, _vp(local_rank.data_ptr()), _vp(block_hist.data_ptr()),
                     _vp(counts.data_ptr())))


def ep_layout_dev(ctx, all_counts, world, rank, num_experts, alignment, capacity, pair_base, group_ends, totals, slot_rows=0):
    _check(_ep_layout(ctx._h, _vp(all_counts.data_ptr()), world, rank, num_experts, alignment, capacity, slot_rows, _vp(pair_base.data_ptr()),
                      _vp(group_ends.data_ptr()), _vp(totals.data_ptr())))


def ep_dispatch_dev(ctx, expert_of_pair, local_rank, block_base, pair_base, pairs, topk, num_experts, world, data, k, sf, sf_stride, sf_cols,
                    peer_data, peer_sf, peer_sf_stride, capacity, pos_of_pair, max_blocks=0, slot_rows=0):
    _check(_ep_dispatch(ctx._h, _vp(expert_of_pair.data_ptr()), _vp(local_rank.data_ptr()), _vp(block_base.data_ptr()),
                        _vp(pair_base.data_ptr()), pairs, topk, num_experts, world, _vp(data.data_ptr()), k, _vp(sf.data_ptr()), sf_stride,
                        sf_cols, _vp(peer_data.data_ptr()), _vp(peer_sf.data_ptr()), peer_sf_stride, capacity, slot_rows,
                        _vp(pos_of_pair.data_ptr()), max_blocks))


def ep_combine_dev(ctx, expert_of_pair, pos_of_pair, weights, tokens, topk, num_experts, world, peer_rows, pitch, n, out, out_pitch,
                   max_blocks=0):
    _check(_ep_combine(ctx._h, _vp(expert_of_pair.data_ptr()), _vp(pos_of_pair.data_ptr()), _vp(weights.data_ptr()), tokens, topk,
                       num_experts, world, _vp(peer_rows.data_ptr()), pitch, n, _vp(out.data_ptr()), out_pitch, max_blocks))


def debug_expire_wait(ctx, limit_us: int = 1000):
    """Launches the bounded-wait self-test; the following ctx.sync() raises DgError(Timeout) once."""
    _check(_expire_wait(ctx._h, limit_us))


def set_mk_alignment_for_contiguous_layout(value: int):
    """types.rs:195 (raises instead of panicking on a bad value)."""
    _check(_set_mk(value))


def get_mk_alignment_for_contiguous_layout() -> int:
    """types.rs:204"""
    return _get_mk()


def get_theoretical_mk_alignment_for_contiguous_layout(arch_major: int) -> int:
    """types.rs:213"""
    return _get_mk_theory(arch_major)


@dataclass
class Sm100Desc:
    """heuristics_sm100.rs:61-87 (fields this build's tile choice reads)."""
    gemm_type: int
    m: int
    n: int
    k: int
    num_groups: int = 1
    expected_m: int = 0
    a_bits: int = 8
    b_bits: int = 8
    gran_a: int = 128
    gran_b: int = 128
    cd_dtype: int = 0
    num_sms: int = 148
    major_a_mn: bool = False
    major_b_mn: bool = False


@dataclass
class Sm100Config:
    """heuristics_sm100.rs:17-57 flattened."""
    swap_ab: bool
    block_m: int
    block_n: int
    block_k: int
    cluster_m: int
    cluster_n: int
    num_stages: int
    num_accum_stages: int
    smem_size: int
    num_tiles: int
    num_splits: int = 1


SM100_SMEM_CAPACITY = 232448


def best_config(desc: Sm100Desc) -> Sm100Config:
    """heuristics_sm100.rs:455"""
    d = _Desc(desc.gemm_type, desc.m, desc.n, desc.k, desc.num_groups, desc.expected_m or desc.m, desc.a_bits, desc.b_bits,
              desc.gran_a, desc.gran_b, desc.cd_dtype, desc.num_sms, int(desc.major_a_mn), int(desc.major_b_mn))
    c = _Config()
    _check(_best_config(C.byref(d), C.byref(c)))
    return Sm100Config(bool(c.swap_ab), c.block_m, c.block_n, c.block_k, c.cluster_m, c.cluster_n, c.num_stages,
                       c.num_accum_stages, c.smem_size, c.num_tiles, c.num_splits)
