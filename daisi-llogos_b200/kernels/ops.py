"""Python face of the CUDA kernels: every function takes torch CUDA tensors, checks them,
and launches on the current stream.  Nothing here computes on the CPU, and nothing falls
back: a tensor that is not on the GPU, or a library that cannot be built, is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_library

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; checked against the library at first use


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t: Optional[torch.Tensor], dtype=None) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"a kernel was given a non-contiguous tensor of shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"expected {dtype}, got {t.dtype}")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current stream of the current device (the raw query: this runs once per launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launches() -> int:
    """Kernels launched (or recorded into a CUDA graph) by this module so far."""
    return _launches


def _check(lib, rc: int, kernels: int = 1) -> None:
    global _launches
    if rc != 0:
        raise KernelError(lib.llg_last_error().decode("utf-8", "replace"))
    _launches += kernels


# ---- libraries and prototypes ---------------------------------------------------------

class _RowScale(Structure):
    _fields_ = [("ss", c_void_p), ("parts", c_int), ("inv_width", c_float), ("eps", c_float)]


class RowScale:
    """What a norm leaves to the consumer of its output when it does not divide by the root mean square itself: the
    output holds ``x * weight`` and ``ss`` (float32 ``[rows, parts]``) the sums of squares of each row of ``x``, whole
    or as partial sums; the consumer multiplies row r of its product by ``1 / sqrt(sum(ss[r]) / width + eps)``."""

    def __init__(self, ss: torch.Tensor, width: int, eps: float):
        if ss.dim() != 2 or ss.dtype != torch.float32:
            raise KernelError("a row scale's sums are float32 [rows, parts]")
        self.ss, self.width, self.eps = ss, int(width), float(eps)

    @property
    def rows(self) -> int:
        return self.ss.shape[0]

    def slice(self, r0: int, r1: int) -> "RowScale":
        return RowScale(self.ss[r0:r1], self.width, self.eps)

    def c(self) -> "_RowScale":
        return _RowScale(_ptr(self.ss, torch.float32), self.ss.shape[1], 1.0 / self.width, self.eps)


def _scale_ref(row_scale: Optional[RowScale], rows: int):
    """ctypes argument for an optional ``const RowScale*``."""
    if row_scale is None:
        return None
    if row_scale.rows != rows:
        raise KernelError(f"a row scale for {row_scale.rows} rows was given to a product of {rows} rows")
    return byref(row_scale.c())


class _QkPrepArgs(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("qkv_dtype", c_int), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("norm_w_dtype", c_int), ("norm_eps", c_float),
        ("bias", c_void_p), ("bias_dtype", c_int),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("rotary_dim", c_int), ("pairing", c_int),
        ("table_positions", c_int), ("positions", c_void_p),
        ("q_out", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p),
        ("table_width", c_int), ("ring_pages", c_int),
        ("seq_of_token", c_void_p), ("slots", c_void_p),
        ("n_tokens", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int),
        ("row_scale", _RowScale),
        ("vd", c_int), ("v_mix", c_void_p), ("v_first_in", c_void_p), ("v_first_out", c_void_p),
    ]


class _PrefillArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p),
        ("page_table", c_void_p), ("table_width", c_int), ("ring_pages", c_int),
        ("tiles", c_void_p), ("cu_tokens", c_void_p), ("len_before", c_void_p), ("slots", c_void_p),
        ("out", c_void_p),
        ("n_tiles", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int),
        ("scale", c_float), ("window", c_int), ("n_tokens", c_int), ("n_pages", c_int),
        ("vd", c_int), ("has_sink", c_int), ("sink_score", c_float), ("gate", c_void_p),
        ("sinks", c_void_p), ("chunked", c_int),
    ]


class _DecodeArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p),
        ("table_width", c_int), ("ring_pages", c_int), ("slots", c_void_p), ("len_before", c_void_p),
        ("part_o", c_void_p), ("part_ml", c_void_p),
        ("n_seqs", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("n_splits", c_int),
        ("scale", c_float), ("window", c_int),
        ("vd", c_int), ("has_sink", c_int), ("sink_score", c_float), ("gate", c_void_p),
        ("sinks", c_void_p), ("chunked", c_int),
    ]


class _HyperNormArgs(Structure):
    _fields_ = [
        ("streams", c_void_p), ("stream_stride", c_longlong), ("n_streams", c_int),
        ("branch", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("mix", c_void_p), ("write", c_void_p), ("read", c_void_p),
        ("weight", c_void_p), ("weight_dtype", c_int), ("eps", c_float),
        ("out", c_void_p), ("out_dtype", c_int), ("rows", c_void_p), ("n_out", c_int), ("hidden", c_int),
    ]


class _QkvRowPrepArgs(Structure):
    _fields_ = [
        ("qkvg", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("bias", c_void_p), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("w_dtype", c_int), ("norm_eps", c_float),
        ("positions", c_void_p), ("q_out", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p), ("table_width", c_int),
        ("ring_pages", c_int), ("seq_of_token", c_void_p), ("slots", c_void_p), ("gate_out", c_void_p),
        ("n_tokens", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("vd", c_int),
    ]


class _DecodeTmaArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("page_table", c_void_p), ("table_width", c_int), ("ring_pages", c_int),
        ("slots", c_void_p), ("len_before", c_void_p), ("part", c_void_p), ("counters", c_void_p), ("out", c_void_p),
        ("n_seqs", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("scale", c_float), ("window", c_int),
        ("has_sink", c_int), ("sink_score", c_float), ("gate", c_void_p),
        ("sinks", c_void_p), ("chunked", c_int),
    ]


_LN_BRANCHES = 4


class _LayerNormArgs(Structure):
    _fields_ = [
        ("residual", c_void_p), ("branch", c_void_p * _LN_BRANCHES), ("n_partials", c_int * _LN_BRANCHES),
        ("partial_stride", c_longlong), ("scale", c_float), ("weight", c_void_p), ("bias", c_void_p), ("w_dtype", c_int),
        ("eps", c_float), ("out", c_void_p), ("out_dtype", c_int), ("rows", c_void_p), ("n_out", c_int), ("hidden", c_int),
    ]


class _GroupNormArgs(Structure):
    _fields_ = [
        ("residual", c_void_p), ("branch", c_void_p), ("n_partials", c_int), ("gate", c_void_p), ("gate_partials", c_int),
        ("partial_stride", c_longlong), ("gate_bias", c_void_p), ("post_w", c_void_p), ("post_groups", c_int),
        ("post_eps", c_float), ("weight", c_void_p), ("w_dtype", c_int), ("groups", c_int), ("eps", c_float),
        ("out", c_void_p), ("out_dtype", c_int), ("rows", c_void_p), ("n_out", c_int), ("hidden", c_int),
    ]


class _MinGruArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong), ("bias", c_void_p), ("state", c_void_p),
        ("slots", c_void_p), ("cu_tokens", c_void_p), ("out", c_void_p), ("out_dtype", c_int), ("carry", c_void_p),
        ("pieces", c_int), ("n_seqs", c_int), ("n_tokens", c_int), ("size", c_int),
    ]


class _AddNormTerm(Structure):
    _fields_ = [("data", c_void_p), ("n_partials", c_int), ("norm_w", c_void_p), ("norm_eps", c_float), ("scale", c_float)]


class _AddNormOut(Structure):
    _fields_ = [("out", c_void_p), ("weight", c_void_p), ("offset", c_float)]


ADDNORM_MAX_TERMS = 4        # terms and outputs of ``multi_add_rmsnorm``; checked against the library at first use
ADDNORM_MAX_OUTS = 2


class _AddNormArgs(Structure):
    _fields_ = [
        ("residual", c_void_p), ("partial_stride", c_longlong), ("terms", _AddNormTerm * ADDNORM_MAX_TERMS), ("n_terms", c_int),
        ("outs", _AddNormOut * ADDNORM_MAX_OUTS), ("n_outs", c_int), ("out_dtype", c_int), ("eps", c_float),
        ("rows", c_void_p), ("n_out", c_int), ("hidden", c_int),
    ]


class _HashEmbedArgs(Structure):
    _fields_ = [
        ("table", c_void_p), ("table_dtype", c_int), ("scale", c_float), ("pair_table", c_void_p), ("pair_dtype", c_int),
        ("buckets", c_int), ("mul_prev", c_longlong), ("mul_cur", c_longlong),
        ("token_ids", c_void_p), ("positions", c_void_p), ("seq_of_token", c_void_p), ("cu_tokens", c_void_p),
        ("slots", c_void_p), ("last_token", c_void_p), ("norm_w", c_void_p), ("norm_offset", c_float), ("eps", c_float),
        ("out", c_void_p), ("n_tokens", c_int), ("vocab", c_int), ("hidden", c_int),
    ]


class _TableGateArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong), ("table", c_void_p),
        ("table_dtype", c_int), ("table_width", c_int), ("col0", c_int), ("token_ids", c_void_p), ("act", c_int),
        ("out", c_void_p), ("out_dtype", c_int), ("n_tokens", c_int), ("width", c_int), ("vocab", c_int),
    ]


class _ConvArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("row_width", c_int), ("col0", c_int), ("channels", c_int), ("taps", c_int),
        ("in_bias", c_void_p), ("weight", c_void_p), ("bias", c_void_p), ("state", c_void_p),
        ("slots", c_void_p), ("cu_tokens", c_void_p), ("seq_of_token", c_void_p), ("len_before", c_void_p),
        ("out", c_void_p), ("out2", c_void_p), ("out2_dtype", c_int), ("n_seqs", c_int), ("n_tokens", c_int),
    ]


class _RgLruArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong), ("row_width", c_int), ("y_col", c_int),
        ("y_bias", c_void_p), ("u", c_void_p), ("gates", c_void_p), ("gate_bias", c_void_p), ("lam", c_void_p),
        ("decay_scale", c_float), ("state", c_void_p), ("slots", c_void_p), ("cu_tokens", c_void_p),
        ("out", c_void_p), ("out_dtype", c_int), ("carry", c_void_p), ("pieces", c_int),
        ("n_seqs", c_int), ("n_tokens", c_int), ("size", c_int), ("block_width", c_int),
    ]


class _RetentionArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("row_width", c_int), ("q_col", c_int), ("k_col", c_int), ("v_col", c_int), ("g_col", c_int),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("rotary_dim", c_int), ("table_positions", c_int),
        ("positions", c_void_p), ("decay", c_void_p), ("k_scale", c_float), ("eps", c_float),
        ("state", c_void_p), ("slots", c_void_p), ("cu_tokens", c_void_p), ("out", c_void_p), ("out_dtype", c_int),
        ("carry", c_void_p), ("pieces", c_int),
        ("n_seqs", c_int), ("n_tokens", c_int), ("nh", c_int), ("dim", c_int), ("vdim", c_int),
    ]


class _RouterRule(Structure):
    _fields_ = [("score", c_int), ("groups", c_int), ("keep_groups", c_int), ("group_top", c_int), ("scale", c_float),
                ("sum_eps", c_float)]


class _LatentPrepArgs(Structure):
    _fields_ = [
        ("rows", c_void_p), ("n_partials", c_int), ("partial_stride", c_longlong),
        ("row_width", c_int), ("q_col", c_int), ("kv_col", c_int), ("cq_col", c_int), ("cq_rank", c_int),
        ("cq_norm_w", c_void_p), ("cq_out", c_void_p), ("pairing", c_int),
        ("c_norm_w", c_void_p), ("w_dtype", c_int), ("norm_eps", c_float),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("table_positions", c_int), ("positions", c_void_p),
        ("q_plain", c_void_p), ("q_out", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("page_table", c_void_p), ("table_width", c_int),
        ("ring_pages", c_int), ("seq_of_token", c_void_p), ("slots", c_void_p),
        ("n_tokens", c_int), ("nh", c_int), ("dim", c_int), ("rdim", c_int), ("rank", c_int),
    ]


class _HeadLinearArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_token_stride", c_longlong), ("x_head_stride", c_longlong), ("w", c_void_p),
        ("y", c_void_p), ("y_token_stride", c_longlong), ("y_head_stride", c_longlong),
        ("n_tokens", c_int), ("nh", c_int), ("n_in", c_int), ("n_out", c_int),
    ]


class _GroupedLinearArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("token_of_row", c_void_p), ("tile_expert", c_void_p), ("w", c_void_p), ("w2", c_void_p),
        ("y", c_void_p), ("rows", c_int), ("n_in", c_int), ("n_out", c_int),
        ("x_row_stride", c_longlong), ("y_row_stride", c_longlong), ("x_group_stride", c_longlong),
        ("y_group_stride", c_longlong), ("n_rows", c_int), ("w_group_stride", c_longlong),
    ]


class _SampleArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("work", c_void_p), ("out", c_void_p), ("probs_out", c_void_p),
        ("seq_ids", c_void_p), ("history", c_void_p), ("history_len", c_void_p), ("history_stride", c_int),
        ("n_seqs", c_int), ("vocab", c_int),
        ("temperature", c_float), ("top_k", c_int),
        ("top_p", c_float), ("min_p", c_float), ("typical_p", c_float), ("min_keep", c_int),
        ("repetition_penalty", c_float), ("frequency_penalty", c_float), ("presence_penalty", c_float),
        ("penalize_newline", c_int), ("seed", c_ulonglong), ("step", c_int),
        ("banned", c_void_p), ("n_banned", c_int),
        ("cand_val", c_void_p), ("cand_idx", c_void_p), ("cand_count", c_void_p), ("n_slices", c_int),
        ("history_rows", c_void_p), ("history_append", c_int),
        ("slice_stats", c_void_p),
    ]


_protos_done = set()


_libs = {}


def _lib(name: str):
    lib = _libs.get(name)
    if lib is not None:
        return lib
    lib = _load_lib(name)
    _libs[name] = lib
    return lib


def _load_lib(name: str):
    lib = load_library(name)
    if name in _protos_done:
        return lib
    if name == "elementwise":
        lib.llg_page_size.restype = c_int
        if lib.llg_page_size() != PAGE:
            raise KernelError(f"the kernels use pages of {lib.llg_page_size()} tokens, Python expects {PAGE}")
        lib.llg_embed_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.llg_embed_rows_copies.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_void_p]
        lib.llg_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float,
                                        c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.llg_qk_prep.argtypes = [POINTER(_QkPrepArgs), c_int, c_void_p]
        lib.llg_kv_write.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.llg_silu_mul.argtypes = [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.llg_gate_mul.argtypes = [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.llg_tanh_cap.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        lib.llg_scatter_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.llg_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.llg_zero_rows.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
        lib.llg_hc_add_rmsnorm.argtypes = [POINTER(_HyperNormArgs), c_void_p]
        lib.llg_qkv_row_prep.argtypes = [POINTER(_QkvRowPrepArgs), c_int, c_void_p]
        lib.llg_act_rows.argtypes = [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_void_p]
    elif name == "gemm_simt":
        lib.llg_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                      POINTER(_RowScale), c_void_p]
    elif name == "gemm_tc":
        lib.llg_gemm_tc_supported.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int]
        lib.llg_gemm_tc_splits.argtypes = [c_int, c_int]
        lib.llg_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    POINTER(_RowScale), c_void_p]
        lib.llg_gemm_tc_gated.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          POINTER(_RowScale), c_void_p]
        lib.llg_gemm_tc_qkv.argtypes = [c_void_p, c_void_p, c_int, c_int, POINTER(_QkPrepArgs), c_void_p]
        lib.llg_gemm_tc_grouped.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                            c_int, c_void_p]
        lib.llg_gemm_tc_act.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        POINTER(_RowScale), c_void_p]
    elif name == "attention_simt":
        lib.llg_attn_prefill_simt.argtypes = [POINTER(_PrefillArgs), c_int, c_void_p]
        lib.llg_attn_decode_simt.argtypes = [POINTER(_DecodeArgs), c_void_p, c_int, c_void_p]
        lib.llg_attn_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_scratch_floats.restype = c_longlong
    elif name == "attention_mma":
        lib.llg_attn_mma_supported.argtypes = [c_int]
        lib.llg_attn_prefill_mma.argtypes = [POINTER(_PrefillArgs), c_void_p]
        lib.llg_attn_decode_mma.argtypes = [POINTER(_DecodeArgs), c_void_p, c_void_p, c_int, c_void_p]
    elif name == "attention_tc":
        lib.llg_attn_tc_supported.argtypes = [c_int]
        lib.llg_attn_prefill_tc.argtypes = [POINTER(_PrefillArgs), c_void_p]
        lib.llg_attn_tc_status.restype = c_int
    elif name == "attention_decode_tma":
        lib.llg_attn_decode_tma_supported.argtypes = [c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_tma_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.llg_attn_decode_tma_scratch_floats.restype = c_longlong
        lib.llg_attn_decode_tma.argtypes = [POINTER(_DecodeTmaArgs), c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.llg_attn_decode_tma_status.restype = c_int
    elif name == "layernorm":
        lib.llg_add_layernorm.argtypes = [POINTER(_LayerNormArgs), c_void_p]
    elif name == "groupnorm":
        lib.llg_gated_add_group_rmsnorm.argtypes = [POINTER(_GroupNormArgs), c_void_p]
        lib.llg_norm_max_groups.restype = c_int
        if lib.llg_norm_max_groups() != NORM_MAX_GROUPS:
            raise KernelError(f"the norm kernel takes {lib.llg_norm_max_groups()} groups, Python expects {NORM_MAX_GROUPS}")
    elif name == "addnorm":
        lib.llg_multi_add_rmsnorm.argtypes = [POINTER(_AddNormArgs), c_void_p]
        lib.llg_hash_embed.argtypes = [POINTER(_HashEmbedArgs), c_void_p]
        lib.llg_table_gate.argtypes = [POINTER(_TableGateArgs), c_void_p]
        if (lib.llg_addnorm_max_terms(), lib.llg_addnorm_max_outs()) != (ADDNORM_MAX_TERMS, ADDNORM_MAX_OUTS):
            raise KernelError("the add-and-norm kernel's limits differ from what Python expects")
    elif name == "recurrent":
        lib.llg_causal_conv.argtypes = [POINTER(_ConvArgs), c_void_p]
        lib.llg_rglru_scan.argtypes = [POINTER(_RgLruArgs), c_int, c_void_p]
        lib.llg_retention.argtypes = [POINTER(_RetentionArgs), c_int, c_void_p]
        if (lib.llg_conv_max_taps(), lib.llg_retention_piece()) != (CONV_MAX_TAPS, RETENTION_PIECE):
            raise KernelError("the convolution's taps or retention's pieces differ from what Python expects")
        lib.llg_mingru_scan.argtypes = [POINTER(_MinGruArgs), c_int, c_void_p]
        lib.llg_mingru_piece.restype = c_int
        if lib.llg_mingru_piece() != MINGRU_PIECE:
            raise KernelError(f"the scan's pieces hold {lib.llg_mingru_piece()} tokens, Python expects {MINGRU_PIECE}")
    elif name == "latent":
        lib.llg_latent_prep.argtypes = [POINTER(_LatentPrepArgs), c_int, c_void_p]
        lib.llg_sigmoid_gate.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_int, c_int,
                                         c_void_p]
        lib.llg_head_linear.argtypes = [POINTER(_HeadLinearArgs), c_int, c_int, c_void_p]
    elif name == "moe":
        lib.llg_moe_route.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      POINTER(_RouterRule), c_void_p, c_void_p]
        lib.llg_head_linear_mma_supported.argtypes = [c_void_p, c_longlong, c_longlong, c_void_p, c_int]
        lib.llg_head_linear_mma.argtypes = [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong,
                                            c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.llg_moe_topk.argtypes = [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     POINTER(_RouterRule), c_void_p, c_void_p]
        lib.llg_moe_plan.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.llg_moe_gather_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.llg_grouped_linear.argtypes = [POINTER(_GroupedLinearArgs), c_int, c_int, c_void_p]
        lib.llg_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_void_p]
    elif name == "init":
        lib.llg_fill_normal.argtypes = [c_void_p, c_int, c_longlong, c_ulonglong, ctypes.c_double, ctypes.c_double, c_void_p]
        lib.llg_fill.argtypes = [c_void_p, c_int, c_longlong, c_float, c_void_p]
        lib.llg_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
    elif name == "sampling":
        lib.llg_argmax.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.llg_sample.argtypes = [POINTER(_SampleArgs), c_void_p]
        lib.llg_sample_slices.argtypes = [c_int]
    _protos_done.add(name)
    return lib


_sm_counts = {}


def sm_count() -> int:
    """Multiprocessors of the current CUDA device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return n


def require_gpu() -> None:
    """Fails loudly when there is no GPU or the kernels cannot be loaded."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library runs on the GPU only and has no CPU path")
    _lib("elementwise")


# ---- kernels ------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, token_ids: torch.Tensor, out_residual: torch.Tensor) -> None:
    """out_residual[n] = table[token_ids[n]] as float32; a residual of several streams ``[S, N, hidden]`` gets the row in
    every stream."""
    lib = _lib("elementwise")
    vocab, hidden = table.shape
    n = token_ids.numel()
    if out_residual.dim() == 3:
        assert out_residual.shape[1:] == (n, hidden)
        _check(lib, lib.llg_embed_rows_copies(_ptr(table), _dt(table), _ptr(token_ids, torch.int32),
                                              _ptr(out_residual, torch.float32), n, hidden, vocab, out_residual.shape[0],
                                              n * hidden, _stream()))
        return
    assert out_residual.shape == (n, hidden)
    _check(lib, lib.llg_embed_rows(_ptr(table), _dt(table), _ptr(token_ids, torch.int32),
                                   _ptr(out_residual, torch.float32), n, hidden, vocab, _stream()))


def add_rmsnorm(residual: torch.Tensor, branch: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, ss_out: Optional[torch.Tensor] = None) -> None:
    """residual += sum of branch partials (if any); out[j] = RMSNorm(residual[rows[j] or j]) * weight.

    ``residual`` is float32 ``[N, H]``; ``branch`` float32 ``[S, N, H]`` or None; ``out`` ``[M, H]``.
    With ``ss_out`` (float32 ``[M, norm_ss_parts(M, H)]``) the division is left to whoever consumes ``out``: ``out[j]``
    is the row times ``weight`` and ``ss_out[j]`` holds the row's sum of squares, whole or as the sums of equal slices
    of the row in their order (see ``RowScale``).
    """
    lib = _lib("elementwise")
    n, hidden = residual.shape
    m = out.shape[0]
    assert out.shape[1] == hidden and weight.shape == (hidden,)
    if rows is not None:
        assert rows.numel() == m
    else:
        assert m == n
    if ss_out is not None:
        assert tuple(ss_out.shape) == (m, norm_ss_parts(m, hidden)), (ss_out.shape, m, hidden)
    n_part, stride = 0, 0
    if branch is not None:
        assert branch.dim() == 3 and branch.shape[1:] == (n, hidden), (branch.shape, residual.shape)
        n_part, stride = branch.shape[0], n * hidden
    _check(lib, lib.llg_add_rmsnorm(_ptr(residual, torch.float32), _ptr(branch, torch.float32), n_part, stride,
                                    _ptr(weight), _dt(weight), float(eps), _ptr(out), _dt(out),
                                    _ptr(rows, torch.int32), m, hidden, _ptr(ss_out, torch.float32), _stream()))


_ss_parts = {}


def norm_ss_parts(n_out: int, hidden: int) -> int:
    """Sums of squares per row that ``add_rmsnorm(..., ss_out=)`` writes for these sizes: one, or for the few rows
    of a decode step one per slice of the row (each slice is a block of its own there)."""
    key = (n_out <= 64, hidden)
    p = _ss_parts.get(key)
    if p is None:
        lib = _lib("elementwise")
        lib.llg_add_rmsnorm_parts.argtypes = [c_int, c_int]
        p = _ss_parts[key] = lib.llg_add_rmsnorm_parts(1 if n_out <= 64 else 65, hidden)
    return p


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale: Optional[RowScale] = None) -> None:
    """out[n, o] = sum_k x[n, k] w[o, k] on the CUDA cores, float32 accumulation; rows times ``row_scale`` if given."""
    lib = _lib("gemm_simt")
    n, k = x.shape
    o, k2 = w.shape
    assert k == k2 and out.shape == (n, o), (x.shape, w.shape, out.shape)
    _check(lib, lib.llg_gemm_simt(_ptr(x), _dt(x), _ptr(w), _dt(w), _ptr(out), _dt(out), n, o, k,
                                  _scale_ref(row_scale, n), _stream()))


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes this product (bfloat16 operands, k a multiple of 8)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not (x.is_cuda and w.is_cuda):
        return False
    # the library's rule (llg_gemm_tc_supported), kept here because this runs before every product
    return x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


_splits_cache = {}


def gemm_tc_splits(k: int, wish: int) -> int:
    """The number of split-K partials the kernel writes when asked for ``wish``."""
    key = (k, wish)
    s = _splits_cache.get(key)
    if s is None:
        s = _splits_cache[key] = _lib("gemm_tc").llg_gemm_tc_splits(k, wish)
    return s


def gated_rows(features: int) -> int:
    """Rows of a gate/up matrix in the gated layout: the gate rows, filled up to a multiple of 128, then
    the up rows in the same way."""
    return -(-features // 128) * 256


GATE_ACTIVATIONS = ("silu", "gelu_tanh")     # what the gate of a gated feed-forward may pass


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, tile_n: int = 0, gated_features: int = 0,
            row_scale: Optional[RowScale] = None, gate_activation: str = "silu") -> None:
    """out[s, n, o] = split-K partials of x[n, k] w[o, k] on the tensor cores (tcgen05, TMA).

    ``out`` is ``[S, N, O]`` float32 with S = ``gemm_tc_splits(k, wish)``, or ``[1, N, O]`` bfloat16.
    With ``gated_features = F`` the matrix ``w`` is in the gated layout (``gated_rows(F)`` rows) and
    ``out`` is ``[1, N, F]`` holding ``act(gate) * up`` with ``act`` = ``gate_activation`` (one of ``GATE_ACTIVATIONS``).  ``row_scale``: what a norm left for the rows of ``x``;
    the rows of the product are multiplied by it (before the gating).
    """
    lib = _lib("gemm_tc")
    n, k = x.shape
    o, k2 = w.shape
    s = out.shape[0]
    assert k == k2 and out.shape == (s, n, gated_features if gated_features else o), (x.shape, w.shape, out.shape)
    if gemm_tc_splits(k, s) != s:
        raise KernelError(f"gemm_tc: {s} splits cannot be had for k = {k}")
    if gate_activation != "silu":
        if gate_activation not in GATE_ACTIVATIONS or not gated_features:
            raise KernelError(f"gemm_tc: gate activation '{gate_activation}' (known: {', '.join(GATE_ACTIVATIONS)}; gated products only)")
        _check(lib, lib.llg_gemm_tc_gated(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(out), _dt(out), n, o, k, tile_n,
                                          gated_features, ACTIVATIONS[gate_activation], _scale_ref(row_scale, n), _stream()))
        return
    _check(lib, lib.llg_gemm_tc(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(out), _dt(out), n, o, k, s,
                                tile_n, gated_features, _scale_ref(row_scale, n), _stream()))


def gemm_tc_act(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, kind: str, row_scale: Optional[RowScale] = None) -> None:
    """out[n, o] = act(x[n, k] w[o, k]) on the tensor cores in one split: the activation (one of ``ACTIVATIONS``) is the
    product's epilogue, applied to the float32 sums before they are rounded to ``out`` (bfloat16)."""
    lib = _lib("gemm_tc")
    n, k = x.shape
    o, k2 = w.shape
    assert k == k2 and out.shape == (n, o), (x.shape, w.shape, out.shape)
    if kind not in ACTIVATIONS:
        raise KernelError(f"gemm_tc_act: activation '{kind}' is not known ({', '.join(ACTIVATIONS)})")
    _check(lib, lib.llg_gemm_tc_act(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(out, torch.bfloat16), _dt(out), n, o, k,
                                    ACTIVATIONS[kind], _scale_ref(row_scale, n), _stream()))


def gemm_tc_status() -> int:
    """Error code a tensor-core product recorded when a wait ran out (0 = none); synchronises."""
    lib = _lib("gemm_tc")
    lib.llg_gemm_tc_status.restype = c_int
    return lib.llg_gemm_tc_status()


def qk_prep(qkv: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
            q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], norm_eps: float,
            bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
            rotary_dim: int, pairing: int, positions: torch.Tensor, q_out: torch.Tensor,
            k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
            k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
            page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
            seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
            row_scale: Optional[RowScale] = None, value_dim: int = 0, v_mix: Optional[torch.Tensor] = None,
            v_first_in: Optional[torch.Tensor] = None, v_first_out: Optional[torch.Tensor] = None) -> None:
    """Per-head norm (optional), bias (optional), rotation, and the writes of q, k, v.

    ``qkv`` is ``[S, N, (nh + nkv) * hd + nkv * vd]`` (partials are summed; ``vd = value_dim or hd``).  Queries go to
    ``q_out``; keys and values go to ``k_new``/``v_new`` (packed, for a prompt step) and/or straight into
    the cache pages (for a one-token step).  ``row_scale``: what a norm left for the token rows; the summed
    partials are multiplied by it before anything else.  Values blended across layers: ``v_first_out`` (float32
    ``[N, nkv, vd]``) receives the values as projected; with ``v_first_in`` and ``v_mix`` (one float32 number lam on the
    device) the values written are ``(1 - lam) v + lam v_first_in``.
    """
    lib = _lib("elementwise")
    s, n, width = qkv.shape
    vd = value_dim or head_dim
    assert width == (n_heads + n_kv_heads) * head_dim + n_kv_heads * vd
    a = _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
                   positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)
    a.qkv, a.qkv_dtype, a.n_partials, a.partial_stride = _ptr(qkv), _dt(qkv), s, n * width
    a.vd = 0 if vd == head_dim else vd
    for t in (v_first_in, v_first_out):
        if t is not None and tuple(t.shape) != (n, n_kv_heads, vd):
            raise KernelError(f"qk_prep: lent values of shape {tuple(t.shape)}, expected {(n, n_kv_heads, vd)}")
    if (v_first_in is None) != (v_mix is None):
        raise KernelError("qk_prep: the values to blend with and the blend's weight come together")
    a.v_mix, a.v_first_in = _ptr(v_mix, torch.float32), _ptr(v_first_in, torch.float32)
    a.v_first_out = _ptr(v_first_out, torch.float32)
    _set_scale(a, row_scale, n)
    _check(lib, lib.llg_qk_prep(byref(a), _dt(q_out), _stream()))


def _set_scale(a: "_QkPrepArgs", row_scale: Optional[RowScale], n: int) -> None:
    if row_scale is not None:
        if row_scale.rows != n:
            raise KernelError(f"a row scale for {row_scale.rows} rows was given to {n} token rows")
        a.row_scale = row_scale.c()


def _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
               positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots) -> "_QkPrepArgs":
    """The argument block of the q/k/v preparation, without the q/k/v input itself."""
    a = _QkPrepArgs()
    a.q_norm_w, a.k_norm_w = _ptr(q_norm_w), _ptr(k_norm_w)
    a.norm_w_dtype = _dt(q_norm_w) if q_norm_w is not None else F32
    a.norm_eps = float(norm_eps)
    a.bias = _ptr(bias)
    a.bias_dtype = _dt(bias) if bias is not None else F32
    if cos is not None:
        assert cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim
        a.cos_table, a.sin_table = _ptr(cos, torch.float32), _ptr(sin, torch.float32)
        a.table_positions = cos.shape[0]
    a.rotary_dim, a.pairing = rotary_dim, pairing
    a.positions = _ptr(positions, torch.int32)
    a.q_out, a.k_new, a.v_new = _ptr(q_out), _ptr(k_new), _ptr(v_new)
    a.k_pages, a.v_pages = _ptr(k_pages), _ptr(v_pages)
    if page_table is not None:
        a.page_table, a.table_width = _ptr(page_table, torch.int32), page_table.shape[1]
    a.ring_pages = ring_pages
    a.seq_of_token, a.slots = _ptr(seq_of_token, torch.int32), _ptr(slots, torch.int32)
    a.n_tokens, a.nh, a.nkv, a.hd = n, n_heads, n_kv_heads, head_dim
    for t in (k_new, v_new, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("qk_prep: all outputs must share one dtype")
    return a


# Rows above which a prompt step's q/k/v product prepares queries and keys in its own epilogue.  With fewer rows (three
# token tiles of 128 or fewer) the product that splits its sums over more blocks, followed by the preparation kernel, is
# faster: measured on a B200 at the 8B layer sizes, 384 rows 7.26 ms per step against 7.63 fused, 448 rows 8.49 against 8.27.
FUSED_QKV_ABOVE = 384
USE_FUSED_QKV = True        # tests switch it off to compare with the product followed by the preparation kernel


def gemm_tc_qkv_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int, pairing: int) -> bool:
    """Whether ``gemm_tc_qkv`` takes this q/k/v projection: tensor-core operands, more than ``FUSED_QKV_ABOVE`` rows (with fewer the
    product splits its sums over blocks, which leaves partial sums and no place for an epilogue), head size 64 or
    128, rotation over the whole head by halves or none (``rotary_dim`` 0)."""
    return (USE_FUSED_QKV and gemm_tc_supported(x, w) and x.shape[0] > FUSED_QKV_ABOVE and head_dim in (64, 128)
            and (rotary_dim == 0 or (pairing == 0 and rotary_dim == head_dim)))


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
                q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], norm_eps: float,
                bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                rotary_dim: int, pairing: int, positions: torch.Tensor, q_out: torch.Tensor,
                k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
                k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
                seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                row_scale: Optional[RowScale] = None) -> None:
    """The q/k/v projection ``x w^T`` on the tensor cores with ``qk_prep`` as its epilogue (one kernel; the float32
    q/k/v array is never written).  Same arguments and results as ``gemm_tc`` followed by ``qk_prep``."""
    lib = _lib("gemm_tc")
    n, k = x.shape
    assert w.shape == ((n_heads + 2 * n_kv_heads) * head_dim, k) and q_out.dtype == torch.bfloat16
    a = _prep_args(n, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim, pairing,
                   positions, q_out, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)
    _set_scale(a, row_scale, n)
    _check(lib, lib.llg_gemm_tc_qkv(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), n, k, byref(a), _stream()))


def hc_max_streams() -> int:
    """Most residual streams ``hc_add_rmsnorm`` takes."""
    return _lib("elementwise").llg_hc_max_streams()


def hc_add_rmsnorm(streams: torch.Tensor, branch: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                   write: Optional[torch.Tensor], read: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                   out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """The residual as ``S`` streams (float32 ``[S, N, H]``): with a branch (float32 partials ``[P, N, H]``, summed to y)
    every stream becomes ``X_t = sum_s mix[s, t] X_s + write[t] y`` (all at once from the old ones, written back); then
    ``u = sum_s read[s] X_s`` (``read`` None: the plain sum) and ``out[j] = RMSNorm(u[rows[j] or j]) * weight``.
    ``mix`` ``[S, S]``, ``write`` and ``read`` ``[S]`` are float32."""
    lib = _lib("elementwise")
    s_n, n, hidden = streams.shape
    m = out.shape[0]
    assert out.shape[1] == hidden and weight.shape == (hidden,)
    assert rows.numel() == m if rows is not None else m == n
    a = _HyperNormArgs()
    a.streams, a.stream_stride, a.n_streams = _ptr(streams, torch.float32), n * hidden, s_n
    if branch is not None:
        assert branch.dim() == 3 and branch.shape[1:] == (n, hidden), (branch.shape, streams.shape)
        assert mix.shape == (s_n, s_n) and write.shape == (s_n,)
        a.branch, a.n_partials, a.partial_stride = _ptr(branch, torch.float32), branch.shape[0], n * hidden
        a.mix, a.write = _ptr(mix, torch.float32), _ptr(write, torch.float32)
    if read is not None:
        assert read.shape == (s_n,)
        a.read = _ptr(read, torch.float32)
    a.weight, a.weight_dtype, a.eps = _ptr(weight), _dt(weight), float(eps)
    a.out, a.out_dtype, a.rows, a.n_out, a.hidden = _ptr(out), _dt(out), _ptr(rows, torch.int32), m, hidden
    _check(lib, lib.llg_hc_add_rmsnorm(byref(a), _stream()))


def qkv_row_prep(qkvg: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int,
                 bias: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                 norm_eps: float, positions: torch.Tensor, q_out: torch.Tensor, gate_out: Optional[torch.Tensor] = None,
                 k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
                 k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                 page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
                 seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None) -> None:
    """Queries, keys, values and head gates from the rows of one product, float32 partials ``[P, N, row]`` with
    ``row = nh hd + nkv hd + nkv vd (+ nh gates)``: partials summed, ``bias`` added (q, k and v parts), an RMS norm over
    the whole q part and one over the whole k part (weights of those sizes; None = none), then the writes of
    ``qk_prep`` (values ``[N, nkv, vd]``) and ``gate_out[n, h] = sigmoid(g)`` in float32."""
    lib = _lib("elementwise")
    p_n, n, width = qkvg.shape
    q_w, k_w, v_w = n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * value_dim
    assert width == q_w + k_w + v_w + (n_heads if gate_out is not None else 0), (width, q_w, k_w, v_w)
    ws = [t for t in (bias, q_norm_w, k_norm_w) if t is not None]
    if len({t.dtype for t in ws}) > 1:
        raise KernelError("qkv_row_prep: bias and norm weights must share a dtype")
    for t in (k_new, v_new, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("qkv_row_prep: all outputs must share one dtype")
    a = _QkvRowPrepArgs()
    a.qkvg, a.n_partials, a.partial_stride = _ptr(qkvg, torch.float32), p_n, n * width
    a.bias, a.q_norm_w, a.k_norm_w = _ptr(bias), _ptr(q_norm_w), _ptr(k_norm_w)
    a.w_dtype = _dt(ws[0]) if ws else F32
    a.norm_eps = float(norm_eps)
    a.positions = _ptr(positions, torch.int32)
    a.q_out, a.k_new, a.v_new = _ptr(q_out), _ptr(k_new), _ptr(v_new)
    a.k_pages, a.v_pages = _ptr(k_pages), _ptr(v_pages)
    if page_table is not None:
        a.page_table, a.table_width = _ptr(page_table, torch.int32), page_table.shape[1]
    a.ring_pages = ring_pages
    a.seq_of_token, a.slots = _ptr(seq_of_token, torch.int32), _ptr(slots, torch.int32)
    a.gate_out = _ptr(gate_out, torch.float32)
    a.n_tokens, a.nh, a.nkv, a.hd, a.vd = n, n_heads, n_kv_heads, head_dim, value_dim
    _check(lib, lib.llg_qkv_row_prep(byref(a), _dt(q_out), _stream()))


def add_layernorm(residual: torch.Tensor, parts, scale: float, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                  out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """residual += scale * (sum of every set of partials in ``parts``); out[j] = layer norm of residual[rows[j] or j]:
    ``(v - mean) / sqrt(mean((v - mean)^2) + eps) * weight + bias``.  ``residual`` float32 ``[N, H]``; ``parts`` a sequence
    of float32 ``[S_i, N, H]`` tensors (up to four; none: nothing is added)."""
    lib = _lib("layernorm")
    n, hidden = residual.shape
    m = out.shape[0]
    assert out.shape[1] == hidden and weight.shape == (hidden,) and bias.shape == (hidden,)
    assert rows.numel() == m if rows is not None else m == n
    if len(parts) > _LN_BRANCHES:
        raise KernelError(f"add_layernorm: {len(parts)} sets of partials, at most {_LN_BRANCHES}")
    if weight.dtype != bias.dtype:
        raise KernelError("add_layernorm: weight and bias must share a dtype")
    a = _LayerNormArgs()
    a.residual = _ptr(residual, torch.float32)
    for i, p in enumerate(parts):
        assert p.dim() == 3 and p.shape[1:] == (n, hidden), (p.shape, residual.shape)
        a.branch[i], a.n_partials[i] = _ptr(p, torch.float32), p.shape[0]
    a.partial_stride, a.scale = n * hidden, float(scale)
    a.weight, a.bias, a.w_dtype, a.eps = _ptr(weight), _ptr(bias), _dt(weight), float(eps)
    a.out, a.out_dtype, a.rows, a.n_out, a.hidden = _ptr(out), _dt(out), _ptr(rows, torch.int32), m, hidden
    _check(lib, lib.llg_add_layernorm(byref(a), _stream()))


def latent_prep(rows: torch.Tensor, *, n_heads: int, head_dim: int, rot_dim: int, kv_rank: int, c_norm_w: torch.Tensor,
                norm_eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                q_plain_out: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None,
                k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
                k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, ring_pages: int = 0,
                seq_of_token: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                pairing: int = 0, q_col: int = 0, kv_col: Optional[int] = None, cq_col: int = -1,
                cq_norm_w: Optional[torch.Tensor] = None, cq_out: Optional[torch.Tensor] = None) -> None:
    """Preparation for latent attention from the rows of one product, float32 partials ``[P, N, width]``.  A row holds up to
    three runs of columns, each starting at a column of its own (negative: absent, its work is left out).  At ``kv_col``
    (default: behind the queries): the latent (``rank`` elements, RMS-normed with ``c_norm_w``) and the shared key part
    (``rdim`` elements, rotated) become the token's key ``[rank + rdim]`` and, where ``v_new`` / ``v_pages`` are given,
    value ``[rank]`` of ONE key/value head (packed and/or into the cache pages).  At ``q_col``: ``nh (dim + rdim)`` query
    elements; every head's unrotated part goes to ``q_plain_out`` ``[N, nh, dim]`` and its rotated part, rotated, to the
    last ``rdim`` elements of ``q_out`` ``[N, nh, rank + rdim]`` (the first ``rank`` are ``head_linear``'s to fill).  At
    ``cq_col``: a latent of the queries, RMS-normed with ``cq_norm_w`` into ``cq_out`` ``[N, cq_rank]``.  ``pairing``: which
    elements a rotation pairs, 0 (i, i + rdim / 2) or 1 (2i, 2i + 1)."""
    lib = _lib("latent")
    p_n, n, width = rows.shape
    kd = kv_rank + rot_dim
    qw = n_heads * (head_dim + rot_dim)
    if kv_col is None:
        kv_col = qw
    outs = [t for t in (q_plain_out, q_out, k_new, v_new, k_pages, v_pages, cq_out) if t is not None]
    if not outs:
        raise KernelError("latent_prep: nothing to write")
    dtype = outs[0].dtype
    if any(t.dtype != dtype for t in outs):
        raise KernelError("latent_prep: all outputs must share one dtype")
    a = _LatentPrepArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.row_width, a.q_col, a.kv_col, a.cq_col, a.pairing = width, q_col, kv_col, cq_col, pairing
    if q_col >= 0:
        assert q_plain_out.shape == (n, n_heads, head_dim) and q_out.shape == (n, n_heads, kd)
        assert q_plain_out.is_contiguous() and q_out.is_contiguous()
    if cq_col >= 0:
        assert cq_out.dim() == 2 and cq_out.shape[0] == n and cq_norm_w.shape == (cq_out.shape[1],) and cq_out.is_contiguous()
        if cq_norm_w.dtype != c_norm_w.dtype:
            raise KernelError("latent_prep: both norm weights must share a dtype")
        a.cq_rank, a.cq_norm_w, a.cq_out = cq_out.shape[1], _ptr(cq_norm_w), _ptr(cq_out)
    a.c_norm_w, a.w_dtype, a.norm_eps = _ptr(c_norm_w), _dt(c_norm_w), float(norm_eps)
    if rot_dim:
        assert cos is not None and cos.shape == sin.shape and cos.shape[1] * 2 == rot_dim
        a.cos_table, a.sin_table, a.table_positions = _ptr(cos, torch.float32), _ptr(sin, torch.float32), cos.shape[0]
    a.positions = _ptr(positions, torch.int32)
    a.q_plain, a.q_out = (_ptr(q_plain_out), _ptr(q_out)) if q_col >= 0 else (None, None)
    a.k_new, a.v_new = _ptr(k_new), _ptr(v_new)
    a.k_pages, a.v_pages = _ptr(k_pages), _ptr(v_pages)
    if k_pages is not None:
        assert k_pages.shape[1] == 1 and k_pages.shape[3] == kd and (v_pages is None or v_pages.shape[3] == kv_rank)
    if page_table is not None:
        a.page_table, a.table_width = _ptr(page_table, torch.int32), page_table.shape[1]
    a.ring_pages = ring_pages
    a.seq_of_token, a.slots = _ptr(seq_of_token, torch.int32), _ptr(slots, torch.int32)
    a.n_tokens, a.nh, a.dim, a.rdim, a.rank = n, n_heads, head_dim, rot_dim, kv_rank
    _check(lib, lib.llg_latent_prep(byref(a), _dtype_code(dtype), _stream()))


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, col0: int, bias: Optional[torch.Tensor] = None) -> None:
    """x[n, j] *= sigmoid(sum of the partials ``gate[:, n, col0 + j]`` + ``bias[j]``), in place: ``x`` ``[N, W]`` contiguous,
    ``gate`` float32 partial sums ``[P, N, width]`` of a product whose columns ``col0 .. col0 + W`` are the gate's arguments."""
    lib = _lib("latent")
    n, w = x.shape
    p_n, n2, width = gate.shape
    assert n2 == n and x.is_contiguous() and (bias is None or bias.shape == (w,))
    _check(lib, lib.llg_sigmoid_gate(_ptr(x), _dt(x), _ptr(gate, torch.float32), p_n, n * width, width, col0,
                                     _ptr(bias, torch.float32), n, w, _stream()))


NORM_MAX_GROUPS = 65536      # groups of a grouped RMS norm; checked against the library at first use


def gated_add_group_rmsnorm(residual: torch.Tensor, branch: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                            gate_bias: Optional[torch.Tensor], post_w: Optional[torch.Tensor], post_groups: int,
                            post_eps: float, weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor,
                            rows: Optional[torch.Tensor] = None) -> None:
    """RMS norm in groups fused with the residual add.  For output row j (token r = ``rows[j]`` or j), with y the sum of
    ``branch``'s partials ``[S, N, H]``: ``y *= sigmoid(sum of gate's partials [S', N, H] + gate_bias)`` where ``gate`` is given;
    ``y = group_rms(y, post_groups, post_eps) * post_w`` where ``post_w`` is given; ``residual[r] += y``;
    ``out[j] = group_rms(residual[r], groups, eps) * weight``.  ``group_rms`` cuts a row into equal consecutive parts and
    divides each by the root of (its mean square + eps).  The residual is float32 ``[N, H]``; without a branch the row is
    only normed."""
    lib = _lib("groupnorm")
    n, hidden = residual.shape
    m = out.shape[0]
    assert out.shape[1] == hidden and weight.shape == (hidden,) and out.is_contiguous()
    assert (rows.numel() == m) if rows is not None else (m == n)
    a = _GroupNormArgs()
    a.residual = _ptr(residual, torch.float32)
    a.partial_stride = n * hidden
    if branch is not None:
        assert branch.dim() == 3 and branch.shape[1:] == (n, hidden), (branch.shape, residual.shape)
        a.branch, a.n_partials = _ptr(branch, torch.float32), branch.shape[0]
        if gate is not None:
            assert gate.dim() == 3 and gate.shape[1:] == (n, hidden), (gate.shape, residual.shape)
            assert gate_bias is None or gate_bias.shape == (hidden,)
            a.gate, a.gate_partials, a.gate_bias = _ptr(gate, torch.float32), gate.shape[0], _ptr(gate_bias, torch.float32)
        if post_w is not None:
            assert post_w.shape == (hidden,)
            if post_w.dtype != weight.dtype:
                raise KernelError("group_rmsnorm: both norm weights must share a dtype")
            a.post_w, a.post_groups, a.post_eps = _ptr(post_w), int(post_groups), float(post_eps)
    elif gate is not None or post_w is not None:
        raise KernelError("group_rmsnorm: a gate or a norm of the branch needs the branch")
    a.weight, a.w_dtype, a.groups, a.eps = _ptr(weight), _dt(weight), int(groups), float(eps)
    a.out, a.out_dtype, a.rows, a.n_out, a.hidden = _ptr(out), _dt(out), _ptr(rows, torch.int32), m, hidden
    _check(lib, lib.llg_gated_add_group_rmsnorm(byref(a), _stream()))


MINGRU_PIECE = 64            # tokens of a piece of the minGRU scan; checked against the library at first use


def mingru_pieces(max_count: int) -> int:
    """Pieces per sequence that ``mingru_scan`` wants a carry for when the longest sequence of a step brings
    ``max_count`` tokens (1: no carry)."""
    return max(1, -(-int(max_count) // MINGRU_PIECE))


def mingru_scan(rows: torch.Tensor, bias: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, cu_tokens: torch.Tensor,
                out: torch.Tensor, carry: Optional[torch.Tensor] = None) -> None:
    """The minGRU recurrence along every sequence of a step.  ``rows``: float32 partials ``[P, N, 3 size]`` holding the
    arguments of z | u | g; ``bias`` float32 ``[2 size]`` (of z and u); per channel ``S_t = (1 - z_t) S_{t-1} + z_t c_t``
    with ``z = sigmoid(.)``, ``c = u + 1/2`` (u >= 0) or ``sigmoid(u)``; ``out[n] = S_t silu(g_t)`` ``[N, size]``.
    ``state`` float32 ``[slots, size]`` holds S before the step at ``slots[b]`` and receives S after it; sequence b's
    tokens are ``cu_tokens[b] .. cu_tokens[b + 1]``.  ``carry`` float32 ``[B, pieces, 2, size]``: scratch that lets a long
    prompt be scanned in pieces side by side (``pieces = mingru_pieces(longest sequence)``); without it every sequence is
    walked token by token by one thread per channel."""
    lib = _lib("recurrent")
    p_n, n, width = rows.shape
    size = out.shape[1]
    n_seqs = slots.numel()
    assert width == 3 * size and out.shape == (n, size) and bias.shape == (2 * size,) and out.is_contiguous()
    assert state.dim() == 2 and state.shape[1] == size and state.is_contiguous() and cu_tokens.numel() == n_seqs + 1
    a = _MinGruArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.bias, a.state = _ptr(bias, torch.float32), _ptr(state, torch.float32)
    a.slots, a.cu_tokens = _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32)
    a.out, a.out_dtype = _ptr(out), _dt(out)
    max_count = 0
    if carry is not None:
        assert carry.dim() == 4 and carry.shape[0] >= n_seqs and carry.shape[2:] == (2, size) and carry.is_contiguous()
        a.carry, a.pieces = _ptr(carry, torch.float32), carry.shape[1]
        max_count = min(n, carry.shape[1] * MINGRU_PIECE)
    a.n_seqs, a.n_tokens, a.size = n_seqs, n, size
    _check(lib, lib.llg_mingru_scan(byref(a), max_count, _stream()), kernels=3 if carry is not None else 1)


def multi_add_rmsnorm(residual: torch.Tensor, terms, outs, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """The residual add of several terms fused with the norm of the sum.  ``terms``: a sequence of ``(data, norm_weight, norm_eps,
    scale)`` with ``data`` float32 partials ``[S, N, H]``; a term with a ``norm_weight`` (float32 ``[H]``) is divided by its
    own root mean square and multiplied by that weight before ``scale`` times it is added to ``residual`` (float32
    ``[N, H]``).  ``outs``: a sequence of ``(out, weight, offset)``: ``out[j] = residual[r] / sqrt(mean(residual[r]^2) + eps) *
    (offset + weight)`` for r = ``rows[j]`` or j, or, with ``weight`` None, the row as it is in ``out``'s type.  All outputs
    share one dtype."""
    lib = _lib("addnorm")
    n, hidden = residual.shape
    if len(terms) > ADDNORM_MAX_TERMS or not 1 <= len(outs) <= ADDNORM_MAX_OUTS:
        raise KernelError(f"multi_add_rmsnorm: {len(terms)} terms (at most {ADDNORM_MAX_TERMS}) and {len(outs)} outputs "
                          f"(1 to {ADDNORM_MAX_OUTS})")
    a = _AddNormArgs()
    a.residual, a.partial_stride = _ptr(residual, torch.float32), n * hidden
    for i, (data, w, w_eps, scale) in enumerate(terms):
        assert data.dim() == 3 and data.shape[1:] == (n, hidden), (data.shape, residual.shape)
        assert w is None or w.shape == (hidden,)
        a.terms[i] = _AddNormTerm(_ptr(data, torch.float32), data.shape[0], _ptr(w, torch.float32), float(w_eps), float(scale))
    a.n_terms = len(terms)
    m = outs[0][0].shape[0]
    assert (rows.numel() == m) if rows is not None else (m == n)
    for i, (out, w, offset) in enumerate(outs):
        assert out.shape == (m, hidden) and (w is None or w.shape == (hidden,))
        if out.dtype != outs[0][0].dtype:
            raise KernelError("multi_add_rmsnorm: all outputs must share one dtype")
        a.outs[i] = _AddNormOut(_ptr(out), _ptr(w, torch.float32), float(offset))
    a.n_outs, a.out_dtype, a.eps = len(outs), _dt(outs[0][0]), float(eps)
    a.rows, a.n_out, a.hidden = _ptr(rows, torch.int32), m, hidden
    _check(lib, lib.llg_multi_add_rmsnorm(byref(a), _stream()))


def hash_embed(table: torch.Tensor, scale: float, pair_table: Optional[torch.Tensor], buckets: int, mul_prev: int, mul_cur: int,
               token_ids: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, cu_tokens: torch.Tensor,
               slots: torch.Tensor, last_token: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], norm_offset: float,
               eps: float, out_residual: torch.Tensor) -> None:
    """out_residual[n] = norm(scale * table[token] + pair_table[(prev * mul_prev + token * mul_cur) mod buckets]) in
    float32, where ``prev`` is the token before in the same sequence and a sequence's first token takes the pair table's
    row ``buckets``.  ``last_token`` (int32 ``[slots, 1]``) gives the token before a step's first one and receives the
    step's last.  ``norm_w`` (float32, or None for no norm): ``x / sqrt(mean(x^2) + eps) * (norm_offset + norm_w)``."""
    lib = _lib("addnorm")
    vocab, hidden = table.shape
    n = token_ids.numel()
    assert out_residual.shape == (n, hidden)
    a = _HashEmbedArgs()
    a.table, a.table_dtype, a.scale = _ptr(table), _dt(table), float(scale)
    if pair_table is not None:
        assert pair_table.shape == (buckets + 1, hidden) and last_token is not None
        a.pair_table, a.pair_dtype = _ptr(pair_table), _dt(pair_table)
        a.buckets, a.mul_prev, a.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        a.last_token = _ptr(last_token, torch.int32)
    a.token_ids, a.positions = _ptr(token_ids, torch.int32), _ptr(positions, torch.int32)
    a.seq_of_token, a.cu_tokens = _ptr(seq_of_token, torch.int32), _ptr(cu_tokens, torch.int32)
    a.slots = _ptr(slots, torch.int32)
    a.norm_w, a.norm_offset, a.eps = _ptr(norm_w, torch.float32), float(norm_offset), float(eps)
    a.out, a.n_tokens, a.vocab, a.hidden = _ptr(out_residual, torch.float32), n, vocab, hidden
    _check(lib, lib.llg_hash_embed(byref(a), _stream()))


def table_gate(rows: torch.Tensor, table: torch.Tensor, col0: int, token_ids: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out[n, j] = act(sum of the partials ``rows[:, n, j]``) * table[token_ids[n], col0 + j]; ``kind`` one of
    ``ACTIVATIONS``."""
    lib = _lib("addnorm")
    p_n, n, width = rows.shape
    assert out.shape == (n, width) and table.dim() == 2 and token_ids.numel() == n
    if kind not in ACTIVATIONS:
        raise KernelError(f"table_gate: activation '{kind}' is not known ({', '.join(ACTIVATIONS)})")
    a = _TableGateArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.table, a.table_dtype, a.table_width, a.col0 = _ptr(table), _dt(table), table.shape[1], int(col0)
    a.token_ids, a.act = _ptr(token_ids, torch.int32), ACTIVATIONS[kind]
    a.out, a.out_dtype, a.n_tokens, a.width, a.vocab = _ptr(out), _dt(out), n, width, table.shape[0]
    _check(lib, lib.llg_table_gate(byref(a), _stream()))


CONV_MAX_TAPS = 16           # taps of a short convolution; checked against the library at first use
RETENTION_PIECE = 128        # tokens of a piece of retention's walk; checked against the library at first use


def retention_supported(dim: int, vdim: int) -> bool:
    """Whether ``retention`` takes heads of these sizes (the rule of csrc/recurrent.cu: the state of a head lies in the
    registers of 256 or 512 threads, at most 32 rows of one column each, or else whole in shared memory)."""
    for threads in (256, 512):
        if vdim <= threads and -(-dim // (threads // vdim)) <= 32:
            return True
    slices = max(1, 256 // vdim)
    return (dim * vdim + 2 * dim + 2 * vdim + slices * vdim) * 4 <= 220 * 1024


def causal_conv(rows: torch.Tensor, col0: int, weight: torch.Tensor, state: Optional[torch.Tensor], slots: torch.Tensor,
                cu_tokens: torch.Tensor, seq_of_token: torch.Tensor, len_before: torch.Tensor, out: torch.Tensor,
                in_bias: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                out2: Optional[torch.Tensor] = None) -> None:
    """A causal convolution per channel along every sequence of a step.  The inputs are the ``C`` columns from ``col0`` of
    float32 partials ``rows`` ``[P, N, width]``, plus ``in_bias``; ``out[n, c] = sum_j weight[c, j] * input(position - K + 1 + j)
    + bias[c]`` (``weight`` float32 ``[C, K]``; zeros before a sequence's start).  ``state`` float32 ``[slots, K - 1, C]`` holds a
    sequence's last ``K - 1`` inputs before the step and receives those after it.  ``out`` float32 ``[N, C]``; ``out2``: the
    same once more in another type."""
    lib = _lib("recurrent")
    p_n, n, width = rows.shape
    c, k = weight.shape
    assert out.shape == (n, c) and (out2 is None or out2.shape == (n, c))
    assert k == 1 or (state is not None and state.shape[1:] == (k - 1, c)), "the state holds taps - 1 rows of inputs"
    a = _ConvArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.row_width, a.col0, a.channels, a.taps = width, int(col0), c, k
    a.in_bias, a.weight, a.bias = _ptr(in_bias, torch.float32), _ptr(weight, torch.float32), _ptr(bias, torch.float32)
    a.state = _ptr(state, torch.float32) if k > 1 else None
    a.slots, a.cu_tokens = _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32)
    a.seq_of_token, a.len_before = _ptr(seq_of_token, torch.int32), _ptr(len_before, torch.int32)
    a.out, a.out2 = _ptr(out, torch.float32), _ptr(out2)
    a.out2_dtype = _dt(out2) if out2 is not None else F32
    a.n_seqs, a.n_tokens = slots.numel(), n
    _check(lib, lib.llg_causal_conv(byref(a), _stream()))


def rglru_scan(rows: torch.Tensor, y_col: int, y_bias: Optional[torch.Tensor], u: torch.Tensor, gates: torch.Tensor,
               gate_bias: torch.Tensor, lam: torch.Tensor, decay_scale: float, state: torch.Tensor, slots: torch.Tensor,
               cu_tokens: torch.Tensor, out: torch.Tensor, carry: Optional[torch.Tensor] = None) -> None:
    """The real-gated linear recurrent unit along every sequence of a step.  Per channel c in block b (of ``bw`` channels,
    o = c mod bw): ``r = sigmoid(gates[n, b, o] + gate_bias[b, o])``, ``i = sigmoid(gates[n, b, bw + o] + gate_bias[b, bw + o])``,
    ``a = exp(-decay_scale r softplus(lam[c]))``, ``S_t = a S_{t-1} + sqrt(1 - a^2) i u[n, c]``; ``out[n, c] = S_t gelu_tanh(y)``
    with y the sum of the partials ``rows[:, n, y_col + c]`` plus ``y_bias[c]``.  ``gates`` float32 ``[N, blocks, 2 bw]``, ``u``
    float32 ``[N, size]``, ``state`` float32 ``[slots, size]``; ``carry`` as in ``mingru_scan``."""
    lib = _lib("recurrent")
    p_n, n, width = rows.shape
    size = out.shape[1]
    blocks, two_bw = gates.shape[1], gates.shape[2]
    n_seqs = slots.numel()
    assert out.shape == (n, size) and u.shape == (n, size) and gates.shape[0] == n and blocks * two_bw == 2 * size
    assert gate_bias.shape == (blocks, two_bw) and lam.shape == (size,) and state.shape[1:] == (size,)
    a = _RgLruArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.row_width, a.y_col, a.y_bias = width, int(y_col), _ptr(y_bias, torch.float32)
    a.u, a.gates, a.gate_bias = _ptr(u, torch.float32), _ptr(gates, torch.float32), _ptr(gate_bias, torch.float32)
    a.lam, a.decay_scale = _ptr(lam, torch.float32), float(decay_scale)
    a.state, a.slots, a.cu_tokens = _ptr(state, torch.float32), _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32)
    a.out, a.out_dtype = _ptr(out), _dt(out)
    max_count = 0
    if carry is not None:
        assert carry.dim() == 4 and carry.shape[0] >= n_seqs and carry.shape[2:] == (2, size) and carry.is_contiguous()
        a.carry, a.pieces = _ptr(carry, torch.float32), carry.shape[1]
        max_count = min(n, carry.shape[1] * MINGRU_PIECE)
    a.n_seqs, a.n_tokens, a.size, a.block_width = n_seqs, n, size, two_bw // 2
    _check(lib, lib.llg_rglru_scan(byref(a), max_count, _stream()), kernels=3 if carry is not None else 1)


def retention_pieces(max_count: int) -> int:
    """Pieces per sequence that ``retention`` wants a carry for when the longest sequence of a step brings ``max_count``
    tokens (1: no carry)."""
    return max(1, -(-int(max_count) // RETENTION_PIECE))


def retention(rows: torch.Tensor, *, q_col: int, k_col: int, v_col: int, g_col: int, n_heads: int, dim: int, vdim: int,
              cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
              decay: torch.Tensor, k_scale: float, eps: float, state: torch.Tensor, slots: torch.Tensor,
              cu_tokens: torch.Tensor, out: torch.Tensor, carry: Optional[torch.Tensor] = None) -> None:
    """Retention along every sequence of a step, from float32 partials ``rows`` ``[P, N, width]`` that hold q, k (``n_heads *
    dim`` columns each), v and the gate's arguments (``n_heads * vdim`` each) at their columns.  q and k are rotated by
    halves over their first ``rotary_dim`` elements, k times ``k_scale``; per head ``S_t = decay[h] S_{t-1} + k_t v_t^T``,
    ``o_t = S_t^T q_t``, ``out[n, h] = o_t / sqrt(mean(o_t^2) + eps) * silu(g)``.  ``state`` float32 ``[slots, n_heads, dim, vdim]``;
    ``carry`` float32 ``[B, pieces, n_heads, dim, vdim]`` lets a long prompt run in pieces side by side (``pieces =
    retention_pieces(longest sequence)``)."""
    lib = _lib("recurrent")
    p_n, n, width = rows.shape
    n_seqs = slots.numel()
    assert out.shape == (n, n_heads * vdim) and state.shape[1:] == (n_heads, dim, vdim) and decay.shape == (n_heads,)
    for col, w_ in ((q_col, n_heads * dim), (k_col, n_heads * dim), (v_col, n_heads * vdim), (g_col, n_heads * vdim)):
        assert 0 <= col and col + w_ <= width
    a = _RetentionArgs()
    a.rows, a.n_partials, a.partial_stride = _ptr(rows, torch.float32), p_n, n * width
    a.row_width, a.q_col, a.k_col, a.v_col, a.g_col = width, q_col, k_col, v_col, g_col
    if cos is not None and rotary_dim:
        assert cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim
        a.cos_table, a.sin_table = _ptr(cos, torch.float32), _ptr(sin, torch.float32)
        a.rotary_dim, a.table_positions = rotary_dim, cos.shape[0]
    a.positions, a.decay = _ptr(positions, torch.int32), _ptr(decay, torch.float32)
    a.k_scale, a.eps = float(k_scale), float(eps)
    a.state, a.slots, a.cu_tokens = _ptr(state, torch.float32), _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32)
    a.out, a.out_dtype = _ptr(out), _dt(out)
    max_count = 0
    if carry is not None:
        assert carry.dim() == 5 and carry.shape[0] >= n_seqs and carry.shape[2:] == (n_heads, dim, vdim) and carry.is_contiguous()
        a.carry, a.pieces = _ptr(carry, torch.float32), carry.shape[1]
        max_count = min(n, carry.shape[1] * RETENTION_PIECE)
    a.n_seqs, a.n_tokens, a.nh, a.dim, a.vdim = n_seqs, n, n_heads, dim, vdim
    _check(lib, lib.llg_retention(byref(a), max_count, _stream()), kernels=3 if carry is not None else 1)


def head_linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> None:
    """y[n, h, :] = w[h] x[n, h, :]: ``x`` ``[N, nh, a]``, ``w`` ``[nh, b, a]`` (contiguous), ``y`` ``[N, nh, b]``.  ``x`` and
    ``y`` may be views into wider rows (their last elements contiguous); float32 sums; ``x`` and ``w`` share a dtype, ``y``
    has it too or is float32 (the sums as they are).
    bfloat16 with rows on 16-byte boundaries runs on the tensor cores (csrc/moe.cu's grouped kernel), the rest on the CUDA
    cores (csrc/latent.cu)."""
    lib = _lib("latent")
    n, nh, k = x.shape
    assert w.shape[0] == nh and w.shape[2] == k and y.shape == (n, nh, w.shape[1]), (x.shape, w.shape, y.shape)
    if not (x.is_cuda and w.is_cuda and y.is_cuda):
        raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")
    if x.dtype != w.dtype or y.dtype not in (x.dtype, torch.float32):
        raise KernelError("head_linear: x and w must share a dtype, and y has it too or is float32")
    if n and (x.stride(2) != 1 or y.stride(2) != 1):
        raise KernelError("head_linear: the innermost elements of x and y must be contiguous")
    if n and x.dtype == torch.bfloat16:
        # the grouped tensor-core kernel of the experts, with the head as the group
        moe = _moe_lib()
        if moe.llg_head_linear_mma_supported(x.data_ptr(), x.stride(0), x.stride(1), _ptr(w), k):
            _check(moe, moe.llg_head_linear_mma(x.data_ptr(), x.stride(0), x.stride(1), _ptr(w), y.data_ptr(), y.stride(0),
                                                y.stride(1), n, nh, k, w.shape[1], _dt(y), _stream()))
            return
    a = _HeadLinearArgs()
    a.x, a.x_token_stride, a.x_head_stride = x.data_ptr(), x.stride(0), x.stride(1)
    a.w = _ptr(w)
    a.y, a.y_token_stride, a.y_head_stride = y.data_ptr(), y.stride(0), y.stride(1)
    a.n_tokens, a.nh, a.n_in, a.n_out = n, nh, k, w.shape[1]
    _check(lib, lib.llg_head_linear(byref(a), _dt(x), _dt(y), _stream()))


MOE_TILE_ROWS = 32          # rows of a tile of the experts' grouped products; checked against the library at first use
MOE_MAX_EXPERTS = 1024
MOE_MAX_TOP = 32


def _moe_lib():
    lib = _lib("moe")
    got = (lib.llg_moe_tile_rows(), lib.llg_moe_max_experts(), lib.llg_moe_max_top())
    if got != (MOE_TILE_ROWS, MOE_MAX_EXPERTS, MOE_MAX_TOP):
        raise KernelError(f"the mixture-of-experts kernels use (tile, experts, top) = {got}, Python expects "
                          f"{(MOE_TILE_ROWS, MOE_MAX_EXPERTS, MOE_MAX_TOP)}")
    return lib


MOE_TC_TILE_ROWS = 128      # rows of a tile of the grouped tcgen05 product (the tensor cores' rows)


def moe_tile_rows(dtype: torch.dtype, pairs: int, n_experts: int, hidden: int, inner: int) -> int:
    """The tile size for a step's layout: the tensor cores' 128 rows where the experts' products can run as the grouped
    tcgen05 product (bfloat16, row lengths the tensor copies take) and the step brings enough pairs that filling every
    expert's run up to 128 rows costs little; else the small tile of the kernels in csrc/moe.cu."""
    if dtype == torch.bfloat16 and hidden % 8 == 0 and inner % 8 == 0 and pairs >= 2 * n_experts * MOE_TC_TILE_ROWS:
        return MOE_TC_TILE_ROWS
    return MOE_TILE_ROWS


def moe_row_capacity(pairs: int, n_experts: int, tile: int = MOE_TILE_ROWS) -> int:
    """Rows that the (token, choice) pairs of a step can take once every expert's run is filled up to whole tiles."""
    cap = pairs + n_experts * (tile - 1)
    return -(-cap // tile) * tile


ROUTER_SCORES = {"softmax": 0, "sigmoid": 1, "softmax_all": 2}


class RouterRule:
    """How logits become a token's experts and weights.  ``score`` "softmax": the ``top`` largest logits, weighted by a
    softmax over them.  "softmax_all": scores are the softmax over every expert's logit; the ``top`` largest, weighted as
    the sigmoid scores are.  "sigmoid": scores ``s = sigmoid(logit)``; with ``groups`` the experts form that many equal groups of
    neighbours, a group is judged by the sum of its ``group_score_top`` largest scores and only the ``keep_groups`` best
    groups' experts can be chosen; the ``top`` largest eligible scores, ``weight = s / (sum of the chosen + weight_sum_eps) *
    weight_scale``."""

    def __init__(self, score: str = "softmax", groups: int = 0, keep_groups: int = 0, group_score_top: int = 2,
                 weight_scale: float = 1.0, weight_sum_eps: float = 0.0):
        if score not in ROUTER_SCORES:
            raise KernelError(f"router rule: score '{score}' is not known ({', '.join(ROUTER_SCORES)})")
        self.c = _RouterRule(ROUTER_SCORES[score], int(groups), int(keep_groups), int(group_score_top),
                             float(weight_scale), float(weight_sum_eps))


def _rule_ref(rule: Optional["RouterRule"]):
    return byref(rule.c) if rule is not None else None


def moe_route(x: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor], choice: torch.Tensor,
              weight: torch.Tensor, rule: Optional[RouterRule] = None, extra_out: Optional[torch.Tensor] = None) -> None:
    """Per token: ``z = w_router x + b_router`` in float32, ``choice[n]`` the ``top`` experts of largest z (largest
    first; of equals the lower index), ``weight[n]`` the softmax over those z, or what ``rule`` says.  ``w_router`` and
    ``b_router`` float32.  With ``extra_out`` ``[N]`` the matrix has one more row behind the experts' and ``extra_out[n]``
    receives the sigmoid of its product with ``x[n]``."""
    lib = _moe_lib()
    n, hidden = x.shape
    top = choice.shape[1]
    n_exp = w_router.shape[0] - (1 if extra_out is not None else 0)
    assert w_router.shape[1] == hidden and choice.shape == (n, top) and weight.shape == (n, top)
    assert b_router is None or b_router.shape == (n_exp,)
    assert extra_out is None or extra_out.shape == (n,)
    _check(lib, lib.llg_moe_route(_ptr(x), _dt(x), _ptr(w_router, torch.float32), _ptr(b_router, torch.float32),
                                  _ptr(choice, torch.int32), _ptr(weight, torch.float32), n, hidden, n_exp, top,
                                  _rule_ref(rule), _ptr(extra_out, torch.float32), _stream()))


def moe_topk(logits: torch.Tensor, b_router: Optional[torch.Tensor], choice: torch.Tensor, weight: torch.Tensor,
             rule: Optional[RouterRule] = None, extra_out: Optional[torch.Tensor] = None) -> None:
    """As ``moe_route``, from router logits that a product has left as float32 partial sums ``[S, N, experts]`` (one more
    column with ``extra_out``): the partials and the bias are added, then the experts are chosen and weighed."""
    lib = _moe_lib()
    s, n, width = logits.shape
    n_exp = width - (1 if extra_out is not None else 0)
    top = choice.shape[1]
    assert choice.shape == (n, top) and weight.shape == (n, top) and (b_router is None or b_router.shape == (n_exp,))
    assert extra_out is None or extra_out.shape == (n,)
    _check(lib, lib.llg_moe_topk(_ptr(logits, torch.float32), s, n * width, _ptr(b_router, torch.float32),
                                 _ptr(choice, torch.int32), _ptr(weight, torch.float32), n, n_exp, top,
                                 _rule_ref(rule), _ptr(extra_out, torch.float32), _stream()))


def moe_plan(choice: torch.Tensor, n_experts: int, row_of_pair: torch.Tensor, token_of_row: torch.Tensor,
             tile_expert: torch.Tensor) -> None:
    """Lays the pairs ``(n, k)`` of ``choice`` ``[N, top]`` out as rows in the order of their experts, every expert's run
    filled up to whole tiles of ``MOE_TILE_ROWS``: ``row_of_pair[n * top + k]`` the pair's row, ``token_of_row[r]`` the
    row's token (-1: a filling row), ``tile_expert[t]`` the expert of tile t (-1: unused).  ``token_of_row`` has
    ``moe_row_capacity(N * top, n_experts, tile)`` entries and ``tile_expert`` one per tile: their sizes say which tile
    size is meant."""
    lib = _moe_lib()
    n, top = choice.shape
    cap = token_of_row.numel()
    tile = _tile_of(cap, tile_expert)
    assert row_of_pair.numel() == n * top
    _check(lib, lib.llg_moe_plan(_ptr(choice, torch.int32), n * top, top, n_experts, _ptr(row_of_pair, torch.int32),
                                 _ptr(token_of_row, torch.int32), _ptr(tile_expert, torch.int32), cap, tile, _stream()))


def _tile_of(rows: int, tile_expert: torch.Tensor) -> int:
    tiles = tile_expert.numel()
    if tiles == 0 or rows % tiles or rows // tiles not in (MOE_TILE_ROWS, MOE_TC_TILE_ROWS):
        raise KernelError(f"a layout of {rows} rows in {tiles} tiles: tiles have {MOE_TILE_ROWS} or {MOE_TC_TILE_ROWS} rows")
    return rows // tiles


def moe_gather_rows(x: torch.Tensor, token_of_row: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = x[token_of_row[r]], zeros for a filling row: the layout's rows as one matrix (for the grouped tcgen05
    product, whose operands arrive by tensor copies)."""
    lib = _moe_lib()
    rows, width = out.shape
    assert x.shape[1] == width and x.dtype == out.dtype and token_of_row.numel() == rows
    _check(lib, lib.llg_moe_gather_rows(_ptr(x), _ptr(token_of_row, torch.int32), _ptr(out), rows, width * x.element_size(), _stream()))


def _grouped_tc(x, tile_expert, w, out, gated_features: int) -> None:
    lib = _lib("gemm_tc")
    rows, k = x.shape
    n_groups, group_rows, k2 = w.shape
    assert k == k2 and tile_expert.numel() * MOE_TC_TILE_ROWS == rows
    _check(lib, lib.llg_gemm_tc_grouped(_ptr(x, torch.bfloat16), _ptr(w, torch.bfloat16), _ptr(out), _dt(out), rows, group_rows, k,
                                        gated_features, _ptr(tile_expert, torch.int32), n_groups, group_rows, _stream()))


def _grouped(x, token_of_row, tile_expert, w, w2_offset, n_out, y) -> None:
    """The kernels of csrc/moe.cu: ``w`` ``[E, rows per expert, n_in]``, of which the first ``n_out`` rows of an expert are the
    (first) matrix and, with ``w2_offset``, the rows from there on the second."""
    lib = _moe_lib()
    rows = y.shape[0]
    n_in = x.shape[1]
    assert w.dim() == 3 and w.shape[2] == n_in and y.shape[1] == n_out and w.shape[1] >= n_out + (w2_offset or 0)
    assert tile_expert.numel() * MOE_TILE_ROWS == rows and (token_of_row is None or token_of_row.numel() == rows)
    assert token_of_row is not None or x.shape[0] == rows
    if x.dtype != w.dtype:
        raise KernelError("grouped products: activations and matrices must share a dtype")
    a = _GroupedLinearArgs()
    a.x, a.token_of_row, a.tile_expert = _ptr(x), _ptr(token_of_row, torch.int32), _ptr(tile_expert, torch.int32)
    a.w, a.y = _ptr(w), _ptr(y)
    a.w2 = (a.w + w2_offset * n_in * w.element_size()) if w2_offset else None
    a.rows, a.n_in, a.n_out = rows, n_in, n_out
    a.w_group_stride = w.shape[1] * n_in
    _check(lib, lib.llg_grouped_linear(byref(a), _dt(x), _dt(y), _stream()))


def moe_gated(x: torch.Tensor, token_of_row: Optional[torch.Tensor], tile_expert: torch.Tensor, w_gate_up: torch.Tensor,
              act: torch.Tensor) -> None:
    """act[r] = silu(gate_e x_r) * (up_e x_r) for every row r of the layout (e its tile's expert); filling rows of a used
    tile get zeros.  ``w_gate_up`` ``[E, 2 P, hidden]`` holds every expert's matrices in the gated layout (gate rows,
    filled up to P = a multiple of 128, then the up rows); ``act`` ``[rows, inner]``.  With tiles of ``MOE_TILE_ROWS``,
    ``x`` is the step's activations and ``token_of_row`` says which row reads which; with tiles of ``MOE_TC_TILE_ROWS``,
    ``x`` is the gathered rows themselves (``moe_gather_rows``) and the product runs on tcgen05."""
    rows, inner = act.shape
    pad = w_gate_up.shape[1] // 2
    assert w_gate_up.shape[1] == gated_rows(inner)
    if _tile_of(rows, tile_expert) == MOE_TC_TILE_ROWS:
        if token_of_row is not None or x.shape[0] != rows:
            raise KernelError("moe_gated: tiles of 128 rows take the gathered rows")
        _grouped_tc(x, tile_expert, w_gate_up, act, inner)
        return
    _grouped(x, token_of_row, tile_expert, w_gate_up, pad, inner, act)


def moe_down(act: torch.Tensor, tile_expert: torch.Tensor, w_down: torch.Tensor, y: torch.Tensor) -> None:
    """y[r] = w_down[e] act[r] in float32 for the rows of used tiles.  ``w_down`` ``[E, hidden, inner]``."""
    if y.dtype != torch.float32:
        raise KernelError("moe_down: the experts' outputs are float32")
    if _tile_of(y.shape[0], tile_expert) == MOE_TC_TILE_ROWS:
        _grouped_tc(act, tile_expert, w_down, y, 0)
        return
    _grouped(act, None, tile_expert, w_down, None, w_down.shape[1], y)


def moe_combine(y: torch.Tensor, row_of_pair: torch.Tensor, weight: torch.Tensor, shared: Optional[torch.Tensor],
                out: torch.Tensor, shared_scale: Optional[torch.Tensor] = None) -> None:
    """out[n] = sum_k weight[n, k] y[row_of_pair[n * top + k]] + the sum of ``shared``'s partials ``[S, N, H]`` (if any),
    that sum times ``shared_scale[n]`` where given (float32 ``[N]``)."""
    lib = _moe_lib()
    n, top = weight.shape
    hidden = y.shape[1]
    assert out.shape == (n, hidden) and row_of_pair.numel() == n * top
    n_shared = 0
    if shared is not None:
        assert shared.dim() == 3 and shared.shape[1:] == (n, hidden)
        n_shared = shared.shape[0]
    assert shared_scale is None or (shared is not None and shared_scale.shape == (n,))
    _check(lib, lib.llg_moe_combine(_ptr(y, torch.float32), _ptr(row_of_pair, torch.int32), _ptr(weight, torch.float32),
                                    _ptr(shared, torch.float32), n_shared, n * hidden, _ptr(shared_scale, torch.float32),
                                    _ptr(out, torch.float32), n, hidden, top, _stream()))


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def act_rows(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out[n, i] = act(sum of the partials ``x[:, n, i]``); ``kind`` is one of ``ACTIVATIONS``: relu2 (the square of
    relu), gelu_tanh, silu, relu."""
    lib = _lib("elementwise")
    if kind not in ACTIVATIONS:
        raise KernelError(f"act_rows: activation '{kind}' is not known ({', '.join(ACTIVATIONS)})")
    p_n, n, width = x.shape
    assert out.shape == (n, width)
    _check(lib, lib.llg_act_rows(_ptr(x), _dt(x), p_n, n * width, _ptr(out), _dt(out), n * width, ACTIVATIONS[kind], _stream()))


def kv_write(k_new, v_new, k_pages, v_pages, page_table, ring_pages, positions, seq_of_token, slots,
             cu_tokens, len_before) -> None:
    """Copies a prompt step's packed keys/values ``[N, nkv, hd]`` into the cache pages (values may have another
    head size than keys)."""
    lib = _lib("elementwise")
    n, nkv, hd = k_new.shape
    assert k_pages.dtype == k_new.dtype == v_new.dtype == v_pages.dtype
    if v_new.shape[2] != hd:
        # two passes of the same kernel, each with keys and values of one size
        for src, dst in ((k_new, k_pages), (v_new, v_pages)):
            _check(lib, lib.llg_kv_write(_ptr(src), _ptr(src), _ptr(dst), _ptr(dst),
                                         _ptr(page_table, torch.int32), page_table.shape[1], ring_pages,
                                         _ptr(positions, torch.int32), _ptr(seq_of_token, torch.int32),
                                         _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32),
                                         _ptr(len_before, torch.int32), n, nkv, src.shape[2], _dt(src), _stream()))
        return
    _check(lib, lib.llg_kv_write(_ptr(k_new), _ptr(v_new), _ptr(k_pages), _ptr(v_pages),
                                 _ptr(page_table, torch.int32), page_table.shape[1], ring_pages,
                                 _ptr(positions, torch.int32), _ptr(seq_of_token, torch.int32),
                                 _ptr(slots, torch.int32), _ptr(cu_tokens, torch.int32),
                                 _ptr(len_before, torch.int32), n, nkv, hd, _dt(k_new), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[n, i] = act(g) * u, act = ``activation`` (one of ``GATE_ACTIVATIONS``; silu by default); the summed partials ``[S, N, gated_rows(I)]`` hold g and u in the gated
    layout (g of feature i at i, u at ``gated_rows(I) / 2 + i``)."""
    lib = _lib("elementwise")
    s, n, two_i = gate_up.shape
    inter = out.shape[1]
    assert out.shape == (n, inter) and two_i == gated_rows(inter)
    if activation != "silu":
        if activation not in GATE_ACTIVATIONS:
            raise KernelError(f"silu_mul: gate activation '{activation}' is not known ({', '.join(GATE_ACTIVATIONS)})")
        _check(lib, lib.llg_gate_mul(_ptr(gate_up), _dt(gate_up), s, n * two_i, _ptr(out), _dt(out), n, inter,
                                     ACTIVATIONS[activation], _stream()))
        return
    _check(lib, lib.llg_silu_mul(_ptr(gate_up), _dt(gate_up), s, n * two_i, _ptr(out), _dt(out), n, inter, _stream()))


def tanh_cap(x: torch.Tensor, cap: float) -> None:
    """x <- cap tanh(x / cap) in place (float32, contiguous)."""
    lib = _lib("elementwise")
    if not x.is_contiguous():
        raise KernelError("tanh_cap: the tensor must be contiguous")
    _check(lib, lib.llg_tanh_cap(_ptr(x, torch.float32), x.numel(), float(cap), _stream()))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.flat[idx[i]] = val[i]."""
    lib = _lib("elementwise")
    assert idx.numel() == val.numel()
    _check(lib, lib.llg_scatter_i32(_ptr(dst, torch.int32), _ptr(idx, torch.int32), _ptr(val, torch.int32),
                                    idx.numel(), _stream()))


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor) -> None:
    """dst[i] = src.flat[idx[i]]."""
    lib = _lib("elementwise")
    assert dst.numel() == idx.numel()
    _check(lib, lib.llg_gather_i32(_ptr(dst, torch.int32), _ptr(src, torch.int32), _ptr(idx, torch.int32),
                                   idx.numel(), _stream()))


def zero_rows(base: torch.Tensor, rows: torch.Tensor) -> None:
    """Zeroes ``base[rows[i]]`` for a 2-D (or flattened-per-row) tensor."""
    lib = _lib("elementwise")
    row_bytes = (base.numel() // base.shape[0]) * base.element_size() if base.shape[0] else 0
    _check(lib, lib.llg_zero_rows(_ptr(base), _ptr(rows, torch.int32), rows.numel(), row_bytes, _stream()))


def _use_mma(dtype: torch.dtype, head_dim: int) -> bool:
    """bfloat16 attention with a head size the tensor-core kernels take (multiples of 16 up to 128)."""
    return dtype == torch.bfloat16 and 16 <= head_dim <= 128 and head_dim % 16 == 0


ATTN_MAX_HEAD_DIM = 384          # what csrc/attention_simt.cu takes; the tensor-core kernels take less and fall back to it
USE_TC_PROMPT_ATTENTION = True     # tests switch it off to reach the mma.sync kernel at head sizes 64 and 128


def _use_tc_attn(dtype: torch.dtype, head_dim: int) -> bool:
    """bfloat16 prompt attention with a head size the tcgen05 kernel takes (64 or 128)."""
    return USE_TC_PROMPT_ATTENTION and dtype == torch.bfloat16 and head_dim in (64, 128)


class AttentionForm:
    """What an attention computes beyond the plain causal softmax over keys and values of one head size:
    ``value_dim`` (elements of a value head; 0 = the key heads' size), ``sink`` (None, or the score of a sink that
    joins every softmax's denominator and carries no value: ``p_j = e^{s_j} / (e^{sink} + sum e^{s_j})``), ``gated``
    (the output of every (token, head) is multiplied by a float32 gate ``[N, nh]`` that the caller passes), ``sinks``
    (a float32 tensor ``[nh]`` on the device: a sink per query head, instead of one score for all), ``chunked`` (the
    ``window`` of the call is a chunk size: a query sees the keys of its own chunk of that many positions, chunks
    counted from position 0, instead of the last ``window`` keys)."""

    def __init__(self, value_dim: int = 0, sink: Optional[float] = None, gated: bool = False,
                 sinks: Optional[torch.Tensor] = None, chunked: bool = False):
        self.value_dim, self.sink, self.gated = int(value_dim), (None if sink is None else float(sink)), bool(gated)
        if sinks is not None and (sinks.dtype != torch.float32 or sinks.dim() != 1):
            raise KernelError("AttentionForm: per-head sinks are a float32 vector [query heads]")
        self.sinks, self.chunked = sinks, bool(chunked)

    def plain(self, head_dim: int) -> bool:
        return (self.value_dim in (0, head_dim) and self.sink is None and self.sinks is None and not self.gated
                and not self.chunked)

    def one_head_size(self, head_dim: int) -> bool:
        """Keys and values of one head size: what the tensor-core kernels take (sink and gate they all apply)."""
        return self.value_dim in (0, head_dim)

    def vd(self, head_dim: int) -> int:
        return self.value_dim or head_dim


PLAIN_ATTENTION = AttentionForm()


def _prefill_kernel(dtype: torch.dtype, head_dim: int, form: AttentionForm) -> str:
    """Which prompt attention kernel takes this geometry and form: the tensor-core kernels want keys and values
    of one head size."""
    if form.one_head_size(head_dim):
        return "tc" if _use_tc_attn(dtype, head_dim) else "mma" if _use_mma(dtype, head_dim) else "simt"
    return "simt"


def prefill_tile_queries(dtype: torch.dtype, head_dim: int, form: AttentionForm = PLAIN_ATTENTION) -> int:
    """Queries per block of the prompt attention kernel that ``attn_prefill`` will run."""
    return {"tc": 256, "mma": 64, "simt": 16}[_prefill_kernel(dtype, head_dim, form)]


def _set_form(a, form: AttentionForm, head_dim: int, gate: Optional[torch.Tensor]) -> None:
    """The fields of a prompt or decode argument block that say which form of attention is wanted."""
    a.vd = 0 if form.value_dim in (0, head_dim) else form.value_dim
    _set_sink(a, form)
    a.gate = _ptr(gate, torch.float32)


def _set_sink(a, form: AttentionForm, n_heads: Optional[int] = None) -> None:
    a.has_sink, a.sink_score = (0, 0.0) if form.sink is None else (1, form.sink)
    if form.sinks is not None:
        if form.sinks.numel() != a.nh:
            raise KernelError(f"attention: {form.sinks.numel()} sinks for {a.nh} query heads")
        a.has_sink, a.sinks = 1, _ptr(form.sinks, torch.float32)
    a.chunked = int(form.chunked)


def attn_tc_status() -> int:
    """Error code the tcgen05 prompt attention recorded when a wait ran out (0 = none); synchronises."""
    return _lib("attention_tc").llg_attn_tc_status()


def attn_prefill(q, k_new, v_new, k_pages, v_pages, page_table, ring_pages, tiles, cu_tokens, len_before,
                 slots, out, *, scale: float, window: int, tile_queries: int,
                 form: AttentionForm = PLAIN_ATTENTION, gate: Optional[torch.Tensor] = None) -> None:
    """Causal attention for a step with several tokens per sequence.

    ``tiles`` is ``[n_tiles, 2]`` (sequence index, first query among its step tokens) cut every
    ``tile_queries`` queries, which must be ``prefill_tile_queries(q.dtype, head_dim)``.  bfloat16 runs on
    the tensor cores: head sizes 64 and 128 with tcgen05 (csrc/attention_tc.cu), other multiples of 16 up
    to 128 with mma.sync (csrc/attention_mma.cu); everything else on the CUDA cores
    (csrc/attention_simt.cu).  ``form`` (an ``AttentionForm``) and ``gate`` ask for values of another head size, a
    sink and gated heads; ``out`` is then ``[N, nh * value_dim]``.
    """
    n, nh, hd = q.shape
    nkv = k_new.shape[1]
    vd = form.vd(hd)
    assert out.shape == (n, nh * vd) and v_new.shape == (k_new.shape[0], nkv, vd) and v_pages.shape[3] == vd
    if tile_queries != prefill_tile_queries(q.dtype, hd, form):
        raise KernelError(f"attn_prefill: tiles of {tile_queries} queries, the kernel works on "
                          f"{prefill_tile_queries(q.dtype, hd, form)}")
    if scale <= 0:
        raise KernelError("attn_prefill: the softmax scale must be positive")
    if form.gated != (gate is not None) or (gate is not None and tuple(gate.shape) != (n, nh)):
        raise KernelError("attn_prefill: a gated form needs a gate [tokens, heads], and only a gated form takes one")
    kernel = _prefill_kernel(q.dtype, hd, form)
    tc, mma = kernel == "tc", kernel == "mma"
    lib = _lib("attention_tc" if tc else "attention_mma" if mma else "attention_simt")
    a = _PrefillArgs()
    a.q, a.k_new, a.v_new = _ptr(q), _ptr(k_new, q.dtype), _ptr(v_new, q.dtype)
    a.k_pages, a.v_pages = _ptr(k_pages, q.dtype), _ptr(v_pages, q.dtype)
    a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
    a.tiles, a.cu_tokens = _ptr(tiles, torch.int32), _ptr(cu_tokens, torch.int32)
    a.len_before, a.slots = _ptr(len_before, torch.int32), _ptr(slots, torch.int32)
    a.out = _ptr(out, q.dtype)
    a.n_tiles, a.nh, a.nkv, a.hd = tiles.shape[0], nh, nkv, hd
    a.scale, a.window = float(scale), int(window)
    a.n_tokens, a.n_pages = k_new.shape[0], k_pages.shape[0]
    _set_form(a, form, hd, gate)
    if tc:
        _check(lib, lib.llg_attn_prefill_tc(byref(a), _stream()))
    elif mma:
        _check(lib, lib.llg_attn_prefill_mma(byref(a), _stream()))
    else:
        _check(lib, lib.llg_attn_prefill_simt(byref(a), _dt(q), _stream()))


# tests switch it off to reach the cp.async kernel at head sizes 64 and 128; LLOGOS_DECODE_ATTENTION=mma does the same
# for a whole process (for comparing the two kernels with the same measurement program)
USE_TMA_DECODE_ATTENTION = os.environ.get("LLOGOS_DECODE_ATTENTION", "tma") != "mma"


def _use_tma_decode(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int, n_seqs: int) -> bool:
    """bfloat16 decode attention with a geometry the TMA kernel takes (csrc/attention_decode_tma.cu)."""
    return (USE_TMA_DECODE_ATTENTION and dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv_heads > 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 8 and n_seqs <= 1024)


class DecodePlan:
    """How ``attn_decode`` will run for one batch shape: which kernel, how the keys are split over blocks, and what
    scratch it wants.  Made by ``attn_decode_plan``; callers only read ``scratch_floats`` and ``n_counters``."""

    def __init__(self, kind: str, n_splits: int, balance: bool, max_len: int, scratch_floats: int, n_counters: int):
        self.kind, self.n_splits, self.balance, self.max_len = kind, n_splits, balance, max_len
        self.scratch_floats, self.n_counters = scratch_floats, n_counters


def _splits_for(n_seqs: int, n_kv_heads: int, max_len: int, n_sms: int, blocks_per_sm: int = 2) -> int:
    """How many blocks share one (sequence, key/value head) in the kernels that take one split count for all.

    With ``pairs = n_seqs * n_kv_heads`` and ``tiles`` 64-key tiles per sequence, ``s`` splits run in
    ``ceil(pairs * s / resident blocks)`` rounds of ``ceil(tiles / s)`` tiles each; the ``s`` with
    the least rounds x tiles wins (the smallest on ties), so that no nearly empty last round of
    blocks doubles the time."""
    pairs = max(1, n_seqs * n_kv_heads)
    tiles = max(1, -(-max_len // PAGE))
    resident = blocks_per_sm * n_sms
    best, best_cost = 1, None
    for s in range(1, min(64, tiles) + 1):
        cost = -(-pairs * s // resident) * (-(-tiles // s) + 3)     # + 3: prologue and join of a block
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attn_decode_plan(dtype: torch.dtype, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, max_len: int,
                     form: AttentionForm = PLAIN_ATTENTION) -> DecodePlan:
    """The plan for a batch of ``n_seqs`` sequences of at most ``max_len`` keys (the new token's included).

    bfloat16 at head sizes 64 / 128: the TMA kernel, which balances the work itself from the lengths it finds on
    the device.  Other multiples of 16 up to 128: the mma.sync kernel with a split count from ``max_len`` (per
    sequence by its length for small batches).  Everything else, and values of another head size than the keys: the
    CUDA-core kernel."""
    plain = form.one_head_size(head_dim)
    if plain and _use_tma_decode(dtype, head_dim, n_heads, n_kv_heads, n_seqs):
        lib = _lib("attention_decode_tma")
        floats = lib.llg_attn_decode_tma_scratch_floats(n_seqs, n_heads, n_kv_heads, head_dim, max_len)
        return DecodePlan("tma", 0, False, max_len, int(floats), n_seqs * n_heads)
    n_sms = sm_count()
    splits = _splits_for(n_seqs, n_kv_heads, max_len, n_sms)
    mma = plain and _use_mma(dtype, head_dim)
    # Sequences of unequal lengths: the kernel gives each as many splits as its length calls for, up to what
    # one long sequence among short ones could use (the blocks the GPU holds, less one per other pair).
    balance = mma and 1 < n_seqs <= 32 and n_seqs * n_kv_heads <= attn_decode_balance_pairs()
    if balance:
        tiles = max(1, -(-max_len // PAGE))
        splits = max(splits, min(64, tiles, 2 * n_sms // n_kv_heads - (n_seqs - 1)))
    return DecodePlan("mma" if mma else "simt", splits, balance, max_len,
                      attn_decode_scratch_floats(n_seqs, n_heads, form.vd(head_dim), splits), n_seqs * n_kv_heads if mma else 0)


def attn_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    """Floats of scratch the split kernels need for the partial results of ``n_splits`` key splits."""
    return n_seqs * n_heads * n_splits * (head_dim + 2)


def attn_decode_balance_pairs() -> int:
    """Most (sequence, key/value head) pairs for which the mma.sync decode kernel balances its splits by length: half
    the blocks of that kernel that the GPU holds at once (two per multiprocessor)."""
    return sm_count()


def attn_decode_uses_counters(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the split kernels want ``counters`` (the tensor-core kernel joins its splits itself)."""
    return _use_mma(dtype, head_dim)


def attn_decode_tma_status() -> int:
    """Error code the TMA decode attention recorded when a wait ran out (0 = none); synchronises."""
    return _lib("attention_decode_tma").llg_attn_decode_tma_status()


def attn_decode(q, k_pages, v_pages, page_table, ring_pages, slots, len_before, out, scratch, *,
                scale: float, window: int, plan: Optional[DecodePlan] = None, n_splits: int = 0,
                counters: Optional[torch.Tensor] = None, balance: bool = False,
                form: AttentionForm = PLAIN_ATTENTION, gate: Optional[torch.Tensor] = None) -> None:
    """Attention of one new token per sequence over the cache; ``scratch`` holds the partial results.

    With ``plan`` (from ``attn_decode_plan`` for this batch shape) the kernel is the plan's.  Without it the
    caller names ``n_splits`` (and ``balance``) and gets the mma.sync kernel (bfloat16, head sizes in steps of 16
    up to 128) or the CUDA-core kernel.

    The tensor-core kernels need ``counters`` (``plan.n_counters``, or ``n_seqs * n_kv_heads`` without a plan):
    int32, zero when first used (the kernels leave them zero), through which the last block of a sequence joins
    the partial results.
    ``balance`` (mma.sync kernel, at most ``attn_decode_balance_pairs()`` (sequence, kv head) pairs):
    ``n_splits`` is the most splits a sequence may have; each gets as many as its length calls for."""
    b, nh, hd = q.shape
    nkv = k_pages.shape[1]
    vd = form.vd(hd)
    if scale <= 0:
        raise KernelError("attn_decode: the softmax scale must be positive")
    if scratch.dtype != torch.float32:
        raise KernelError("attn_decode: the scratch must be float32")
    if form.gated != (gate is not None) or (gate is not None and tuple(gate.shape) != (b, nh)):
        raise KernelError("attn_decode: a gated form needs a gate [sequences, heads], and only a gated form takes one")
    if not form.one_head_size(hd) and plan is not None and plan.kind != "simt":
        raise KernelError(f"attn_decode: the {plan.kind} kernel takes keys and values of one head size")
    assert out.shape == (b, nh * vd) and v_pages.shape[3] == vd
    if plan is not None and plan.kind == "tma":
        lib = _lib("attention_decode_tma")
        if scratch.numel() < plan.scratch_floats:
            raise KernelError(f"attn_decode: scratch of {scratch.numel()} floats, {plan.scratch_floats} needed")
        if counters is None or counters.numel() < b * nh:
            raise KernelError(f"attn_decode: needs {b * nh} zeroed int32 counters")
        a = _DecodeTmaArgs()
        a.q = _ptr(q, torch.bfloat16)
        a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
        a.slots, a.len_before = _ptr(slots, torch.int32), _ptr(len_before, torch.int32)
        a.part, a.counters, a.out = _ptr(scratch), _ptr(counters, torch.int32), _ptr(out, torch.bfloat16)
        a.n_seqs, a.nh, a.nkv, a.hd = b, nh, nkv, hd
        a.scale, a.window = float(scale), int(window)
        _set_sink(a, form)
        a.gate = _ptr(gate, torch.float32)
        _check(lib, lib.llg_attn_decode_tma(byref(a), _ptr(k_pages, torch.bfloat16), _ptr(v_pages, torch.bfloat16),
                                            k_pages.shape[0], int(plan.max_len), _stream()))
        return
    if plan is not None:
        n_splits, balance = plan.n_splits, plan.balance
    mma = form.one_head_size(hd) and _use_mma(q.dtype, hd)
    lib = _lib("attention_mma" if mma else "attention_simt")
    need = b * nh * n_splits * (vd + 2)
    if n_splits < 1 or scratch.numel() < need:
        raise KernelError(f"attn_decode: {n_splits} splits, scratch of {scratch.numel()} floats, {need} needed")
    a = _DecodeArgs()
    a.q, a.k_pages, a.v_pages = _ptr(q), _ptr(k_pages, q.dtype), _ptr(v_pages, q.dtype)
    a.page_table, a.table_width, a.ring_pages = _ptr(page_table, torch.int32), page_table.shape[1], ring_pages
    a.slots, a.len_before = _ptr(slots, torch.int32), _ptr(len_before, torch.int32)
    base = _ptr(scratch)
    a.part_o = base
    a.part_ml = base + 4 * b * nh * n_splits * vd
    a.n_seqs, a.nh, a.nkv, a.hd, a.n_splits = b, nh, nkv, hd, n_splits
    a.scale, a.window = float(scale), int(window)
    _set_form(a, form, hd, gate)
    if mma:
        if counters is None or counters.numel() < b * nkv:
            raise KernelError(f"attn_decode: needs {b * nkv} zeroed int32 counters")
        _check(lib, lib.llg_attn_decode_mma(byref(a), _ptr(out, q.dtype), _ptr(counters, torch.int32),
                                            int(bool(balance) and b * nkv <= attn_decode_balance_pairs() and b <= 32), _stream()))
    else:
        _check(lib, lib.llg_attn_decode_simt(byref(a), _ptr(out, q.dtype), _dt(q), _stream()), kernels=2)


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * z(key, i): the counter-based normal values of csrc/init.cu, which
    weights/random_init.py restates for the host."""
    lib = _lib("init")
    _check(lib, lib.llg_fill_normal(_ptr(out), _dt(out), out.numel(), int(key) & 0xFFFFFFFFFFFFFFFF, float(mean),
                                    float(std), _stream()))


def fill(out: torch.Tensor, value: float) -> None:
    lib = _lib("init")
    _check(lib, lib.llg_fill(_ptr(out), _dt(out), out.numel(), float(value), _stream()))


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst = src converted between float32 and bfloat16 (to bfloat16: round to nearest even)."""
    lib = _lib("init")
    assert src.numel() == dst.numel()
    _check(lib, lib.llg_cast(_ptr(src), _dt(src), _ptr(dst), _dt(dst), src.numel(), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    lib = _lib("sampling")
    b, v = logits.shape
    _check(lib, lib.llg_argmax(_ptr(logits, torch.float32), b, v, _ptr(out, torch.int32), _stream()))


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int = 0,
           top_p: float = 1.0, min_p: float = 0.0, typical_p: float = 1.0, min_keep: int = 1,
           repetition_penalty: float = 1.0, frequency_penalty: float = 0.0, presence_penalty: float = 0.0,
           penalize_newline: bool = False, seed: int = 0, step: int = 0,
           seq_ids: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_len: Optional[torch.Tensor] = None, banned: Optional[torch.Tensor] = None,
           probs_out: Optional[torch.Tensor] = None, candidates: bool = True,
           history_rows: Optional[torch.Tensor] = None, history_append: bool = False) -> None:
    """One token per row of ``logits`` by the sampling pipeline of csrc/sampling.cu.

    ``history`` holds recent tokens per sequence, ``history_len`` how many each has seen: a row is a ring of
    ``history.shape[1]`` entries of which the last ``min(len, width)`` count.  Row of sequence b:
    ``history_rows[b]`` (default b).  With ``history_append`` the kernel writes the token it drew into the
    ring and raises the count, so that the next step needs nothing from the host.

    ``candidates=False`` keeps the kernels on the general way over the whole vocabulary (tests compare the
    two ways)."""
    lib = _lib("sampling")
    b, v = logits.shape
    assert work.numel() >= b * v and work.dtype == torch.float32
    a = _SampleArgs()
    a.logits, a.work, a.out = _ptr(logits, torch.float32), _ptr(work), _ptr(out, torch.int32)
    a.probs_out = _ptr(probs_out, torch.float32)
    a.seq_ids = _ptr(seq_ids, torch.int32)
    if history is not None:
        a.history, a.history_len = _ptr(history, torch.int32), _ptr(history_len, torch.int32)
        a.history_stride = history.shape[1]
        a.history_rows = _ptr(history_rows, torch.int32)
        a.history_append = int(bool(history_append))
    a.n_seqs, a.vocab = b, v
    a.temperature, a.top_k = float(temperature), int(top_k)
    a.top_p, a.min_p, a.typical_p, a.min_keep = float(top_p), float(min_p), float(typical_p), int(min_keep)
    a.repetition_penalty = float(repetition_penalty)
    a.frequency_penalty, a.presence_penalty = float(frequency_penalty), float(presence_penalty)
    a.penalize_newline = int(bool(penalize_newline))
    a.seed, a.step = int(seed) & 0xFFFFFFFFFFFFFFFF, int(step)
    if banned is not None and banned.numel():
        a.banned, a.n_banned = _ptr(banned, torch.int32), banned.numel()
    if candidates:
        # scratch of the two-stage way (top-k up to the candidate cap): the kernels decide whether they take it
        slices, cap = lib.llg_sample_slices(v), lib.llg_sample_candidate_cap()
        key = (logits.device, b, slices)
        ws = _sample_scratch.get(key)
        if ws is None:
            ws = _sample_scratch[key] = (torch.empty(b * slices * cap, dtype=torch.float32, device=logits.device),
                                         torch.empty(b * slices * cap, dtype=torch.int32, device=logits.device),
                                         torch.empty(b * slices, dtype=torch.int32, device=logits.device),
                                         torch.empty(b * slices * 3, dtype=torch.float32, device=logits.device))
        a.cand_val, a.cand_idx, a.cand_count, a.n_slices = _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]), slices
        a.slice_stats = _ptr(ws[3])
    _check(lib, lib.llg_sample(byref(a), _stream()))


_sample_scratch = {}
