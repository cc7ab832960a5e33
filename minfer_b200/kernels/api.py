"""Python face of the CUDA launchers: each function checks its tensors, passes raw device
pointers and the current stream to an ``extern "C"`` launcher, and raises on any error.

There is no CPU path: a tensor that is not on a CUDA device is an error, and so is a
library that cannot be built or loaded.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
PAGE = 64
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {2001: "a size or dtype this kernel does not take", 2002: "inconsistent arguments",
           2003: "the tensor-map encoder of the CUDA driver is not available",
           2004: "the CUDA driver refused a tensor map"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


launches = 0      # kernels launched by this module since import (benchmarks read the difference)


def _check(code: int, what: str, n_kernels: int = 1) -> None:
    global launches
    launches += n_kernels
    if code != 0:
        why = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {why}")


def _ptr(t: Optional[torch.Tensor], what: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what} must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (called once per launch: the short way where torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _i32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t, what)


def _f32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
    return _ptr(t, what)


def _f64(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.float64:
        raise KernelError(f"{what} must be float64, got {t.dtype}")
    return _ptr(t, what)


_configured: set[str] = set()


def _lib(name: str) -> ctypes.CDLL:
    lib = load_library(name)
    if name not in _configured:
        _SIGNATURES[name](lib)
        _configured.add(name)
    return lib


def _sig_ops(lib: ctypes.CDLL) -> None:
    lib.mf_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                             c_void_p, c_void_p]
    lib.mf_embed_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]
    lib.mf_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                               c_void_p]
    lib.mf_rope_kvstore.argtypes = ([c_void_p, c_int, c_void_p] + [c_void_p] * 10 + [c_int] * 9 +
                                    [c_void_p, c_void_p])
    lib.mf_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                   c_int, c_int, c_float, c_void_p]
    lib.mf_swiglu.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.mf_gather_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.mf_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
    lib.mf_add_rows.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                c_void_p]
    lib.mf_norm_shift.argtypes = ([c_void_p, c_void_p, c_int] + [c_void_p] * 9 +
                                  [c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    lib.mf_xielu.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_longlong, c_void_p]
    lib.mf_tanh_cap.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
    lib.mf_add_stream.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mf_poly_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lib.mf_depth_mix.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, c_int, c_void_p]
    lib.mf_norm_add.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                c_float, c_float, c_void_p, c_void_p]
    lib.mf_unary_act.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p]
    lib.mf_gated_act.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float,
                                 c_void_p, c_longlong, c_int, c_void_p]
    lib.mf_row_gate_mul.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p]
    lib.mf_gate_mul.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_float,
                                c_void_p]
    lib.mf_table_gate.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]


def _sig_gemm_simt(lib: ctypes.CDLL) -> None:
    lib.mf_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                                 c_void_p]


def _sig_attention(lib: ctypes.CDLL) -> None:
    lib.mf_attention_packed.argtypes = [c_void_p] * 7 + [c_int] * 5 + [c_float, c_int, c_void_p]
    lib.mf_attention_paged.argtypes = ([c_void_p] * 6 + [c_int, c_int, c_void_p, c_void_p] +
                                       [c_int] * 7 + [c_float, c_int, c_int, c_longlong, c_void_p,
                                                      c_int, c_void_p])


def _sig_attention_sink(lib: ctypes.CDLL) -> None:
    lib.mf_unit_norm_kvstore.argtypes = ([c_void_p, c_int] + [c_void_p] * 9 + [c_int] * 7 +
                                         [c_float, c_int, c_int, c_void_p, c_void_p])
    lib.mf_sink_attention_packed.argtypes = ([c_void_p] * 9 + [c_int] * 8 +
                                             [c_float, c_void_p, c_float, c_int, c_int, c_void_p])
    lib.mf_sink_attention_paged.argtypes = ([c_void_p] * 6 + [c_int, c_int] + [c_void_p] * 3 +
                                            [c_int] * 8 + [c_float, c_void_p, c_float, c_int, c_int,
                                                           c_void_p])


    lib.mf_sink_attention_mma_supported.argtypes = [c_int, c_int]
    lib.mf_sink_attention_mma.argtypes = ([c_void_p] * 6 + [c_int, c_int] + [c_void_p] * 3 +
                                          [c_int] * 9 + [c_float, c_void_p, c_float, c_int, c_void_p])


    lib.mf_sink_decode_plan.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p]
    lib.mf_sink_attention_decode.argtypes = ([c_void_p] * 6 + [c_int, c_int] + [c_void_p] * 4 +
                                             [c_int] * 8 + [c_float, c_int, c_void_p, c_float, c_int,
                                                            c_void_p])


def _sig_sampling(lib: ctypes.CDLL) -> None:
    lib.mf_sample.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_float, c_int, c_float, c_float, c_float, c_float,
                              c_ulonglong, c_int, c_void_p]
    lib.mf_sampler_state_ints.argtypes = []


def _sig_gemm_tc(lib: ctypes.CDLL) -> None:
    lib.mf_gemm_tc.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                               c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p]
    lib.mf_splitk_reduce.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                     c_int, c_int, c_void_p]
    lib.mf_gemm_tc_workspace_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mf_gemm_tc_workspace_floats.restype = c_longlong
    lib.mf_gemm_tc_plan.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.mf_gemm_pair_plan.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p]
    lib.mf_gemm_pair_dual_mode.argtypes = [c_int]
    lib.mf_gemm_pair_dual_mode.restype = None
    lib.mf_gemm_pair_group_m.argtypes = [c_int]
    lib.mf_gemm_pair_group_m.restype = None
    lib.mf_gemm_tc_fused.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                                     c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_float, c_void_p, c_longlong, c_void_p,
                                     c_void_p, c_void_p, c_void_p]
    lib.mf_gemm_tc_xielu.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                                     c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int,
                                     c_int, c_float, c_void_p, c_void_p]
    lib.mf_gemm_tc_gated.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                                     c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p]
    lib.mf_gemm_tc_prep_parts.argtypes = [c_int, c_int, c_int]
    lib.mf_wait_probe.argtypes = [c_void_p, ctypes.c_uint, c_ulonglong, c_void_p, c_void_p]


def _sig_attention_prefill(lib: ctypes.CDLL) -> None:
    lib.mf_attention_prefill_mma.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_float, c_void_p]


def _sig_attention_prefill_tc(lib: ctypes.CDLL) -> None:
    lib.mf_attention_prefill_tc.argtypes = [c_void_p] * 5 + [c_int] * 7 + [c_float, c_void_p, c_void_p]
    lib.mf_attention_prefill_tc_paged.argtypes = ([c_void_p] * 6 + [c_int, c_int, c_void_p] + [c_int] * 7 +
                                                  [c_float, c_longlong, c_void_p, c_void_p])


    lib.mf_sink_attention_tc.argtypes = ([c_void_p] * 6 + [c_int, c_int] + [c_void_p] * 3 + [c_int] * 9 +
                                         [c_float, c_longlong, c_void_p, c_float, c_int, c_void_p, c_void_p])


def _sig_recurrent(lib: ctypes.CDLL) -> None:
    lib.mf_conv_silu.argtypes = ([c_void_p, c_longlong, c_int, c_int, c_int] + [c_void_p] * 7 +
                                 [c_int, c_int, c_int, c_void_p])
    lib.mf_ssm_scan.argtypes = ([c_void_p, c_void_p, c_longlong, c_int, c_int] + [c_void_p] * 7 +
                                [c_int] * 6 + [c_void_p])
    lib.mf_gated_group_norm.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_float, c_void_p]
    lib.mf_selective_scan.argtypes = [c_void_p, c_int, c_void_p]


def _sig_retention(lib: ctypes.CDLL) -> None:
    lib.mf_retention_scan.argtypes = [c_void_p, c_void_p]
    lib.mf_unit_norm_gate.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int,
                                      c_int, c_int, c_float, c_int, c_float, c_void_p]


def _sig_mixer_prep(lib: ctypes.CDLL) -> None:
    lib.mf_qk_prepare.argtypes = [c_void_p, c_int, c_int, c_void_p]
    lib.mf_head_linear.argtypes = [c_void_p, c_int, c_void_p]
    lib.mf_head_prepare.argtypes = [c_void_p, c_int, c_int, c_void_p]


def _sig_delta_rule(lib: ctypes.CDLL) -> None:
    lib.mf_delta_scan.argtypes = [c_void_p, c_int, c_int, c_void_p]
    lib.mf_delta_prep_width.argtypes = [c_int, c_int, c_int, c_int]
    lib.mf_delta_prep_width.restype = c_int
    lib.mf_head_norm_gate.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]


def _sig_attention_talk(lib: ctypes.CDLL) -> None:
    lib.mf_talk_attention.argtypes = [c_void_p, c_int, c_int, c_void_p]
    lib.mf_talk_attention_scratch.argtypes = [c_int, c_int, c_int, c_int]
    lib.mf_talk_attention_scratch.restype = c_longlong
    lib.mf_talk_attention_tile.argtypes = [c_void_p, c_int, c_void_p]
    lib.mf_talk_tile_cluster.argtypes = [c_int, c_int, c_int, c_int]
    lib.mf_value_mix.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p,
                                 c_int, c_int, c_void_p]


def _sig_moe(lib: ctypes.CDLL) -> None:
    lib.mf_moe_route.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mf_router_logits.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_void_p]
    lib.mf_moe_route_scored.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_void_p]
    lib.mf_moe_experts.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_longlong,
                                   c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_float, c_void_p]
    lib.mf_moe_counts.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
    lib.mf_moe_place.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_void_p]
    lib.mf_moe_gather.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mf_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_void_p]


_SIGNATURES = {"retention": _sig_retention, "delta_rule": _sig_delta_rule, "attention_talk": _sig_attention_talk, "moe": _sig_moe,
               "attention_prefill_tc": _sig_attention_prefill_tc, "recurrent": _sig_recurrent,
               "mixer_prep": _sig_mixer_prep,
               "attention_sink": _sig_attention_sink,
               "attention_prefill": _sig_attention_prefill, "gemm_tc": _sig_gemm_tc, "ops": _sig_ops, "gemm_simt": _sig_gemm_simt, "attention": _sig_attention,
               "sampling": _sig_sampling}


# ---------------------------------------------------------------------------------------
# row-wise ops
# ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0, rows: Optional[torch.Tensor] = None,
          row_index: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[ids[t]] * scale in float32; an id outside the table sets status bit 1.
    ``rows`` [m, width] with ``row_index`` [tokens]: out[t] += rows[row_index[t]] (unscaled; an
    index outside sets status bit 2 and adds nothing)."""
    n, width = out.shape
    vocab = table.shape[0]
    if table.shape[1] != width or ids.numel() != n:
        raise KernelError("embed: shapes do not fit")
    if rows is not None:
        if row_index is None or row_index.numel() != n or rows.dim() != 2 or rows.shape[1] != width:
            raise KernelError("embed: the added rows do not fit")
        _check(_lib("ops").mf_embed_rows(
            _ptr(table, "table"), dtype_code(table.dtype), _i32(ids, "ids"), _f32(out, "out"), n,
            width, vocab, float(scale), _ptr(rows, "rows"), dtype_code(rows.dtype),
            _i32(row_index, "row_index"), rows.shape[0], _i32(status, "status"), _stream()), "embed")
        return
    _check(_lib("ops").mf_embed(_ptr(table, "table"), dtype_code(table.dtype), _i32(ids, "ids"),
                                _f32(out, "out"), n, width, vocab, float(scale),
                                _i32(status, "status"), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight.  ``weight`` and ``rows`` are read while
    the kernel before this one may still run: weights, or inputs of the step."""
    n, width = out.shape
    if x.shape[1] != width or weight.numel() != width:
        raise KernelError("rmsnorm: shapes do not fit")
    if rows is None and x.shape[0] != n:
        raise KernelError("rmsnorm: row counts do not fit")
    _check(_lib("ops").mf_rmsnorm(_f32(x, "x"), _f32(weight, "weight"), _i32(rows, "rows"),
                                  _ptr(out, "out"), dtype_code(out.dtype), n, width, float(eps),
                                  _stream()), "rmsnorm")


def add_rmsnorm(h: torch.Tensor, partial: Optional[torch.Tensor], n_partials: int,
                bias: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """h += bias + sum of the K splits in ``partial`` [n_partials, rows, width]; out = rmsnorm(h)."""
    n, width = out.shape
    if h.shape != (n, width) or weight.numel() != width:
        raise KernelError("add_rmsnorm: shapes do not fit")
    if n_partials > 0 and (partial is None or partial.numel() < n_partials * n * width):
        raise KernelError("add_rmsnorm: the partial sums are too small")
    _check(_lib("ops").mf_add_rmsnorm(_f32(h, "h"), _f32(partial, "partial"), int(n_partials),
                                      _f32(bias, "bias"), _f32(weight, "weight"), _ptr(out, "out"),
                                      dtype_code(out.dtype), n, width, float(eps), _stream()),
           "add_rmsnorm")


def rope_kvstore(qkv: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                 seq_end: torch.Tensor, inv_freq: Optional[torch.Tensor], q_out: torch.Tensor,
                 k_out: Optional[torch.Tensor], v_out: Optional[torch.Tensor],
                 k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                 page_table: Optional[torch.Tensor], table_stride: int, ring: int,
                 n_heads: int, n_kv: int, head_dim: int, rotary_dim: int, style: int,
                 status: torch.Tensor, n_partials: int = 0,
                 bias: Optional[torch.Tensor] = None) -> None:
    """``n_partials`` > 0: ``qkv`` is [n_partials, tokens, width], the K splits a deferred
    projection left; they are added here in split order, with ``bias``.

    The kernel reads ``positions``, ``token_row``, ``seq_end``, ``page_table``, ``inv_freq`` and
    ``bias`` while the kernel before it may still run (it only waits for that kernel before it
    touches ``qkv``).  They must therefore be final before the step's first kernel starts, as
    the engine's step inputs are (one copy to the device in front of the step), or be written
    by an ordinary launch, which this kernel waits for in full."""
    if n_partials > 0:
        if qkv.dim() != 3 or qkv.shape[0] != n_partials:
            raise KernelError("rope_kvstore: partial sums must be [splits, tokens, width]")
        n, width = qkv.shape[1], qkv.shape[2]
    else:
        n, width = qkv.shape
    if width != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_kvstore: qkv has the wrong width")
    if bias is not None and bias.numel() != width:
        raise KernelError("rope_kvstore: bias has the wrong length")
    dt = q_out.dtype
    for t in (k_out, v_out, k_cache, v_cache):
        if t is not None and t.dtype != dt:
            raise KernelError("rope_kvstore: q, k, v and the cache must share one dtype")
    if (k_cache is None) != (v_cache is None) or (k_cache is not None and page_table is None):
        raise KernelError("rope_kvstore: the cache needs keys, values and a page table")
    _check(_lib("ops").mf_rope_kvstore(
        _f32(qkv, "qkv"), int(n_partials), _f32(bias, "bias"), _i32(positions, "positions"),
        _i32(token_row, "token_row"),
        _i32(seq_end, "seq_end"), _f64(inv_freq, "inv_freq"), _ptr(q_out, "q_out"),
        _ptr(k_out, "k_out"), _ptr(v_out, "v_out"), _ptr(k_cache, "k_cache"),
        _ptr(v_cache, "v_cache"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        n, n_heads, n_kv, head_dim, rotary_dim, style, dtype_code(dt), _i32(status, "status"),
        _stream()), "rope_kvstore")


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False,
           activation: str = "silu") -> None:
    """out = act(gate) * up, act the silu or the tanh form of gelu; ``interleaved``: the columns
    of ``gate_up`` alternate gate, up instead of all gates first."""
    n, nf = out.shape
    if gate_up.shape != (n, 2 * nf):
        raise KernelError("swiglu: shapes do not fit")
    _check(_lib("ops").mf_swiglu(_ptr(gate_up, "gate_up"), dtype_code(gate_up.dtype),
                                 _ptr(out, "out"), dtype_code(out.dtype), n, nf,
                                 1 if interleaved else 0, GATE_ACTIVATIONS[activation], _stream()),
           "swiglu")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    n, width = out.shape
    if x.shape[1] != width or rows.numel() != n:
        raise KernelError("gather_rows: shapes do not fit")
    _check(_lib("ops").mf_gather_rows(_f32(x, "x"), _i32(rows, "rows"), _f32(out, "out"), n, width,
                                      _stream()), "gather_rows")


def cast(src: torch.Tensor, out: torch.Tensor) -> None:
    if src.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check(_lib("ops").mf_cast(_ptr(src, "src"), dtype_code(src.dtype), _ptr(out, "out"),
                               dtype_code(out.dtype), src.numel(), _stream()), "cast")


def add_rows(h: torch.Tensor, table: torch.Tensor, index: torch.Tensor, status: torch.Tensor) -> None:
    """h[t] += table[index[t]] in float32 (learned position vectors); an index outside the
    table sets status bit 2 and adds nothing."""
    n, width = h.shape
    if table.dim() != 2 or table.shape[1] != width or index.numel() != n:
        raise KernelError("add_rows: shapes do not fit")
    _check(_lib("ops").mf_add_rows(_f32(h, "h"), _ptr(table, "table"), dtype_code(table.dtype),
                                   _i32(index, "index"), n, width, table.shape[0],
                                   _i32(status, "status"), _stream()), "add_rows")


def norm_shift(x: torch.Tensor, weight: torch.Tensor, shift: torch.Tensor, eps: float,
               positions: torch.Tensor, token_row: torch.Tensor, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, state: torch.Tensor, out: torch.Tensor, multi: bool,
               partial: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> None:
    """n = rmsnorm(x) * weight; out[t] = n[t] + (n[t-1] - n[t]) * shift, where n[t-1] of the
    first token a sequence brings is ``state[slot]`` (zeros at position 0); ``state[slot]``
    takes n of the last token a sequence brings.  ``multi``: some row may bring more than one
    token.  ``partial`` [splits, tokens, width] (only without ``multi``): the K splits of the
    projection before, added into ``x`` first, with ``bias``."""
    n, width = out.shape
    n_rows = slots.numel()
    if x.shape != (n, width) or weight.numel() != width or shift.numel() != width:
        raise KernelError("norm_shift: shapes do not fit")
    if state.dim() != 2 or state.shape[1] != width or cu_seqlens.numel() != n_rows + 1:
        raise KernelError("norm_shift: the state or the row bounds do not fit")
    n_partials = 0
    if partial is not None:
        if multi or partial.dim() != 3 or partial.shape[1:] != (n, width):
            raise KernelError("norm_shift: partial sums must be [splits, tokens, width], one token a row")
        n_partials = partial.shape[0]
    _check(_lib("ops").mf_norm_shift(
        _f32(x, "x"), _f32(partial, "partial"), n_partials, _f32(bias, "bias"),
        _f32(weight, "weight"), _f32(shift, "shift"), _i32(positions, "positions"),
        _i32(token_row, "token_row"), _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"),
        _f32(state, "state"), _ptr(out, "out"), dtype_code(out.dtype), n, n_rows, width, float(eps),
        1 if multi else 0, _stream()), "norm_shift", 2 if multi else 1)


def tanh_cap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _check(_lib("ops").mf_tanh_cap(_f32(x, "x"), x.numel(), float(cap), _stream()), "tanh_cap")


def add_stream(h: torch.Tensor, other: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> None:
    """h[t] += other[t] + vec (each optional), float32 rows; ``vec`` [width] in any dtype."""
    n, width = h.shape
    if other is not None and other.shape != h.shape:
        raise KernelError("add_stream: the added rows have another shape")
    if vec is not None and vec.numel() != width:
        raise KernelError("add_stream: the added vector has another width")
    _check(_lib("ops").mf_add_stream(_f32(h, "h"), _f32(other, "other"), _ptr(vec, "vec"),
                                     dtype_code(vec.dtype) if vec is not None else F32, n, width,
                                     _stream()), "add_stream")


def xielu(x: torch.Tensor, params: torch.Tensor, out: torch.Tensor) -> None:
    """out = softplus(a0) z^2 + z/2 for z > 0, (1/2 + softplus(a1)) (exp(z) - 1 - z) + z/2
    otherwise; ``params`` = (a0, a1) float32 on the device."""
    if x.shape != out.shape or params.numel() != 2:
        raise KernelError("xielu: shapes do not fit")
    _check(_lib("ops").mf_xielu(_ptr(x, "x"), dtype_code(x.dtype), _ptr(out, "out"),
                                dtype_code(out.dtype), _f32(params, "params"), x.numel(),
                                _stream()), "xielu")


# ---------------------------------------------------------------------------------------
# matrix product on the FP32 pipe
# ---------------------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              accumulate: bool = False) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T + bias.  Rows may be strided (last dim contiguous)."""
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, "
                          f"out {tuple(out.shape)}")
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"gemm: {what} must live on a CUDA device (there is no CPU path)")
        if t.stride(1) != 1:
            raise KernelError(f"gemm: {what} must be contiguous along its last dimension")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    _check(_lib("gemm_simt").mf_gemm_simt(
        a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype), _f32(bias, "bias"),
        out.data_ptr(), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
        1 if accumulate else 0, _stream()), "gemm_simt")


# ---------------------------------------------------------------------------------------
# matrix product on the tensor cores (bfloat16 x bfloat16, float32 accumulation)
# ---------------------------------------------------------------------------------------
EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2
# the gated epilogue with the tanh form of gelu on the gate instead of silu (the activation's
# code rides in the second byte of the epilogue code)
EPI_GEGLU_TANH = EPI_SWIGLU | (1 << 8)


def gated_epilogue(activation: str) -> int:
    return EPI_SWIGLU | (GATE_ACTIVATIONS[activation] << 8)


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel takes bfloat16 operands whose rows start on 16-byte
    boundaries (TMA); anything else goes to the FP32-pipe kernel."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2
            and w.dim() == 2 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


_PLANS: dict = {}


def gemm_tc_plan(m: int, n: int, k: int, epi: int = EPI_STORE) -> tuple[int, int]:
    """(token tile, K splits) the kernel uses for these sizes (a function of the sizes only:
    asked once per shape)."""
    return _gemm_tc_shape(m, n, k, epi)[:2]


def gemm_pair_plan(m: int, n: int, k: int) -> tuple[int, bool]:
    """(token tile, two token tiles a pair at once) of the CTA-pair kernel, which runs products
    of 256 tokens and more."""
    nt, dual = ctypes.c_int(0), ctypes.c_int(0)
    _lib("gemm_tc").mf_gemm_pair_plan(m, n, k, ctypes.addressof(nt), ctypes.addressof(dual))
    return nt.value, bool(dual.value)


def gemm_pair_dual_mode(mode: int) -> None:
    """0: a pair never takes two token tiles at once; 1: where the kernel's cost model says so
    (the default); 2: always.  The result's bits are the same in every mode."""
    _lib("gemm_tc").mf_gemm_pair_dual_mode(int(mode))


def gemm_pair_group_m(group_m: int) -> None:
    """The CTA-pair kernel walks the token tiles in groups of this many (0: chosen from the sizes,
    the default).  The order of the tiles changes no bits."""
    _lib("gemm_tc").mf_gemm_pair_group_m(int(group_m))


def _gemm_tc_shape(m: int, n: int, k: int, epi: int) -> tuple[int, int, int]:
    """(token tile, K splits, workspace floats) of a product of these sizes."""
    key = (m, n, k, epi)
    got = _PLANS.get(key)
    if got is None:
        lib = _lib("gemm_tc")
        nt, sp = ctypes.c_int(0), ctypes.c_int(0)
        lib.mf_gemm_tc_plan(m, n, k, epi, ctypes.addressof(nt), ctypes.addressof(sp))
        got = (nt.value, sp.value, int(lib.mf_gemm_tc_workspace_floats(m, n, k, epi)))
        _PLANS[key] = got
    return got


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            epi: int, status: torch.Tensor) -> None:
    """out (+)= x @ w^T + bias on tcgen05.  EPI_SWIGLU: w's rows alternate gate, up and out is
    [M, N/2] bfloat16 = silu(gate) * up."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}")
    want_cols = n // 2 if (epi & 0xff) == EPI_SWIGLU else n
    if out.shape != (m, want_cols) or out.stride(1) != 1:
        raise KernelError(f"gemm: out has shape {tuple(out.shape)}, expected {(m, want_cols)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    lib = _lib("gemm_tc")
    need = _gemm_tc_shape(m, n, k, epi & 0xff)[2]
    ws = torch.empty(need, dtype=torch.float32, device=x.device) if need else None
    _check(lib.mf_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _f32(bias, "bias"),
                          out.data_ptr(), out.stride(0), dtype_code(out.dtype), m, n, k, epi,
                          _ptr(ws, "workspace"), None, _i32(status, "status"), _stream()),
           "gemm_tc", 2 if need else 1)


def gemm_tc_xielu(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act_p: float, act_n: float,
                  status: torch.Tensor, row_scale: Optional["RowScale"] = None) -> None:
    """out = f(x @ w^T) on tcgen05, f the xIELU activation with its two coefficients
    (act_p = softplus(a0), act_n = 1/2 + softplus(a1)) applied to the float32 sums in the
    product's epilogue.  ``row_scale`` as in ``gemm_tc_fused``."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, "
                          f"out {tuple(out.shape)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    rs = row_scale
    if rs is not None and (rs.ssq.dim() != 2 or rs.ssq.shape[1] != m):
        raise KernelError("gemm: the sums of squares must be [parts, rows]")
    _check(_lib("gemm_tc").mf_gemm_tc_xielu(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
        dtype_code(out.dtype), m, n, k, float(act_p), float(act_n),
        _f32(rs.ssq, "ssq") if rs is not None else None, rs.ssq.shape[0] if rs is not None else 0,
        rs.width if rs is not None else 0, rs.eps if rs is not None else 0.0,
        _i32(status, "status"), _stream()), "gemm_tc_xielu")


GATE_CODES = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def gemm_tc_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str, p0: float,
                  p1: float, status: torch.Tensor) -> None:
    """out [M, N/2] (bfloat16) = act(gate, up) over the interleaved gate, up rows of ``w`` on tcgen05,
    the activation applied to the float32 sums in the product's epilogue: "silu", "gelu_tanh", or
    "clamped_swish" with its limit ``p0`` and the factor ``p1`` inside the sigmoid."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or n % 2 != 0 or out.shape != (m, n // 2) or out.stride(1) != 1 \
            or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, "
                          f"out {tuple(out.shape)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    _check(_lib("gemm_tc").mf_gemm_tc_gated(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), m, n, k,
        GATE_CODES[activation], float(p0), float(p1), _i32(status, "status"), _stream()), "gemm_tc_gated")


class RowScale:
    """A norm whose 1/rms is still to be applied to the rows of an activation: the rows hold
    x' = h * g (g: the norm's weight), ``ssq`` [parts, rows] the sums of h^2 per group of
    columns, as the product before left them.  The product that reads x' multiplies row t's
    results by ``rsqrt(ssq[:, t].sum() / width + eps)``."""

    __slots__ = ("ssq", "width", "eps")

    def __init__(self, ssq: torch.Tensor, width: int, eps: float):
        self.ssq, self.width, self.eps = ssq, int(width), float(eps)


_PREP_PARTS: dict = {}


def gemm_tc_prep_parts(m: int, n: int, k: int) -> int:
    """Column groups whose sums of squares a residual-completing product of these sizes writes
    (the first dimension of its ``ssq``), or 0 if no kernel folds the next norm in at these
    sizes."""
    key = (m, n, k)
    got = _PREP_PARTS.get(key)
    if got is None:
        got = int(_lib("gemm_tc").mf_gemm_tc_prep_parts(m, n, k))
        _PREP_PARTS[key] = got
    return got


def gemm_tc_fused(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  epi: int, status: torch.Tensor, row_scale: Optional[RowScale] = None,
                  prep_x: Optional[torch.Tensor] = None, prep_weight: Optional[torch.Tensor] = None,
                  prep_ssq: Optional[torch.Tensor] = None, defer: bool = False) -> Optional[torch.Tensor]:
    """``gemm_tc`` with a norm folded in on either side.  ``row_scale``: ``x`` holds x' = h * g
    of a norm and row t's results are multiplied by its 1/rms.  ``prep_x`` [M, N] bfloat16,
    ``prep_weight`` [N] float32 and ``prep_ssq`` [gemm_tc_prep_parts(M, N, K), M] float32
    (EPI_ACCUM only): ``out`` is complete when the call returns and the three hold what the
    norm that reads ``out`` next needs.  ``defer``: if the product is split along K, returns the
    float32 partial sums [splits, M, N] (``out`` untouched, may be None) instead of adding them."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if not gemm_tc_supported(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows")
    want_cols = n // 2 if (epi & 0xff) == EPI_SWIGLU else n
    if out is not None and (out.shape != (m, want_cols) or out.stride(1) != 1):
        raise KernelError(f"gemm: out has shape {tuple(out.shape)}, expected {(m, want_cols)}")
    if bias is not None and bias.numel() != n:
        raise KernelError("gemm: bias has the wrong length")
    if row_scale is not None and (row_scale.ssq.dim() != 2 or row_scale.ssq.shape[1] != m):
        raise KernelError("gemm: the sums of squares must be [parts, rows]")
    if prep_x is not None:
        parts = gemm_tc_prep_parts(m, n, k)
        if parts == 0:
            raise KernelError("gemm: no kernel folds the next norm in at these sizes")
        if (prep_x.shape != (m, n) or prep_x.dtype != torch.bfloat16 or prep_x.stride(1) != 1
                or prep_weight is None or prep_weight.numel() != n or prep_ssq is None
                or prep_ssq.shape != (parts, m)):
            raise KernelError("gemm: the next norm's tensors have the wrong shapes")
    lib = _lib("gemm_tc")
    need = _gemm_tc_shape(m, n, k, epi & 0xff)[2]
    ws = None
    if need and prep_x is None:
        ws = torch.empty(need, dtype=torch.float32, device=x.device)
    splits = ctypes.c_int(0)
    if defer:
        if ws is None:
            return None
        target, ldo, code = ws, n, F32
    else:
        target, ldo, code = out, out.stride(0), dtype_code(out.dtype)
    _check(lib.mf_gemm_tc_fused(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _f32(bias, "bias") if not defer else None,
        target.data_ptr(), ldo, code, m, n, k, epi, _ptr(ws, "workspace"),
        ctypes.addressof(splits) if defer else None,
        _f32(row_scale.ssq, "ssq") if row_scale is not None else None,
        row_scale.ssq.shape[0] if row_scale is not None else 0,
        row_scale.width if row_scale is not None else 0,
        row_scale.eps if row_scale is not None else 0.0,
        _ptr(prep_x, "prep_x"), prep_x.stride(0) if prep_x is not None else 0,
        _f32(prep_weight, "prep_weight"), _f32(prep_ssq, "prep_ssq"), _i32(status, "status"),
        _stream()), "gemm_tc", 2 if (need and prep_x is None and not defer) else 1)
    if defer:
        if splits.value < 1:
            raise KernelError("gemm_tc: a split product reported no splits")
        return ws[:splits.value * m * n].view(splits.value, m, n)
    return None


def gemm_tc_partial_sums(x: torch.Tensor, w: torch.Tensor,
                         status: torch.Tensor) -> Optional[torch.Tensor]:
    """If the kernel would split x @ w^T along K, runs only the splits and returns their
    float32 partial sums [splits, M, N] for the caller's next kernel to add; returns None
    (and runs nothing) if the product is not split."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_tc_supported(x, w) or w.shape[1] != k:
        return None
    need = _gemm_tc_shape(m, n, k, EPI_STORE)[2]
    if need == 0:
        return None
    lib = _lib("gemm_tc")
    ws = torch.empty(need, dtype=torch.float32, device=x.device)
    splits = ctypes.c_int(0)
    _check(lib.mf_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None,
                          ws.data_ptr(), n, F32, m, n, k, EPI_STORE, ws.data_ptr(),
                          ctypes.addressof(splits), _i32(status, "status"), _stream()),
           "gemm_tc")
    if splits.value < 1:
        raise KernelError("gemm_tc: a split product reported no splits")
    return ws[:splits.value * m * n].view(splits.value, m, n)


def wait_probe(status: torch.Tensor, max_tries: int, max_wait_ns: int,
               waited_ns: Optional[torch.Tensor] = None) -> None:
    """Runs the product kernels' bounded barrier wait on a barrier that nothing arrives at,
    with the given limits (never above the kernels' own).  The wait runs out, bit 4 of
    ``status`` is set and the kernel returns; ``waited_ns`` (int64 [1]) receives how long the
    wait lasted.  Nothing faults and nothing is left in flight."""
    if waited_ns is not None and (waited_ns.dtype != torch.int64 or not waited_ns.is_cuda):
        raise KernelError("wait_probe: waited_ns must be an int64 tensor on the device")
    _check(_lib("gemm_tc").mf_wait_probe(_i32(status, "status"), int(max_tries), int(max_wait_ns),
                                         None if waited_ns is None else waited_ns.data_ptr(),
                                         _stream()), "wait_probe")


def splitk_reduce(partial: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  accumulate: bool) -> None:
    """out (+)= bias + the sum of ``partial`` [splits, M, N] over its first dimension."""
    splits, m, n = partial.shape
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("splitk_reduce: out has the wrong shape")
    _check(_lib("gemm_tc").mf_splitk_reduce(_f32(partial, "partial"), splits, _f32(bias, "bias"),
                                            out.data_ptr(), out.stride(0), dtype_code(out.dtype),
                                            m, n, 1 if accumulate else 0, _stream()),
           "splitk_reduce")


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------
def attention_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row_seq: torch.Tensor,
                     row_pos: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor,
                     n_heads: int, n_kv: int, head_dim: int, window: int, scale: float) -> None:
    rows = q.shape[0]
    if q.dtype != k.dtype or q.dtype != v.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, k, v and out must share one dtype")
    _check(_lib("attention").mf_attention_packed(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"), rows, n_heads, n_kv, head_dim,
        int(window), float(scale), dtype_code(q.dtype), _stream()), "attention_packed")


def attention_prefill_supported(q: torch.Tensor, n_heads: int, n_kv: int, head_dim: int) -> bool:
    """The tensor-core kernel for whole prompts takes bfloat16 and head sizes 64 and 128."""
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % n_kv == 0


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                      out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                      head_dim: int, window: int, scale: float) -> None:
    """Causal attention of whole sequences (positions 0..len-1) packed one after another, on
    tensor cores.  ``max_len`` is the longest sequence (it sizes the grid)."""
    for t in (q, k, v, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill takes bfloat16")
    _check(_lib("attention_prefill").mf_attention_prefill_mma(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"),
        int(n_seqs), int(max_len), n_heads, n_kv, head_dim, int(window), float(scale), _stream()),
        "attention_prefill")


def attention_prefill_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                         out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                         head_dim: int, window: int, scale: float, status: torch.Tensor) -> None:
    """The same attention of whole sequences on tcgen05 (S and O in tensor memory)."""
    for t in (q, k, v, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill_tc takes bfloat16")
    _check(_lib("attention_prefill_tc").mf_attention_prefill_tc(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"),
        int(q.shape[0]), int(n_seqs), int(max_len), n_heads, n_kv, head_dim, int(window), float(scale),
        _i32(status, "status"), _stream()), "attention_prefill_tc")


def attention_prefill_tc_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                               cu_seqlens: torch.Tensor, seq_end: torch.Tensor,
                               page_table: torch.Tensor, table_stride: int, ring: int,
                               out: torch.Tensor, n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                               head_dim: int, window: int, scale: float,
                               status: torch.Tensor) -> None:
    """Attention of a step's packed tokens over the paged cache on tcgen05: sequence ``b``
    brings tokens ``cu_seqlens[b] .. cu_seqlens[b+1]-1`` at positions
    ``seq_end[b] - count .. seq_end[b] - 1``; the cache holds every position up to there, the
    step's own included.  ``max_len`` is the most tokens one sequence brings."""
    for t in (q, k_cache, v_cache, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_prefill_tc_paged takes bfloat16")
    _check(_lib("attention_prefill_tc").mf_attention_prefill_tc_paged(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
        _i32(cu_seqlens, "cu_seqlens"), _i32(seq_end, "seq_end"), _i32(page_table, "page_table"),
        int(table_stride), int(ring), _ptr(out, "out"), int(q.shape[0]), int(n_seqs), int(max_len),
        n_heads, n_kv, head_dim, int(window), float(scale), int(k_cache.shape[0]),
        _i32(status, "status"), _stream()), "attention_prefill_tc_paged")


def attention_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    row_seq: torch.Tensor, row_pos: torch.Tensor, page_table: torch.Tensor,
                    table_stride: int, ring: int, out: torch.Tensor,
                    partial: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                    window: int, chunk: int, n_chunks: int, scale: float,
                    force_generic: bool = False, status: Optional[torch.Tensor] = None,
                    old_keys_final: bool = False) -> None:
    """Attention of ``rows`` queries over the paged cache.  ``partial`` (float32,
    rows*n_heads*n_chunks*(head_dim+2)) is scratch for the key chunks; with it, bfloat16 and
    head size 64 or 128 run on the tensor-core kernels, everything else on the generic one.
    With ``status`` (the device status word) the tensor-core kernel is the one that streams the
    keys through a TMA ring, whose bounded waits report there.  ``old_keys_final``: each row is the only new
    token of its sequence in this step (the keys below its position were cached before the step
    began), which lets that kernel fetch them while the kernel before it still runs."""
    rows = q.shape[0]
    if q.dtype != k_cache.dtype or q.dtype != v_cache.dtype or q.dtype != out.dtype:
        raise KernelError("attention: q, the cache and out must share one dtype")
    need = rows * n_heads * n_chunks * (head_dim + 2)
    if partial is not None and partial.numel() < need:
        raise KernelError("attention: the scratch for key chunks is too small")
    if n_chunks > 1 and partial is None:
        raise KernelError("attention: several key chunks need scratch to merge them")
    _check(_lib("attention").mf_attention_paged(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"), _i32(row_seq, "row_seq"),
        _i32(row_pos, "row_pos"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(partial, "partial"), rows, n_heads, n_kv, head_dim, int(window),
        int(chunk), int(n_chunks), float(scale), dtype_code(q.dtype), 1 if force_generic else 0,
        int(k_cache.shape[0]), _i32(status, "status"), 1 if old_keys_final else 0,
        _stream()), "attention_paged", 2 if n_chunks > 1 else 1)


# ---------------------------------------------------------------------------------------
# state-space mixer (csrc/recurrent.cu)
# ---------------------------------------------------------------------------------------
def conv_silu(proj: torch.Tensor, x_off: int, channels: int, weight: torch.Tensor,
              bias: Optional[torch.Tensor], state: torch.Tensor, token_row: torch.Tensor,
              cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, n_rows: int,
              single: bool) -> None:
    """out[t][c] = silu(bias[c] + sum_j weight[c][j] * in[t - (taps - 1 - j)][c]) over the columns
    x_off .. x_off + channels of ``proj`` (float32 [tokens, width]); inputs before a row's first
    token come from ``state`` [slots, channels, taps - 1], which then takes the row's last ones."""
    n = proj.shape[0]
    taps = weight.shape[1]
    if (weight.shape[0] != channels or out.shape != (n, channels) or state.shape[1:] != (channels, max(taps - 1, 0))
            or x_off + channels > proj.shape[1]):
        raise KernelError("conv_silu: shapes do not fit")
    _check(_lib("recurrent").mf_conv_silu(
        _f32(proj, "proj"), proj.shape[1], int(x_off), int(channels), int(taps), _f32(weight, "weight"),
        _f32(bias, "bias"), _f32(state, "state"), _i32(token_row, "token_row"),
        _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"), _f32(out, "out"), n, int(n_rows),
        1 if single else 0, _stream()), "conv_silu", 1 if single or taps < 2 else 2)


def ssm_scan(u: torch.Tensor, proj: torch.Tensor, dt_off: int, dt_bias: torch.Tensor,
             a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor,
             cu_seqlens: torch.Tensor, slots: torch.Tensor, y: torch.Tensor, n_rows: int,
             heads: int, head_dim: int, n_state: int, groups: int) -> None:
    """The selective recurrence per (row, head), tokens one after another:
    dt = softplus(proj[t][dt_off + h] + dt_bias[h]); S <- exp(-exp(a_log[h]) dt) S + dt B x^T;
    y = S^T C + d_skip[h] x, with x | B | C the columns of ``u`` (float32 [tokens, channels]) and
    S float32 in ``state`` [slots, heads, head_dim, n_state]."""
    n = u.shape[0]
    inner = heads * head_dim
    if (u.shape[1] != inner + 2 * groups * n_state or y.shape != (n, inner)
            or state.shape[1:] != (heads, head_dim, n_state) or proj.shape[0] != n):
        raise KernelError("ssm_scan: shapes do not fit")
    _check(_lib("recurrent").mf_ssm_scan(
        _f32(u, "u"), _f32(proj, "proj"), proj.shape[1], int(dt_off), u.shape[1],
        _f32(dt_bias, "dt_bias"), _f32(a_log, "a_log"), _f32(d_skip, "d_skip"), _f32(state, "state"),
        _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots"), _f32(y, "y"), n, int(n_rows), heads,
        head_dim, n_state, groups, _stream()), "ssm_scan")


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, z_off: int, weight: torch.Tensor,
                     out: torch.Tensor, groups: int, eps: float) -> None:
    """v = y * silu(z), z the columns z_off .. of ``proj``; each of ``groups`` equal parts of v
    divided by its root mean square, times ``weight``."""
    n, inner = y.shape
    if out.shape != (n, inner) or weight.numel() != inner or inner % groups != 0:
        raise KernelError("gated_group_norm: shapes do not fit")
    _check(_lib("recurrent").mf_gated_group_norm(
        _f32(y, "y"), _f32(proj, "proj"), proj.shape[1], int(z_off), _f32(weight, "weight"),
        _ptr(out, "out"), dtype_code(out.dtype), n, inner, int(groups), float(eps), _stream()),
        "gated_group_norm")


# ---------------------------------------------------------------------------------------
# between an attention mixer's projection and its attention (csrc/mixer_prep.cu)
# ---------------------------------------------------------------------------------------
class _PrepArgs(ctypes.Structure):
    _fields_ = ([("proj", c_void_p), ("in_width", c_longlong)] +
                [(n, c_void_p) for n in ("positions", "token_row", "seq_end", "inv_freq", "q_norm_w",
                                         "k_norm_w", "q_out", "k_out", "v_out", "k_cache", "v_cache",
                                         "page_table")] +
                [(n, c_int) for n in ("table_stride", "ring", "q_off", "n_heads", "qw", "q_norm_n",
                                      "q_rot_off", "k_off", "n_kv", "kw", "k_norm_n", "k_rot_off",
                                      "v_off", "vw", "v_from_k", "rot_dims", "rot_style")] +
                [("rot_mag", c_float), ("eps", c_float), ("status", c_void_p)])


def qk_prepare(proj: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
               seq_end: torch.Tensor, q_out: torch.Tensor, k_out: Optional[torch.Tensor],
               v_out: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
               table_stride: int, ring: int, *, q_off: int, n_heads: int, q_width: int,
               k_off: int, n_kv: int, k_width: int, v_off: int, v_width: int, v_from_k: bool,
               q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
               inv_freq: Optional[torch.Tensor], rot_dims: int, rot_style: int, rot_magnitude: float,
               q_rot_off: int, k_rot_off: int, status: torch.Tensor) -> None:
    """From the float32 projection rows: the query segment (``n_heads`` heads of ``q_width`` at
    column ``q_off``) and the key segment (``n_kv`` heads of ``k_width`` at ``k_off``), each with
    its first ``len(norm weight)`` elements RMS-normed as a whole, ``rot_dims`` dimensions of
    every head rotated from ``q_rot_off`` / ``k_rot_off`` on; values from column ``v_off`` or,
    with ``v_from_k``, the first ``v_width`` elements of each prepared key head.  Writes q, the
    step's k and v, and the cache's pages."""
    n = proj.shape[0]
    dt = q_out.dtype
    for t in (k_out, v_out, k_cache, v_cache):
        if t is not None and t.dtype != dt:
            raise KernelError("qk_prepare: q, k, v and the cache must share one dtype")
    if q_out.numel() != n * n_heads * q_width:
        raise KernelError("qk_prepare: q has the wrong size")
    if k_cache is not None and (k_cache.shape[-1] != k_width or k_cache.shape[1] != n_kv or
                                (v_cache is not None and v_cache.shape[-1] != v_width)):
        raise KernelError("qk_prepare: the cache has other key or value widths")
    need = max(q_off + n_heads * q_width, k_off + n_kv * k_width,
               0 if v_from_k else v_off + n_kv * v_width)
    if proj.dim() != 2 or proj.shape[1] < need:
        raise KernelError("qk_prepare: the projection is narrower than its segments")
    a = _PrepArgs()
    a.proj, a.in_width = _f32(proj, "proj"), proj.shape[1]
    a.positions, a.token_row = _i32(positions, "positions"), _i32(token_row, "token_row")
    a.seq_end, a.inv_freq = _i32(seq_end, "seq_end"), _f64(inv_freq, "inv_freq")
    a.q_norm_w, a.k_norm_w = _f32(q_norm, "q_norm"), _f32(k_norm, "k_norm")
    a.q_out, a.k_out, a.v_out = _ptr(q_out, "q_out"), _ptr(k_out, "k_out"), _ptr(v_out, "v_out")
    a.k_cache, a.v_cache = _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache")
    a.page_table, a.table_stride, a.ring = _i32(page_table, "page_table"), int(table_stride), int(ring)
    a.q_off, a.n_heads, a.qw = int(q_off), int(n_heads), int(q_width)
    a.q_norm_n = q_norm.numel() if q_norm is not None else 0
    a.q_rot_off = int(q_rot_off)
    a.k_off, a.n_kv, a.kw = int(k_off), int(n_kv), int(k_width)
    a.k_norm_n = k_norm.numel() if k_norm is not None else 0
    a.k_rot_off = int(k_rot_off)
    a.v_off, a.vw, a.v_from_k = int(v_off), int(v_width), 1 if v_from_k else 0
    a.rot_dims, a.rot_style = int(rot_dims), int(rot_style)
    a.rot_mag, a.eps = float(rot_magnitude), float(eps)
    a.status = _i32(status, "status")
    _check(_lib("mixer_prep").mf_qk_prepare(ctypes.addressof(a), n, dtype_code(dt), _stream()),
           "qk_prepare")


class _HeadLinearArgs(ctypes.Structure):
    _fields_ = ([(n, c_void_p) for n in ("x", "w", "y", "gate")] +
                [(n, c_longlong) for n in ("x_row", "y_row", "gate_row")] +
                [(n, c_int) for n in ("x_head", "x_off", "y_head", "gate_off", "n_tokens", "heads",
                                      "J", "D", "tail", "x_tail_off")])


def head_linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, *, x_head: int, x_off: int,
                y_head: int, gate: Optional[torch.Tensor] = None, gate_off: int = 0,
                tail: int = 0, x_tail_off: int = 0) -> None:
    """y[t][h][j] = sum_d w[h][j][d] * x[t][h * x_head + x_off + d] for every head (``w``
    [heads, J, D]; ``x`` and ``y`` 2-D rows, head h of y at column h * y_head), times
    sigmoid(gate[t][gate_off + h * J + j]) if ``gate`` (float32 rows) is given; then ``tail``
    elements x[t][h * x_head + x_tail_off ..] copied behind the J outputs."""
    heads, J, D = w.shape
    n = x.shape[0]
    if x.dtype != w.dtype or y.dtype != x.dtype or y.shape[0] != n:
        raise KernelError("head_linear: x, w and y must share one dtype and row count")
    if (heads - 1) * x_head + x_off + D > x.shape[1] or (heads - 1) * y_head + J + tail > y.shape[1]:
        raise KernelError("head_linear: a head reaches beyond its row")
    a = _HeadLinearArgs()
    a.x, a.w, a.y, a.gate = _ptr(x, "x"), _ptr(w, "w"), _ptr(y, "y"), _f32(gate, "gate")
    a.x_row, a.y_row = x.shape[1], y.shape[1]
    a.gate_row = gate.shape[1] if gate is not None else 0
    a.x_head, a.x_off, a.y_head, a.gate_off = int(x_head), int(x_off), int(y_head), int(gate_off)
    a.n_tokens, a.heads, a.J, a.D = n, heads, J, D
    a.tail, a.x_tail_off = int(tail), int(x_tail_off)
    _check(_lib("mixer_prep").mf_head_linear(ctypes.addressof(a), dtype_code(x.dtype), _stream()),
           "head_linear")


# ---------------------------------------------------------------------------------------
# row-wise ops of the residual stream and the feed-forward (csrc/ops.cu)
# ---------------------------------------------------------------------------------------
def poly_norm(z: torch.Tensor, coef: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row of ``z`` (float32), powers element by
    element, N(u) = u / sqrt(mean(u^2) + eps); ``coef`` = (a, b, c, e), float32 on the device."""
    if z.dim() != 2 or out.shape != z.shape or coef.numel() != 4:
        raise KernelError("poly_norm: shapes do not fit")
    _check(_lib("ops").mf_poly_norm(_f32(z, "z"), _f32(coef, "coef"), _ptr(out, "out"),
                                    dtype_code(out.dtype), z.shape[0], z.shape[1], float(eps),
                                    _stream()), "poly_norm")


def depth_mix(history: torch.Tensor, n_hist: int, rows: Optional[torch.Tensor], last: torch.Tensor,
              weights: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = sum_{j < n_hist} weights[j] history[j][rows[r] or r] + weights[n_hist] last[r]:
    ``history`` float32 [slots >= n_hist, tokens, width], ``last`` and ``out`` [rows, width]
    (``out`` may be ``last``: every element is read before it is written, by its own thread)."""
    if (history.dim() != 3 or last.dim() != 2 or out.shape != last.shape
            or history.shape[2] != last.shape[1] or n_hist > history.shape[0]
            or weights.numel() != n_hist + 1):
        raise KernelError("depth_mix: shapes do not fit")
    if rows is None and history.shape[1] != last.shape[0]:
        raise KernelError("depth_mix: without a row index the streams must have the same rows")
    if rows is not None and rows.numel() != last.shape[0]:
        raise KernelError("depth_mix: one row index per output row")
    _check(_lib("ops").mf_depth_mix(_f32(history, "history"), history.stride(0), int(n_hist),
                                    _i32(rows, "rows"), _f32(last, "last"), _f32(weights, "weights"),
                                    _f32(out, "out"), last.shape[0], last.shape[1], _stream()),
           "depth_mix")


# ---------------------------------------------------------------------------------------
# the gated delta rule (csrc/delta_rule.cu)
# ---------------------------------------------------------------------------------------
class _DeltaArgs(ctypes.Structure):
    _fields_ = [("u", c_void_p), ("u_width", c_longlong), ("q_off", c_int), ("k_off", c_int),
                ("v_off", c_int), ("beta", c_void_p), ("beta_width", c_longlong),
                ("beta_off", c_int), ("decay", c_void_p), ("decay_width", c_longlong),
                ("decay_off", c_int), ("dt_bias", c_void_p), ("a_log", c_void_p),
                ("state", c_void_p), ("cu_seqlens", c_void_p), ("slots", c_void_p),
                ("out", c_void_p), ("prep", c_void_p), ("prep_width", c_longlong)] + [
                    (n, c_int) for n in ("n_rows", "heads", "kv_heads", "D", "Dv", "per_channel")]


def delta_scan(u: torch.Tensor, q_off: int, k_off: int, v_off: int, beta: torch.Tensor,
               beta_off: int, decay: torch.Tensor, decay_off: int, dt_bias: torch.Tensor,
               a_log: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, out: torch.Tensor, n_rows: int, max_row_tokens: int, heads: int,
               kv_heads: int, key_dim: int, value_dim: int, per_channel: bool) -> None:
    """The gated delta rule per (row, head), tokens one after another, on float32 rows: q, k, v at
    the columns ``q_off``, ``k_off``, ``v_off`` of ``u`` (after convolution and silu); raw beta at
    column ``beta_off + h`` of ``beta``; the raw decay input at ``decay_off + h`` of ``decay`` (or
    ``decay_off + h * key_dim + d`` with ``per_channel``).  q and k become unit vectors per head,
    q times key_dim^(-1/2); g = exp(-exp(a_log[h]) softplus(raw + dt_bias)); S <- g S;
    u = sigmoid(beta) (v - S^T k); S <- S + k u^T; out = S^T q.  ``state`` float32
    [slots, heads, value_dim, key_dim] goes on from what the row's slot holds.  When a row may
    bring several tokens, what does not depend on the state (unit vectors, q . k, beta, decays) is
    prepared for all tokens by a kernel of its own and the scan streams it."""
    n = u.shape[0]
    n_decay = heads * key_dim if per_channel else heads
    if (out.shape != (n, heads * value_dim) or state.shape[1:] != (heads, value_dim, key_dim)
            or beta.shape[0] != n or decay.shape[0] != n or dt_bias.numel() != n_decay
            or a_log.numel() != heads or beta_off + heads > beta.shape[1]
            or decay_off + n_decay > decay.shape[1]
            or max(q_off, k_off) + kv_heads * key_dim > u.shape[1]
            or v_off + heads * value_dim > u.shape[1]):
        raise KernelError("delta_scan: shapes do not fit")
    a = _DeltaArgs()
    a.u, a.u_width, a.q_off, a.k_off, a.v_off = _f32(u, "u"), u.shape[1], int(q_off), int(k_off), int(v_off)
    a.beta, a.beta_width, a.beta_off = _f32(beta, "beta"), beta.shape[1], int(beta_off)
    a.decay, a.decay_width, a.decay_off = _f32(decay, "decay"), decay.shape[1], int(decay_off)
    a.dt_bias, a.a_log, a.state = _f32(dt_bias, "dt_bias"), _f32(a_log, "a_log"), _f32(state, "state")
    a.cu_seqlens, a.slots = _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots")
    a.out = _f32(out, "out")
    a.n_rows, a.heads, a.kv_heads, a.D, a.Dv = int(n_rows), heads, kv_heads, key_dim, value_dim
    a.per_channel = 1 if per_channel else 0
    prep = None
    if max_row_tokens > 1:
        width = _lib("delta_rule").mf_delta_prep_width(heads, kv_heads, key_dim, a.per_channel)
        prep = torch.empty((n, width), dtype=torch.float32, device=u.device)
    a.prep, a.prep_width = _f32(prep, "prep"), prep.shape[1] if prep is not None else 0
    _check(_lib("delta_rule").mf_delta_scan(ctypes.addressof(a), int(max_row_tokens), n, _stream()),
           "delta_scan", 2 if prep is not None else 1)


HEAD_GATES = {"silu": 0, "sigmoid": 1}


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, gate_off: int, weight: torch.Tensor,
                   out: torch.Tensor, heads: int, value_dim: int, eps: float, gate_act: str) -> None:
    """out[t][h] = o[t][h] / sqrt(mean(o[t][h]^2) + eps) * weight * act(gate[t][gate_off + h * Dv ..]),
    ``weight`` [value_dim] shared by the heads, act silu or sigmoid; o and gate float32 rows."""
    n = o.shape[0]
    if (o.shape != (n, heads * value_dim) or out.shape != o.shape or weight.numel() != value_dim
            or gate.shape[0] != n or gate_off + heads * value_dim > gate.shape[1]):
        raise KernelError("head_norm_gate: shapes do not fit")
    _check(_lib("delta_rule").mf_head_norm_gate(
        _f32(o, "o"), _f32(gate, "gate"), gate.shape[1], int(gate_off), _f32(weight, "weight"),
        _ptr(out, "out"), dtype_code(out.dtype), n, heads, value_dim, float(eps),
        HEAD_GATES[gate_act], _stream()), "head_norm_gate")


# ---------------------------------------------------------------------------------------
# attention whose heads' scores are mixed before the softmax (csrc/attention_talk.cu)
# ---------------------------------------------------------------------------------------
class _TalkArgs(ctypes.Structure):
    _fields_ = ([(n, c_void_p) for n in ("q", "k", "v", "row_seq", "row_pos", "cu_seqlens",
                                         "page_table")] +
                [("table_stride", c_int), ("ring", c_int), ("talk", c_void_p), ("gate", c_void_p),
                 ("gate_width", c_longlong), ("gate_off", c_int), ("out", c_void_p),
                 ("scratch", c_void_p)] +
                [(n, c_int) for n in ("rows", "heads", "n_kv", "hd", "vd", "window", "splits")] +
                [("scale", c_float), ("q_cu", c_void_p)] +
                [(n, c_int) for n in ("n_seq", "max_q_tiles", "cluster", "nkv", "raw_bufs")])


def talk_attention_splits(rows: int, reach_keys: int) -> int:
    """Stretches a query's keys are cut into: enough blocks to fill the GPU when the queries are
    few and their keys many (at least a tile of 32 keys a stretch)."""
    if rows <= 0:
        return 1
    want = max(1, (4 * 148) // rows)
    return max(1, min(want, reach_keys // 32, 32))


def talk_tile_cluster(n_heads: int, n_kv: int, head_dim: int, value_dim: int) -> int:
    """Blocks of the cluster that the tiled kernel of talking attention runs a tile of 16 queries
    on for this shape (each block a share of the heads); 0: the shape is not taken."""
    return int(_lib("attention_talk").mf_talk_tile_cluster(n_heads, n_kv, head_dim, value_dim))


def talk_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row_seq: torch.Tensor,
                   row_pos: torch.Tensor, cu_seqlens: Optional[torch.Tensor],
                   page_table: Optional[torch.Tensor], table_stride: int, ring: int,
                   talk: torch.Tensor, gate: Optional[torch.Tensor], gate_off: int,
                   out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, value_dim: int,
                   window: int, scale: float, reach_keys: int = 0,
                   q_cu_seqlens: Optional[torch.Tensor] = None, n_seq: int = 0,
                   max_row_tokens: int = 0) -> None:
    """Softmax attention with s'_h = sum_g talk[h][g] (q_g . k) * scale, causal with an optional
    window, over the step's packed keys (``page_table`` None: key j of batch row b at token
    cu_seqlens[b] + j) or over the cache's pages; head h's output times sigmoid(gate[row][gate_off
    + h]) if ``gate`` (float32 rows) is given.  ``reach_keys``: a bound on the keys a query sees,
    used to cut long stretches over several blocks.  With ``q_cu_seqlens`` (the queries of batch row
    b are rows q_cu_seqlens[b] .. q_cu_seqlens[b + 1], at consecutive positions), ``n_seq`` batch rows
    and ``max_row_tokens``, bfloat16 inputs of a shape the tiled kernel takes run as tiles of 16
    queries on the tensor cores, the heads spread over a thread-block cluster (few queries over
    many keys: the key tiles dealt to several clusters and merged)."""
    rows = q.shape[0]
    paged = page_table is not None
    cluster = (talk_tile_cluster(n_heads, n_kv, head_dim, value_dim)
               if q_cu_seqlens is not None and n_seq > 0 and max_row_tokens >= 1
               and q.dtype == torch.bfloat16 else 0)
    tiled = cluster > 0
    if out.shape != (rows, n_heads * value_dim) or talk.shape != (n_heads, n_heads):
        raise KernelError("talk_attention: shapes do not fit")
    if k.dtype != q.dtype or v.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("talk_attention: q, k, v and the output must share one dtype")
    if tiled:
        # blocks of the tiled kernel: rows x tiles of 16 queries x the cluster; two key tiles a
        # stretch at least
        blocks = n_seq * ((int(max_row_tokens) + 15) // 16) * cluster
        splits = max(1, min((3 * 148) // blocks, reach_keys // 64, 32)) if reach_keys > 0 else 1
    else:
        splits = talk_attention_splits(rows, reach_keys) if reach_keys > 0 else 1
    scratch = None
    if splits > 1:
        scratch = torch.empty(rows * splits * n_heads * (value_dim + 2), dtype=torch.float32,
                              device=q.device)
    a = _TalkArgs()
    a.q, a.k, a.v = _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v")
    a.row_seq, a.row_pos = _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos")
    a.cu_seqlens, a.page_table = _i32(cu_seqlens, "cu_seqlens"), _i32(page_table, "page_table")
    a.table_stride, a.ring = int(table_stride), int(ring)
    a.talk, a.gate = _f32(talk, "talk"), _f32(gate, "gate")
    a.gate_width = gate.shape[1] if gate is not None else 0
    a.gate_off, a.out, a.scratch = int(gate_off), _ptr(out, "out"), _f32(scratch, "scratch")
    a.rows, a.heads, a.n_kv, a.hd, a.vd = rows, n_heads, n_kv, head_dim, value_dim
    a.window, a.splits, a.scale = int(window), splits, float(scale)
    if tiled:
        a.q_cu, a.n_seq = _i32(q_cu_seqlens, "q_cu_seqlens"), int(n_seq)
        a.max_q_tiles = (int(max_row_tokens) + 15) // 16
        code = _lib("attention_talk").mf_talk_attention_tile(ctypes.addressof(a), 1 if paged else 0,
                                                             _stream())
        if code != 2001:             # a grid the tiled kernel does not take goes to the kernel below
            _check(code, "talk_attention_tile", 2 if splits > 1 else 1)
            return
    _check(_lib("attention_talk").mf_talk_attention(ctypes.addressof(a), 1 if paged else 0,
                                                    dtype_code(q.dtype), _stream()),
           "talk_attention", 2 if splits > 1 else 1)


def value_mix(proj: torch.Tensor, v_off: int, first: torch.Tensor, first_off: int,
              lam: torch.Tensor, width: int) -> None:
    """proj[:, v_off : v_off + width] <- (1 - lam) that + lam first[:, first_off : ..] on float32
    rows; ``lam`` one float32 number on the device."""
    n = proj.shape[0]
    if first.shape[0] != n or v_off + width > proj.shape[1] or first_off + width > first.shape[1]:
        raise KernelError("value_mix: shapes do not fit")
    _check(_lib("attention_talk").mf_value_mix(
        _f32(proj, "proj"), proj.shape[1], int(v_off), _f32(first, "first"), first.shape[1],
        int(first_off), _f32(lam, "lam"), n, int(width), _stream()), "value_mix")


# ---------------------------------------------------------------------------------------
# routed experts (csrc/moe.cu)
# ---------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, top: int) -> None:
    """Per row of ``logits`` (float32 [tokens, experts]): the ``top`` largest (ties: the lower
    index) into ``idx`` (int32 [tokens, top]) and the softmax over the chosen into ``wts``."""
    n, experts = logits.shape
    if idx.shape != (n, top) or wts.shape != (n, top):
        raise KernelError("moe_route: shapes do not fit")
    _check(_lib("moe").mf_moe_route(_f32(logits, "logits"), _i32(idx, "idx"), _f32(wts, "wts"), n,
                                    experts, int(top), _stream()), "moe_route")


EXPERT_ACTIVATIONS = {"silu": 0, "clamped_swish": 2}


def router_logits(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                  out: torch.Tensor) -> None:
    """out[t][e] = bias[e] + x[t] . w[e] in float32: the product of a router (few outputs, a wide
    input), ``w`` float32 [outputs, width], ``x`` float32 or bfloat16."""
    n, width = x.shape
    outputs = w.shape[0]
    if w.shape[1] != width or out.shape != (n, outputs) or (bias is not None and bias.numel() != outputs):
        raise KernelError("router_logits: shapes do not fit")
    _check(_lib("moe").mf_router_logits(_ptr(x, "x"), dtype_code(x.dtype), _f32(w, "w"),
                                        _f32(bias, "bias"), _f32(out, "out"), n, outputs, width,
                                        _stream()), "router_logits")


def moe_route_scored(logits: torch.Tensor, correction: Optional[torch.Tensor], idx: torch.Tensor,
                     wts: torch.Tensor, top: int, outputs: int) -> None:
    """Per row of ``logits`` (float32 [tokens, >= outputs]; only the first ``outputs`` columns are
    the router's): scores = softmax over the outputs; the ``top`` largest of score + correction
    (ties: the lower index) into ``idx``, and their scores (uncorrected, not renormalized) into
    ``wts``."""
    n = logits.shape[0]
    if (idx.shape != (n, top) or wts.shape != (n, top) or logits.shape[1] < outputs
            or logits.stride(1) != 1 or (correction is not None and correction.numel() != outputs)):
        raise KernelError("moe_route_scored: shapes do not fit")
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise KernelError("moe_route_scored: logits must be float32 on a CUDA device")
    _check(_lib("moe").mf_moe_route_scored(
        logits.data_ptr(), logits.stride(0), _f32(correction, "correction"), _i32(idx, "idx"),
        _f32(wts, "wts"), n, int(outputs), int(top), _stream()), "moe_route_scored")


def moe_experts(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                idx: torch.Tensor, wts: torch.Tensor, hidden: torch.Tensor, h: torch.Tensor,
                activation: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> None:
    """h[t] += sum_k wts[t][k] Wd_e (silu(Wg_e x_t) * (Wu_e x_t)), e = idx[t][k]; with
    ``activation`` "clamped_swish" an expert's hidden values are g' sigmoid(alpha g') (u' + 1),
    g' = min(g, limit), u' = clamp(u, -limit, limit).  A choice e >= the number of stacked experts
    names an expert without weights that returns the token's input: h[t] += wts[t][k] x_t.  ``w_gate`` and
    ``w_up`` [experts, ff, width] are two stacks or strided views of one stack with alternating
    rows (equal strides, rows contiguous); ``w_down`` [experts, width, ff]; ``hidden``
    [tokens, top, ff] in the type of ``x`` is scratch; ``h`` float32.  For steps of few tokens (a
    product per token)."""
    n, width = x.shape
    experts, ff, _ = w_gate.shape
    top = idx.shape[1]
    if (w_up.shape != w_gate.shape or w_down.shape != (experts, width, ff) or w_gate.shape[2] != width
            or hidden.shape != (n, top, ff) or hidden.dtype != x.dtype or h.shape != (n, width)
            or w_up.dtype != w_gate.dtype or w_down.dtype != w_gate.dtype
            or w_gate.stride() != w_up.stride() or w_gate.stride(2) != 1):
        raise KernelError("moe_experts: shapes do not fit")
    if not (w_gate.is_cuda and w_up.is_cuda):
        raise KernelError("moe_experts: the weights must live on a CUDA device")
    _check(_lib("moe").mf_moe_experts(
        _ptr(x, "x"), dtype_code(x.dtype), w_gate.data_ptr(), w_up.data_ptr(), w_gate.stride(1),
        w_gate.stride(0), _ptr(w_down, "w_down"), dtype_code(w_gate.dtype), _i32(idx, "idx"),
        _f32(wts, "wts"), _ptr(hidden, "hidden"), _f32(h, "h"), n, width, ff, top, int(experts),
        EXPERT_ACTIVATIONS[activation], float(limit), float(alpha), _stream()),
        "moe_experts", 2)


def moe_counts(idx: torch.Tensor, counts: torch.Tensor) -> None:
    """counts[e] += number of entries of ``idx`` equal to e (int32; zero it first)."""
    _check(_lib("moe").mf_moe_counts(_i32(idx, "idx"), _i32(counts, "counts"), idx.numel(),
                                     _stream()), "moe_counts")


def moe_place(idx: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor,
              where: torch.Tensor) -> None:
    """Groups the (token, choice) pairs of ``idx`` by expert: offsets[e] = first row of expert e
    (int32 [experts + 1]), where[pair] = the pair's row, order[row] = its pair; an expert's pairs
    keep their order."""
    n_pairs, experts = idx.numel(), counts.numel()
    if offsets.numel() != experts + 1 or order.numel() != n_pairs or where.numel() != n_pairs:
        raise KernelError("moe_place: shapes do not fit")
    _check(_lib("moe").mf_moe_place(_i32(idx, "idx"), _i32(counts, "counts"), _i32(offsets, "offsets"),
                                    _i32(order, "order"), _i32(where, "where"), n_pairs, experts,
                                    _stream()), "moe_place", 2)


def moe_gather(x: torch.Tensor, pairs: torch.Tensor, out: torch.Tensor, top: int) -> None:
    """out[i] = x[pairs[i] // top]: the rows of the tokens behind the (token, choice) pairs."""
    if out.shape != (pairs.numel(), x.shape[1]) or out.dtype != x.dtype:
        raise KernelError("moe_gather: shapes do not fit")
    _check(_lib("moe").mf_moe_gather(_ptr(x, "x"), dtype_code(x.dtype), _i32(pairs, "pairs"),
                                     _ptr(out, "out"), pairs.numel(), x.shape[1], int(top),
                                     _stream()), "moe_gather")


def moe_combine(y: torch.Tensor, where: torch.Tensor, wts: torch.Tensor, h: torch.Tensor) -> None:
    """h[t] += sum_k wts[t][k] y[where[t][k]], the choices in order; y float32 rows."""
    n, top = where.shape
    if wts.shape != (n, top) or h.shape != (n, y.shape[1]):
        raise KernelError("moe_combine: shapes do not fit")
    _check(_lib("moe").mf_moe_combine(_f32(y, "y"), _i32(where, "where"), _f32(wts, "wts"),
                                      _f32(h, "h"), n, y.shape[1], top, _stream()), "moe_combine")



# ---------------------------------------------------------------------------------------
# layers that norm a sublayer's output; activations on float32 products (csrc/ops.cu)
# ---------------------------------------------------------------------------------------
def norm_add(h: torch.Tensor, y: Optional[torch.Tensor], weight: torch.Tensor, eps: float, mult: float,
             partial: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
             x_out: Optional[torch.Tensor] = None) -> None:
    """h[t] += mult * v[t] / sqrt(mean(v[t]^2) + eps) * weight, with v = ``y`` (float32 [rows, width],
    may be None) plus the K splits of a product ``partial`` [splits, rows, width] (may be None),
    added in split order, plus ``bias``.  ``x_out`` (bfloat16 [rows, width], optional) takes the new
    h rounded, for the product that reads the stream next."""
    if x_out is not None and (x_out.dtype != torch.bfloat16 or x_out.shape != h.shape):
        raise KernelError("norm_add: x_out must be bfloat16 and shaped like the stream")
    n, width = h.shape
    if y is not None and y.dim() == 3 and partial is None:
        y, partial = None, y
    if y is None and partial is None:
        raise KernelError("norm_add: nothing to add")
    if y is not None and y.shape != (n, width):
        raise KernelError("norm_add: shapes do not fit")
    splits = 0
    if partial is not None:
        splits = partial.shape[0]
        if partial.dim() != 3 or partial.shape[1:] != (n, width):
            raise KernelError("norm_add: the partial sums do not fit the stream")
    if weight.numel() != width:
        raise KernelError("norm_add: the weight has another width")
    _check(_lib("ops").mf_norm_add(_f32(h, "h"), _f32(y, "y"), _f32(partial, "partial"), splits,
                                   _f32(bias, "bias"), _f32(weight, "weight"), n, width, float(eps),
                                   float(mult), _ptr(x_out, "x_out"), _stream()), "norm_add")


UNARY_ACTIVATIONS = {"gelu": 0}
GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def unary_act(z: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(z), z float32; "gelu" is the erf form 0.5 z (1 + erf(z / sqrt 2))."""
    if out.shape != z.shape:
        raise KernelError("unary_act: shapes do not fit")
    _check(_lib("ops").mf_unary_act(_f32(z, "z"), _ptr(out, "out"), dtype_code(out.dtype), z.numel(),
                                    UNARY_ACTIVATIONS[activation], _stream()), "unary_act")


def row_gate_mul(o: torch.Tensor, row_gate: torch.Tensor) -> None:
    """o[t] <- o[t] * sigmoid(row_gate[t]), in place; ``row_gate`` float32, one number a row (any
    row stride)."""
    n, width = o.shape
    if row_gate.dtype != torch.float32 or not row_gate.is_cuda or row_gate.shape[0] != n or row_gate.dim() != 1:
        raise KernelError("row_gate_mul: the row gate must be float32 on the device, one a row")
    _check(_lib("ops").mf_row_gate_mul(_ptr(o, "o"), dtype_code(o.dtype), row_gate.data_ptr(),
                                       row_gate.stride(0), n, width, _stream()), "row_gate_mul")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, limit: float = 0.0,
              alpha: float = 1.0, row_gate: Optional[torch.Tensor] = None,
              interleaved: bool = False) -> None:
    """From float32 rows [gate (ff) | up (ff)] (``interleaved``: gate, up, gate, up, ..): silu(g) u, gelu_tanh(g) u, or ("clamped_swish")
    g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit); times
    sigmoid(row_gate[t]) if ``row_gate`` (float32, one number a row, any row stride) is given."""
    n, ff = out.shape
    if gate_up.shape != (n, 2 * ff):
        raise KernelError("gated_act: shapes do not fit")
    rg, rg_stride = None, 0
    if row_gate is not None:
        if row_gate.dtype != torch.float32 or not row_gate.is_cuda or row_gate.shape[0] != n:
            raise KernelError("gated_act: the row gate must be float32 on the device, one a row")
        rg, rg_stride = row_gate.data_ptr(), row_gate.stride(0)
    _check(_lib("ops").mf_gated_act(_f32(gate_up, "gate_up"), _ptr(out, "out"), dtype_code(out.dtype),
                                    n, ff, GATED_ACTIVATIONS[activation], float(limit), float(alpha),
                                    rg, rg_stride, 1 if interleaved else 0, _stream()), "gated_act")


def gate_mul(o: torch.Tensor, gate: torch.Tensor, gate_off: int, mul: float = 1.0) -> None:
    """o[t][c] <- o[t][c] * sigmoid(gate[t][gate_off + c]) * mul, in place; ``gate`` float32 rows."""
    n, width = o.shape
    if gate.shape[0] != n or gate_off + width > gate.shape[1]:
        raise KernelError("gate_mul: shapes do not fit")
    _check(_lib("ops").mf_gate_mul(_ptr(o, "o"), dtype_code(o.dtype), _f32(gate, "gate"),
                                   gate.shape[1], int(gate_off), n, width, float(mul), _stream()),
           "gate_mul")


def table_gate(a: torch.Tensor, table: torch.Tensor, off: int, ids: torch.Tensor,
               rows: Optional[torch.Tensor], out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t][d] = gelu_tanh(a[t][d]) * table[ids[rows[t] if rows else t]][off + d]."""
    n, dim = a.shape
    if out.shape != (n, dim) or off + dim > table.shape[1] or (rows is not None and rows.numel() != n):
        raise KernelError("table_gate: shapes do not fit")
    _check(_lib("ops").mf_table_gate(_f32(a, "a"), _ptr(table, "table"), dtype_code(table.dtype),
                                     table.shape[1], int(off), _i32(ids, "ids"), _i32(rows, "rows"),
                                     _ptr(out, "out"), dtype_code(out.dtype), n, dim, table.shape[0],
                                     _i32(status, "status"), _stream()), "table_gate")


# ---------------------------------------------------------------------------------------
# heads prepared one by one (csrc/mixer_prep.cu)
# ---------------------------------------------------------------------------------------
class _HeadPrepArgs(ctypes.Structure):
    _fields_ = ([("proj", c_void_p), ("in_width", c_longlong)] +
                [(n, c_void_p) for n in ("positions", "token_row", "seq_end", "inv_freq", "q_norm_w",
                                         "k_norm_w", "q_out", "k_out", "v_out", "k_cache", "v_cache",
                                         "page_table")] +
                [(n, c_int) for n in ("table_stride", "ring", "q_off", "n_heads", "qw", "k_off", "n_kv",
                                      "kw", "v_off", "vw", "rot_dims", "rot_style")] +
                [(n, c_float) for n in ("rot_mag", "eps", "q_mul", "k_mul")] + [("status", c_void_p)])


def head_prepare(proj: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                 seq_end: torch.Tensor, q_out: torch.Tensor, k_out: Optional[torch.Tensor],
                 v_out: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                 v_cache: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                 table_stride: int, ring: int, *, q_off: int, n_heads: int, q_width: int, k_off: int,
                 n_kv: int, k_width: int, v_off: int, v_width: int,
                 q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                 inv_freq: Optional[torch.Tensor], rot_dims: int, rot_style: int,
                 rot_magnitude: float, q_mul: float, k_mul: float, status: torch.Tensor) -> None:
    """From the float32 projection rows: every query head (``n_heads`` of ``q_width`` at column
    ``q_off``) and key head (``n_kv`` of ``k_width`` at ``k_off``) RMS-normed BY ITSELF with a weight
    of the head's width shared by all heads (None: no norm), its first ``rot_dims`` dimensions
    rotated, the result times ``q_mul`` / ``k_mul``; values (``n_kv`` heads of ``v_width`` at
    ``v_off``) copied.  Writes q, the step's k and v and the cache's pages (each optional except q),
    in the type of ``q_out``."""
    n = proj.shape[0]
    dt = q_out.dtype
    for t in (k_out, v_out, k_cache, v_cache):
        if t is not None and t.dtype != dt:
            raise KernelError("head_prepare: q, k, v and the cache must share one dtype")
    if q_out.numel() != n * n_heads * q_width:
        raise KernelError("head_prepare: q has the wrong size")
    if k_cache is not None and (k_cache.shape[-1] != k_width or k_cache.shape[1] != n_kv
                                or v_cache is None or v_cache.shape[-1] != v_width):
        raise KernelError("head_prepare: the cache has other key or value widths")
    wants_v = v_out is not None or v_cache is not None
    need = max(q_off + n_heads * q_width, k_off + n_kv * k_width,
               v_off + n_kv * v_width if wants_v else 0)
    if proj.dim() != 2 or proj.shape[1] < need:
        raise KernelError("head_prepare: the projection is narrower than its segments")
    for w, width in ((q_norm, q_width), (k_norm, k_width)):
        if w is not None and w.numel() != width:
            raise KernelError("head_prepare: a norm weight has another width than its heads")
    a = _HeadPrepArgs()
    a.proj, a.in_width = _f32(proj, "proj"), proj.shape[1]
    a.positions, a.token_row = _i32(positions, "positions"), _i32(token_row, "token_row")
    a.seq_end, a.inv_freq = _i32(seq_end, "seq_end"), _f64(inv_freq, "inv_freq")
    a.q_norm_w, a.k_norm_w = _f32(q_norm, "q_norm"), _f32(k_norm, "k_norm")
    a.q_out, a.k_out, a.v_out = _ptr(q_out, "q_out"), _ptr(k_out, "k_out"), _ptr(v_out, "v_out")
    a.k_cache, a.v_cache = _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache")
    a.page_table, a.table_stride, a.ring = _i32(page_table, "page_table"), int(table_stride), int(ring)
    a.q_off, a.n_heads, a.qw = int(q_off), int(n_heads), int(q_width)
    a.k_off, a.n_kv, a.kw = int(k_off), int(n_kv), int(k_width)
    a.v_off, a.vw = int(v_off), int(v_width)
    a.rot_dims, a.rot_style = int(rot_dims), int(rot_style)
    a.rot_mag, a.eps, a.q_mul, a.k_mul = float(rot_magnitude), float(eps), float(q_mul), float(k_mul)
    a.status = _i32(status, "status")
    _check(_lib("mixer_prep").mf_head_prepare(ctypes.addressof(a), n, dtype_code(dt), _stream()),
           "head_prepare")


# ---------------------------------------------------------------------------------------
# retention and the selective scan (csrc/retention.cu, csrc/recurrent.cu)
# ---------------------------------------------------------------------------------------
class _RetentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("v_width", c_longlong),
                ("v_off", c_int), ("decay", c_void_p), ("state", c_void_p), ("cu_seqlens", c_void_p),
                ("slots", c_void_p), ("out", c_void_p), ("n_rows", c_int), ("heads", c_int),
                ("D", c_int), ("Dv", c_int)]


def retention_scan(q: torch.Tensor, k: torch.Tensor, proj: torch.Tensor, v_off: int,
                   decay: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                   slots: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """Per (row, head), tokens one after another: S <- decay[h] S + k v^T; out = S^T q.  ``q``, ``k``
    float32 [tokens, heads, D] (prepared); v the columns v_off .. of ``proj`` (float32 rows, heads of
    Dv); S float32 in ``state`` [slots, heads, Dv, D]; ``out`` float32 [tokens, heads * Dv]."""
    n, heads, d = q.shape
    dv = state.shape[2]
    if (k.shape != q.shape or state.shape[1:] != (heads, dv, d) or out.shape != (n, heads * dv)
            or proj.shape[0] != n or v_off + heads * dv > proj.shape[1] or decay.numel() != heads):
        raise KernelError("retention_scan: shapes do not fit")
    a = _RetentionArgs()
    a.q, a.k, a.v = _f32(q, "q"), _f32(k, "k"), _f32(proj, "proj")
    a.v_width, a.v_off = proj.shape[1], int(v_off)
    a.decay, a.state = _f32(decay, "decay"), _f32(state, "state")
    a.cu_seqlens, a.slots = _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots")
    a.out, a.n_rows, a.heads, a.D, a.Dv = _f32(out, "out"), int(n_rows), heads, d, dv
    _check(_lib("retention").mf_retention_scan(ctypes.addressof(a), _stream()), "retention_scan")


def unit_norm_gate(o: torch.Tensor, gate: torch.Tensor, gate_off: int, out: torch.Tensor,
                   heads: int, eps: float, activation: str = "silu", mul: float = 1.0) -> None:
    """Each head of ``o`` (float32 [tokens, heads * Dv]) divided by its root mean square (eps inside
    the root, no weight), times silu or sigmoid of the gate (columns gate_off .. of float32 rows),
    times ``mul``."""
    n = o.shape[0]
    dv = o.shape[1] // heads
    if out.shape != o.shape or gate.shape[0] != n or gate_off + heads * dv > gate.shape[1]:
        raise KernelError("unit_norm_gate: shapes do not fit")
    _check(_lib("retention").mf_unit_norm_gate(
        _f32(o, "o"), _f32(gate, "gate"), gate.shape[1], int(gate_off), _ptr(out, "out"),
        dtype_code(out.dtype), n, heads, dv, float(eps), HEAD_GATES[activation], float(mul),
        _stream()), "unit_norm_gate")


class _SelectiveArgs(ctypes.Structure):
    _fields_ = [("u", c_void_p), ("dt_raw", c_void_p), ("bc", c_void_p), ("bc_width", c_longlong),
                ("b_off", c_int), ("c_off", c_int), ("z", c_void_p), ("z_width", c_longlong),
                ("z_off", c_int), ("a_log", c_void_p), ("d_skip", c_void_p), ("state", c_void_p),
                ("cu_seqlens", c_void_p), ("slots", c_void_p), ("out", c_void_p), ("n_rows", c_int),
                ("channels", c_int), ("n_state", c_int), ("mul", c_float)]


def selective_scan(u: torch.Tensor, dt_raw: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int,
                   z: torch.Tensor, z_off: int, a_log: torch.Tensor, d_skip: torch.Tensor,
                   state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                   out: torch.Tensor, n_rows: int, mul: float = 1.0) -> None:
    """Per (row, channel c), tokens one after another: dt = softplus(dt_raw[t][c]);
    S[c][n] <- exp(-exp(a_log[c][n]) dt) S[c][n] + dt u[t][c] B[t][n]; y = sum_n S[c][n] C[t][n] +
    d_skip[c] u[t][c]; out = y silu(z[t][z_off + c]) mul.  B and C are columns of ``bc``; everything
    float32 but ``out``; S in ``state`` [slots, channels, n_state]."""
    n, channels = u.shape
    n_state = a_log.shape[1]
    if (dt_raw.shape != u.shape or out.shape != u.shape or a_log.shape[0] != channels
            or state.shape[1:] != (channels, n_state) or d_skip.numel() != channels
            or bc.shape[0] != n or max(b_off, c_off) + n_state > bc.shape[1]
            or z.shape[0] != n or z_off + channels > z.shape[1]):
        raise KernelError("selective_scan: shapes do not fit")
    a = _SelectiveArgs()
    a.u, a.dt_raw, a.bc = _f32(u, "u"), _f32(dt_raw, "dt_raw"), _f32(bc, "bc")
    a.bc_width, a.b_off, a.c_off = bc.shape[1], int(b_off), int(c_off)
    a.z, a.z_width, a.z_off = _f32(z, "z"), z.shape[1], int(z_off)
    a.a_log, a.d_skip, a.state = _f32(a_log, "a_log"), _f32(d_skip, "d_skip"), _f32(state, "state")
    a.cu_seqlens, a.slots = _i32(cu_seqlens, "cu_seqlens"), _i32(slots, "slots")
    a.out, a.n_rows, a.channels, a.n_state, a.mul = _ptr(out, "out"), int(n_rows), channels, n_state, float(mul)
    _check(_lib("recurrent").mf_selective_scan(ctypes.addressof(a), dtype_code(out.dtype), _stream()),
           "selective_scan")


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
# ---------------------------------------------------------------------------------------
# attention with changed scores and a sink (csrc/attention_sink.cu)
# ---------------------------------------------------------------------------------------
def unit_norm_kvstore(qkv: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                      seq_end: torch.Tensor, q_out: torch.Tensor, k_out: Optional[torch.Tensor],
                      v_out: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                      v_cache: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                      table_stride: int, ring: int, n_heads: int, n_kv: int, head_dim: int,
                      value_dim: int, eps: float, norm_qk: bool, status: torch.Tensor,
                      n_partials: int = 0) -> None:
    """The float32 output of a q|k|v projection (``n_partials`` > 0: its K splits
    [splits, tokens, width], added here in split order) -> q and k divided by their root mean
    square per head (``norm_qk``), v unchanged; written as the step's q, k, v and into the
    cache's pages."""
    if n_partials > 0:
        if qkv.dim() != 3 or qkv.shape[0] != n_partials:
            raise KernelError("unit_norm_kvstore: partial sums must be [splits, tokens, width]")
        n, width = qkv.shape[1], qkv.shape[2]
    else:
        n, width = qkv.shape
    if width != (n_heads + n_kv) * head_dim + n_kv * value_dim:
        raise KernelError("unit_norm_kvstore: qkv has the wrong width")
    dt = q_out.dtype
    for t in (k_out, v_out, k_cache, v_cache):
        if t is not None and t.dtype != dt:
            raise KernelError("unit_norm_kvstore: q, k, v and the cache must share one dtype")
    if k_cache is not None and (k_cache.shape[-1] != head_dim or v_cache.shape[-1] != value_dim):
        raise KernelError("unit_norm_kvstore: the cache has other key or value widths")
    _check(_lib("attention_sink").mf_unit_norm_kvstore(
        _f32(qkv, "qkv"), int(n_partials), _i32(positions, "positions"),
        _i32(token_row, "token_row"), _i32(seq_end, "seq_end"), _ptr(q_out, "q_out"),
        _ptr(k_out, "k_out"), _ptr(v_out, "v_out"), _ptr(k_cache, "k_cache"),
        _ptr(v_cache, "v_cache"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        n, n_heads, n_kv, head_dim, value_dim, float(eps), 1 if norm_qk else 0, dtype_code(dt),
        _i32(status, "status"), _stream()), "unit_norm_kvstore")


def sink_attention_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, row_seq: torch.Tensor,
                          row_pos: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor,
                          r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], n_heads: int,
                          n_kv: int, head_dim: int, value_dim: int, window: int, chunk: int,
                          sink: bool, scale: float, sink_logit: Optional[torch.Tensor] = None,
                          softcap: float = 0.0, keep_first: int = 0) -> None:
    """Attention of the step's own packed keys and values (whole prompts): scores
    (q . k) * scale - r1 ln(1 + r2 (i - j)), causal, optional window and chunk mask, a sink
    of score 0 in the softmax if ``sink`` (of score ``sink_logit[h]`` if given), the scores
    soft-capped first (cap * tanh(s / cap)) if ``softcap`` > 0; with ``keep_first`` the keys at
    positions below it stay visible however far the window has moved on."""
    rows = q.shape[0]
    if out.shape != (rows, n_heads * value_dim) or (r1 is None) != (r2 is None):
        raise KernelError("sink_attention_packed: shapes do not fit")
    _check(_lib("attention_sink").mf_sink_attention_packed(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(cu_seqlens, "cu_seqlens"), _ptr(out, "out"), _f32(r1, "r1"), _f32(r2, "r2"), rows,
        n_heads, n_kv, head_dim, value_dim, int(window), int(chunk), 1 if sink else 0, float(scale),
        _f32(sink_logit, "sink_logit"), float(softcap), int(keep_first), dtype_code(q.dtype),
        _stream()), "sink_attention_packed")


def sink_attention_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         row_seq: torch.Tensor, row_pos: torch.Tensor, page_table: torch.Tensor,
                         table_stride: int, ring: int, out: torch.Tensor,
                         r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], n_heads: int,
                         n_kv: int, head_dim: int, value_dim: int, window: int, chunk: int,
                         sink: bool, scale: float, sink_logit: Optional[torch.Tensor] = None,
                         softcap: float = 0.0, keep_first: int = 0) -> None:
    """The same over the paged cache: every row of ``q`` is a query at its own position."""
    rows = q.shape[0]
    if out.shape != (rows, n_heads * value_dim) or (r1 is None) != (r2 is None):
        raise KernelError("sink_attention_paged: shapes do not fit")
    _check(_lib("attention_sink").mf_sink_attention_paged(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"), _i32(row_seq, "row_seq"),
        _i32(row_pos, "row_pos"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(r1, "r1"), _f32(r2, "r2"), rows, n_heads, n_kv, head_dim, value_dim,
        int(window), int(chunk), 1 if sink else 0, float(scale), _f32(sink_logit, "sink_logit"),
        float(softcap), int(keep_first), dtype_code(q.dtype), _stream()), "sink_attention_paged")


def sink_attention_mma_supported(dtype: torch.dtype, head_dim: int, value_dim: int) -> bool:
    """The tensor-core kernels of this attention take bfloat16 with key and value sizes that are
    multiples of 8 up to 128."""
    return (dtype == torch.bfloat16 and
            bool(_lib("attention_sink").mf_sink_attention_mma_supported(int(head_dim), int(value_dim))))


def sink_attention_mma(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                       seq_end: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                       table_stride: int, ring: int, out: torch.Tensor, r1: Optional[torch.Tensor],
                       r2: Optional[torch.Tensor], n_rows: int, max_row_tokens: int, n_heads: int,
                       n_kv: int, head_dim: int, value_dim: int, window: int, chunk: int, sink: bool,
                       scale: float, sink_logit: Optional[torch.Tensor] = None,
                       softcap: float = 0.0, keep_first: int = 0) -> None:
    """The step's packed queries (sequence b brings tokens cu_seqlens[b] .. cu_seqlens[b+1]-1)
    on tensor cores.  ``page_table`` None: ``k``, ``v`` are the step's own packed rows and every
    sequence starts at position 0; else they are the cache and sequence b ends at
    ``seq_end[b]`` after the step."""
    if q.dtype != torch.bfloat16 or out.shape != (q.shape[0], n_heads * value_dim):
        raise KernelError("sink_attention_mma: bfloat16 only, out [tokens, heads * value size]")
    if (r1 is None) != (r2 is None) or (page_table is None) != (seq_end is None):
        raise KernelError("sink_attention_mma: inconsistent arguments")
    _check(_lib("attention_sink").mf_sink_attention_mma(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_end, "seq_end"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(r1, "r1"), _f32(r2, "r2"), int(n_rows), int(max_row_tokens), n_heads,
        n_kv, head_dim, value_dim, int(window), int(chunk), 1 if sink else 0, float(scale),
        _f32(sink_logit, "sink_logit"), float(softcap), int(keep_first), _stream()),
        "sink_attention_mma")


def sink_attention_tc_supported(dtype: torch.dtype, head_dim: int, value_dim: int) -> bool:
    """The tcgen05 kernel takes bfloat16 with keys and values of one size, 64 or 128."""
    return dtype == torch.bfloat16 and head_dim == value_dim and head_dim in (64, 128)


def sink_attention_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                      seq_end: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                      table_stride: int, ring: int, out: torch.Tensor, r1: Optional[torch.Tensor],
                      r2: Optional[torch.Tensor], n_rows: int, max_row_tokens: int, n_heads: int,
                      n_kv: int, head_dim: int, window: int, chunk: int, sink: bool, scale: float,
                      status: torch.Tensor, sink_logit: Optional[torch.Tensor] = None,
                      softcap: float = 0.0, keep_first: int = 0) -> None:
    """``sink_attention_mma``'s job on the 5th-generation tensor cores (tcgen05, tensor memory):
    the step's packed queries over the step's own keys (``page_table`` None) or over the cache."""
    n = q.shape[0]
    if q.dtype != torch.bfloat16 or out.shape != (n, n_heads * head_dim):
        raise KernelError("sink_attention_tc: bfloat16 only, out [tokens, heads * head size]")
    if (r1 is None) != (r2 is None) or (page_table is None) != (seq_end is None):
        raise KernelError("sink_attention_tc: inconsistent arguments")
    pages = k.shape[0] if page_table is not None else 0
    _check(_lib("attention_prefill_tc").mf_sink_attention_tc(
        _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_end, "seq_end"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(r1, "r1"), _f32(r2, "r2"), n, int(n_rows), int(max_row_tokens),
        n_heads, n_kv, head_dim, int(window), int(chunk), 1 if sink else 0, float(scale), int(pages),
        _f32(sink_logit, "sink_logit"), float(softcap), int(keep_first), _i32(status, "status"),
        _stream()), "sink_attention_tc")


_SINK_PLANS: dict = {}


def sink_decode_plan(rows: int, n_kv: int, reach_keys: int) -> tuple[int, int]:
    """(tiles of 32 keys per CTA, key splits) of the kernel for single queries."""
    key = (rows, n_kv, reach_keys)
    got = _SINK_PLANS.get(key)
    if got is None:
        tpc, sp = ctypes.c_int(0), ctypes.c_int(0)
        _lib("attention_sink").mf_sink_decode_plan(rows, n_kv, reach_keys, ctypes.addressof(tpc),
                                                   ctypes.addressof(sp))
        got = (tpc.value, sp.value)
        _SINK_PLANS[key] = got
    return got


def sink_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          row_seq: torch.Tensor, row_pos: torch.Tensor, page_table: torch.Tensor,
                          table_stride: int, ring: int, out: torch.Tensor,
                          r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], n_heads: int,
                          n_kv: int, head_dim: int, value_dim: int, window: int, chunk: int,
                          sink: bool, scale: float, reach_keys: int,
                          sink_logit: Optional[torch.Tensor] = None, softcap: float = 0.0, keep_first: int = 0) -> None:
    """Every row of ``q`` a query at its own position over the paged cache, on tensor cores
    (bfloat16; the query heads of a key/value head in blocks of up to 16).  ``reach_keys``: the most keys a query
    sees (its chunk or window, or the longest sequence's length)."""
    rows = q.shape[0]
    if q.dtype != torch.bfloat16 or out.shape != (rows, n_heads * value_dim):
        raise KernelError("sink_attention_decode: bfloat16 only, out [rows, heads * value size]")
    if (r1 is None) != (r2 is None):
        raise KernelError("sink_attention_decode: inconsistent arguments")
    head_blocks = n_kv * ((n_heads // n_kv + 15) // 16)
    _, splits = sink_decode_plan(rows, head_blocks, int(reach_keys))
    partial = None
    if splits > 1:
        partial = torch.empty(rows * n_heads * splits * (value_dim + 2), dtype=torch.float32,
                              device=q.device)
    _check(_lib("attention_sink").mf_sink_attention_decode(
        _ptr(q, "q"), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"), _i32(row_seq, "row_seq"),
        _i32(row_pos, "row_pos"), _i32(page_table, "page_table"), int(table_stride), int(ring),
        _ptr(out, "out"), _f32(partial, "partial"), _f32(r1, "r1"), _f32(r2, "r2"), rows, n_heads,
        n_kv, head_dim, value_dim, int(window), int(chunk), 1 if sink else 0, float(scale),
        int(reach_keys), _f32(sink_logit, "sink_logit"), float(softcap), int(keep_first), _stream()),
        "sink_attention_decode", 2 if splits > 1 else 1)


def sampler_state_ints() -> int:
    return int(_lib("sampling").mf_sampler_state_ints())


def sample(logits: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int,
           top_p: float, repeat_penalty: float, frequency_penalty: float,
           presence_penalty: float, seed: int, slots: Optional[torch.Tensor] = None,
           state: Optional[torch.Tensor] = None, stream_ids: Optional[torch.Tensor] = None,
           update_state: bool = True) -> None:
    """Samples one token per row of ``logits`` (float32, changed in place) into ``out``."""
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits must be contiguous along the vocabulary")
    if not logits.is_cuda:
        raise KernelError("sample: logits must live on a CUDA device (there is no CPU path)")
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _check(_lib("sampling").mf_sample(
        logits.data_ptr(), logits.stride(0), rows, vocab, _i32(slots, "slots"),
        _i32(state, "state"), _i32(stream_ids, "stream_ids"), _i32(out, "out"), float(temperature),
        int(top_k), float(top_p), float(repeat_penalty), float(frequency_penalty),
        float(presence_penalty), int(seed) & 0xFFFFFFFFFFFFFFFF, 1 if update_state else 0,
        _stream()), "sample")
