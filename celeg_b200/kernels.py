"""Python face of the CUDA kernel library: loads (building it first if needed) the shared
object made from ``celeg_b200/csrc`` and wraps each entry point for torch tensors.

There is no fallback: if the library cannot be built or loaded, :func:`library` raises
:class:`KernelLibraryError`, and every wrapper raises it when a kernel reports an error.
Kernels run on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import build as _build

FLOAT32 = 0
BFLOAT16 = 1


class KernelLibraryError(RuntimeError):
    pass


_LIB: Optional[ctypes.CDLL] = None


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FLOAT32
    if dtype == torch.bfloat16:
        return BFLOAT16
    raise KernelLibraryError(f"the kernels handle float32 and bfloat16, not {dtype}")


_SIGNATURES = {
    "celeg_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "celeg_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                          c_void_p],
    "celeg_rmsnorm_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "celeg_short_conv": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_int, c_void_p, c_int, c_void_p],
    "celeg_attention_generic": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_int,
                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
    "celeg_qkv_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float, c_int, c_int,
                          c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                          c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_void_p, c_int, c_void_p],
    "celeg_add_layernorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
                            c_int, c_void_p],
    "celeg_rmsnorm_strided": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_float, c_int,
                              c_void_p],
    "celeg_sigmoid_gate": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_bias_store_kv": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_int, c_void_p],
    "celeg_embedding_sinusoid": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "celeg_lru_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_block_diagonal_product": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_lru_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                       c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_lru_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_retention_decode_raw": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_int,
                                   c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "celeg_activation_columns": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_glu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_scaled_sum": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "celeg_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_attention_decode_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                     c_void_p],
    "celeg_attention_decode_solo_items": [c_longlong],
    "celeg_attention_decode_resident_blocks": [c_int],
    "celeg_attention_prefill": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "celeg_attention_prefill_tcgen05": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "celeg_attention_decode_biased": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "celeg_gemv_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                        c_void_p, c_longlong, c_void_p, c_void_p],
    "celeg_gemv_prefetch_next": [c_void_p, c_longlong],
    "celeg_gemv_bf16_split_norm": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                   c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
                                   c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
    "celeg_embedding_split_norm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                   c_void_p, c_int, c_void_p],
    "celeg_gemm_tcgen05": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                           c_int, c_void_p],
    "celeg_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "celeg_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_sample_scratch_elements": [],
    "celeg_sample_greedy": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p],
    "celeg_mark_seen": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "celeg_attention_decode_sinks": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_qk_whole_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                       c_int, c_void_p, c_void_p, c_int, c_void_p],
    "celeg_add_dyt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                      c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p],
    "celeg_join_stream_embedding": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_float, c_int, c_void_p],
    "celeg_activation": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p],
    "celeg_softcap": [c_void_p, c_longlong, c_float, c_void_p],
    "celeg_recurrent_scan": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                             c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "celeg_recurrent_decode": [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                               c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float, c_float, c_void_p, c_longlong,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p],
    "celeg_mlstm_gates": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p],
    "celeg_delta_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_float, c_void_p],
    "celeg_gated_head_norm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_int,
                              c_int, c_void_p],
    "celeg_retention_segmented": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                  c_void_p, c_void_p, c_void_p],
    "celeg_depth_average": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                            c_float, c_int, c_int, c_int, c_void_p],
    "celeg_latent_prepare": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "celeg_head_project": [c_void_p, c_int, c_int, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_int, c_int,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_head_gate": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_moe_route": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "celeg_moe_group": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_moe_gather_rows": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_gemm_tcgen05_grouped": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                   c_int, c_int, c_void_p, c_int, c_void_p],
    "celeg_expert_product": [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_int,
                             c_int, c_int, c_int, c_int, c_void_p],
    "celeg_expert_rows": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_void_p],
    "celeg_moe_combine": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_void_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; built at the first call in a fresh checkout."""
    global _LIB
    if _LIB is None:
        try:
            path = _build.ensure_built()
            lib = ctypes.CDLL(path)
        except (_build.BuildError, OSError) as exc:
            raise KernelLibraryError(f"the CUDA kernel library of celeg_b200 is not available: {exc}") from exc
        lib.celeg_last_error.restype = ctypes.c_char_p
        lib.celeg_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = lib
    return _LIB


def library_path() -> str:
    library()
    return _LIB._name  # type: ignore[union-attr]


LAUNCHES = 0        # entry-point calls made so far (each is one kernel launch unless it returned early)


def _check(code: int) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        raise KernelLibraryError(library().celeg_last_error().decode("utf-8", "replace"))


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    if tensor is None:
        return None
    return tensor.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(tensor: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if tensor.dtype != dtype or not tensor.is_cuda or not tensor.is_contiguous():
        raise KernelLibraryError(f"{name} must be a contiguous CUDA tensor of {dtype}, got {tensor.dtype} "
                                 f"on {tensor.device}, contiguous={tensor.is_contiguous()}")


# ------------------------------------------------------------------------------ wrappers
class SplitNorm:
    """An RMSNorm split over the two products around it (csrc/gemv_bf16.cu, GemvNormArgs): ``xw`` holds
    bfloat16 rows of residual * weight, ``sumsq[row, :partials]`` the pieces of each row's sum of squares;
    the product that takes ``xw`` as its operand multiplies its sums by 1 / sqrt(sum / width + eps)."""
    __slots__ = ("xw", "sumsq", "partials", "eps", "width")

    def __init__(self, xw: torch.Tensor, sumsq: torch.Tensor, partials: int, eps: float, width: int):
        self.xw, self.sumsq, self.partials, self.eps, self.width = xw, sumsq, partials, eps, width


def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, multiplier: float = 1.0,
              prepare: Optional[SplitNorm] = None, next_weight: Optional[torch.Tensor] = None,
              positions: Optional[torch.Tensor] = None, frequencies: Optional[torch.Tensor] = None) -> None:
    """out[t] = multiplier * table[tokens[t]]. With ``prepare``: also the first half of the norm whose
    weight is ``next_weight`` (``prepare.xw`` and one sum of squares per row are written). With ``positions`` and
    ``frequencies`` (float32 [(hidden + 1) // 2]): plus a sinusoidal vector of the position, entry 2i
    sin(p f_i), entry 2i + 1 cos(p f_i)."""
    rows = tokens.shape[0]
    _need(tokens, torch.int32, "tokens")
    _need(out, torch.float32, "out")
    vocab, hidden = table.shape
    assert out.shape[0] >= rows and out.shape[1] == hidden
    if frequencies is not None:
        _need(frequencies, torch.float32, "frequencies")
        _need(positions, torch.int32, "positions")
        assert frequencies.numel() >= (hidden + 1) // 2 and positions.numel() >= rows
        if prepare is not None:
            _need(next_weight, torch.float32, "next_weight")
            assert prepare.xw.dtype == torch.bfloat16 and prepare.xw.stride(0) == hidden and prepare.partials == 1
        _check(library().celeg_embedding_sinusoid(
            _ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(positions), _ptr(frequencies), _ptr(out), rows,
            hidden, vocab, multiplier, _ptr(next_weight) if prepare is not None else None,
            _ptr(prepare.xw) if prepare is not None else None, _ptr(prepare.sumsq) if prepare is not None else None,
            prepare.sumsq.stride(0) if prepare is not None else 0, _stream()))
        return
    if prepare is None:
        _check(library().celeg_embedding(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), rows, hidden,
                                         vocab, multiplier, _stream()))
        return
    _need(next_weight, torch.float32, "next_weight")
    assert prepare.xw.dtype == torch.bfloat16 and prepare.xw.stride(0) == hidden and prepare.partials == 1
    _check(library().celeg_embedding_split_norm(
        _ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), rows, hidden, vocab, multiplier,
        _ptr(next_weight), _ptr(prepare.xw), _ptr(prepare.sumsq), prepare.sumsq.stride(0), _stream()))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                write_residual: bool = True) -> None:
    """out[i] = rmsnorm(residual[r] + delta[r]) * weight; residual[r] updated when not gathering."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "weight")
    width = residual.shape[-1]
    if n_rows is None:
        n_rows = rows.shape[0] if rows is not None else residual.shape[0]
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == width
    _check(library().celeg_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows,
                                       width, eps, int(write_residual and rows is None), dtype_code(out.dtype),
                                       _stream()))


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, n_rows: int) -> None:
    _need(weight, torch.float32, "weight")
    _check(library().celeg_rmsnorm_rows(_ptr(x), _ptr(weight), _ptr(out), n_rows, x.shape[-1], eps,
                                        dtype_code(x.dtype), _stream()))


def short_conv(proj: torch.Tensor, kernel: torch.Tensor, state: torch.Tensor, slot_stride: int, out: torch.Tensor,
               token_span: torch.Tensor, span_begin: torch.Tensor, span_slot: torch.Tensor, tokens: int, spans: int,
               hidden: int, taps: int, max_span: Optional[int] = None) -> None:
    """``state`` points at this layer's state inside slot 0; ``slot_stride`` floats separate slots.
    ``max_span``: the longest span of the step if the caller knows it (saves a launch when no span is
    longer than the kernel); default: as long as the batch."""
    _need(kernel, torch.float32, "conv kernel")
    assert state.dtype == torch.float32
    _check(library().celeg_short_conv(_ptr(proj), _ptr(kernel), _ptr(state), slot_stride, _ptr(out),
                                      _ptr(token_span), _ptr(span_begin), _ptr(span_slot), tokens, spans, hidden,
                                      taps, tokens if max_span is None else max_span, dtype_code(proj.dtype),
                                      _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       inv_freq: Optional[torch.Tensor], positions: torch.Tensor, token_span: torch.Tensor,
                       block_table: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       tokens: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int, page_tokens: int,
                       eps: float, store_kv, error_flag: torch.Tensor) -> None:
    """k_cache / v_cache: one layer's pages, [pages, kv_heads, page_tokens, head_dim]. ``store_kv``: False/0 = q
    heads only; True/1 = k (normalised, rotated) and v are written to the cache; 2 = k heads are normalised and
    rotated in place like the q heads, v heads and the cache are left alone."""
    page_stride = k_cache.stride(0) if k_cache is not None else 0
    _check(library().celeg_qk_norm_rope_store(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _ptr(positions), _ptr(token_span),
        _ptr(block_table), block_table.stride(0), _ptr(k_cache), _ptr(v_cache), page_stride, tokens, q_heads,
        kv_heads, head_dim, rotary_dim, page_tokens, eps, int(store_kv), _ptr(error_flag), dtype_code(qkv.dtype),
        _stream()))


def qk_whole_norm_rope_store(qk: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                             inv_freq: Optional[torch.Tensor], positions: torch.Tensor, token_span: torch.Tensor,
                             block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tokens: int,
                             q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int, page_tokens: int, eps: float,
                             values_are_keys: bool, row_scales: torch.Tensor, error_flag: torch.Tensor) -> None:
    """q and k normalised over the whole projection (weights [q_heads*head_dim], [kv_heads*head_dim]), rotated, q in
    place, k into the cache; ``values_are_keys``: rows are [q heads | k heads] and a key as projected is stored as
    its own value (else rows are [q | k | v heads]). ``row_scales``: float32 scratch of 2*tokens."""
    _need(row_scales, torch.float32, "row_scales")
    assert row_scales.numel() >= 2 * tokens
    _check(library().celeg_qk_whole_norm_rope_store(
        _ptr(qk), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _ptr(positions), _ptr(token_span),
        _ptr(block_table), block_table.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), tokens, q_heads,
        kv_heads, head_dim, rotary_dim, page_tokens, eps, int(values_are_keys), _ptr(row_scales), _ptr(error_flag),
        dtype_code(qk.dtype), _stream()))
    global LAUNCHES
    LAUNCHES += 1 if (q_weight is not None or k_weight is not None) else 0      # the scales are a launch of their own


def attention_generic(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                      block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                      page_tokens: int, window: Optional[int], scale: float, error_flag: torch.Tensor,
                      sinks: Optional[torch.Tensor] = None, value_dim: Optional[int] = None,
                      chunk: Optional[int] = None, distance_bias: Optional[torch.Tensor] = None) -> None:
    """``sinks``: float32 [q_heads] or None; a head's sink is a score that enters the denominator of each of its
    rows once, unscaled, without key or value. ``value_dim``: the values' size when it is not the keys' (``out`` is
    then [tokens, q_heads * value_dim]). ``chunk``: a query reads only the keys of its own chunk of that many
    positions, counted from position 0 (no window then). ``distance_bias``: float32 [q_heads, n + 1] or None; entry
    [h, min(distance, n)] is added to head h's scaled score of a key ``distance`` positions back."""
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
    bias_ptr, bias_last = _distance_bias(distance_bias, q_heads)
    _check(library().celeg_attention_generic(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), v_cache.stride(0),
        int(value_dim or 0), int(chunk or 0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, _ptr(sinks), bias_ptr, bias_last, _ptr(error_flag), dtype_code(q.dtype),
        _stream()))


def _distance_bias(table: Optional[torch.Tensor], q_heads: int) -> Tuple[Optional[int], int]:
    """(address, last column) of a table of score biases by distance, [q_heads, last + 1] float32, or (None, 0)."""
    if table is None:
        return None, 0
    _need(table, torch.float32, "distance_bias")
    assert table.dim() == 2 and table.shape[0] == q_heads and table.is_contiguous() and table.shape[1] >= 1
    return _ptr(table), int(table.shape[1]) - 1


def qkv_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor, positions: torch.Tensor,
                token_span: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                tokens: int, q_heads: int, kv_heads: int, head_dim: int, value_dim: int, key_store: int,
                value_store: int, page_tokens: int, error_flag: torch.Tensor, *,
                q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                frequencies: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                temperature: Optional[Tuple[float, int]] = None, blend: int = 0, lam: float = 0.0,
                first_values: Optional[torch.Tensor] = None) -> None:
    """Float32 rows [q heads | k heads | v heads | ...] as projected become queries in ``q_out`` and keys and values
    in the tokens' places of the paged cache (csrc/attention_prepare.cu), after, in this order: the biases; one RMS
    norm over the whole q projection and one over the whole k projection (``q_norm`` / ``k_norm``, as wide as the
    projections); the rotation of the first ``rotary_dim`` entries of every q and k head in pairs (i, i + half) by
    position x ``frequencies``; ``temperature`` = (coef, every): q times 1 + coef ln(floor((position + 1) / every) + 1);
    ``blend`` 1: the values are noted in ``first_values`` (float32 [tokens, kv_heads * value_dim]); 2: v becomes
    (1 - lam) v + lam first_values. One rounding."""
    _need(proj, torch.float32, "proj")
    for vector in (bias, q_norm, k_norm, frequencies, first_values):
        if vector is not None:
            _need(vector, torch.float32, "a vector of qkv_prepare")
    assert q_out.dtype == k_cache.dtype == v_cache.dtype and q_out.stride(-1) == 1 and proj.stride(-1) == 1
    coef, every = temperature if temperature else (0.0, 0)
    _check(library().celeg_qkv_prepare(
        _ptr(proj), proj.stride(0), _ptr(bias), _ptr(q_norm), _ptr(k_norm), norm_eps, _ptr(frequencies), rotary_dim,
        float(coef), int(every), blend, lam, _ptr(first_values), first_values.stride(0) if first_values is not None else 0,
        _ptr(q_out), q_out.stride(0), _ptr(positions), _ptr(token_span), _ptr(block_table), block_table.stride(0),
        _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), v_cache.stride(0), tokens, q_heads, kv_heads, head_dim, value_dim,
        key_store, value_store, page_tokens, _ptr(error_flag), dtype_code(q_out.dtype), _stream()))


def add_layernorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                  eps: float, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                  bias: Optional[torch.Tensor] = None) -> None:
    """out[i] = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight (+ bias) of x = residual[r] + delta[r];
    residual[r] is updated when not gathering (csrc/layernorm.cu)."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "weight")
    width = residual.shape[-1]
    if n_rows is None:
        n_rows = rows.shape[0] if rows is not None else residual.shape[0]
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == width
    _check(library().celeg_add_layernorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(bias), _ptr(out), _ptr(rows),
                                         n_rows, width, eps, int(rows is None), dtype_code(out.dtype), _stream()))


def rmsnorm_strided(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, n_rows: int) -> None:
    """RMS norm of the rows of a 2-D view (a slice of a wider buffer's columns) into another."""
    _need(weight, torch.float32, "weight")
    assert x.dtype == out.dtype and x.stride(-1) == 1 and out.stride(-1) == 1 and x.shape[-1] == out.shape[-1]
    _check(library().celeg_rmsnorm_strided(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), n_rows,
                                           x.shape[-1], eps, dtype_code(x.dtype), _stream()))


def sigmoid_gate(values: torch.Tensor, gate: torch.Tensor, tokens: int, width: int) -> None:
    """values[t, c] *= sigmoid(gate[t, c]) for c < width, in place; ``gate`` float32 or of the values' type."""
    assert values.stride(-1) == 1 and gate.stride(-1) == 1
    _check(library().celeg_sigmoid_gate(_ptr(values), values.stride(0), _ptr(gate), gate.stride(0), tokens, width,
                                        dtype_code(values.dtype), dtype_code(gate.dtype), _stream()))


def bias_store_kv(proj: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor, positions: torch.Tensor,
                  token_span: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  tokens: int, q_heads: int, kv_heads: int, head_dim: int, value_dim: int, key_store: int,
                  value_store: int, page_tokens: int, error_flag: torch.Tensor) -> None:
    """Float32 rows [q heads | k heads | v heads] as projected (values ``value_dim`` wide): ``bias`` (float32, a row's
    width, or None) is added and the sums are rounded once, q into ``q_out`` and k and v into the tokens' places in
    the paged cache. ``key_store`` / ``value_store``: the sizes of a stored head (queries and keys / values); what a
    stored head has beyond the projected one is written as zeros."""
    _need(proj, torch.float32, "proj")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        assert bias.numel() == q_heads * head_dim + kv_heads * (head_dim + value_dim)
    assert q_out.dtype == k_cache.dtype == v_cache.dtype and q_out.stride(-1) == 1 and proj.stride(-1) == 1
    _check(library().celeg_bias_store_kv(
        _ptr(proj), proj.stride(0), _ptr(bias), _ptr(q_out), q_out.stride(0), _ptr(positions), _ptr(token_span),
        _ptr(block_table), block_table.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), v_cache.stride(0),
        tokens, q_heads, kv_heads, head_dim, value_dim, key_store, value_store, page_tokens, _ptr(error_flag),
        dtype_code(q_out.dtype), _stream()))


def attention_decode_supported(q_heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Shapes the split-key decode kernel takes; everything else goes to the general kernel."""
    return (dtype == torch.bfloat16 and q_heads % kv_heads == 0 and q_heads // kv_heads <= 16
            and head_dim % 8 == 0 and head_dim <= 256)


def attention_decode_resident_blocks(head_dim: int) -> int:
    """Blocks of the decode attention (its one-stage form) that the current device holds at a time; 0 if unknown."""
    return max(0, int(library().celeg_attention_decode_resident_blocks(int(head_dim))))


def attention_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                     block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                     page_tokens: int, window: Optional[int], scale: float, chunk: int, max_splits: int,
                     partial_o: torch.Tensor, partial_ml: torch.Tensor, counters: torch.Tensor,
                     error_flag: torch.Tensor, sinks: Optional[torch.Tensor] = None,
                     distance_bias: Optional[torch.Tensor] = None) -> None:
    """One query token per row, keys split into chunks of ``chunk``; scratch: partial_o float32
    [tokens*q_heads*max_splits*head_dim], partial_ml float32 [tokens*q_heads*max_splits*2],
    counters int32 [tokens*kv_heads] (zero before the first call, left zero by every call).
    ``sinks``: as for :func:`attention_generic`. ``window`` = -c (negative) stands for a chunked mask: a query reads the
    keys of its own chunk of c positions, chunks counted from position 0; the prompt kernels read it the same way."""
    assert partial_o.numel() >= tokens * q_heads * max_splits * head_dim
    assert partial_ml.numel() >= tokens * q_heads * max_splits * 2
    assert counters.numel() >= tokens * kv_heads
    if distance_bias is not None:
        if sinks is not None:
            _need(sinks, torch.float32, "sinks")
        bias_ptr, bias_last = _distance_bias(distance_bias, q_heads)
        _check(library().celeg_attention_decode_biased(
            _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
            _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
            page_tokens, int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml),
            _ptr(counters), _ptr(error_flag), _ptr(sinks), bias_ptr, bias_last, _stream()))
        return
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        _check(library().celeg_attention_decode_sinks(
            _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
            _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
            page_tokens, int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml),
            _ptr(counters), _ptr(error_flag), _ptr(sinks), _stream()))
        return
    _check(library().celeg_attention_decode(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml),
        _ptr(counters), _ptr(error_flag), _stream()))


def attention_decode_fused(qkv: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                           block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                           page_tokens: int, window: Optional[int], scale: float, chunk: int, max_splits: int,
                           partial_o: torch.Tensor, partial_ml: torch.Tensor, counters: torch.Tensor,
                           error_flag: torch.Tensor, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                           eps: float) -> None:
    """Decode attention over the raw q|k|v projection: per-head norm and rotation of q and of the token's own
    key, the cache write of that key and its value, and the attention, in one launch."""
    _check(library().celeg_attention_decode_fused(
        _ptr(qkv), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim, page_tokens,
        int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml), _ptr(counters),
        _ptr(error_flag), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), rotary_dim, eps, _stream()))


def attention_prefill_supported(q_heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Shapes the tensor-core kernel for prompt portions takes; the rest goes to the general kernel."""
    return dtype == torch.bfloat16 and q_heads % kv_heads == 0 and head_dim % 8 == 0 and head_dim <= 256


def attention_prefill(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, positions: torch.Tensor, span_begin: torch.Tensor,
                      block_table: torch.Tensor, tokens: int, spans: int, q_heads: int, kv_heads: int,
                      head_dim: int, page_tokens: int, window: Optional[int], scale: float,
                      error_flag: torch.Tensor, sinks: Optional[torch.Tensor] = None,
                      distance_bias: Optional[torch.Tensor] = None) -> None:
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
    bias_ptr, bias_last = _distance_bias(distance_bias, q_heads)
    _check(library().celeg_attention_prefill(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(span_begin), _ptr(block_table), block_table.stride(0), tokens, spans, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, _ptr(sinks), bias_ptr, bias_last, _ptr(error_flag), _stream()))


def attention_prefill_tcgen05_supported(q_heads: int, kv_heads: int, head_dim: int, page_tokens: int,
                                        dtype: torch.dtype) -> bool:
    """Shapes the tcgen05 kernel for prompt portions takes: head size 64, pages of 8, 16, 32 or 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim == 64 and kv_heads > 0 and q_heads % kv_heads == 0
            and page_tokens >= 8 and page_tokens % 8 == 0 and 64 % page_tokens == 0)


def attention_prefill_tcgen05(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                              v_cache: torch.Tensor, positions: torch.Tensor, span_begin: torch.Tensor,
                              block_table: torch.Tensor, tokens: int, spans: int, tile_count: int, q_heads: int,
                              kv_heads: int, head_dim: int, page_tokens: int, window: Optional[int], scale: float,
                              error_flag: torch.Tensor, sinks: Optional[torch.Tensor] = None,
                              distance_bias: Optional[torch.Tensor] = None) -> None:
    """Prompt-portion attention on tcgen05 (S and O' in tensor memory, Q/K/V by TMA).
    ``tile_count`` = sum over the spans of ceil(length / 128). ``distance_bias``: as for :func:`attention_generic`."""
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelLibraryError("attention_prefill_tcgen05 needs contiguous cache layers")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
    bias_ptr, bias_last = _distance_bias(distance_bias, q_heads)
    _check(library().celeg_attention_prefill_tcgen05(
        _ptr(q), q_row_stride, q.shape[0], _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(positions),
        _ptr(span_begin), _ptr(block_table), block_table.stride(0), tokens, spans, tile_count, q_heads, kv_heads,
        head_dim, page_tokens, int(window or 0), scale, _ptr(sinks), bias_ptr, bias_last, _ptr(error_flag), _stream()))


ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU, ACT_RELU_SQUARED, ACT_RELU = 0, 1, 2, 3, 4      # codes of csrc/common.cuh: activate()
GEMV_MAX_ROWS = 16
GEMV_STORE, GEMV_STORE_F32, GEMV_ADD_RESIDUAL, GEMV_SWIGLU, GEMV_CONV, GEMV_ACTIVATION = 0, 1, 2, 3, 4, 5


def gemv_supported(rows: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < rows <= GEMV_MAX_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemv_bf16(x, w: torch.Tensor, y: torch.Tensor, rows: int, mode: int = GEMV_STORE, *,
              conv_w: Optional[torch.Tensor] = None, taps: int = 0, state: Optional[torch.Tensor] = None,
              slot_stride: int = 0, span_slot: Optional[torch.Tensor] = None,
              prepare: Optional[SplitNorm] = None, next_weight: Optional[torch.Tensor] = None,
              ahead: Optional[Tuple[int, int]] = None) -> None:
    """y[:rows] = x[:rows] @ w.T for at most 16 rows, streaming w once. mode GEMV_STORE: y bfloat16;
    GEMV_STORE_F32: y float32; GEMV_ADD_RESIDUAL: y float32, accumulated; GEMV_SWIGLU: w is
    [2*inner, k] (gate rows, then up rows) and y bfloat16 [rows, inner] = silu(gate) * up (``taps`` = 1 + ACT_*:
    that function of the gate instead); GEMV_CONV: w is
    [3*channels, k] (B, C, X rows of the short convolution's input projection), y bfloat16
    [rows, channels] = C * conv(B*X) over each request's carried state, which is shifted; row i is the
    single token of request i, whose state slot is span_slot[i]. GEMV_ACTIVATION: y bfloat16 = act(x w^T) with
    ``taps`` = ACT_GELU_ERF, ACT_GELU_TANH or ACT_SILU (the product rounded to bfloat16 first, as a plain product
    stores it).
    ``x`` may be a :class:`SplitNorm` (the operand still lacks its row scale; applied to the sums here).
    With ``prepare`` (GEMV_ADD_RESIDUAL only): the first half of the norm that follows, weight
    ``next_weight``, is written too: ``prepare.xw`` and this product's pieces of the sums of squares.
    ``ahead`` = (device address, bytes) of the weights that the step's next product will read: this launch
    asks them into the L2 (the memory must outlive every graph that captures the launch)."""
    if ahead is not None and ahead[1] > 0:
        if library().celeg_gemv_prefetch_next(ctypes.c_void_p(ahead[0]), ahead[1]) != 0:      # (no launch)
            raise KernelLibraryError(library().celeg_last_error().decode("utf-8", "replace"))
    blocks = {GEMV_SWIGLU: 2, GEMV_CONV: 3}.get(mode, 1)
    n = w.shape[0] // blocks
    k = w.shape[1]
    scaled = x if isinstance(x, SplitNorm) else None
    operand = scaled.xw if scaled is not None else x
    assert operand.shape[-1] == k and y.shape[-1] >= n
    want = torch.float32 if mode in (GEMV_STORE_F32, GEMV_ADD_RESIDUAL) else torch.bfloat16
    if y.dtype != want:
        raise KernelLibraryError(f"gemv_bf16 mode {mode} writes {want}, got {y.dtype}")
    if scaled is None and prepare is None:
        _check(library().celeg_gemv_bf16(_ptr(operand), operand.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0),
                                         rows, n, k, mode, _ptr(conv_w), taps, _ptr(state), slot_stride,
                                         _ptr(span_slot), _stream()))
        return
    if prepare is not None:
        _need(next_weight, torch.float32, "next_weight")
        if prepare.partials != (n + 15) // 16 or prepare.sumsq.stride(0) < prepare.partials:
            raise KernelLibraryError(f"a product of {n} columns writes {(n + 15) // 16} pieces of the sums, "
                                     f"not {prepare.partials}")
    _check(library().celeg_gemv_bf16_split_norm(
        _ptr(operand), operand.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0), rows, n, k, mode,
        _ptr(conv_w), taps, _ptr(state), slot_stride, _ptr(span_slot),
        _ptr(scaled.sumsq) if scaled else None, scaled.partials if scaled else 0,
        scaled.sumsq.stride(0) if scaled else 0, scaled.eps if scaled else 0.0, scaled.width if scaled else 0,
        _ptr(next_weight) if prepare else None, _ptr(prepare.xw) if prepare else None,
        prepare.xw.stride(0) if prepare else 0, _ptr(prepare.sumsq) if prepare else None,
        prepare.sumsq.stride(0) if prepare else 0, _stream()))


TC_STORE, TC_STORE_F32, TC_SWIGLU = 0, 1, 2
TC_ACTIVATION = 3          # + ACT_GELU_ERF, ACT_GELU_TANH or ACT_SILU: y bfloat16 = act(x w^T)
TC_GATED = 16              # + a code of ACT_*: as TC_SWIGLU with that function of the gate in place of SiLU


def gemm_tcgen05_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, rows: int, epilogue: int,
                 error_flag: torch.Tensor, variant: int = -1) -> None:
    """y[:rows] = x[:rows] @ w.T on tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    TC_STORE: y bfloat16; TC_STORE_F32: y float32; TC_SWIGLU: w is [2*inner, k] (gate rows, then up rows),
    y bfloat16 [rows, inner] = silu(gate) * up; TC_GATED + kind: the same with another function of the gate.
    ``variant``: -1 lets the library choose the tile shape,
    0..3 force one (128x128 with 6 or 3 stages, 128x256, persistent with two accumulators)."""
    n = w.shape[0] // 2 if epilogue == TC_SWIGLU or epilogue >= TC_GATED else w.shape[0]
    k = w.shape[1]
    want = torch.float32 if epilogue == TC_STORE_F32 else torch.bfloat16
    if y.dtype != want:
        raise KernelLibraryError(f"gemm_tcgen05 epilogue {epilogue} writes {want}, got {y.dtype}")
    assert x.shape[-1] == k and y.shape[-1] >= n
    _check(library().celeg_gemm_tcgen05(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0), rows, n, k,
                                        epilogue, _ptr(error_flag), int(variant), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, tokens: int, inner: int) -> None:
    _check(library().celeg_swiglu(_ptr(gate_up), _ptr(out), tokens, inner, dtype_code(gate_up.dtype), _stream()))


def glu(gate_up: torch.Tensor, out: torch.Tensor, tokens: int, inner: int, kind: int) -> None:
    """out[:tokens] = act(gate) * up of rows [gate | up] (``inner`` each), ``kind`` one of ACT_*."""
    _check(library().celeg_glu(_ptr(gate_up), _ptr(out), tokens, inner, kind, dtype_code(gate_up.dtype), _stream()))


def gemm_f32(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, accumulate: bool = False) -> None:
    """y[:m] (+)= x[:m] @ w.T with float32 operands and FFMA accumulation."""
    _need(w, torch.float32, "w")
    assert x.dtype == torch.float32 and y.dtype == torch.float32
    n, k = w.shape
    assert x.stride(-1) == 1 and y.stride(-1) == 1 and x.shape[-1] == k and y.shape[-1] == n
    _check(library().celeg_gemm_f32(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0),
                                    int(accumulate), _stream()))


def sample_scratch(device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Scratch that lets :func:`sample` cut the rows of a small batch into pieces (one block each): candidate
    scores, candidate tokens and their counts."""
    elements = int(library().celeg_sample_scratch_elements())
    return (torch.zeros(elements, dtype=torch.float32, device=device),
            torch.zeros(elements, dtype=torch.int32, device=device),
            torch.zeros(elements // 128, dtype=torch.int32, device=device))


def sample(logits: torch.Tensor, rows: int, row_slot: Optional[torch.Tensor], seen: Optional[torch.Tensor],
           rng: Optional[torch.Tensor], temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], penalty: Optional[torch.Tensor], out: torch.Tensor,
           scratch: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> None:
    """One token per row with celeg's rules. ``scratch`` (:func:`sample_scratch`): with it, a batch of at most
    32 rows over a large vocabulary runs as 16 blocks per row and a merge; without it, one block per row."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    parts = scratch or (None, None, None)
    _check(library().celeg_sample(_ptr(logits), logits.stride(0), logits.shape[1], rows, _ptr(row_slot), _ptr(seen),
                                  _ptr(rng), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty), _ptr(out),
                                  _ptr(parts[0]), _ptr(parts[1]), _ptr(parts[2]), _stream()))


def sample_greedy(logits: torch.Tensor, rows: int, row_slot: Optional[torch.Tensor], seen: Optional[torch.Tensor],
                  penalty: Optional[torch.Tensor], out: torch.Tensor, partial_score: torch.Tensor,
                  partial_token: torch.Tensor) -> None:
    """Arg-max (first maximum) of every row after the repetition penalty; scratch: rows*64 each."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    assert partial_score.numel() >= rows * 64 and partial_token.numel() >= rows * 64
    _check(library().celeg_sample_greedy(_ptr(logits), logits.stride(0), logits.shape[1], rows, _ptr(row_slot),
                                         _ptr(seen), _ptr(penalty), _ptr(out), _ptr(partial_score),
                                         _ptr(partial_token), _stream()))
    global LAUNCHES
    LAUNCHES += 1                                     # two kernels


def mark_seen(seen: torch.Tensor, tokens: torch.Tensor, token_span: torch.Tensor, span_slot: torch.Tensor,
              count: int) -> None:
    _check(library().celeg_mark_seen(_ptr(seen), seen.shape[1], _ptr(tokens), _ptr(token_span), _ptr(span_slot),
                                     count, _stream()))


# ------------------------------------------------------- Dynamic Tanh blocks, matrix-state mixers
def add_dyt(residual: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor], n_rows: int,
            first: Tuple[torch.Tensor, torch.Tensor, float, torch.Tensor],
            second: Optional[Tuple[torch.Tensor, torch.Tensor, float, torch.Tensor]] = None,
            rows: Optional[torch.Tensor] = None) -> None:
    """x = residual (+ delta_a) (+ delta_b), written back unless ``rows`` gathers; ``first`` and ``second`` are
    (weight, bias, alpha, out): out = tanh(alpha x) weight + bias in the activation type of ``out``."""
    _need(residual, torch.float32, "residual")
    width = residual.shape[-1]
    w1, b1, alpha1, out1 = first
    w2, b2, alpha2, out2 = second if second is not None else (None, None, 0.0, None)
    for delta in (delta_a, delta_b):
        if delta is not None:
            assert delta.dtype == out1.dtype and delta.shape[-1] == width
    _check(library().celeg_add_dyt(_ptr(residual), _ptr(delta_a), _ptr(delta_b), _ptr(rows), n_rows, width,
                                   int(rows is None), _ptr(w1), _ptr(b1), alpha1, _ptr(out1), _ptr(w2), _ptr(b2), alpha2,
                                   _ptr(out2), dtype_code(out1.dtype), _stream()))


def add_to_residual(residual: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                    n_rows: int) -> None:
    """residual[:n_rows] += delta_a (+ delta_b), float32 sums."""
    _need(residual, torch.float32, "residual")
    given = delta_a if delta_a is not None else delta_b
    if given is None:
        return
    _check(library().celeg_add_dyt(_ptr(residual), _ptr(delta_a), _ptr(delta_b), None, n_rows, residual.shape[-1], 1,
                                   None, None, 0.0, None, None, None, 0.0, None, dtype_code(given.dtype), _stream()))


def join_stream_embedding(residual: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                          table: torch.Tensor, tokens: torch.Tensor, joined: torch.Tensor, n_rows: int,
                          multiplier: float = 1.0) -> None:
    """joined[t] = [residual[t] (+ deltas) | multiplier * table[tokens[t]]] in the type of ``joined`` (= the table's)."""
    _need(residual, torch.float32, "residual")
    _need(tokens, torch.int32, "tokens")
    width = residual.shape[-1]
    assert joined.shape[-1] == 2 * width and table.shape[1] == width and table.dtype == joined.dtype
    _check(library().celeg_join_stream_embedding(_ptr(residual), _ptr(delta_a), _ptr(delta_b), _ptr(table), _ptr(tokens),
                                                 _ptr(joined), n_rows, width, table.shape[0], multiplier,
                                                 dtype_code(joined.dtype), _stream()))


def activation(x: torch.Tensor, out: torch.Tensor, rows: int, kind: int) -> None:
    """out[:rows] = act(x[:rows]) element by element (in place allowed); both contiguous, same shape."""
    assert x.is_contiguous() and out.is_contiguous() and x.shape[1:] == out.shape[1:] and x.dtype == out.dtype
    _check(library().celeg_activation(_ptr(x), _ptr(out), rows * x.shape[1], kind, dtype_code(x.dtype), _stream()))


def activation_columns(x: torch.Tensor, columns: int, rows: int, kind: int) -> None:
    """act() of the first ``columns`` columns of x[:rows], in place; the other columns are left alone."""
    assert x.stride(-1) == 1 and columns <= x.shape[1]
    _check(library().celeg_activation_columns(_ptr(x), x.stride(0), columns, rows, kind, dtype_code(x.dtype), _stream()))


def scaled_sum(a: torch.Tensor, b: Optional[torch.Tensor], bias_a: Optional[torch.Tensor], scale_a: float, scale_b: float,
               out: torch.Tensor, rows: int) -> None:
    """out[:rows] = scale_a (a + bias_a) + scale_b b; a, b float32 [rows, width] (b None: no second term), float32
    arithmetic, rounded once."""
    _need(a, torch.float32, "a")
    assert a.is_contiguous() and a.shape[1] == out.shape[1] and out.is_contiguous()
    if b is not None:
        _need(b, torch.float32, "b")
        assert b.is_contiguous() and b.shape[1] == a.shape[1]
    _check(library().celeg_scaled_sum(_ptr(a), _ptr(b), _ptr(bias_a), scale_a, scale_b, _ptr(out), rows, a.shape[1],
                                      dtype_code(out.dtype), _stream()))


def softcap(logits: torch.Tensor, rows: int, cap: float) -> None:
    """logits[:rows] = cap * tanh(logits[:rows] / cap), in place (float32, contiguous)."""
    _need(logits, torch.float32, "logits")
    _check(library().celeg_softcap(_ptr(logits), rows * logits.shape[1], cap, _stream()))


SCAN_DELTA, SCAN_MLSTM, SCAN_RETENTION = 0, 1, 2
SCAN_MAX_DIM = 256


def recurrent_scan(mode: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, out: torch.Tensor,
                   state: torch.Tensor, slot_stride: int, span_begin: torch.Tensor, span_slot: torch.Tensor, spans: int,
                   heads: int, kv_heads: int, dim: int, vdim: int, q_scale: float) -> None:
    """The matrix-state recurrences of csrc/recurrent_scan.cu over the step's spans. q, k, v: float32 column
    views of [tokens, *] buffers (row strides are taken from them); gates float32 [tokens, 2*heads] (retention:
    [heads], each head's decay); out float32
    [tokens, heads*vdim]; ``state`` points at this part's floats inside slot 0."""
    for tensor in (q, k, v, gates, out, state):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert gates.is_contiguous() and out.is_contiguous() and out.shape[1] == heads * vdim
    assert gates.shape == (heads,) if mode == SCAN_RETENTION else gates.shape[1] == 2 * heads
    _check(library().celeg_recurrent_scan(mode, _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0),
                                          _ptr(gates), _ptr(out), _ptr(state), slot_stride, _ptr(span_begin),
                                          _ptr(span_slot), spans, heads, kv_heads, dim, vdim, q_scale, _stream()))


def retention_segmented(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, out: torch.Tensor,
                        state: torch.Tensor, slot_stride: int, span_begin: torch.Tensor, span_slot: torch.Tensor, spans: int,
                        tokens: int, heads: int, dim: int, vdim: int, q_scale: float, segment: int, max_segments: int,
                        float_scratch: torch.Tensor, int_scratch: torch.Tensor, identity: torch.Tensor) -> None:
    """The retention (mode SCAN_RETENTION of :func:`recurrent_scan`) with every span cut into segments of ``segment``
    tokens that are scanned side by side, the states at their starts carried from one to the next, and the carried
    share added to the read-outs (csrc/recurrent_scan.cu). Scratch: float32 [2 * max_segments * heads * dim * vdim],
    int32 [max_segments + spans + 2], ``identity`` = arange(max_segments) int32."""
    for tensor in (q, k, v, decay, out, state, float_scratch):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert out.is_contiguous() and out.shape[1] == heads * vdim and decay.shape == (heads,)
    assert max_segments >= tokens // segment + spans and identity.numel() >= max_segments
    assert float_scratch.numel() >= 2 * max_segments * heads * dim * vdim and int_scratch.numel() >= max_segments + spans + 2
    _check(library().celeg_retention_segmented(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(decay),
                                               _ptr(out), _ptr(state), slot_stride, _ptr(span_begin), _ptr(span_slot), spans,
                                               tokens, heads, dim, vdim, q_scale, segment, max_segments,
                                               _ptr(float_scratch), _ptr(int_scratch), _ptr(identity), _stream()))
    global LAUNCHES
    LAUNCHES += 4          # the plan, the scan, the carried states, their share of the read-outs (and a memset)


def recurrent_decode(mode: int, proj: torch.Tensor, offsets: Tuple[int, int, int, int, int, int],
                     conv_kernel: Optional[torch.Tensor], carried: Optional[torch.Tensor], taps: int, channels: int,
                     bias0: torch.Tensor, bias1: torch.Tensor, cap: float, norm_weight: torch.Tensor,
                     norm_per_head: bool, eps: float, unit_eps: float, state: torch.Tensor, slot_stride: int,
                     span_begin: torch.Tensor, span_slot: torch.Tensor, tokens: int, heads: int, kv_heads: int,
                     dim: int, vdim: int, q_scale: float, out: torch.Tensor) -> None:
    """A decoding step of a matrix-state mixer between its two projections, one launch (the delta rule's carried
    inputs: a second): row i of ``proj`` (float32) is the one token of request i. ``offsets``: columns of
    (q, k, v, output gate, first gate, second gate) in a row. See csrc/recurrent_scan.cu."""
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and out.is_contiguous() and out.shape[1] == heads * vdim
    _check(library().celeg_recurrent_decode(
        mode, _ptr(proj), proj.stride(0), *offsets, _ptr(conv_kernel), _ptr(carried), taps, channels, _ptr(bias0),
        _ptr(bias1), cap, _ptr(norm_weight), int(norm_per_head), eps, unit_eps, _ptr(state), slot_stride,
        _ptr(span_begin), _ptr(span_slot), tokens, heads, kv_heads, dim, vdim, q_scale, _ptr(out),
        dtype_code(out.dtype), _stream()))
    global LAUNCHES
    LAUNCHES += 1 if (mode == SCAN_DELTA and taps > 1) else 0


def mlstm_gates(pre_i: torch.Tensor, pre_f: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
                gates: torch.Tensor, tokens: int, heads: int) -> None:
    """gates[t] = [cap tanh((pre_i + bias_i) / cap) | logsigmoid(cap tanh((pre_f + bias_f) / cap))], float32."""
    assert pre_i.dtype == torch.float32 and pre_f.dtype == torch.float32 and pre_i.stride(0) == pre_f.stride(0)
    _check(library().celeg_mlstm_gates(_ptr(pre_i), _ptr(pre_f), pre_i.stride(0), _ptr(bias_i), _ptr(bias_f), cap,
                                       _ptr(gates), tokens, heads, _stream()))


def delta_prepare(proj: torch.Tensor, kernel: torch.Tensor, carried: torch.Tensor, slot_stride: int,
                  token_span: torch.Tensor, span_begin: torch.Tensor, span_slot: torch.Tensor, conv_out: torch.Tensor,
                  pre_beta: torch.Tensor, pre_a: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  gates: torch.Tensor, tokens: int, spans: int, channels: int, taps: int, qk_heads: int, dim: int,
                  heads: int, unit_eps: float) -> None:
    """The gated delta rule's token-parallel part: short causal convolutions (carried inputs before a span's
    start) with SiLU over the first ``channels`` columns of ``proj`` ([q | k | v]), unit q and k heads, beta and
    decay; then the carried inputs are moved on (a second launch). All float32."""
    assert proj.dtype == torch.float32 and conv_out.dtype == torch.float32 and conv_out.shape[1] == channels
    assert pre_beta.stride(0) == proj.stride(0) and pre_a.stride(0) == proj.stride(0)
    _check(library().celeg_delta_prepare(_ptr(proj), proj.stride(0), _ptr(kernel), _ptr(carried), slot_stride,
                                         _ptr(token_span), _ptr(span_begin), _ptr(span_slot), _ptr(conv_out),
                                         _ptr(pre_beta), _ptr(pre_a), _ptr(a_log), _ptr(dt_bias), _ptr(gates), tokens,
                                         spans, channels, taps, qk_heads, dim, heads, unit_eps, _stream()))
    global LAUNCHES
    LAUNCHES += 1 if taps > 1 else 0


GATE_SIGMOID, GATE_SILU = 0, 1


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], weight_per_head: bool,
                    out: torch.Tensor, tokens: int, heads: int, vdim: int, eps: float, gate_kind: int) -> None:
    """out = o / sqrt(mean_head(o^2) + eps) * weight * act(gate) per (token, head); o and gate float32; ``weight``
    None: no weight."""
    assert o.dtype == torch.float32 and gate.dtype == torch.float32 and o.is_contiguous() and gate.stride(-1) == 1
    _check(library().celeg_gated_head_norm(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), int(weight_per_head),
                                           _ptr(out), tokens, heads, vdim, eps, gate_kind, dtype_code(out.dtype),
                                           _stream()))


def retention_decode_raw(proj: torch.Tensor, offsets: Tuple[int, int, int], decay: torch.Tensor, state: torch.Tensor,
                         slot_stride: int, span_slot: torch.Tensor, tokens: int, heads: int, dim: int, vdim: int,
                         q_scale: float, input_act: int, raw_out: torch.Tensor) -> None:
    """A decoding step of the retention (S <- d S + k v^T, read-out S^T q) that leaves the read-outs as they are in
    ``raw_out`` (float32 [tokens, heads * vdim]); ``input_act``: an activation of q, k and v as they are read out of
    ``proj`` (a code of ACT_*, or -1). ``offsets``: columns of (q, k, v) in a row of ``proj`` (float32)."""
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and raw_out.dtype == torch.float32
    assert raw_out.is_contiguous() and raw_out.shape[1] == heads * vdim and decay.shape == (heads,)
    _check(library().celeg_retention_decode_raw(_ptr(proj), proj.stride(0), *offsets, _ptr(decay), _ptr(state),
                                                slot_stride, _ptr(span_slot), tokens, heads, dim, vdim, q_scale,
                                                input_act, _ptr(raw_out), _stream()))


# ------------------------------------------------------------- gated linear recurrent unit over channels
def lru_prepare(proj: torch.Tensor, bias: Optional[torch.Tensor], taps: torch.Tensor, conv_bias: Optional[torch.Tensor],
                carried: torch.Tensor, slot_stride: int, token_span: torch.Tensor, span_begin: torch.Tensor,
                span_slot: torch.Tensor, y_out: torch.Tensor, u_out: torch.Tensor, tokens: int, spans: int, width: int,
                n_taps: int) -> None:
    """Rows [y | x] of ``proj`` (float32): y_out = gelu_tanh(y + b_y), u_out = conv(x + b_x) + b_c over each span with
    the carried inputs before its start; then the carried inputs are moved on (a second launch)."""
    for tensor in (proj, taps, carried, y_out, u_out):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert y_out.is_contiguous() and u_out.is_contiguous() and y_out.shape[1] == width and u_out.shape[1] == width
    _check(library().celeg_lru_prepare(_ptr(proj), proj.stride(0), _ptr(bias), _ptr(taps), _ptr(conv_bias), _ptr(carried),
                                       slot_stride, _ptr(token_span), _ptr(span_begin), _ptr(span_slot), _ptr(y_out),
                                       _ptr(u_out), tokens, spans, width, n_taps, _stream()))
    global LAUNCHES
    LAUNCHES += 1 if n_taps > 1 else 0


def block_diagonal_product(x: torch.Tensor, x_parts: int, w: torch.Tensor, y: torch.Tensor, rows: int) -> None:
    """y[:rows, z n:(z + 1) n] = x[:rows, (z % x_parts) k:...] @ w[z]^T for every z; w float32 [batches, n, k]."""
    batches, n, k = w.shape
    for tensor in (x, w, y):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert w.is_contiguous()
    _check(library().celeg_block_diagonal_product(_ptr(x), x.stride(0), x_parts, _ptr(w), _ptr(y), y.stride(0), rows, n,
                                                  k, batches, _stream()))


def lru_scan(gates: torch.Tensor, u: torch.Tensor, gate_bias: Optional[torch.Tensor], lam: torch.Tensor, c: float,
             y: torch.Tensor, out: torch.Tensor, state: torch.Tensor, slot_stride: int, span_begin: torch.Tensor,
             span_slot: torch.Tensor, tokens: int, spans: int, width: int) -> None:
    """gates float32 [tokens, 2 * width] (the gates' sums; rewritten as decay | input), then S <- a S + b along every
    span with S in the slots, out = S y in the activation type (two launches)."""
    for tensor in (gates, u, lam, y, state):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert gates.is_contiguous() and gates.shape[1] == 2 * width and u.is_contiguous() and y.is_contiguous()
    assert out.is_contiguous() and out.shape[1] == width
    _check(library().celeg_lru_scan(_ptr(gates), _ptr(u), _ptr(gate_bias), _ptr(lam), c, _ptr(y), _ptr(out), _ptr(state),
                                    slot_stride, _ptr(span_begin), _ptr(span_slot), tokens, spans, width,
                                    dtype_code(out.dtype), _stream()))
    global LAUNCHES
    LAUNCHES += 1


def lru_decode(proj: torch.Tensor, bias: Optional[torch.Tensor], taps: torch.Tensor, conv_bias: Optional[torch.Tensor],
               carried: torch.Tensor, state: torch.Tensor, slot_stride: int, span_slot: torch.Tensor,
               gate_w: torch.Tensor, gate_bias: Optional[torch.Tensor], lam: torch.Tensor, c: float, out: torch.Tensor,
               tokens: int, width: int, n_taps: int, blocks: int) -> None:
    """One token a request: the whole unit between its two projections in one launch (csrc/linear_recurrence.cu)."""
    for tensor in (proj, taps, carried, state, gate_w, lam):
        assert tensor.dtype == torch.float32 and tensor.stride(-1) == 1
    assert gate_w.is_contiguous() and out.is_contiguous() and out.shape[1] == width
    _check(library().celeg_lru_decode(_ptr(proj), proj.stride(0), _ptr(bias), _ptr(taps), _ptr(conv_bias), _ptr(carried),
                                      _ptr(state), slot_stride, _ptr(span_slot), _ptr(gate_w), _ptr(gate_bias), _ptr(lam),
                                      c, _ptr(out), tokens, width, n_taps, blocks, dtype_code(out.dtype), _stream()))


# ------------------------------------------- depth average, latent attention, mixture of experts
def depth_average(stream: torch.Tensor, delta_a: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                  history: torch.Tensor, weights: torch.Tensor, index: int, n_rows: int,
                  norm_weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """X_(index+1) = stream (+ deltas) goes into ``history`` (float32 [entries, rows, width]; block 0 also stores its
    input as X_0), the stream becomes sum_j weights[j] X_j, and with ``norm_weight`` its RMSNorm is written to ``out``."""
    _need(stream, torch.float32, "stream")
    _need(history, torch.float32, "history")
    _need(weights, torch.float32, "weights")
    width = stream.shape[-1]
    assert history.shape[0] >= index + 2 and history.shape[-1] == width and weights.numel() == index + 2
    given = delta_a if delta_a is not None else delta_b
    act = out.dtype if out is not None else (given.dtype if given is not None else torch.float32)
    for delta in (delta_a, delta_b):
        assert delta is None or (delta.dtype == act and delta.shape[-1] == width and delta.is_contiguous())
    _check(library().celeg_depth_average(_ptr(stream), _ptr(delta_a), _ptr(delta_b), _ptr(history), history.stride(0),
                                         _ptr(weights), index, _ptr(norm_weight), _ptr(out), eps, n_rows, width,
                                         dtype_code(act), _stream()))


def latent_prepare(q: torch.Tensor, down: torch.Tensor, norm_weight: torch.Tensor, frequencies: torch.Tensor,
                   magnitude: float, eps: float, positions: torch.Tensor, token_span: torch.Tensor,
                   block_table: torch.Tensor, cache: torch.Tensor, page_tokens: int, query: torch.Tensor, tokens: int,
                   heads: int, dim: int, rot: int, rotated: int, rank: int, error_flag: torch.Tensor,
                   halves: bool = False) -> None:
    """The latent attention's token-parallel step (csrc/latent_attention.cu): the normalised latent vector and the
    rotated shared key part go to the token's place in ``cache`` (pages of [page_tokens, rank + rot]), every head's
    rotated query part to ``query[t, h, rank:]`` ([tokens, heads * (rank + rot)]). Of the ``rot`` dimensions of a
    rotated part the first ``rotated`` turn (pairs of neighbours, or with ``halves`` pairs (i, i + rotated / 2)), the
    rest pass unchanged."""
    assert q.dtype == down.dtype == cache.dtype == query.dtype and q.stride(-1) == 1 and down.stride(-1) == 1
    assert query.stride(-1) == 1 and cache.is_contiguous()
    _check(library().celeg_latent_prepare(
        _ptr(q), q.stride(0), _ptr(down), down.stride(0), _ptr(norm_weight), _ptr(frequencies), magnitude, eps,
        _ptr(positions), _ptr(token_span), _ptr(block_table), block_table.stride(0), _ptr(cache), cache.stride(0),
        page_tokens, _ptr(query), query.stride(0), tokens, heads, dim, rot, rotated, rank, int(halves), _ptr(error_flag),
        dtype_code(q.dtype), _stream()))


def head_project(x: torch.Tensor, in_head: int, matrix: torch.Tensor, contract_rows: bool, out: torch.Tensor,
                 out_head: int, tokens: int, heads: int, n: int, k: int, gate: Optional[torch.Tensor] = None,
                 gate_per_element: bool = False) -> None:
    """out[t, h * out_head + j] = sum_i x[t, h * in_head + i] M_h[i, j] (times sigmoid(gate[t, h])) for j < n, i < k.
    ``matrix`` is a stored projection [heads * rows, columns]: with ``contract_rows`` M_h[i, j] = matrix[h * k + i, j]
    (the sum runs over the head's rows), else M_h[i, j] = matrix[h * n + j, i] (over its columns). With
    ``gate_per_element`` the gate is [tokens, heads * n] and the factor sigmoid(gate[t, h * n + j])."""
    assert x.dtype == matrix.dtype == out.dtype and x.stride(-1) == 1 and out.stride(-1) == 1 and matrix.is_contiguous()
    columns = matrix.shape[1]
    if contract_rows:
        m_head, m_k, m_n = k * columns, columns, 1
    else:
        m_head, m_k, m_n = n * columns, 1, columns
    if gate is not None:
        assert gate.dtype == x.dtype and gate.stride(-1) == 1
    _check(library().celeg_head_project(_ptr(x), x.stride(0), in_head, _ptr(matrix), m_head, m_k, m_n, _ptr(out),
                                        out.stride(0), out_head, _ptr(gate), gate.stride(0) if gate is not None else 0,
                                        n if gate_per_element else 1, tokens, heads, n, k, dtype_code(x.dtype), _stream()))


def head_gate(values: torch.Tensor, head_width: int, gate: torch.Tensor, tokens: int, heads: int) -> None:
    """values[t, h * head_width + j] *= sigmoid(gate[t, h]), in place."""
    assert values.dtype == gate.dtype and values.stride(-1) == 1 and gate.stride(-1) == 1
    _check(library().celeg_head_gate(_ptr(values), values.stride(0), head_width, _ptr(gate), gate.stride(0), tokens,
                                     heads, dtype_code(values.dtype), _stream()))


MOE_TILE = 64


def moe_max_tiles(pairs: int, experts: int, tile_rows: int = MOE_TILE) -> int:
    """The most row tiles that ``pairs`` (token, choice) pairs can make, however they fall on the experts."""
    return pairs // tile_rows + min(pairs, experts)


def moe_route(logits: torch.Tensor, experts: int, correction: Optional[torch.Tensor], gate_column: Optional[int],
              chosen: torch.Tensor, weights: torch.Tensor, shared_gate: Optional[torch.Tensor], tokens: int,
              top: int, bias: Optional[torch.Tensor] = None) -> None:
    """From router logits (float32 [tokens, >= experts], a product with float32 sums; ``bias`` float32 [experts] is
    added to them first): chosen int32 [tokens, top] and weights float32 [tokens, top], the ``top`` experts with the
    largest softmax(logits[:, :experts]) + correction and their softmax scores divided by their sum (without a
    correction that is: the largest logits choose, and the weights are the softmax over the chosen logits alone);
    shared_gate float32 [tokens] = sigmoid(logits[:, gate_column])."""
    _need(chosen, torch.int32, "chosen")
    _need(weights, torch.float32, "weights")
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1 and logits.shape[-1] >= experts
    if bias is not None:
        _need(bias, torch.float32, "bias")
        assert bias.numel() >= experts
    _check(library().celeg_moe_route(_ptr(logits), logits.stride(0), _ptr(bias), _ptr(correction),
                                     -1 if gate_column is None else gate_column, _ptr(chosen), _ptr(weights),
                                     _ptr(shared_gate), tokens, experts, top, _stream()))


def moe_group(chosen: torch.Tensor, tokens: int, experts: int, top: int, place_of_pair: torch.Tensor,
              source_of_place: torch.Tensor, table: torch.Tensor, tile_rows: int = MOE_TILE) -> None:
    """Orders the (token, choice) pairs by expert: place_of_pair [tokens * top], source_of_place [tokens * top] (the
    token of each place) and the tile table int32 [4 + 3 * moe_max_tiles] (count, then (expert, first place, rows) for
    runs of at most ``tile_rows`` places of one expert)."""
    assert table.numel() >= 4 + 3 * moe_max_tiles(tokens * top, experts, tile_rows)
    _check(library().celeg_moe_group(_ptr(chosen), tokens, experts, top, tile_rows, _ptr(place_of_pair),
                                     _ptr(source_of_place), _ptr(table), _stream()))


def moe_gather_rows(x: torch.Tensor, source: torch.Tensor, out: torch.Tensor, places: int) -> None:
    """out[place] = x[source[place]]: the step's rows in the order of the experts that chose them."""
    assert x.dtype == out.dtype and x.stride(-1) == 1 and out.stride(-1) == 1 and x.shape[-1] == out.shape[-1]
    _check(library().celeg_moe_gather_rows(_ptr(x), x.stride(0), _ptr(source), _ptr(out), out.stride(0), places,
                                           x.shape[-1], dtype_code(x.dtype), _stream()))


def expert_product_tcgen05_supported(x: torch.Tensor, weights: torch.Tensor) -> bool:
    """Shapes the grouped tcgen05 product takes: bfloat16, k and the row strides multiples of 8, 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and weights.dtype == torch.bfloat16 and weights.is_contiguous()
            and weights.shape[2] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(-1) == 1
            and x.data_ptr() % 16 == 0 and weights.data_ptr() % 16 == 0)


def expert_product_tcgen05(x: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, table: torch.Tensor,
                           max_tiles: int, activation: int, error_flag: torch.Tensor, wide_tiles: int = -1) -> None:
    """out[place] = act(x[place] @ weights[expert of the place]^T) on tcgen05 over a tile table of 128-row tiles;
    ``x`` holds the rows in the order of their places. ``activation``: a code of ACT_* or -1. ``wide_tiles``: output
    tiles of 256 columns (1) or 128 (0); -1: chosen from the shape."""
    _, n, k = weights.shape
    assert out.dtype == torch.bfloat16 and out.stride(-1) == 1 and out.shape[-1] == n and x.shape[-1] == k
    _check(library().celeg_gemm_tcgen05_grouped(_ptr(x), x.stride(0), x.shape[0], _ptr(weights), weights.stride(1),
                                                weights.shape[0], _ptr(out), out.stride(0), _ptr(table), max_tiles, n, k,
                                                TC_STORE if activation < 0 else TC_ACTIVATION + activation,
                                                _ptr(error_flag), wide_tiles, _stream()))


def expert_product(x: torch.Tensor, source: Optional[torch.Tensor], weights: torch.Tensor, out: torch.Tensor,
                   table: torch.Tensor, max_tiles: int, activation: int) -> None:
    """out[place] = act(x[source[place]] @ weights[expert of the place]^T) over the tile table; ``weights``
    [experts, n, k]; ``activation`` a code of ACT_* or -1."""
    assert x.dtype == weights.dtype == out.dtype and weights.is_contiguous() and x.stride(-1) == 1 and out.stride(-1) == 1
    _, n, k = weights.shape
    _check(library().celeg_expert_product(_ptr(x), x.stride(0), _ptr(source), _ptr(weights), weights.stride(0),
                                          weights.stride(1), _ptr(out), out.stride(0), _ptr(table), max_tiles, n, k,
                                          activation, dtype_code(x.dtype), _stream()))


def expert_rows(x: torch.Tensor, pairs_per_row: int, chosen: torch.Tensor, weights: torch.Tensor, out: torch.Tensor,
                pairs: int, activation: int) -> None:
    """out[pair] = act(x[pair // pairs_per_row] @ weights[chosen[pair]]^T) for few pairs (the weights stream once)."""
    assert x.dtype == weights.dtype == out.dtype and weights.is_contiguous() and x.stride(-1) == 1 and out.stride(-1) == 1
    _, n, k = weights.shape
    _check(library().celeg_expert_rows(_ptr(x), x.stride(0), pairs_per_row, _ptr(chosen), _ptr(weights),
                                       weights.stride(0), weights.stride(1), _ptr(out), out.stride(0), pairs, n, k,
                                       activation, dtype_code(x.dtype), _stream()))


def moe_combine(expert_out: torch.Tensor, place_of_pair: Optional[torch.Tensor], weights: torch.Tensor,
                shared: Optional[torch.Tensor], shared_gate: Optional[torch.Tensor], y: torch.Tensor, tokens: int,
                top: int) -> None:
    """y[t] = sum_k weights[t, k] expert_out[place_of_pair[t * top + k]] (+ shared_gate[t] shared[t])."""
    width = y.shape[-1]
    assert expert_out.dtype == y.dtype and expert_out.stride(-1) == 1 and y.is_contiguous()
    assert shared is None or (shared.dtype == y.dtype and shared.is_contiguous() and shared.shape[-1] == width)
    _check(library().celeg_moe_combine(_ptr(expert_out), expert_out.stride(0), _ptr(place_of_pair), _ptr(weights),
                                       _ptr(shared), _ptr(shared_gate), _ptr(y), tokens, width, top,
                                       dtype_code(y.dtype), _stream()))
