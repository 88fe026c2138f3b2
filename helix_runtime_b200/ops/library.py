"""Python face of the CUDA kernel library: one function per entry point.

The functions take ``torch`` tensors, check dtypes and contiguity, and pass raw
device pointers plus the current CUDA stream to the C interface.  Nothing here
computes: there is no CPU path and no library stand-in.  If the shared object
cannot be built or loaded the import of this module's :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Sequence, Tuple

import torch

from ..csrc import build as _build

HX_F32 = 0
HX_BF16 = 1

EPI_STORE = 0        # compute dtype out
EPI_STORE_F32 = 1    # float32 out
EPI_ADD_F32 = 2      # float32 out += product
EPI_SWIGLU = 3       # tensor-core kernel only
EPI_GEGLU_TANH = 5   # tensor-core kernel only: gelu_tanh(gate) * up

GATE_SILU = 0        # what a gated feed-forward passes its gate through
GATE_GELU_TANH = 1
GATE_RELU = 2             # max(gate, 0) * up
GATE_CLAMPED_SIGMOID = 3  # g = min(gate, L), u = clamp(up, -L, L): g * sigmoid(1.702 g) * (u + 1)
GATE_ACTIVATIONS = {"silu": GATE_SILU, "gelu_tanh": GATE_GELU_TANH, "relu": GATE_RELU,
                    "clamped_sigmoid": GATE_CLAMPED_SIGMOID}

FLAG_BAD_TOKEN = 1
FLAG_BAD_PAGE = 2
FLAG_WAIT_TIMEOUT = 4
FLAG_NONFINITE = 8
FLAG_BAD_POSITION = 16

_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_float = ctypes.c_float
_c_longlong = ctypes.c_longlong

_lock = threading.Lock()
_library: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def _declare(library: ctypes.CDLL) -> None:
    library.hx_last_error.restype = ctypes.c_char_p
    library.hx_last_error.argtypes = []
    library.hx_abi_version.restype = _c_int
    library.hx_sm_count.restype = _c_int
    library.hx_sm_count.argtypes = []
    library.hx_embed.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_embed_scaled.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                        _c_float, _c_ptr, _c_ptr]
    library.hx_add_rows.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr]
    library.hx_layernorm.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int,
                                     _c_float, _c_ptr]
    library.hx_gated_activation.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_ptr]
    library.hx_short_conv_append.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_sigmoid_gate.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                        _c_ptr, _c_int, _c_int, _c_ptr]
    library.hx_paged_attention_kept.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_rmsnorm.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_float, _c_ptr]
    library.hx_swiglu.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_rope_append.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
        _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_ptr, _c_ptr, _c_int, _c_ptr]
    library.hx_gemm_simt.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_ptr]
    library.hx_gemm_tc.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                   _c_ptr]
    library.hx_gemm_tc_gated.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr,
                                         _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr,
                                         _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_gemm_tc_gated.restype = _c_int
    library.hx_gemm_tc_rope_append.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_gemm_tc_rope_append.restype = _c_int
    library.hx_gemm_tc_rope_append_min_tokens.argtypes = []
    library.hx_gemm_tc_rope_append_min_tokens.restype = _c_int
    library.hx_gemm_tc_supports.argtypes = [_c_int] * 5
    library.hx_gemm_tc_token_tile.argtypes = [_c_int]
    library.hx_paged_attention.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_prefill_attention.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr]
    library.hx_prefill_attention.restype = _c_int
    library.hx_prefill_attention_supports.argtypes = [_c_int, _c_int]
    library.hx_prefill_attention_supports.restype = _c_int
    library.hx_prefill_attention_windowed.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int,
        _c_ptr, _c_ptr]
    library.hx_prefill_attention_windowed.restype = _c_int
    library.hx_prefill_attention_packed.argtypes = library.hx_prefill_attention_windowed.argtypes
    library.hx_prefill_attention_packed.restype = _c_int
    library.hx_prefill_attention_packed_tokens.argtypes = [_c_int, _c_int]
    library.hx_prefill_attention_packed_tokens.restype = _c_int
    library.hx_prefill_attention_tc_windowed.argtypes = \
        library.hx_prefill_attention_windowed.argtypes
    library.hx_prefill_attention_tc_windowed.restype = _c_int
    library.hx_prefill_attention_tc.argtypes = library.hx_prefill_attention.argtypes
    library.hx_prefill_attention_tc.restype = _c_int
    library.hx_prefill_attention_tc_supports.argtypes = [_c_int, _c_int]
    library.hx_prefill_attention_tc_supports.restype = _c_int
    library.hx_paged_attention_scratch_floats.restype = ctypes.c_longlong
    library.hx_paged_attention_scratch_floats.argtypes = [_c_int] * 4
    library.hx_paged_attention_scratch_floats_for.restype = ctypes.c_longlong
    library.hx_paged_attention_scratch_floats_for.argtypes = [_c_int] * 7
    library.hx_argmax.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_sample.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr]
    library.hx_set_dependent_launch.argtypes = [_c_int]
    library.hx_set_dependent_launch.restype = None
    library.hx_launch_count.restype = ctypes.c_longlong
    library.hx_launch_count.argtypes = []
    library.hx_feed_tokens.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr]
    library.hx_feed_tokens.restype = _c_int
    library.hx_bounded_wait_check.argtypes = [_c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_bounded_wait_check.restype = _c_int
    library.hx_streams_spread.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_streams_read_norm.argtypes = [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr,
                                             _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr]
    library.hx_streams_write.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                         _c_int, _c_ptr]
    library.hx_scaled_sum.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_add_bias.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr]
    library.hx_biased_activation.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                             _c_int, _c_int, _c_float, _c_float, _c_ptr]
    library.hx_causal_filter.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr,
                                         _c_ptr, _c_longlong, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                         _c_ptr, _c_ptr, _c_ptr]
    library.hx_scan_state_floats.argtypes = [_c_int, _c_int]
    library.hx_scan_state_floats.restype = _c_int
    library.hx_state_space_scan.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int,
                                            _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_longlong, _c_int, _c_ptr,
                                            _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_ptr]
    library.hx_token_shift.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_longlong,
                                       _c_ptr, _c_longlong, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                       _c_ptr]
    library.hx_outer_product_scan.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int,
                                              _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_longlong,
                                              _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                              _c_int, _c_ptr]
    library.hx_gated_group_norm.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr,
                                            _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr]
    library.hx_norm_rotary_append.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_rotate_back.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                       _c_int, _c_int, _c_ptr]
    _c_double_ptr = _c_ptr
    library.hx_linear_state_scan.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_double_ptr, _c_int, _c_int, _c_int,
        _c_float, _c_float, _c_float, _c_ptr, _c_longlong, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_gated_residual_add.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int,
                                              _c_ptr]
    library.hx_join_rows.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_route_top.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr,
                                     _c_ptr]
    library.hx_expert_gate_up.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                          _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_expert_down.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                       _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_expert_tile_bound.argtypes = [_c_int, _c_int, _c_int]
    library.hx_expert_rows.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_expert_gather.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                         _c_int, _c_int, _c_ptr]
    library.hx_expert_combine.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                          _c_int, _c_int, _c_ptr]
    library.hx_gemm_tc_grouped.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                           _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                           _c_int, _c_ptr, _c_ptr, _c_ptr]
    for name in ("hx_expert_tile_bound", "hx_expert_rows", "hx_expert_gather",
                 "hx_expert_combine", "hx_gemm_tc_grouped"):
        getattr(library, name).restype = _c_int
    library.hx_latent_prepare.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr,
        _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
        _c_ptr]
    library.hx_latent_queries.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr]
    library.hx_biased_gated_activation.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                                   _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr]
    library.hx_route_top_ruled.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                           _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_expert_gate_up_limited.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                  _c_float, _c_ptr]
    library.hx_expert_identity_add.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                               _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_gemm_tc_grouped_gated.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int,
                                                 _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                                 _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr,
                                                 _c_ptr]
    library.hx_paged_attention_biased.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr]
    library.hx_prefill_attention_biased.argtypes = [
        *library.hx_prefill_attention_windowed.argtypes[:-2], _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr]
    library.hx_prefill_attention_tc_biased.argtypes = [
        *library.hx_prefill_attention_windowed.argtypes[:-2], _c_ptr, _c_ptr, _c_ptr, _c_ptr]
    library.hx_prefill_attention_tc_biased.restype = _c_int
    library.hx_norm_residual_add.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_float, _c_float, _c_ptr,
                                             _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_biased_normed_rows.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_float,
        _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
        _c_ptr, _c_ptr]
    library.hx_head_gate.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_token_gate.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                      _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    for name in ("hx_biased_gated_activation", "hx_route_top_ruled", "hx_expert_gate_up_limited",
                 "hx_expert_identity_add", "hx_gemm_tc_grouped_gated", "hx_paged_attention_biased",
                 "hx_prefill_attention_biased", "hx_norm_residual_add", "hx_biased_normed_rows",
                 "hx_head_gate", "hx_token_gate"):
        getattr(library, name).restype = _c_int
    library.hx_head_products.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                         _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    for name in ("hx_linear_state_scan", "hx_gated_residual_add", "hx_join_rows", "hx_route_top",
                 "hx_expert_gate_up", "hx_expert_down", "hx_latent_prepare", "hx_latent_queries",
                 "hx_head_products"):
        getattr(library, name).restype = _c_int
    for name in ("hx_streams_spread", "hx_streams_read_norm", "hx_streams_write", "hx_scaled_sum",
                 "hx_add_bias", "hx_biased_activation", "hx_causal_filter", "hx_state_space_scan",
                 "hx_token_shift", "hx_outer_product_scan", "hx_gated_group_norm",
                 "hx_norm_rotary_append", "hx_rotate_back"):
        getattr(library, name).restype = _c_int
    for name in ("hx_embed", "hx_rmsnorm", "hx_swiglu", "hx_rope_append", "hx_gemm_simt",
                 "hx_gemm_tc", "hx_gemm_tc_supports", "hx_gemm_tc_token_tile",
                 "hx_paged_attention", "hx_argmax", "hx_sample", "hx_embed_scaled",
                 "hx_add_rows", "hx_layernorm", "hx_gated_activation", "hx_short_conv_append",
                 "hx_sigmoid_gate", "hx_paged_attention_kept"):
        getattr(library, name).restype = _c_int


def lib() -> ctypes.CDLL:
    """Load (building at first use) the kernel library; raise if that is impossible."""
    global _library
    if _library is None:
        with _lock:
            if _library is None:
                path = _build.build()
                library = ctypes.CDLL(path)
                _declare(library)
                _library = library
    return _library


_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device, asked of the device once."""
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        count = int(lib().hx_sm_count())
        if count <= 0:
            raise KernelError(lib().hx_last_error().decode("utf-8", "replace"))
        _sm_counts[device] = count
    return _sm_counts[device]


def library_file() -> str:
    lib()
    return _build.library_path()


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(lib().hx_last_error().decode("utf-8", "replace") or f"kernel error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return HX_F32
    if dtype == torch.bfloat16:
        return HX_BF16
    raise KernelError(f"unsupported compute dtype {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Every launch asks for it, and a step has hundreds of
    launches: the direct accessor costs a fraction of a microsecond where building a
    ``torch.cuda.Stream`` object costs fourteen (measured: 3.6 ms of a 2,048-token step's
    10 ms of host time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need(tensor: torch.Tensor, dtype: torch.dtype, name: str, last_dim_contiguous: bool = True) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if last_dim_contiguous and tensor.dim() > 0 and tensor.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """out[t] (float32) = table[ids[t]] * scale."""
    _need(ids, torch.int32, "ids")
    _need(out, torch.float32, "out")
    vocab, hidden = table.shape
    tokens = ids.shape[0]
    assert table.is_contiguous() and out.is_contiguous() and out.shape[1] == hidden
    _check(lib().hx_embed_scaled(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                 out.data_ptr(), tokens, hidden, vocab, float(scale),
                                 _ptr(status), _stream()))


def add_rows(x: torch.Tensor, y: torch.Tensor, tokens: int) -> None:
    """x[:tokens] += y[:tokens]; both float32 with the same row width."""
    _need(x, torch.float32, "x")
    _need(y, torch.float32, "y")
    assert x.is_contiguous() and y.is_contiguous() and x.shape[1] == y.shape[1]
    assert x.shape[0] >= tokens and y.shape[0] >= tokens
    _check(lib().hx_add_rows(x.data_ptr(), y.data_ptr(), tokens, x.shape[1], _stream()))


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
              out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x[r'] - mean) / sqrt(var + eps) * weight + bias with r' = rows[r] or r and var
    the mean of the squared deviations; x, weight and bias float32."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "weight")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    assert x.is_contiguous() and out.is_contiguous()
    hidden = x.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
        assert rows.shape[0] >= n_rows
    else:
        assert x.shape[0] >= n_rows
    _check(lib().hx_layernorm(x.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(),
                              dtype_code(out.dtype), _ptr(rows), n_rows, hidden, float(eps),
                              _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight; x and weight float32."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "weight")
    assert x.is_contiguous() and out.is_contiguous()
    hidden = x.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
        assert rows.shape[0] >= n_rows
    else:
        assert x.shape[0] >= n_rows
    _check(lib().hx_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                            _ptr(rows), n_rows, hidden, float(eps), _stream()))


def swiglu(gate_up: torch.Tensor, act: torch.Tensor, zero_input: bool = False,
           activation: int = GATE_SILU, gate_bias: Optional[torch.Tensor] = None,
           up_bias: Optional[torch.Tensor] = None, limit: float = 0.0) -> None:
    """act[t, i] = f(gate_up[t, i] + gate_bias[i]) * (gate_up[t, I + i] + up_bias[i]) with f =
    silu (or ``activation``: any of GATE_ACTIVATIONS; the clamped form takes ``limit``);
    gate_up and the optional biases float32, act compute dtype.
    ``zero_input`` clears what was read (gate_up is a split-K accumulator)."""
    tokens, intermediate = act.shape
    _need(gate_up, torch.float32, "gate_up")
    assert act.is_contiguous()
    for bias in (gate_bias, up_bias):
        if bias is not None:
            _need(bias, torch.float32, "bias")
            assert bias.numel() == intermediate
    _check(lib().hx_biased_gated_activation(
        gate_up.data_ptr(), _ptr(gate_bias), _ptr(up_bias), act.data_ptr(), dtype_code(act.dtype),
        tokens, intermediate, gate_up.stride(0), 1 if zero_input else 0, int(activation),
        float(limit), _stream()))


def short_conv_append(raw: Optional[torch.Tensor], accum: Optional[torch.Tensor],
                      out: torch.Tensor, filter_taps: torch.Tensor, state: Optional[torch.Tensor],
                      positions: torch.Tensor, token_request: torch.Tensor,
                      request_slot: torch.Tensor, request_start: torch.Tensor,
                      block_tables: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                      v_cache: Optional[torch.Tensor], tokens: int, heads: int, kv_heads: int,
                      head_dim: int, total: int, page_size: int, num_pages: int,
                      status: torch.Tensor) -> None:
    """Causal filter over time on the columns ``[q heads | k heads | v heads]`` of the
    projected rows (``raw`` in the compute dtype, or ``accum``: their float32 sums, which are
    NOT cleared), ``filter_taps`` float32 ``[channels, taps]`` with the last tap on the token
    itself; ``state`` ``[slot, taps - 1, channels]`` holds each request's last projected values
    and is updated.  Queries go to ``out``; keys and values to their pages when ``k_cache`` is
    given, else to ``out`` too.  Columns from ``channels`` to ``total`` are copied to ``out``."""
    _need(filter_taps, torch.float32, "filter_taps")
    channels = (heads + 2 * kv_heads) * head_dim
    taps = filter_taps.shape[1]
    assert filter_taps.is_contiguous() and filter_taps.shape[0] == channels
    if taps > 1:
        assert state is not None and state.dtype == out.dtype and state.is_contiguous()
        assert tuple(state.shape[1:]) == (taps - 1, channels)
    if raw is not None:
        assert raw.dtype == out.dtype and raw.stride(-1) == 1
    if accum is not None:
        _need(accum, torch.float32, "accum")
    write = k_cache is not None
    _check(lib().hx_short_conv_append(
        _ptr(raw), 0 if raw is None else raw.stride(0), _ptr(accum),
        0 if accum is None else accum.stride(0), out.data_ptr(), out.stride(0),
        dtype_code(out.dtype), filter_taps.data_ptr(), _ptr(state), taps, positions.data_ptr(),
        token_request.data_ptr(), request_slot.data_ptr(), request_start.data_ptr(),
        _ptr(block_tables) if write else None, block_tables.stride(0) if write else 0,
        _ptr(k_cache), _ptr(v_cache), 1 if write else 0, tokens, heads, kv_heads, head_dim, total,
        page_size, num_pages, _ptr(status), _stream()))


def sigmoid_gate(context: torch.Tensor, gate: torch.Tensor, tokens: int, width: int,
                 clear: Optional[torch.Tensor] = None) -> None:
    """context[:tokens, :width] *= sigmoid(gate[:tokens, :width]) (float32 product, one
    rounding).  ``clear``: a float32 accumulator whose first ``tokens`` rows are zeroed."""
    assert context.dtype == gate.dtype and context.stride(-1) == 1 and gate.stride(-1) == 1
    if clear is not None:
        _need(clear, torch.float32, "clear")
    _check(lib().hx_sigmoid_gate(context.data_ptr(), context.stride(0), gate.data_ptr(),
                                 gate.stride(0), dtype_code(context.dtype), tokens, width,
                                 _ptr(clear), 0 if clear is None else clear.stride(0),
                                 0 if clear is None else clear.shape[1], _stream()))


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, token_request: torch.Tensor,
                request_table_row: torch.Tensor, block_tables: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                cos_table: torch.Tensor, sin_table: torch.Tensor, tokens: int, heads: int,
                kv_heads: int, head_dim: int, rotary_dim: int, pairing: int, page_size: int,
                num_pages: int, status: torch.Tensor,
                accum: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k of ``qkv[:tokens]`` in place and write k, v into their pages.  With
    ``accum`` (float32 ``[rows, width]``) the projection is read from there instead, rounded
    to the storage type, and ``accum`` is cleared."""
    write = k_cache is not None
    _check(lib().hx_rope_append(
        qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), positions.data_ptr(),
        token_request.data_ptr(), request_table_row.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0), _ptr(k_cache), _ptr(v_cache), 1 if write else 0,
        cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0], tokens, heads, kv_heads,
        head_dim, rotary_dim, pairing, page_size, num_pages, _ptr(status), _ptr(accum),
        0 if accum is None else accum.stride(0), _stream()))


def gemm_tc_supports(tokens: int, features: int, depth: int, ldx: int, ldw: int) -> bool:
    return bool(lib().hx_gemm_tc_supports(tokens, features, depth, ldx, ldw))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tokens: int, epilogue: int) -> None:
    """out[:tokens] (op)= x[:tokens] @ w.T on the CUDA cores (float32 or bfloat16 storage)."""
    assert x.dtype == w.dtype and x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    features, depth = w.shape
    _check(lib().hx_gemm_simt(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                              out.stride(0), dtype_code(x.dtype), tokens, features, depth, epilogue,
                              _stream()))


WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH = 128, 64


def tile_weights(matrix: torch.Tensor) -> torch.Tensor:
    """``[rows, depth]`` -> ``[ceil(rows / 128), ceil(depth / 64), 128, 64]``, zero padded:
    every [128 x 64] box the tensor-core product loads becomes 16 contiguous kilobytes."""
    rows, depth = matrix.shape
    row_tiles = -(-rows // WEIGHT_TILE_ROWS)
    k_tiles = -(-depth // WEIGHT_TILE_DEPTH)
    padded = torch.zeros((row_tiles * WEIGHT_TILE_ROWS, k_tiles * WEIGHT_TILE_DEPTH),
                         dtype=matrix.dtype, device=matrix.device)
    padded[:rows, :depth] = matrix
    return padded.view(row_tiles, WEIGHT_TILE_ROWS, k_tiles, WEIGHT_TILE_DEPTH) \
        .permute(0, 2, 1, 3).contiguous()


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tokens: int, features: int,
            epilogue: int, status: torch.Tensor, up_row_offset: int = 0, k_splits: int = 1,
            weight_shape: Optional[Tuple[int, int]] = None, gate_activation: Optional[int] = None,
            gate_limit: float = 0.0, gate_bias: Optional[torch.Tensor] = None,
            up_bias: Optional[torch.Tensor] = None) -> None:
    """out[:tokens, :features] (op)= x[:tokens] @ w.T on the tensor cores (bfloat16).  ``w``
    is the matrix ``[rows, depth]`` or its tiles from :func:`tile_weights` (then
    ``weight_shape`` gives rows and depth).  With ``gate_activation`` (any of GATE_ACTIVATIONS)
    the epilogue is that gated activation of ``[gate; up]`` whatever ``epilogue`` says, with the
    optional float32 biases ``gate_bias`` and ``up_bias`` ``[features]`` added first."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    tiled = w.dim() == 4
    if tiled:
        if weight_shape is None:
            raise ValueError("tiled weights need weight_shape=(rows, depth)")
        rows, depth = weight_shape
        if tuple(w.shape) != (-(-rows // WEIGHT_TILE_ROWS), -(-depth // WEIGHT_TILE_DEPTH),
                              WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH) or not w.is_contiguous():
            raise ValueError(f"tiles of shape {tuple(w.shape)} do not hold a {rows} x {depth} matrix")
        ldw = 0
    else:
        rows, depth = w.shape
        ldw = w.stride(0)
    if gate_activation is not None:
        for bias in (gate_bias, up_bias):
            if bias is not None:
                _need(bias, torch.float32, "bias")
                assert bias.numel() == features and bias.is_contiguous()
        _check(lib().hx_gemm_tc_gated(x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), ldw,
                                      rows, out.data_ptr(), out.stride(0), tokens, features, depth,
                                      int(gate_activation), float(gate_limit), _ptr(gate_bias),
                                      _ptr(up_bias), up_row_offset, 1 if tiled else 0,
                                      status.data_ptr(), _stream()))
        return
    _check(lib().hx_gemm_tc(x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), ldw, rows,
                            out.data_ptr(), out.stride(0), tokens, features, depth, epilogue,
                            up_row_offset, k_splits, 1 if tiled else 0, status.data_ptr(),
                            _stream()))


def gemm_tc_rope_append_min_tokens() -> int:
    return int(lib().hx_gemm_tc_rope_append_min_tokens())


def gemm_tc_rope_append(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, tokens: int,
                        positions: torch.Tensor, token_request: torch.Tensor,
                        request_table_row: torch.Tensor, block_tables: Optional[torch.Tensor],
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                        cos_table: torch.Tensor, sin_table: torch.Tensor, heads: int,
                        kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                        num_pages: int, status: torch.Tensor,
                        weight_shape: Optional[Tuple[int, int]] = None) -> None:
    """The fused QKV product of a prompt portion (more than 64 tokens, bfloat16) with the
    rotary encoding and the cache append as its epilogue: ``qkv[:tokens, :heads * head_dim]``
    receives the rotated queries (the key and value columns of ``qkv`` are NOT written), keys
    (rotated) and values go to their pages.  Adjacent pairs; ``w`` as for :func:`gemm_tc`."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(qkv, torch.bfloat16, "qkv")
    tiled = w.dim() == 4
    if tiled:
        if weight_shape is None:
            raise ValueError("tiled weights need weight_shape=(rows, depth)")
        rows, depth = weight_shape
        if tuple(w.shape) != (-(-rows // WEIGHT_TILE_ROWS), -(-depth // WEIGHT_TILE_DEPTH),
                              WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH) or not w.is_contiguous():
            raise ValueError(f"tiles of shape {tuple(w.shape)} do not hold a {rows} x {depth} matrix")
        ldw = 0
    else:
        rows, depth = w.shape
        ldw = w.stride(0)
    write = k_cache is not None
    _check(lib().hx_gemm_tc_rope_append(
        x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), ldw, rows, qkv.data_ptr(),
        qkv.stride(0), tokens, depth, 1 if tiled else 0, positions.data_ptr(),
        token_request.data_ptr(), request_table_row.data_ptr(),
        _ptr(block_tables) if write else None,
        block_tables.stride(0) if write else 0, _ptr(k_cache), _ptr(v_cache),
        cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0], heads, kv_heads, head_dim,
        rotary_dim, page_size, num_pages, status.data_ptr(), _stream()))


def attention_scratch_floats(tokens: int, heads: int, head_dim: int, max_splits: int,
                             dtype: Optional[torch.dtype] = None, page_size: int = 0,
                             window: int = 0) -> int:
    """Floats of scratch ``paged_attention`` needs; with ``dtype`` and ``page_size`` given, what
    the kernel that will run for them needs (the streaming kernel: a fixed few megabytes)."""
    if dtype is None:
        return int(lib().hx_paged_attention_scratch_floats(tokens, heads, head_dim, max_splits))
    return int(lib().hx_paged_attention_scratch_floats_for(
        dtype_code(dtype), tokens, heads, head_dim, page_size, window, max_splits))


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_request: torch.Tensor,
                    request_table_row: torch.Tensor, block_tables: torch.Tensor, out: torch.Tensor,
                    partial: Optional[torch.Tensor], tokens: int, heads: int, kv_heads: int,
                    head_dim: int, page_size: int, num_pages: int, window: int, scale: float,
                    split_keys: int, max_splits: int, status: torch.Tensor,
                    request_start: Optional[torch.Tensor] = None, skip_query_len: int = 0,
                    arrivals: Optional[torch.Tensor] = None, keep_first: int = 0,
                    sinks: Optional[torch.Tensor] = None,
                    slopes: Optional[torch.Tensor] = None) -> None:
    """out[t, h*D:(h+1)*D] = attention of query (t, h) over its request's pages.  With
    ``skip_query_len > 0`` tokens of requests that bring at least that many tokens are left
    out (the tensor-core kernel takes them).  With a window, keys at positions below
    ``keep_first`` stay visible behind it.  The call needs scratch, made here when it is
    not given: ``partial`` (float32, :func:`attention_scratch_floats` elements) and
    ``arrivals`` (int32, one counter per (token, head), zero on entry; the kernel leaves it
    zero).  ``sinks`` (float32 ``[heads]``): the softmax's denominator also holds
    ``exp(sinks[h])``, a term without key or value.  ``slopes`` (float32 ``[heads]``): the score
    of key ``j`` for the query at position ``i`` is lowered by ``slopes[h] * (i - j)``."""
    for per_head in (sinks, slopes):
        if per_head is not None:
            _need(per_head, torch.float32, "sinks and slopes")
            assert per_head.numel() == heads
    if arrivals is None:
        arrivals = torch.zeros(max(1, tokens * heads), dtype=torch.int32, device=q.device)
    if partial is None:
        partial = torch.empty(attention_scratch_floats(tokens, heads, head_dim, max_splits,
                                                       q.dtype, page_size, window),
                              dtype=torch.float32, device=q.device)
    _check(lib().hx_paged_attention_biased(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), dtype_code(q.dtype),
        positions.data_ptr(), token_request.data_ptr(), request_table_row.data_ptr(),
        block_tables.data_ptr(), block_tables.stride(0), _ptr(request_start), skip_query_len,
        out.data_ptr(), out.stride(0),
        _ptr(partial), _ptr(arrivals), tokens, heads, kv_heads, head_dim, page_size, num_pages, window,
        int(keep_first), float(scale), split_keys, max_splits, _ptr(sinks), _ptr(slopes),
        _ptr(status), _stream()))


PREFILL_TILE_ROWS = 64        # query rows of a CTA of the ``mma.sync`` prompt kernel
PREFILL_TILE_ROWS_TC = 256    # and of the tcgen05 prompt kernel


def prefill_attention_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().hx_prefill_attention_supports(head_dim, page_size))


def prefill_attention_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().hx_prefill_attention_tc_supports(head_dim, page_size))


def prefill_attention_packed_tokens(heads: int, kv_heads: int) -> int:
    """Tokens a query tile of the packed kernel holds; 0 where it does not apply."""
    return int(lib().hx_prefill_attention_packed_tokens(heads, kv_heads))


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      request_start: torch.Tensor, request_context: torch.Tensor,
                      request_table_row: torch.Tensor, block_tables: torch.Tensor,
                      out: torch.Tensor, requests: int, tile_bound: int, heads: int,
                      kv_heads: int, head_dim: int, page_size: int, num_pages: int, scale: float,
                      min_query_len: int, status: torch.Tensor,
                      tensor_memory: Optional[bool] = None,
                      query_lengths: Optional[Sequence[int]] = None, window: int = 0,
                      keep_first: int = 0, packed: bool = False,
                      sinks: Optional[torch.Tensor] = None,
                      slopes: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention (bfloat16) of every request that brings at least
    ``min_query_len`` tokens; ``tile_bound`` bounds the number of query tiles of 64 tokens
    (the tensor-memory kernel, whose tiles hold 256 tokens, needs no more).  A CTA that finds
    no tile leaves at once, but it holds an SM's shared memory while it looks, so a caller
    that knows the requests' token counts on the host passes them (``query_lengths``) and the
    grid is exactly the tiles there are.
    ``tensor_memory``: take the tcgen05 kernel (scores, probabilities and output in tensor
    memory; pages of at least 16 keys) or the ``mma.sync`` kernel; default: tcgen05 where it
    applies.  ``window`` > 0: the query at position p sees key j <= p when p - j < window or
    j < ``keep_first``; both kernels skip the tiles of keys that no row of a query tile sees.
    ``packed``: the ``mma.sync`` kernel with the heads of a key/value head side by side in a
    tile's rows (``prefill_attention_packed_tokens`` tokens a tile), which reads keys and
    values once for all of them; it takes single decoded tokens as well.  ``sinks`` and
    ``slopes`` as in :func:`paged_attention`; all three kernels take them."""
    biased = sinks is not None or slopes is not None
    for per_head in (sinks, slopes):
        if per_head is not None:
            _need(per_head, torch.float32, "sinks and slopes")
            assert per_head.numel() == heads
    _need(q, torch.bfloat16, "q")
    _need(k_cache, torch.bfloat16, "k_cache")
    _need(out, torch.bfloat16, "out")
    if packed:
        tensor_memory = False
    elif tensor_memory is None:
        tensor_memory = prefill_attention_tc_supports(head_dim, page_size)
    if query_lengths is not None:
        rows = PREFILL_TILE_ROWS_TC if tensor_memory else PREFILL_TILE_ROWS
        if packed:
            rows = prefill_attention_packed_tokens(heads, kv_heads)
        tile_bound = sum(-(-length // rows) for length in query_lengths
                         if length >= min_query_len)
        if tile_bound == 0:
            return
    arguments = (
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), request_start.data_ptr(),
        request_context.data_ptr(), request_table_row.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0), out.data_ptr(), out.stride(0), requests, tile_bound, heads,
        kv_heads, head_dim, page_size, num_pages, float(scale), min_query_len)
    if biased and tensor_memory:
        _check(lib().hx_prefill_attention_tc_biased(*arguments, int(window), int(keep_first),
                                                    _ptr(sinks), _ptr(slopes), _ptr(status),
                                                    _stream()))
    elif biased:
        _check(lib().hx_prefill_attention_biased(*arguments, int(window), int(keep_first),
                                                 1 if packed else 0, _ptr(sinks), _ptr(slopes),
                                                 _ptr(status), _stream()))
    elif packed:
        _check(lib().hx_prefill_attention_packed(*arguments, int(window), int(keep_first),
                                                 _ptr(status), _stream()))
    elif tensor_memory:
        _check(lib().hx_prefill_attention_tc_windowed(*arguments, int(window), int(keep_first),
                                                      _ptr(status), _stream()))
    else:
        _check(lib().hx_prefill_attention_windowed(*arguments, int(window), int(keep_first),
                                                   _ptr(status), _stream()))


# ------------------------------------------------------------ residual streams, biased sums

def streams_spread(x: torch.Tensor, streams: torch.Tensor, tokens: int, count: int) -> None:
    """streams[t, s] = x[t] for every stream s; ``streams`` is ``[rows, count * hidden]``."""
    _need(x, torch.float32, "x")
    _need(streams, torch.float32, "streams")
    hidden = x.shape[1]
    assert x.is_contiguous() and streams.is_contiguous() and streams.shape[1] == count * hidden
    _check(lib().hx_streams_spread(x.data_ptr(), streams.data_ptr(), tokens, hidden, count,
                                   _stream()))


def streams_read_norm(streams: torch.Tensor, read: Optional[torch.Tensor], count: int,
                      weight: torch.Tensor, out: torch.Tensor, eps: float, n_rows: int,
                      clear: Optional[torch.Tensor] = None,
                      rows: Optional[torch.Tensor] = None,
                      initial: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(sum_s read[s] * streams[r', s]) * weight with r' = rows[r] or r
    (``read`` None: every stream counts once).  ``clear`` (float32 ``[rows, hidden]``): its
    first ``n_rows`` rows are zeroed, for the sublayer to sum its output into, or set to
    ``initial`` (float32 ``[hidden]``: a bias that output starts from)."""
    _need(streams, torch.float32, "streams")
    _need(weight, torch.float32, "weight")
    hidden = weight.shape[0]
    assert streams.is_contiguous() and out.is_contiguous() and out.shape[1] == hidden
    assert streams.shape[1] == count * hidden
    if read is not None:
        _need(read, torch.float32, "read")
        assert read.numel() == count
    if clear is not None:
        _need(clear, torch.float32, "clear")
        assert clear.is_contiguous() and clear.shape[1] == hidden and rows is None
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if initial is not None:
        _need(initial, torch.float32, "initial")
        assert clear is not None and initial.numel() == hidden and initial.is_contiguous()
    _check(lib().hx_streams_read_norm(streams.data_ptr(), _ptr(read), count, weight.data_ptr(),
                                      out.data_ptr(), dtype_code(out.dtype), _ptr(clear),
                                      _ptr(initial), _ptr(rows), n_rows, hidden, float(eps),
                                      _stream()))


def streams_write(streams: torch.Tensor, y: torch.Tensor, mixing: Optional[torch.Tensor],
                  write: Optional[torch.Tensor], scale: Optional[torch.Tensor], count: int,
                  tokens: int) -> None:
    """streams[t, r] = sum_s mixing[s, r] * streams[t, s] + write[r] * scale * y[t], all streams
    at once from the old ones (``mixing``, ``write`` None: ones; ``scale`` None: one)."""
    _need(streams, torch.float32, "streams")
    _need(y, torch.float32, "y")
    hidden = y.shape[1]
    assert streams.is_contiguous() and y.is_contiguous() and streams.shape[1] == count * hidden
    for name, tensor, size in (("mixing", mixing, count * count), ("write", write, count),
                               ("scale", scale, hidden)):
        if tensor is not None:
            _need(tensor, torch.float32, name)
            assert tensor.is_contiguous() and tensor.numel() == size
    _check(lib().hx_streams_write(streams.data_ptr(), y.data_ptr(), _ptr(mixing), _ptr(write),
                                  _ptr(scale), count, tokens, hidden, _stream()))


def scaled_sum(x: torch.Tensor, sources: Sequence[torch.Tensor], scales: Sequence[float],
               tokens: int) -> None:
    """x[:tokens] += sum_i scales[i] * sources[i][:tokens]; the sources' rows are zeroed."""
    _need(x, torch.float32, "x")
    width = x.shape[1]
    for source in sources:
        _need(source, torch.float32, "source")
        assert source.is_contiguous() and source.shape[1] == width and source.shape[0] >= tokens
    assert x.is_contiguous() and len(sources) == len(scales)
    pointers = (ctypes.c_void_p * len(sources))(*[source.data_ptr() for source in sources])
    factors = (ctypes.c_float * len(scales))(*[float(scale) for scale in scales])
    _check(lib().hx_scaled_sum(x.data_ptr(), pointers, factors, len(sources), tokens, width,
                               _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor, tokens: int) -> None:
    """x[:tokens] += bias (float32)."""
    _need(x, torch.float32, "x")
    _need(bias, torch.float32, "bias")
    assert x.is_contiguous() and bias.numel() == x.shape[1]
    _check(lib().hx_add_bias(x.data_ptr(), bias.data_ptr(), tokens, x.shape[1], _stream()))


ACT_XIELU = 0        # softplus(p) z^2 + z/2 above zero, (1/2 + softplus(q)) (e^z - 1 - z) + z/2 below
ACT_TANH = 1


def biased_activation(sums: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                      tokens: int, activation: int, p0: float = 0.0, p1: float = 0.0) -> None:
    """out[:tokens] = f(sums[:tokens] + bias): ``sums`` float32, ``out`` the compute dtype.
    For ACT_XIELU ``p0 = softplus(p)`` and ``p1 = 1/2 + softplus(q)``."""
    _need(sums, torch.float32, "sums")
    width = out.shape[1]
    assert sums.shape[1] == width and sums.stride(-1) == 1 and out.stride(-1) == 1
    if bias is not None:
        _need(bias, torch.float32, "bias")
        assert bias.numel() == width
    _check(lib().hx_biased_activation(sums.data_ptr(), sums.stride(0), _ptr(bias), out.data_ptr(),
                                      out.stride(0), dtype_code(out.dtype), tokens, width,
                                      int(activation), float(p0), float(p1), _stream()))


# ------------------------------------------------------------------------ recurrent mixers

def scan_rows_per_thread(rows: int) -> int:
    """Consecutive rows of a column that one lane of a recurrence keeps (the kernels' constant)."""
    return 16


def scan_state_floats(columns: int, rows: int) -> int:
    """Floats that a head's ``rows x columns`` matrix takes in a request's state row.  The
    recurrences give a run of consecutive rows of a column to a lane, ``parts`` lanes (a power of
    two) to a column, and keep the matrix in that order, padded to whole runs.  Computed here so
    that a model can be sized without a GPU; the kernels refuse a state that is smaller than
    their own count."""
    run = scan_rows_per_thread(rows)
    parts = 1
    while parts * run < rows:
        parts *= 2
    if parts > 32:
        raise KernelError(f"a recurrence over {rows} rows is more than 512")
    return parts * run * columns


def causal_filter(raw: torch.Tensor, out: torch.Tensor, taps: torch.Tensor,
                  bias: Optional[torch.Tensor], state: Optional[torch.Tensor], tokens: int,
                  silu: bool, token_request: torch.Tensor, request_slot: torch.Tensor,
                  request_start: torch.Tensor) -> None:
    """out[t, c] = f(bias[c] + sum_j taps[c, j] * raw[t - (n - 1) + j, c]) along each request's
    tokens, ``f`` silu or nothing; ``raw`` (a view of the filtered columns) and ``out`` in the
    compute dtype.  ``state`` ``[slots, >= (n - 1) * channels]`` float32 holds each request's
    last ``n - 1`` inputs and is updated."""
    _need(taps, torch.float32, "taps")
    channels, count = taps.shape
    assert raw.dtype == out.dtype and raw.stride(-1) == 1 and out.stride(-1) == 1
    assert raw.shape[1] == channels and out.shape[1] == channels and taps.is_contiguous()
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if count > 1:
        _need(state, torch.float32, "state")
        assert state.shape[1] >= (count - 1) * channels
    _check(lib().hx_causal_filter(raw.data_ptr(), raw.stride(0), out.data_ptr(), out.stride(0),
                                  dtype_code(out.dtype), taps.data_ptr(), _ptr(bias), _ptr(state),
                                  0 if state is None else state.stride(0), count, channels,
                                  1 if silu else 0, tokens, token_request.data_ptr(),
                                  request_slot.data_ptr(), request_start.data_ptr(), _stream()))


def state_space_scan(x: torch.Tensor, b: torch.Tensor, c: torch.Tensor, dt: torch.Tensor,
                     dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor,
                     state: torch.Tensor, y: torch.Tensor, request_start: torch.Tensor,
                     request_slot: torch.Tensor, requests: int, heads: int, width: int, rows: int,
                     groups: int, tokens: Optional[int] = None) -> None:
    """The selective state-space recurrence over each request's tokens: per head
    ``S = exp(-exp(a_log) d) S + d B x'``, ``y = S' C + skip x`` with ``d = softplus(dt +
    dt_bias)``.  ``x`` ``[tokens, heads * width]``, ``b``, ``c`` ``[tokens, groups * rows]`` (views
    of one buffer), ``dt`` ``[tokens, heads]``; ``state`` ``[slots, >= heads * rows * width]`` and
    ``y`` ``[tokens, heads * width]`` float32.  ``tokens`` (default: the rows of ``x``) is the
    step's token count; when it equals ``requests`` the decode kernel runs."""
    for name, tensor in (("dt_bias", dt_bias), ("a_log", a_log), ("skip", skip), ("state", state),
                         ("y", y)):
        _need(tensor, torch.float32, name)
    assert x.dtype == b.dtype == c.dtype == dt.dtype
    assert x.stride(0) == b.stride(0) == c.stride(0) and x.stride(-1) == 1 and dt.stride(-1) == 1
    assert y.is_contiguous() and y.shape[1] == heads * width
    head_stride = scan_state_floats(width, rows)
    assert state.shape[1] >= heads * head_stride
    _check(lib().hx_state_space_scan(x.data_ptr(), b.data_ptr(), c.data_ptr(), x.stride(0),
                                     dt.data_ptr(), dt.stride(0), dtype_code(x.dtype),
                                     dt_bias.data_ptr(), a_log.data_ptr(), skip.data_ptr(),
                                     state.data_ptr(), state.stride(0), head_stride, y.data_ptr(),
                                     request_start.data_ptr(), request_slot.data_ptr(), requests,
                                     x.shape[0] if tokens is None else tokens, heads, width, rows,
                                     groups, _stream()))


def token_shift(h: torch.Tensor, mu: torch.Tensor, out: torch.Tensor, state: torch.Tensor,
                tokens: int, token_request: torch.Tensor, request_slot: torch.Tensor,
                request_start: torch.Tensor) -> None:
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]; the row before a request's first token of
    this step is its ``state`` row (``[slots, >= hidden]`` float32), which becomes the step's
    last row.  ``out`` is ``[mixes, rows, hidden]`` in the compute dtype."""
    _need(mu, torch.float32, "mu")
    _need(state, torch.float32, "state")
    mixes, hidden = mu.shape
    assert out.dtype == h.dtype and out.is_contiguous() and out.shape[0] == mixes
    assert out.shape[2] == hidden and h.stride(-1) == 1 and mu.is_contiguous()
    _check(lib().hx_token_shift(h.data_ptr(), h.stride(0), dtype_code(h.dtype), mu.data_ptr(), mixes,
                                out.data_ptr(), out.stride(0), state.data_ptr(), state.stride(0),
                                tokens, hidden, token_request.data_ptr(), request_slot.data_ptr(),
                                request_start.data_ptr(), _stream()))


def outer_product_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_log: torch.Tensor,
                       w0: torch.Tensor, bonus: torch.Tensor, state: torch.Tensor, o: torch.Tensor,
                       request_start: torch.Tensor, request_slot: torch.Tensor, requests: int,
                       heads: int, dim: int, tokens: Optional[int] = None) -> None:
    """Per head ``o = (S + diag(bonus) k v')' r`` then ``S = diag(w) S + k v'`` with
    ``w = exp(-exp(decay_log + w0))``; ``r``, ``k``, ``v`` ``[tokens, heads * dim]`` in the compute
    dtype, ``decay_log`` and ``o`` float32, ``state`` ``[slots, >= heads * scan_state_floats(dim,
    dim)]`` float32."""
    for name, tensor in (("decay_log", decay_log), ("w0", w0), ("bonus", bonus), ("state", state),
                         ("o", o)):
        _need(tensor, torch.float32, name)
    assert r.dtype == k.dtype == v.dtype and o.is_contiguous() and o.shape[1] == heads * dim
    head_stride = scan_state_floats(dim, dim)
    assert state.shape[1] >= heads * head_stride
    _check(lib().hx_outer_product_scan(r.data_ptr(), r.stride(0), k.data_ptr(), k.stride(0),
                                       v.data_ptr(), v.stride(0), dtype_code(r.dtype),
                                       decay_log.data_ptr(), decay_log.stride(0), w0.data_ptr(),
                                       bonus.data_ptr(), state.data_ptr(), state.stride(0),
                                       head_stride, o.data_ptr(), request_start.data_ptr(),
                                       request_slot.data_ptr(), requests,
                                       r.shape[0] if tokens is None else tokens, heads, dim,
                                       _stream()))


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                     tokens: int, groups: int, eps: float, gate_after: bool) -> None:
    """Channels in ``groups`` equal parts, each over its own root mean square, times ``weight``;
    the gate ``silu(gate)`` multiplies before the norm, or after it (``gate_after``).  ``y``
    float32, ``gate`` and ``out`` in the compute dtype."""
    _need(y, torch.float32, "y")
    _need(weight, torch.float32, "weight")
    channels = weight.numel()
    assert gate.dtype == out.dtype and gate.stride(-1) == 1 and out.stride(-1) == 1
    assert y.stride(-1) == 1 and y.shape[1] == channels
    _check(lib().hx_gated_group_norm(y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0),
                                     dtype_code(out.dtype), weight.data_ptr(), out.data_ptr(),
                                     out.stride(0), tokens, channels, groups, float(eps),
                                     1 if gate_after else 0, _stream()))


# ----------------------------------------------- linear attention with a matrix state

def linear_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor,
                      o: torch.Tensor, request_start: torch.Tensor, request_slot: torch.Tensor,
                      requests: int, heads: int, qk_heads: int, dim: int, vdim: int, *,
                      delta: bool, decay_in: Optional[torch.Tensor] = None,
                      beta_in: Optional[torch.Tensor] = None,
                      a_log: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None,
                      fixed_decay: Optional[torch.Tensor] = None,
                      fixed_decay_m1: Optional[torch.Tensor] = None,
                      positions: Optional[torch.Tensor] = None,
                      freq: Optional[torch.Tensor] = None,
                      freq_exact: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                      rotary_layout: int = 1, unit_norm: bool = False, unit_eps: float = 0.0,
                      q_scale: float = 1.0, k_scale: float = 1.0,
                      tokens: Optional[int] = None) -> None:
    """Linear attention with one ``[dim, vdim]`` matrix per head, token by token along each
    request: ``S <- g S + k v'`` (plain) or ``S <- g S; u = beta (v - S' k); S <- S + k u'``
    (``delta``), then ``o = S' q``.  ``q, k`` ``[tokens, qk_heads * dim]`` and ``v``
    ``[tokens, heads * vdim]`` in the compute dtype (views with a row stride).  The decay is
    ``exp(-exp(a_log) softplus(decay_in + dt_bias))`` from the column ``decay_in[:, head]``, or
    the head's constant ``fixed_decay`` (with ``fixed_decay_m1``, the same minus one); ``beta =
    sigmoid(beta_in[:, head])``.  Queries and keys are prepared in float32: unit vectors per
    head (``unit_norm``: ``x / sqrt(sum x^2 + unit_eps)``) or rotated over their first
    ``rotary_dim`` coordinates by ``positions * freq`` (layout as ``ROTARY_LAYOUTS``), then
    times ``q_scale`` / ``k_scale``.  ``state`` ``[slots, >= heads * scan_state_floats(vdim,
    dim)]`` and ``o`` ``[tokens, heads * vdim]`` float32."""
    _need(state, torch.float32, "state")
    _need(o, torch.float32, "o")
    assert q.dtype == k.dtype == v.dtype and q.stride(-1) == k.stride(-1) == v.stride(-1) == 1
    assert o.is_contiguous() and o.shape[1] == heads * vdim
    head_stride = scan_state_floats(vdim, dim)
    assert state.shape[1] >= heads * head_stride
    ld_gates = 0
    for gate in (decay_in, beta_in):
        if gate is not None:
            assert gate.dtype == q.dtype and gate.stride(-1) == 1
            assert ld_gates in (0, gate.stride(0))
            ld_gates = gate.stride(0)
    for name, tensor in (("a_log", a_log), ("dt_bias", dt_bias), ("fixed_decay", fixed_decay),
                         ("fixed_decay_m1", fixed_decay_m1), ("freq", freq)):
        if tensor is not None:
            _need(tensor, torch.float32, name)
    if freq_exact is not None:
        _need(freq_exact, torch.float64, "freq_exact")
    _check(lib().hx_linear_state_scan(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
        dtype_code(q.dtype), 1 if delta else 0, _ptr(decay_in), _ptr(beta_in), ld_gates,
        _ptr(a_log), _ptr(dt_bias), _ptr(fixed_decay), _ptr(fixed_decay_m1), _ptr(positions),
        _ptr(freq), _ptr(freq_exact), rotary_dim, rotary_layout, 1 if unit_norm else 0,
        float(unit_eps), float(q_scale), float(k_scale), state.data_ptr(), state.stride(0),
        head_stride, o.data_ptr(), request_start.data_ptr(), request_slot.data_ptr(), requests,
        q.shape[0] if tokens is None else tokens, heads, qk_heads, dim, vdim, _stream()))


# ------------------------------------------------------------- gated residual connection

def gated_residual_add(residual: torch.Tensor, output: torch.Tensor, gate: torch.Tensor,
                       bias: torch.Tensor, tokens: int) -> None:
    """residual[:tokens] += output[:tokens] * sigmoid(gate[:tokens] + bias); all float32."""
    for name, tensor in (("residual", residual), ("output", output), ("gate", gate),
                         ("bias", bias)):
        _need(tensor, torch.float32, name)
    width = residual.shape[1]
    assert residual.is_contiguous() and output.is_contiguous() and output.shape[1] == width
    assert gate.shape[1] >= width and bias.numel() == width
    _check(lib().hx_gated_residual_add(residual.data_ptr(), output.data_ptr(), gate.data_ptr(),
                                       gate.stride(0), bias.data_ptr(), tokens, width, _stream()))


def join_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, tokens: int) -> None:
    """out[:tokens] = [a[:tokens] | b[:tokens]] in ``out``'s dtype; ``a``, ``b`` float32."""
    _need(a, torch.float32, "a")
    _need(b, torch.float32, "b")
    width = a.shape[1]
    assert a.is_contiguous() and b.is_contiguous() and b.shape[1] == width
    assert out.stride(-1) == 1 and out.shape[1] >= 2 * width
    _check(lib().hx_join_rows(a.data_ptr(), b.data_ptr(), out.data_ptr(), out.stride(0),
                              dtype_code(out.dtype), tokens, width, _stream()))


# ------------------------------------------------ norms between a product and what follows

def norm_residual_add(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                      mult: float, tokens: int, cast_out: Optional[torch.Tensor] = None) -> None:
    """residual[:tokens] += mult * y / sqrt(mean(y^2) + eps) * weight (float32 rows); with
    ``cast_out`` the updated rows are also written there in its dtype."""
    _need(residual, torch.float32, "residual")
    _need(y, torch.float32, "y")
    _need(weight, torch.float32, "weight")
    width = residual.shape[1]
    assert residual.is_contiguous() and y.is_contiguous() and y.shape[1] == width
    assert weight.numel() == width
    code = dtype_code(cast_out.dtype) if cast_out is not None else HX_F32
    _check(lib().hx_norm_residual_add(residual.data_ptr(), y.data_ptr(), weight.data_ptr(),
                                      float(eps), float(mult), _ptr(cast_out),
                                      cast_out.stride(0) if cast_out is not None else 0, code,
                                      tokens, width, _stream()))


def biased_normed_rows(projected: torch.Tensor, clear: bool, rows: torch.Tensor, tokens: int,
                       heads: int, kv_heads: int, head_dim: int, value_dim: int, row_dim: int,
                       positions: torch.Tensor, q_bias: Optional[torch.Tensor] = None,
                       k_bias: Optional[torch.Tensor] = None,
                       v_bias: Optional[torch.Tensor] = None,
                       q_weight: Optional[torch.Tensor] = None,
                       k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                       temp_coef: float = 0.0, temp_every: int = 0, value_mix: int = 0,
                       mix: float = 0.0, value_source: Optional[torch.Tensor] = None,
                       gates: Optional[torch.Tensor] = None,
                       token_request: Optional[torch.Tensor] = None,
                       request_table_row: Optional[torch.Tensor] = None,
                       block_tables: Optional[torch.Tensor] = None,
                       k_cache: Optional[torch.Tensor] = None,
                       v_cache: Optional[torch.Tensor] = None, page_size: int = 0,
                       num_pages: int = 0, status: Optional[torch.Tensor] = None) -> None:
    """From the float32 projection ``[q | k | v | head gate sums]`` of every token: biases, one RMS
    norm over all query coordinates and one over all key coordinates, the query times ``1 +
    temp_coef * ln(floor((p + 1) / temp_every) + 1)``, values kept in (``value_mix`` 1) or
    blended with (2: ``(1 - mix) v + mix * source``) ``value_source``; ``rows`` gets ``[heads |
    kv_heads | kv_heads]`` rows of ``row_dim`` and ``gates`` ``[tokens, heads]`` the sigmoid of
    the gate sums.  ``clear``: the projection is an accumulator and is left zero.  With
    ``k_cache`` and ``v_cache`` (and the step's ``token_request``, ``request_table_row``,
    ``block_tables``) keys and values are appended to the token's pages instead of written to
    ``rows``, which then holds the queries only."""
    _need(projected, torch.float32, "projected")
    for vector in (q_bias, k_bias, v_bias, q_weight, k_weight, value_source, gates):
        if vector is not None:
            _need(vector, torch.float32, "a float32 argument")
            assert vector.is_contiguous()
    assert rows.stride(-1) == 1
    _check(lib().hx_biased_normed_rows(
        projected.data_ptr(), projected.stride(0), 1 if clear else 0, _ptr(q_bias), _ptr(k_bias),
        _ptr(v_bias), _ptr(q_weight), _ptr(k_weight), float(eps), positions.data_ptr(),
        float(temp_coef), int(temp_every), int(value_mix), float(mix), _ptr(value_source),
        rows.data_ptr(), rows.stride(0), _ptr(gates), dtype_code(rows.dtype), tokens, heads,
        kv_heads, head_dim, value_dim, row_dim, _ptr(token_request), _ptr(request_table_row),
        _ptr(block_tables), block_tables.stride(0) if block_tables is not None else 0,
        _ptr(k_cache), _ptr(v_cache), int(page_size), int(num_pages), _ptr(status), _stream()))


def head_gate(context: torch.Tensor, gates: torch.Tensor, tokens: int, heads: int,
              row_dim: int) -> None:
    """context[t, h * row_dim:(h + 1) * row_dim] *= gates[t, h] (gates float32)."""
    _need(gates, torch.float32, "gates")
    assert gates.is_contiguous() and gates.shape[1] == heads and context.stride(-1) == 1
    _check(lib().hx_head_gate(context.data_ptr(), context.stride(0), gates.data_ptr(),
                              dtype_code(context.dtype), tokens, heads, row_dim, _stream()))


def token_gate(sums: torch.Tensor, clear: bool, table: torch.Tensor, offset: int,
               token_ids: torch.Tensor, out: torch.Tensor, tokens: int, dim: int,
               status: Optional[torch.Tensor]) -> None:
    """out[t, c] = gelu_tanh(sums[t, c]) * table[token_ids[t], offset + c] for ``c < dim``."""
    _need(sums, torch.float32, "sums")
    _need(token_ids, torch.int32, "token_ids")
    assert table.dtype == out.dtype and table.stride(-1) == 1 and out.stride(-1) == 1
    _check(lib().hx_token_gate(sums.data_ptr(), sums.stride(0), 1 if clear else 0,
                               table.data_ptr(), table.stride(0), offset, table.shape[0],
                               token_ids.data_ptr(), out.data_ptr(), out.stride(0),
                               dtype_code(out.dtype), tokens, dim, _ptr(status), _stream()))


# ------------------------------------------------------------------------ routed experts

def route_top(sums: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, tokens: int,
              experts: int, top: int, scale: float, softmax: bool = False,
              correction: Optional[torch.Tensor] = None, normalize: bool = True) -> None:
    """Per token the ``top`` largest of ``sigmoid(sums[:, :experts])`` (lowest index among
    equals) into ``chosen`` (int32 ``[tokens, top]``), and their scores over their sum
    (``+ 1e-20``) times ``scale`` into ``weights`` (float32).  ``softmax``: the scores are
    ``softmax(sums[:, :experts])``; ``correction`` (float32 ``[experts]``) is added to the scores
    for the choice only; ``normalize=False``: the weights are the chosen scores times ``scale``."""
    if correction is not None:
        _need(correction, torch.float32, "correction")
        assert correction.numel() == experts
    _need(sums, torch.float32, "sums")
    _need(chosen, torch.int32, "chosen")
    _need(weights, torch.float32, "weights")
    assert chosen.is_contiguous() and weights.is_contiguous()
    assert chosen.shape[1] == top and weights.shape[1] == top
    _check(lib().hx_route_top_ruled(sums.data_ptr(), sums.stride(0), tokens, experts, top,
                                    float(scale), 1 if softmax else 0, _ptr(correction),
                                    1 if normalize else 0, chosen.data_ptr(), weights.data_ptr(),
                                    _stream()))


def expert_gate_up(x: torch.Tensor, gate_up: torch.Tensor, chosen: torch.Tensor,
                   act: torch.Tensor, tokens: int, top: int, activation: int = GATE_SILU,
                   limit: float = 0.0) -> None:
    """act[t * top + k] = f(gate_e x[t]) * (up_e x[t]) with ``e = chosen[t, k]``; ``gate_up``
    ``[experts, 2 * ff, width]`` holds an expert's gate rows, then its up rows.  A choice that
    names no expert (``e >= experts``) is left out."""
    experts, rows, width = gate_up.shape
    ff = rows // 2
    assert x.dtype == gate_up.dtype == act.dtype and gate_up.is_contiguous()
    assert x.stride(-1) == 1 and x.shape[1] == width
    assert act.is_contiguous() and act.shape[1] == ff and act.shape[0] >= tokens * top
    _check(lib().hx_expert_gate_up_limited(x.data_ptr(), x.stride(0), gate_up.data_ptr(),
                                           chosen.data_ptr(), act.data_ptr(), dtype_code(x.dtype),
                                           tokens, top, ff, width, experts, int(activation),
                                           float(limit), _stream()))


def expert_identity_add(x: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor,
                        out: torch.Tensor, tokens: int, top: int, experts: int) -> None:
    """out[t] += x[t] * (the weights of the token's choices with an index ``>= experts``): the
    router's outputs behind the experts return their input.  ``out`` float32."""
    _need(out, torch.float32, "out")
    width = x.shape[1]
    assert x.stride(-1) == 1 and out.shape[1] >= width
    _check(lib().hx_expert_identity_add(x.data_ptr(), x.stride(0), chosen.data_ptr(),
                                        weights.data_ptr(), out.data_ptr(), out.stride(0),
                                        dtype_code(x.dtype), tokens, top, width, experts,
                                        _stream()))


def expert_down(act: torch.Tensor, down: torch.Tensor, chosen: torch.Tensor,
                weights: torch.Tensor, out: torch.Tensor, tokens: int, top: int) -> None:
    """out[t] += sum_k weights[t, k] * down_e act[t * top + k] (``k`` ascending); ``down``
    ``[experts, width, ff]``, ``out`` float32."""
    experts, width, ff = down.shape
    _need(out, torch.float32, "out")
    assert act.dtype == down.dtype and down.is_contiguous() and act.is_contiguous()
    assert act.shape[1] == ff and out.shape[1] >= width
    _check(lib().hx_expert_down(act.data_ptr(), down.data_ptr(), chosen.data_ptr(),
                                weights.data_ptr(), out.data_ptr(), out.stride(0),
                                dtype_code(act.dtype), tokens, top, ff, width, experts, _stream()))


GROUPED_TILES = (16, 32, 64, 128)


def expert_tile(pairs: int, experts: int) -> int:
    """The token tile of the grouped products: the smallest that holds an expert's average
    share of the pairs, so that padding stays below the work."""
    share = -(-pairs // experts)
    for tile in GROUPED_TILES:
        if share <= tile:
            return tile
    return GROUPED_TILES[-1]


def expert_tile_bound(pairs: int, experts: int, tile: int) -> int:
    """Tiles that ``pairs`` pairs, laid out expert by expert in whole tiles, can take."""
    return int(lib().hx_expert_tile_bound(pairs, experts, tile))


def expert_rows(chosen: torch.Tensor, pair_row: torch.Tensor, tile_group: torch.Tensor, pairs: int,
                experts: int, tile: int, max_tiles: int) -> None:
    """The pairs sorted by expert: ``pair_row[pair]`` is the pair's row in an order where every
    expert's rows are a whole number of tiles, ``tile_group[t]`` the expert of tile ``t`` (-1
    behind the last one in use)."""
    _need(chosen, torch.int32, "chosen")
    _need(pair_row, torch.int32, "pair_row")
    _need(tile_group, torch.int32, "tile_group")
    assert pair_row.numel() >= pairs and tile_group.numel() >= max_tiles
    _check(lib().hx_expert_rows(chosen.data_ptr(), pairs, experts, tile, max_tiles,
                                pair_row.data_ptr(), tile_group.data_ptr(), _stream()))


def expert_gather(x: torch.Tensor, pair_row: torch.Tensor, grouped: torch.Tensor, tokens: int,
                  top: int) -> None:
    """grouped[pair_row[t * top + k]] = x[t]."""
    assert x.dtype == grouped.dtype and x.stride(-1) == 1 and grouped.stride(-1) == 1
    _check(lib().hx_expert_gather(x.data_ptr(), x.stride(0), pair_row.data_ptr(),
                                  grouped.data_ptr(), grouped.stride(0), dtype_code(x.dtype),
                                  tokens, top, x.shape[1], _stream()))


def expert_combine(y: torch.Tensor, pair_row: torch.Tensor, weights: torch.Tensor,
                   out: torch.Tensor, tokens: int, top: int, width: int) -> None:
    """out[t] += sum_k weights[t, k] * y[pair_row[t * top + k]], ``k`` ascending."""
    _need(y, torch.float32, "y")
    _need(out, torch.float32, "out")
    _check(lib().hx_expert_combine(y.data_ptr(), y.stride(0), pair_row.data_ptr(),
                                   weights.data_ptr(), out.data_ptr(), out.stride(0), tokens, top,
                                   width, _stream()))


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, features: int,
                    epilogue: int, up_row_offset: int, token_tile: int, tile_group: torch.Tensor,
                    status: torch.Tensor, gate_activation: Optional[int] = None,
                    gate_limit: float = 0.0) -> None:
    """Tile ``t`` of ``token_tile`` rows of ``x`` times matrix ``tile_group[t]`` of ``w``
    ``[groups, group_rows, depth]`` on the tensor cores; ``rows`` bounds the rows in use (a
    multiple of the tile).  Epilogues: plain store, float32 store, gated activation; with
    ``gate_activation`` (any of GATE_ACTIVATIONS, ``gate_limit`` for the clamped form) the
    epilogue is that gated activation whatever ``epilogue`` says."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    assert w.is_contiguous() and x.stride(-1) == 1 and out.stride(-1) == 1
    groups, group_rows, depth = w.shape
    if gate_activation is not None:
        _check(lib().hx_gemm_tc_grouped_gated(
            x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), depth, group_rows, groups,
            out.data_ptr(), out.stride(0), rows, features, depth, int(gate_activation),
            float(gate_limit), up_row_offset, token_tile, tile_group.data_ptr(),
            status.data_ptr(), _stream()))
        return
    _check(lib().hx_gemm_tc_grouped(x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), depth,
                                    group_rows, groups, out.data_ptr(), out.stride(0), rows,
                                    features, depth, epilogue, up_row_offset, token_tile,
                                    tile_group.data_ptr(), status.data_ptr(), _stream()))


# ---------------------------------------------------------- attention over a cached latent

def latent_prepare(down: torch.Tensor, q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float,
                   positions: torch.Tensor, freq: Optional[torch.Tensor],
                   freq_exact: Optional[torch.Tensor], rotary_dims: int, layout: int,
                   query_latent: torch.Tensor, rows: torch.Tensor, key_offset: int, tokens: int,
                   q_rank: int, kv_rank: int, rot: int, row_dim: int,
                   amplitude: float = 1.0) -> None:
    """From the float32 down-projection ``[q_rank | kv_rank | rot]`` of every token: the normed
    query latent into ``query_latent``; the key row ``[c | rot(kr) | 0]`` at column
    ``key_offset`` of ``rows`` and the value row ``[c | 0]`` behind it (``row_dim`` wide each),
    ``c`` the normed key/value latent."""
    _need(down, torch.float32, "down")
    _need(q_weight, torch.float32, "q_weight")
    _need(kv_weight, torch.float32, "kv_weight")
    assert query_latent.dtype == rows.dtype and down.stride(-1) == 1
    _check(lib().hx_latent_prepare(
        down.data_ptr(), down.stride(0), q_weight.data_ptr(), kv_weight.data_ptr(), float(eps),
        positions.data_ptr(), _ptr(freq), _ptr(freq_exact), rotary_dims, layout,
        query_latent.data_ptr(), query_latent.stride(0), rows.data_ptr(), rows.stride(0),
        key_offset, dtype_code(rows.dtype), tokens, q_rank, kv_rank, rot, row_dim,
        float(amplitude), _stream()))


def latent_queries(q: torch.Tensor, rot_offset: int, rows: torch.Tensor, positions: torch.Tensor,
                   freq: Optional[torch.Tensor], freq_exact: Optional[torch.Tensor],
                   rotary_dims: int, layout: int, tokens: int, heads: int, kv_rank: int, rot: int,
                   row_dim: int, amplitude: float = 1.0) -> None:
    """The rotated part of every head's query (``q[:, rot_offset + head * rot:][:rot]``) turned
    by the token's position into ``rows[:, head * row_dim + kv_rank:]``, zeros to the head's
    end."""
    assert q.dtype == rows.dtype and q.stride(-1) == 1 and rows.stride(-1) == 1
    _check(lib().hx_latent_queries(q.data_ptr(), q.stride(0), rot_offset, rows.data_ptr(),
                                   rows.stride(0), positions.data_ptr(), _ptr(freq),
                                   _ptr(freq_exact), rotary_dims, layout, dtype_code(rows.dtype),
                                   tokens, heads, kv_rank, rot, row_dim, float(amplitude),
                                   _stream()))


def head_products(x: torch.Tensor, x_stride: int, w: torch.Tensor, out: torch.Tensor,
                  out_stride: int, tokens: int) -> None:
    """out[t, h * out_stride + o] = sum_i w[h, o, i] * x[t, h * x_stride + i]: one small product
    per head, ``w`` ``[heads, out_dim, in_dim]``, everything in the compute dtype."""
    heads, out_dim, in_dim = w.shape
    assert x.dtype == w.dtype == out.dtype and w.is_contiguous()
    assert x.stride(-1) == 1 and out.stride(-1) == 1
    _check(lib().hx_head_products(x.data_ptr(), x.stride(0), x_stride, w.data_ptr(),
                                  out.data_ptr(), out.stride(0), out_stride, dtype_code(x.dtype),
                                  tokens, heads, out_dim, in_dim, _stream()))


# ------------------------------------------------- rotation from positions, normed heads

ROTARY_LAYOUTS = {"interleaved": 0, "halves": 1}


def norm_rotary_append(qkv: torch.Tensor, positions: torch.Tensor, token_request: torch.Tensor,
                       request_table_row: torch.Tensor, block_tables: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       freq: torch.Tensor, value_freq: Optional[torch.Tensor],
                       q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                       tokens: int, heads: int, kv_heads: int, head_dim: int, value_dim: int,
                       row_dim: int, rotary_dim: int, layout: int, value_layout: int,
                       page_size: int, num_pages: int, status: torch.Tensor,
                       accum: Optional[torch.Tensor] = None) -> None:
    """Per-head RMS norm of q and k (when the weights are given), rotation of their first
    ``rotary_dim`` coordinates by ``position * freq``, rotation of the values over ``value_dim``
    by ``position * value_freq`` (when given), queries back into ``qkv``, keys and values into
    their pages.  ``accum`` as for :func:`rope_append`."""
    _need(freq, torch.float32, "freq")
    write = k_cache is not None
    _check(lib().hx_norm_rotary_append(
        qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), _ptr(accum),
        0 if accum is None else accum.stride(0), positions.data_ptr(), token_request.data_ptr(),
        request_table_row.data_ptr(), _ptr(block_tables) if write else None,
        block_tables.stride(0) if write else 0, _ptr(k_cache), _ptr(v_cache), 1 if write else 0,
        freq.data_ptr(), _ptr(value_freq), _ptr(q_norm), _ptr(k_norm), float(eps), tokens, heads,
        kv_heads, head_dim, value_dim, row_dim, rotary_dim, layout, value_layout, page_size,
        num_pages, _ptr(status), _stream()))


def rotate_back(rows: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, tokens: int,
                heads: int, row_dim: int, dims: int, layout: int) -> None:
    """Every head of ``rows[:tokens]`` turned by minus its token's position over its first
    ``dims`` coordinates, in place."""
    _need(freq, torch.float32, "freq")
    assert rows.stride(-1) == 1
    _check(lib().hx_rotate_back(rows.data_ptr(), dtype_code(rows.dtype), rows.stride(0),
                                positions.data_ptr(), freq.data_ptr(), tokens, heads, row_dim, dims,
                                layout, _stream()))


def argmax(logits: torch.Tensor, tokens_out: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need(logits, torch.float32, "logits")
    _need(tokens_out, torch.int32, "tokens_out")
    rows, vocab = logits.shape
    _check(lib().hx_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, tokens_out.data_ptr(),
                           _ptr(status), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           tokens_out: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(uniform, torch.float32, "uniform")
    _need(tokens_out, torch.int32, "tokens_out")
    rows, vocab = logits.shape
    _check(lib().hx_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
                           uniform.data_ptr(), tokens_out.data_ptr(), _ptr(status), _stream()))


def feed_tokens(token_ids: torch.Tensor, sampled: torch.Tensor, rows: torch.Tensor,
                count: int) -> None:
    """token_ids[i] = max(sampled[rows[i]], 0) for i < count: the tokens of a step that was
    prepared before the host had read what the step before it sampled."""
    _need(token_ids, torch.int32, "token_ids")
    _need(sampled, torch.int32, "sampled")
    _need(rows, torch.int32, "rows")
    _check(lib().hx_feed_tokens(token_ids.data_ptr(), sampled.data_ptr(), rows.data_ptr(), count,
                                sampled.shape[0], _stream()))


def launch_count() -> int:
    """Kernels this library has launched (or recorded into a graph) since it was loaded."""
    return int(lib().hx_launch_count())


def set_dependent_launch(enabled: bool) -> None:
    """Switch programmatic dependent launch of the kernels off (debugging) or on (default)."""
    lib().hx_set_dependent_launch(1 if enabled else 0)


def bounded_wait_check(polls: int, arrive: bool, status: torch.Tensor) -> bool:
    """Run the kernels' bounded mbarrier wait on a barrier of its own with a limit of ``polls``
    polls.  ``arrive`` False: nobody arrives, the wait runs out, the kernel sets
    FLAG_WAIT_TIMEOUT in ``status`` and returns.  Returns whether the wait succeeded."""
    succeeded = torch.full((1,), -1, dtype=torch.int32, device=status.device)
    _check(lib().hx_bounded_wait_check(int(polls), 1 if arrive else 0, _ptr(status),
                                       _ptr(succeeded), _stream()))
    return int(succeeded.item()) == 1
