"""Python launchers of the sm_100a kernels in libmir_b200/csrc.

Every function takes torch CUDA tensors, checks what the kernel cannot check itself (device, dtype,
contiguity), and launches on torch's current stream, so launches are captured when a CUDA graph is
being recorded.  There is no fallback: if the native library cannot be built or loaded, or a kernel
refuses its sizes, a KernelError is raised.
"""

from __future__ import annotations

import contextlib
import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build
from ..errors import KernelError

_LIBS: dict = {}
_VERBOSE_BUILD = True

_SIGNATURES = {
    "core": {
        "mir_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "mir_rms_norm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "mir_silu_mul": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "mir_add_bias": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "mir_cast": [c_int, c_void_p, c_void_p, c_size_t, c_void_p],
        "mir_qk_rope_store": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_longlong, c_int, c_void_p],
        "mir_paged_attention_generic": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                        c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_float, c_void_p, c_int,
                                        c_void_p],
        "mir_qk_prepare": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
        "mir_layer_norm": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_float, c_void_p],
        "mir_streams_write": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "mir_streams_write_norm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_float, c_void_p],
        "mir_streams_spread": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "mir_streams_sum": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "mir_embed_pairs": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_longlong, c_longlong, c_float, c_void_p],
        "mir_gelu_tanh": [c_int, c_void_p, c_size_t, c_void_p],
        "mir_add_normed_branches": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float,
                                    c_void_p],
        "mir_short_conv_silu": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mir_delta_rule_prepare": [c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                   c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mir_delta_rule_scan": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mir_delta_rule_set_lanes": [c_int],
        "mir_gated_head_norm": [c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_float, c_int, c_int, c_void_p],
        "mir_activation": [c_int, c_int, c_void_p, c_size_t, c_void_p],
        "mir_softcap": [c_void_p, c_size_t, c_float, c_void_p],
        "mir_add_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "mir_rms_norm_pair": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "mir_latent_prepare": [c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                               c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "mir_rope_rows": [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p,
                          c_float, c_int, c_int, c_int, c_int, c_void_p],
        "mir_sigmoid_gate": [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p],
        "mir_head_linear": [c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p,
                            c_longlong, c_int, c_int, c_int, c_int, c_void_p],
        "mir_wkv_mix": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_void_p],
        "mir_retention_scan": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_float,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_void_p],
        "mir_wkv_scan": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mir_moe_route": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_float, c_int, c_int, c_void_p],
        "mir_moe_tile_slots": [c_int, c_int, c_int],
        "mir_moe_sort": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p],
        "mir_moe_gate_up": [c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mir_moe_down": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_int, c_int, c_void_p],
        "mir_moe_gather_rows": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
        "mir_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                            c_int, c_void_p, c_longlong, c_void_p],
        "mir_gemm_f32": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                         c_void_p],
        "mir_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                       c_void_p, c_int, c_void_p],
        "mir_repetition_penalty": [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mir_decode_prepare": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "mir_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    },
    "bf16": {
        "mir_decode_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                      c_longlong, c_void_p],
        "mir_decode_attention_kept_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                           c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                           c_longlong, c_void_p, c_int, c_void_p],
        "mir_decode_attention_extra_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                            c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong],
        "mir_decode_attention_scored_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p,
                                             c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float,
                                             c_void_p, c_int],
        "mir_prefill_attention_tc_scored_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                                 c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_float, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float,
                                                 c_void_p, c_int],
        "mir_decode_attention_paged_scored_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong,
                                                   c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                   c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
                                                   c_void_p, c_longlong, c_int, c_float, c_void_p, c_int],
        "mir_prefill_attention_scored_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                              c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_void_p,
                                              c_int],
        "mir_decode_attention_paged_extra_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong,
                                                  c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                  c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p,
                                                  c_void_p, c_longlong],
        "mir_prefill_attention_extra_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                             c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong],
        "mir_prefill_attention_tc_extra_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                                c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong],
        "mir_decode_attention_paged_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                            c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_int, c_void_p, c_longlong, c_void_p],
        "mir_decode_attention_tc_takes": [c_int, c_int, c_int],
        "mir_head_logits_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_int, c_void_p, c_size_t, c_void_p, c_void_p],
        "mir_gemm_tc_stream_head_candidates": [c_int],
        "mir_decode_partition_keys": [c_int, c_int, c_int, c_int, c_int, c_int],
        "mir_decode_attention_plan": [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "mir_decode_attention_tc_error": [],
        "mir_prefill_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mir_prefill_attention_kept_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_void_p],
        "mir_prefill_attention_tc_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                          c_void_p],
        "mir_prefill_attention_tc_kept_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                               c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                               c_float, c_int, c_int, c_void_p],
        "mir_prefill_attention_tc_takes": [c_int, c_int],
        "mir_prefill_attention_tc_error": [],
        "mir_prefill_attention_tc_set_streams": [c_int],
        "mir_prefill_attention_tc_set_shared": [c_int],
        "mir_gemm_tc_stream_bf16": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mir_gemm_tc_stream_error": [],
        "mir_gemm_tc_stream_set_splits": [c_int, c_int, c_int],
        "mir_gemm_tc_bf16": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_void_p],
        "mir_gemm_tc_grouped_bf16": [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mir_gemm_tc_set_width": [c_int],
        "mir_gemm_tc_error": [],
        "mir_linear_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_void_p,
                            c_void_p],
        "mir_gate_up_silu_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float,
                                  c_void_p, c_void_p, c_size_t, c_void_p],
        "mir_latent_attention_takes": [c_int, c_int],
        "mir_latent_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p],
        "mir_set_option": [ctypes.c_char_p, c_int],
        "mir_get_option": [ctypes.c_char_p],
        "mir_gemm_bf16_lt_batched": [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int,
                                     c_int, c_void_p, c_size_t, c_void_p],
        "mir_gemm_bf16_lt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_void_p, c_size_t, c_void_p],
    },
}


def set_build_verbosity(verbose: bool) -> None:
    global _VERBOSE_BUILD
    _VERBOSE_BUILD = verbose


_TRACED = False


def use_traced_kernels() -> None:
    """Load the bfloat16 library with time stamps inside its kernels (csrc/trace.cuh) instead of the plain one.
    To be called before the first bfloat16 kernel runs; read_trace() returns what they recorded."""
    global _TRACED
    if "bf16" in _LIBS and not _TRACED:
        raise KernelError("use_traced_kernels: the plain bfloat16 library is loaded already")
    _TRACED = True


def read_trace() -> dict:
    """The records of the traced kernels since the last call, per group ("stream", "decode", "merge", "rope"):
    int64 arrays [records, 16] of %globaltimer nanoseconds (0 = not reached), [:, 14] a value, [:, 15] a tag; the
    sources say which time stamp is what.  Synchronises the device."""
    import numpy as np
    _require(_TRACED, "read_trace: call use_traced_kernels() first")
    lib = library("bf16")
    capacity = 4096
    host = (ctypes.c_ulonglong * (16 * capacity))()
    records = {}
    for group in ("stream", "decode", "merge", "rope"):
        reader = getattr(lib, f"mir_trace_read_{group}")
        reader.argtypes = [c_void_p, c_int]
        reader.restype = c_int
        count = reader(host, capacity)
        _require(count >= 0, f"read_trace: reading the {group} records failed")
        records[group] = np.array(host[: count * 16], dtype=np.uint64).reshape(count, 16).astype(np.int64)
    return records


def read_prompt_attention_trace():
    """Cycle stamps of the first CTA of the last tcgen05 prompt-attention launch (traced kernels only): an int64 array
    [256, 16]; row g is the CTA's g-th key tile, rows 200 + n the end of its n-th item; csrc/attention_tc.cu says
    which column is what.  0 = not reached.  Synchronises the device."""
    import numpy as np
    _require(_TRACED, "read_prompt_attention_trace: call use_traced_kernels() first")
    lib = library("bf16")
    rows = 256
    host = (ctypes.c_longlong * (16 * rows))()
    lib.mir_trace_read_prompt_tiles.argtypes = [c_void_p, c_int]
    lib.mir_trace_read_prompt_tiles.restype = c_int
    count = lib.mir_trace_read_prompt_tiles(host, rows)
    _require(count == rows, "read_prompt_attention_trace: reading the records failed")
    return np.array(host, dtype=np.int64).reshape(rows, 16)


def library(name: str) -> ctypes.CDLL:
    """The loaded native library `name`, compiled first if its sources changed or it was never built."""
    lib = _LIBS.get(name)
    if lib is not None:
        return lib
    path = _build.build("bf16_trace" if name == "bf16" and _TRACED else name, verbose=_VERBOSE_BUILD)
    try:
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)
    except OSError as error:
        raise KernelError(f"cannot load {path}: {error}") from error
    lib.mir_last_error.restype = ctypes.c_char_p
    lib.mir_last_error.argtypes = []
    for symbol, argtypes in _SIGNATURES.get(name, {}).items():
        function = getattr(lib, symbol)
        function.argtypes = argtypes
        function.restype = c_int
    _LIBS[name] = lib
    return lib


def set_programmatic_launch(mode) -> None:
    """How kernels are launched: 0 / False plainly; 1 / True all with programmatic stream serialization (a
    kernel's start overlaps the previous kernel's end; every kernel waits for its predecessor before it touches
    activations); 2 only the weight-streaming products, whose first weights are then on their way while the
    kernel before them drains."""
    for name in ("core", "bf16"):
        lib = library(name)
        lib.mir_set_pdl.argtypes = [c_int]
        lib.mir_set_pdl.restype = None
        lib.mir_set_pdl(int(mode))


def launch_counts(reset: bool = False) -> dict:
    """How often each kernel of the loaded libraries was launched, by the name its launcher gives
    ("decode_attention", "prefill_attention_tc", "paged_attention_generic", "tc_stream", "gemm_bf16_lt", ...).
    A launch recorded into a CUDA graph counts once, however often the graph is replayed."""
    counts: dict = {}
    for lib in _LIBS.values():
        lib.mir_launch_counts.argtypes = [ctypes.c_char_p, c_int]
        lib.mir_launch_counts.restype = c_int
        buffer = ctypes.create_string_buffer(lib.mir_launch_counts(None, 0))
        lib.mir_launch_counts(buffer, len(buffer))
        for line in buffer.value.decode().splitlines():
            name, _, count = line.partition("=")
            counts[name] = counts.get(name, 0) + int(count)
        if reset:
            lib.mir_reset_launch_counts.argtypes = []
            lib.mir_reset_launch_counts.restype = None
            lib.mir_reset_launch_counts()
    return counts


def loaded_libraries() -> dict:
    """Paths of the native libraries this process has loaded (for reports)."""
    return {name: lib._name for name, lib in _LIBS.items()}


# Whether an RMSNorm between two few-rows products is folded into them (NormedResidual): the product before it
# leaves the sums of squares and the weighted rows, the product after it scales its results.  Two kernels fewer
# per layer in a decode step.
FUSE_NORM_INTO_PRODUCT = True
# Whether the tanh GELU of a feed-forward runs in the epilogue of the product before it (our tcgen05 kernels) instead
# of as a kernel of its own after a library product.
FUSE_GELU_INTO_PRODUCT = True
# Whether layers of the built-in kind are run by the native executor (csrc/executor.cu), one call per run of such
# layers; False runs every layer part by part from Python (the same kernels, launched from the interpreter).
NATIVE_LAYERS = True
REPLAYED_LAUNCHES = 0   # launches that ran as part of replayed CUDA graphs (a replay counts what its capture counted)


def launches() -> int:
    """Kernels and library products launched so far by this process's native libraries, replays of captured graphs
    included (for reports)."""
    return sum(launch_counts().values()) + REPLAYED_LAUNCHES


MIR_CANNOT_FOLD = 4     # a product was given a folded norm's rows that it cannot take over (launchers.h)


def set_option(name: str, value: int) -> None:
    """A threshold of the bfloat16 product dispatch (csrc/ops_bf16.cu): few_rows_max, folded_norm_max_rows,
    tensor_core_min_rows, few_rows_modes (bits: store, accumulate, float32, SwiGLU), decode_tensor_cores,
    decode_partition_keys, decode_tc_partition_keys."""
    lib = library("bf16")
    _check(lib, lib.mir_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(library("bf16").mir_get_option(name.encode()))


@contextlib.contextmanager
def option(name: str, value: int):
    """An option of the native dispatch set for the duration of a `with` block (measurements, tests)."""
    before = get_option(name)
    set_option(name, value)
    try:
        yield
    finally:
        set_option(name, before)


def _check(lib: ctypes.CDLL, status: int) -> None:
    if status != 0:
        raise KernelError(lib.mir_last_error().decode(errors="replace") or f"kernel launch failed with status {status}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle (asked for at every launch, so by the short way where torch has one)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _is_bf16(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {tensor.dtype}")


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise KernelError(message)


def _cuda(*tensors) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("kernels take CUDA tensors only: there is no CPU path")


# --------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[r] = float(table[ids[r]]) * scale; out is the 32-bit residual [rows, hidden]."""
    _cuda(table, ids, out)
    rows, hidden = out.shape
    _require(table.is_contiguous() and out.is_contiguous() and ids.dtype == torch.int32 and ids.numel() == rows
             and out.dtype == torch.float32 and table.shape[1] == hidden, "embed: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_embed(_is_bf16(table), table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, hidden,
                              table.shape[0], scale, _stream()))


def embed_pairs(table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, previous: torch.Tensor, out: torch.Tensor,
                mul_previous: int, mul_current: int, scale: float = 1.0) -> None:
    """out[r] = float(table[ids[r]]) * scale + float(pairs[bucket]) with bucket = (previous[r] * mul_previous +
    ids[r] * mul_current) mod (rows of pairs - 1), and the last row of `pairs` where previous[r] < 0 (a request's
    first token)."""
    _cuda(table, pairs, ids, previous, out)
    rows, hidden = out.shape
    _require(table.is_contiguous() and pairs.is_contiguous() and out.is_contiguous() and ids.dtype == torch.int32
             and previous.dtype == torch.int32 and ids.numel() == rows and previous.numel() >= rows
             and out.dtype == torch.float32 and table.shape[1] == hidden and pairs.shape[1] == hidden
             and pairs.dtype == table.dtype and pairs.shape[0] >= 2, "embed_pairs: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_embed_pairs(_is_bf16(table), table.data_ptr(), pairs.data_ptr(), ids.data_ptr(),
                                    previous.data_ptr(), out.data_ptr(), rows, hidden, table.shape[0],
                                    pairs.shape[0] - 1, int(mul_previous), int(mul_current), scale, _stream()))


def gelu_tanh(x: torch.Tensor) -> None:
    """x <- 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))) in place, computed in 32-bit."""
    _cuda(x)
    _require(x.is_contiguous(), "gelu_tanh: a contiguous tensor is needed")
    lib = library("core")
    _check(lib, lib.mir_gelu_tanh(_is_bf16(x), x.data_ptr(), x.numel(), _stream()))


def add_normed_branches(branches, weights, residual: torch.Tensor, eps: float, scale: float,
                        rounded: Optional[torch.Tensor] = None) -> None:
    """residual += scale * sum_b rmsnorm(branches[b]) * weights[b]; every tensor 32-bit, branches [rows, hidden].
    `rounded` (bfloat16 [rows, hidden], contiguous) also receives the updated residual, for the product that reads it
    next."""
    _cuda(residual, rounded, *branches, *weights)
    _require(rounded is None or (rounded.dtype == torch.bfloat16 and rounded.shape == residual.shape
                                 and rounded.is_contiguous()), "add_normed_branches: rounded is bfloat16 [rows, hidden]")
    rows, hidden = residual.shape
    _require(1 <= len(branches) <= 4 and len(weights) == len(branches) and residual.dtype == torch.float32
             and residual.is_contiguous(), "add_normed_branches: one to four branches and a 32-bit residual")
    for branch, weight in zip(branches, weights):
        _require(branch.dtype == torch.float32 and branch.shape == residual.shape and branch.is_contiguous()
                 and weight.dtype == torch.float32 and weight.numel() == hidden and weight.is_contiguous(),
                 "add_normed_branches: branches are float32 [rows, hidden], weights float32 [hidden]")
    pointers = (c_void_p * len(branches))(*[b.data_ptr() for b in branches])
    weight_pointers = (c_void_p * len(weights))(*[w.data_ptr() for w in weights])
    lib = library("core")
    _check(lib, lib.mir_add_normed_branches(pointers, weight_pointers, len(branches), residual.data_ptr(), _ptr(rounded),
                                            rows, hidden, eps, scale, _stream()))


def short_conv_silu(x: torch.Tensor, weight: torch.Tensor, tail: torch.Tensor, row_of_token: torch.Tensor,
                    query_starts: torch.Tensor, state_slots: torch.Tensor, positions: torch.Tensor,
                    out: torch.Tensor) -> None:
    """out[t, c] = silu(sum_j weight[c, j] * x[t - (taps - 1) + j, c]) within each request, 32-bit: x is a column
    range [tokens, channels] of the packed projection (a view with unit column stride), weight [channels, taps] with
    the current token's tap last, tail [slots, taps - 1, channels] the request's last inputs (32-bit, zero at its
    start), read for what lies before the portion and then moved on."""
    _cuda(x, weight, tail, row_of_token, query_starts, state_slots, positions, out)
    tokens, channels = x.shape
    taps = weight.shape[1]
    rows = query_starts.numel() - 1
    _require(x.stride(1) == 1 and weight.is_contiguous() and weight.shape[0] == channels and weight.dtype == x.dtype
             and tail.dtype == torch.float32 and tail.is_contiguous() and tail.shape[1:] == (max(taps - 1, 0), channels)
             and out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, channels),
             "short_conv_silu: shapes or dtypes do not fit")
    _require(all(t.dtype == torch.int32 for t in (row_of_token, query_starts, state_slots, positions)),
             "short_conv_silu: the batch description is int32")
    lib = library("core")
    _check(lib, lib.mir_short_conv_silu(_is_bf16(x), x.data_ptr(), x.stride(0), weight.data_ptr(), tail.data_ptr(),
                                        row_of_token.data_ptr(), query_starts.data_ptr(), state_slots.data_ptr(),
                                        positions.data_ptr(), out.data_ptr(), tokens, rows, channels, taps, _stream()))


def delta_rule_prepare(x: torch.Tensor, weight: torch.Tensor, tail: torch.Tensor, beta_raw: torch.Tensor,
                       decay_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, row_of_token: torch.Tensor,
                       query_starts: torch.Tensor, state_slots: torch.Tensor, positions: torch.Tensor,
                       qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, heads: int, kv_heads: int,
                       key_dim: int, value_dim: int) -> None:
    """What the gated delta rule needs of every token, in 32-bit: qkv [tokens, 2 kv_heads key_dim + heads value_dim]
    = silu(short convolution) of the q | k | v columns `x` of the packed projection (as short_conv_silu, with the
    request's `tail` read and moved on), q and k then unit vectors per head (x / sqrt(sum x^2 + 1e-6)) and q times
    key_dim^-1/2; beta = sigmoid(beta_raw) [tokens, heads]; decay = exp(-exp(a_log) * softplus(decay_raw + dt_bias))
    [tokens, heads] or [tokens, heads * key_dim] (one decay per key channel), as wide as decay_raw.  beta_raw and
    decay_raw are views with unit column stride in x's dtype (decay_raw may be float32)."""
    _cuda(x, weight, tail, beta_raw, decay_raw, dt_bias, a_log, row_of_token, query_starts, state_slots, positions, qkv,
          beta, decay)
    tokens, channels = x.shape
    taps = weight.shape[1]
    rows = query_starts.numel() - 1
    decay_width = decay_raw.shape[1]
    _require(channels == 2 * kv_heads * key_dim + heads * value_dim and x.stride(1) == 1 and weight.is_contiguous()
             and weight.shape[0] == channels and weight.dtype == x.dtype and tail.dtype == torch.float32
             and tail.is_contiguous() and tail.shape[1:] == (max(taps - 1, 0), channels),
             "delta_rule_prepare: the convolved columns, their weights or their tail do not fit")
    _require(beta_raw.shape == (tokens, heads) and beta_raw.stride(1) == 1 and beta_raw.dtype == x.dtype
             and decay_raw.shape[0] == tokens and decay_raw.stride(1) == 1
             and decay_raw.dtype in (x.dtype, torch.float32) and decay_width in (heads, heads * key_dim)
             and dt_bias.dtype == torch.float32 and dt_bias.numel() == decay_width and dt_bias.is_contiguous()
             and a_log.dtype == torch.float32 and a_log.numel() == heads, "delta_rule_prepare: bad gates")
    for tensor, shape in ((qkv, (tokens, channels)), (beta, (tokens, heads)), (decay, (tokens, decay_width))):
        _require(tensor.dtype == torch.float32 and tensor.is_contiguous() and tensor.shape == shape,
                 "delta_rule_prepare: outputs are contiguous float32")
    _require(all(t.dtype == torch.int32 for t in (row_of_token, query_starts, state_slots, positions)),
             "delta_rule_prepare: the batch description is int32")
    lib = library("core")
    _check(lib, lib.mir_delta_rule_prepare(
        _is_bf16(x), int(decay_raw.dtype == torch.float32), x.data_ptr(), x.stride(0), weight.data_ptr(), tail.data_ptr(),
        beta_raw.data_ptr(), beta_raw.stride(0), decay_raw.data_ptr(), decay_raw.stride(0), dt_bias.data_ptr(),
        a_log.data_ptr(), row_of_token.data_ptr(), query_starts.data_ptr(), state_slots.data_ptr(), positions.data_ptr(),
        qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(), tokens, rows, heads, kv_heads, key_dim, value_dim, decay_width,
        taps, _stream()))


def delta_rule_scan(qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                    query_starts: torch.Tensor, state_slots: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                    heads: int, kv_heads: int, key_dim: int, value_dim: int) -> None:
    """The gated delta rule over the tokens of each request row, from and into state [slots, heads, value_dim,
    key_dim] (32-bit): per head S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  qkv, beta and
    decay as delta_rule_prepare leaves them (decay [tokens, heads * key_dim] means one decay per key channel); out
    [tokens, heads * value_dim] 32-bit."""
    _cuda(qkv, beta, decay, state, query_starts, state_slots, positions, out)
    tokens = qkv.shape[0]
    rows = query_starts.numel() - 1
    per_channel = decay.shape[1] != heads
    for tensor, shape in ((qkv, (tokens, 2 * kv_heads * key_dim + heads * value_dim)), (beta, (tokens, heads)),
                          (decay, (tokens, heads * key_dim if per_channel else heads)),
                          (out, (tokens, heads * value_dim))):
        _require(tensor.dtype == torch.float32 and tensor.is_contiguous() and tensor.shape == shape,
                 "delta_rule_scan: qkv, beta, decay and out are contiguous float32 of the stated shapes")
    _require(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, value_dim, key_dim),
             "delta_rule_scan: the state is float32 [slots, heads, value_dim, key_dim]")
    lib = library("core")
    _check(lib, lib.mir_delta_rule_scan(int(per_channel), qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(),
                                        state.data_ptr(), query_starts.data_ptr(), state_slots.data_ptr(),
                                        positions.data_ptr(), out.data_ptr(), tokens, rows, heads, kv_heads, key_dim,
                                        value_dim, _stream()))


def set_delta_rule_lanes(lanes: int) -> None:
    """For measurements: how many lanes share one column of the delta rule's state (8, 16 or 32; 0: the launcher's
    own choice)."""
    for name in _LIBS or {"core": None}:
        lib = library(name)
        if hasattr(lib, "mir_delta_rule_set_lanes"):
            lib.mir_delta_rule_set_lanes.argtypes = [c_int]
            lib.mir_delta_rule_set_lanes.restype = c_int
            _check(lib, lib.mir_delta_rule_set_lanes(int(lanes)))


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, heads: int,
                    value_dim: int, eps: float, sigmoid_gate: bool) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * act(gate[t, h]) per head, act = sigmoid or silu; o 32-bit
    [tokens, heads * value_dim], gate a view with unit column stride in out's dtype or in float32, out contiguous.
    The weight holds value_dim numbers (the same for every head) or heads * value_dim (a row per head)."""
    _cuda(o, gate, weight, out)
    tokens = o.shape[0]
    _require(o.dtype == torch.float32 and o.is_contiguous() and o.shape[1] == heads * value_dim
             and gate.shape == o.shape and gate.stride(1) == 1 and out.shape == o.shape and out.is_contiguous()
             and gate.dtype in (out.dtype, torch.float32) and weight.dtype == torch.float32
             and weight.numel() in (value_dim, heads * value_dim) and weight.is_contiguous(),
             "gated_head_norm: shapes or dtypes do not fit")
    lib = library("core")
    _check(lib, lib.mir_gated_head_norm(_is_bf16(out), int(gate.dtype == torch.float32), o.data_ptr(), gate.data_ptr(),
                                        gate.stride(0), weight.data_ptr(),
                                        out.data_ptr(), tokens, heads, value_dim, eps, int(sigmoid_gate),
                                        int(heads > 1 and weight.numel() == heads * value_dim), _stream()))


def gelu_erf(x: torch.Tensor) -> None:
    """x <- 0.5 x (1 + erf(x / sqrt 2)) in place, computed in 32-bit."""
    _cuda(x)
    _require(x.is_contiguous(), "gelu_erf: a contiguous tensor is needed")
    lib = library("core")
    _check(lib, lib.mir_activation(1, _is_bf16(x), x.data_ptr(), x.numel(), _stream()))


def tanh(x: torch.Tensor) -> None:
    """x <- tanh(x) in place, computed in 32-bit."""
    _cuda(x)
    _require(x.is_contiguous(), "tanh: a contiguous tensor is needed")
    lib = library("core")
    _check(lib, lib.mir_activation(2, _is_bf16(x), x.data_ptr(), x.numel(), _stream()))


def relu_squared(x: torch.Tensor) -> None:
    """x <- max(x, 0)^2 in place, computed in 32-bit."""
    _cuda(x)
    _require(x.is_contiguous(), "relu_squared: a contiguous tensor is needed")
    lib = library("core")
    _check(lib, lib.mir_activation(3, _is_bf16(x), x.data_ptr(), x.numel(), _stream()))


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap) in place on contiguous 32-bit logits."""
    _cuda(logits)
    _require(logits.dtype == torch.float32 and logits.is_contiguous(), "softcap: contiguous float32 logits are needed")
    lib = library("core")
    _check(lib, lib.mir_softcap(logits.data_ptr(), logits.numel(), float(cap), _stream()))


def add_rows(residual: torch.Tensor, rows: Optional[torch.Tensor], vector: Optional[torch.Tensor]) -> None:
    """residual[r] += rows[r] + vector on the 32-bit residual stream (either may be None)."""
    _cuda(residual, rows, vector)
    n, hidden = residual.shape
    _require(residual.dtype == torch.float32 and residual.is_contiguous()
             and (rows is None or (rows.dtype == torch.float32 and rows.shape == residual.shape and rows.is_contiguous()))
             and (vector is None or (vector.dtype == torch.float32 and vector.numel() == hidden and vector.is_contiguous())),
             "add_rows: float32 rows of the residual's shape and a float32 vector of its width")
    if rows is None and vector is None:
        return
    lib = library("core")
    _check(lib, lib.mir_add_rows(residual.data_ptr(), _ptr(rows), _ptr(vector), n, hidden, _stream()))


def rms_norm_pair(x: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float, out_a: torch.Tensor,
                  out_b: torch.Tensor) -> None:
    """out_a = rmsnorm(x) * weight_a and out_b = rmsnorm(x) * weight_b in one pass over the 32-bit rows x."""
    _cuda(x, weight_a, weight_b, out_a, out_b)
    rows, hidden = x.shape
    _require(x.dtype == torch.float32 and x.is_contiguous() and out_a.shape == x.shape and out_b.shape == x.shape
             and out_a.is_contiguous() and out_b.is_contiguous() and out_a.dtype == out_b.dtype
             and all(w.dtype == torch.float32 and w.numel() == hidden and w.is_contiguous() for w in (weight_a, weight_b)),
             "rms_norm_pair: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_rms_norm_pair(_is_bf16(out_a), x.data_ptr(), weight_a.data_ptr(), weight_b.data_ptr(),
                                      out_a.data_ptr(), out_b.data_ptr(), rows, hidden, eps, _stream()))


# --------------------------------------------------------------------------- latent attention
def latent_prepare(packed: torch.Tensor, q_offset: int, q_rank: int, kv_offset: int, kv_rank: int, rotary_dim: int,
                   q_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float, positions: torch.Tensor,
                   slot_mapping: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], magnitude: float,
                   interleaved: bool, latent_q: torch.Tensor, pages: Optional[torch.Tensor]) -> None:
    """Per token of the packed projection `packed` [tokens, >= offsets + widths]: latent_q = rmsnorm(packed[q_offset :
    + q_rank]) * q_norm; the token's cache row pages[slot] = [rmsnorm(packed[kv_offset : + kv_rank]) * kv_norm | the
    rotary_dim columns behind it rotated by the token's position].  Norms and angles are 32-bit.  A token whose slot
    is negative (or with slot_mapping None) writes no cache row."""
    _cuda(packed, q_norm, kv_norm, positions, slot_mapping, inv_freq, latent_q, pages)
    tokens = packed.shape[0]
    _require(packed.stride(1) == 1 and q_offset + q_rank <= packed.shape[1]
             and kv_offset + kv_rank + rotary_dim <= packed.shape[1] and latent_q.dtype == packed.dtype
             and latent_q.is_contiguous() and latent_q.shape == (tokens, q_rank)
             and q_norm.dtype == torch.float32 and q_norm.numel() == q_rank and kv_norm.dtype == torch.float32
             and kv_norm.numel() == kv_rank and positions.dtype == torch.int32 and positions.numel() >= tokens,
             "latent_prepare: shapes or dtypes do not fit")
    if slot_mapping is not None:
        _require(slot_mapping.dtype == torch.int32 and pages is not None and pages.dtype == packed.dtype
                 and pages.is_contiguous() and pages[0].numel() == kv_rank + rotary_dim,
                 "latent_prepare: cache rows of kv_rank + rotary_dim elements in the activations' dtype are needed")
    if rotary_dim:
        _require(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
                 "latent_prepare: the angle table must hold rotary_dim / 2 float32 values")
    lib = library("core")
    _check(lib, lib.mir_latent_prepare(_is_bf16(packed), packed.data_ptr(), packed.stride(0), q_offset, q_rank, kv_offset,
                                       kv_rank, rotary_dim, q_norm.data_ptr(), kv_norm.data_ptr(), eps,
                                       positions.data_ptr(), _ptr(slot_mapping), _ptr(inv_freq), float(magnitude),
                                       int(interleaved), latent_q.data_ptr(), _ptr(pages), tokens, _stream()))


def rope_rows(src: torch.Tensor, dst: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, magnitude: float,
              interleaved: bool) -> None:
    """dst[t, h, :r] = src[t, h, :r] rotated by positions[t], r = 2 * len(inv_freq): pairs (i, i + r/2) or, interleaved,
    (2i, 2i + 1); cos and sin times `magnitude`; angles are 32-bit.  src and dst are [tokens, heads, >= r] views with
    unit stride in the last dimension and may be the same tensor."""
    _cuda(src, dst, positions, inv_freq)
    tokens, heads = src.shape[0], src.shape[1]
    rotary = 2 * inv_freq.numel()
    _require(src.dim() == 3 and dst.dim() == 3 and dst.shape[:2] == src.shape[:2] and src.stride(2) == 1
             and dst.stride(2) == 1 and src.shape[2] >= rotary and dst.shape[2] >= rotary and src.dtype == dst.dtype
             and positions.dtype == torch.int32 and positions.numel() >= tokens and inv_freq.dtype == torch.float32,
             "rope_rows: [tokens, heads, dims] views of one dtype are needed")
    lib = library("core")
    _check(lib, lib.mir_rope_rows(_is_bf16(src), src.data_ptr(), src.stride(0), src.stride(1), dst.data_ptr(),
                                  dst.stride(0), dst.stride(1), positions.data_ptr(), inv_freq.data_ptr(),
                                  float(magnitude), int(interleaved), tokens, heads, rotary, _stream()))


HEAD_LINEAR_LIBRARY = True       # False: the products per head always run the 32-bit multiply-add kernel


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = weight[h]^T x[t, h, :] for weight [heads, in, out] (a product per head; 32-bit accumulation),
    times sigmoid(gate[t, h, :]) if a gate [tokens, heads * out] (unit column stride) is given.  x [tokens, heads, in]
    and out [tokens, heads, out] are views with unit stride in the last dimension.  bfloat16 views whose rows and
    heads start on 16-byte boundaries run as one batched library product (the heads are the batch) followed by the
    gate's kernel; everything else runs our kernel, in which every output is one ascending chain."""
    _cuda(x, weight, out, gate)
    tokens, heads, in_dim = x.shape
    out_dim = weight.shape[2]
    _require(weight.shape == (heads, in_dim, out_dim) and weight.is_contiguous() and out.shape == (tokens, heads, out_dim)
             and x.stride(2) == 1 and out.stride(2) == 1 and x.dtype == weight.dtype == out.dtype,
             "head_linear: x [tokens, heads, in], weight [heads, in, out], out [tokens, heads, out] of one dtype")
    if gate is not None:
        _require(gate.shape == (tokens, heads * out_dim) and gate.stride(1) == 1 and gate.dtype == x.dtype,
                 "head_linear: the gate is [tokens, heads * out] in the activations' dtype")
    aligned = all(v % 8 == 0 for v in (in_dim, out_dim, x.stride(0), x.stride(1), out.stride(0), out.stride(1))) \
        and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
    if HEAD_LINEAR_LIBRARY and x.dtype == torch.bfloat16 and aligned and tokens > 0:
        lib = library("bf16")
        workspace = _lt_workspace(x.device)
        _check(lib, lib.mir_gemm_bf16_lt_batched(x.data_ptr(), x.stride(0), x.stride(1), weight.data_ptr(), out.data_ptr(),
                                                 out.stride(0), out.stride(1), tokens, out_dim, in_dim, heads,
                                                 workspace.data_ptr(), workspace.numel(), _stream()))
        if gate is not None:
            _require(out.stride(1) == out_dim, "head_linear: a gated result has its heads side by side")
            core = library("core")
            _check(core, core.mir_sigmoid_gate(1, out.data_ptr(), out.stride(0), gate.data_ptr(), gate.stride(0), tokens,
                                               heads * out_dim, _stream()))
        return
    lib = library("core")
    _check(lib, lib.mir_head_linear(_is_bf16(x), x.data_ptr(), x.stride(0), x.stride(1), weight.data_ptr(), out.data_ptr(),
                                    out.stride(0), out.stride(1), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                    tokens, heads, in_dim, out_dim, _stream()))


LATENT_TENSOR_CORES = True       # False: attention over cached latents always runs the reference kernel


def latent_attention_takes(width: int, rank: int) -> bool:
    """Whether the tensor-core kernel for attention over cached latents takes rows of `width` numbers whose first
    `rank` are the value (bfloat16 only)."""
    return bool(LATENT_TENSOR_CORES and library("bf16").mir_latent_attention_takes(width, rank))


def latent_attention_plan(num_rows: int, max_pairs: int, max_context: int) -> tuple:
    """(keys per partition, partitions) for a step of `num_rows` request rows, the largest of which brings max_pairs
    (token, head) pairs, over at most max_context keys: the keys are split where the query rows alone would leave
    most of the GPU idle (decoded tokens)."""
    blocks = max(1, num_rows * (-(-max_pairs // 64)))
    tiles = max(1, -(-max_context // 64))
    sms = 148
    # one wave of CTAs, two tiles or more a partition (measured at 8 rows x 2,049 keys: 31 us with 17 partitions, 43
    # with 33, 65 with 4; at 64 rows 123 us with 2, 133 with 4)
    partitions = max(1, min(max(1, tiles // 2), sms // blocks, 64))
    per_partition = -(-tiles // partitions) * 64
    return per_partition, -(-max_context // per_partition) if max_context > 0 else 1


def latent_attention(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     query_starts: torch.Tensor, context_lens: torch.Tensor, page_size: int, heads: int, width: int,
                     rank: int, scale: float, max_pairs: int, partition_keys: int, partitions: int, alloc) -> None:
    """out[t, h] = softmax over the cached rows of token t's request up to its own position, on tensor cores: q
    [tokens, heads * width] bfloat16 folded queries, pages [cache rows, 1, width] of which the first `rank` numbers of
    a row are its value, out [tokens, heads * rank].  Request row r brings the tokens query_starts[r] ..
    query_starts[r + 1] and has context_lens[r] keys after the step.  With partitions > 1 the keys are walked in
    shares of partition_keys and merged by a second kernel (scratch from `alloc`)."""
    _cuda(q, out, pages, block_table, query_starts, context_lens)
    tokens = q.shape[0]
    rows = query_starts.numel() - 1
    _require(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
             and q.stride(1) == 1 and q.shape[1] == heads * width and out.is_contiguous()
             and out.shape == (tokens, heads * rank) and pages.is_contiguous() and pages[0].numel() == width
             and block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
             and block_table.shape[0] >= rows and query_starts.dtype == torch.int32 and context_lens.dtype == torch.int32
             and context_lens.numel() >= rows, "latent_attention: shapes or dtypes do not fit")
    partial_o = partial_ml = None
    if partitions > 1:
        partial_o = alloc((tokens * heads * partitions, rank), torch.float32)
        partial_ml = alloc((tokens * heads * partitions, 2), torch.float32)
    lib = library("bf16")
    _check(lib, lib.mir_latent_attention_bf16(q.data_ptr(), q.stride(0), out.data_ptr(), pages.data_ptr(),
                                              block_table.data_ptr(), block_table.shape[1], query_starts.data_ptr(),
                                              context_lens.data_ptr(), rows, tokens, max_pairs, page_size, heads, width,
                                              rank, scale, partition_keys, partitions, _ptr(partial_o), _ptr(partial_ml),
                                              _stream()))


# --------------------------------------------------------------------------- wkv
def wkv_mix(h: torch.Tensor, tail: torch.Tensor, mu: torch.Tensor, row_of_token: torch.Tensor,
            query_starts: torch.Tensor, state_slots: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
            single_tokens_only: bool = False) -> None:
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s] for the five mixes s; h[t - 1] of a portion's first token is the
    request's tail [slots, width] (32-bit; zeros at its start), which moves on to the portion's last row.
    `single_tokens_only`: every request brings one token (the tails then move on inside the one kernel)."""
    _cuda(h, tail, mu, row_of_token, query_starts, state_slots, positions, out)
    tokens, width = h.shape
    rows = query_starts.numel() - 1
    _require(h.stride(1) == 1 and tail.dtype == torch.float32 and tail.is_contiguous() and tail.shape[1] == width
             and mu.dtype == torch.float32 and mu.is_contiguous() and mu.shape == (5, width)
             and out.dtype == h.dtype and out.is_contiguous() and out.shape == (5, tokens, width),
             "wkv_mix: shapes or dtypes do not fit")
    _require(all(t.dtype == torch.int32 for t in (row_of_token, query_starts, state_slots, positions)),
             "wkv_mix: the batch description is int32")
    lib = library("core")
    _check(lib, lib.mir_wkv_mix(_is_bf16(h), h.data_ptr(), h.stride(0), tail.data_ptr(), mu.data_ptr(),
                                row_of_token.data_ptr(), query_starts.data_ptr(), state_slots.data_ptr(),
                                positions.data_ptr(), out.data_ptr(), tokens, rows, width, int(single_tokens_only),
                                _stream()))


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_raw: torch.Tensor, decay_bias: torch.Tensor,
             bonus: torch.Tensor, state: torch.Tensor, query_starts: torch.Tensor, state_slots: torch.Tensor,
             positions: torch.Tensor, out: torch.Tensor, heads: int, dim: int) -> None:
    """The wkv recurrence over the tokens of each request row, from and into state [slots, heads, dim (value channel),
    dim (key channel)] (32-bit): per head o = S^T r + (sum_i r_i u_i k_i) v; S <- diag(w) S + k v^T with
    w = exp(-exp(decay_raw + decay_bias)).  r, k, v [tokens, heads * dim] (one row stride, the activations' dtype);
    decay_raw 32-bit [tokens, heads * dim]; decay_bias, bonus (u) 32-bit [heads * dim]; out 32-bit [tokens, heads * dim]."""
    _cuda(r, k, v, decay_raw, decay_bias, bonus, state, query_starts, state_slots, positions, out)
    tokens = r.shape[0]
    rows = query_starts.numel() - 1
    width = heads * dim
    _require(all(t.shape == (tokens, width) and t.stride(1) == 1 and t.stride(0) == r.stride(0) and t.dtype == r.dtype
                 for t in (r, k, v)), "wkv_scan: r, k, v are [tokens, heads * dim] with one row stride and dtype")
    _require(decay_raw.dtype == torch.float32 and decay_raw.is_contiguous() and decay_raw.shape == (tokens, width)
             and out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, width)
             and all(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == width for t in (decay_bias, bonus))
             and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, dim),
             "wkv_scan: decays, bonus, state and out are contiguous float32 of the stated shapes")
    lib = library("core")
    _check(lib, lib.mir_wkv_scan(_is_bf16(r), r.data_ptr(), k.data_ptr(), v.data_ptr(), r.stride(0), decay_raw.data_ptr(),
                                 decay_bias.data_ptr(), bonus.data_ptr(), state.data_ptr(), query_starts.data_ptr(),
                                 state_slots.data_ptr(), positions.data_ptr(), out.data_ptr(), tokens, rows, heads, dim,
                                 _stream()))


# --------------------------------------------------------------------------- retention
def retention_prepared_floats(tokens: int, heads: int, dim: int) -> int:
    """How many 32-bit numbers retention_scan's `prepared` scratch holds: per token and head the rotated q and k, padded
    to the kernel's width for heads of `dim` key channels, and q . k."""
    padded = next((width for width in (32, 64, 128, 192, 256) if dim <= width), dim)
    return tokens * heads * (2 * padded + 4)


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, inv_freq: Optional[torch.Tensor],
                   decays: torch.Tensor, key_scale: float, state: torch.Tensor, query_starts: torch.Tensor,
                   state_slots: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, heads: int, dim: int,
                   value_dim: int, prepared: Optional[torch.Tensor] = None) -> None:
    """The retention recurrence over the tokens of each request row, from and into state [slots, heads, value_dim, dim]
    (32-bit): per head S <- decay_h S + k v^T, o = S^T q, with q and k rotated by the token's position (half-split pairs
    of the first 2 * len(inv_freq) channels, 32-bit angles) and k times `key_scale` after the rotation.  q, k [tokens,
    heads * dim] and v [tokens, heads * value_dim]: views with one row stride in the activations' dtype; decays 32-bit
    [heads]; out 32-bit [tokens, heads * value_dim].  With `prepared` (32-bit scratch of retention_prepared_floats
    numbers) a step that brings more than single tokens rotates in a kernel of its own, once per token and head, and
    the walk copies what that left; the results are the same bits either way."""
    _cuda(q, k, v, inv_freq, decays, state, query_starts, state_slots, positions, out, prepared)
    _require(prepared is None or (prepared.dtype == torch.float32 and prepared.is_contiguous()
                                  and prepared.numel() >= retention_prepared_floats(q.shape[0], heads, dim)),
             "retention_scan: prepared is float32 scratch of retention_prepared_floats numbers")
    tokens = q.shape[0]
    rows = query_starts.numel() - 1
    rotary = 0 if inv_freq is None else 2 * inv_freq.numel()
    _require(q.shape == (tokens, heads * dim) and k.shape == q.shape and v.shape == (tokens, heads * value_dim)
             and all(t.stride(1) == 1 and t.stride(0) == q.stride(0) and t.dtype == q.dtype for t in (q, k, v)),
             "retention_scan: q, k, v are views with one row stride and dtype")
    _require(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (tokens, heads * value_dim)
             and decays.dtype == torch.float32 and decays.is_contiguous() and decays.numel() == heads
             and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, value_dim, dim)
             and (inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.is_contiguous() and rotary <= dim)),
             "retention_scan: decays, state and out are contiguous float32 of the stated shapes")
    _require(all(t.dtype == torch.int32 for t in (query_starts, state_slots, positions)),
             "retention_scan: the batch description is int32")
    lib = library("core")
    _check(lib, lib.mir_retention_scan(_is_bf16(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0),
                                       _ptr(inv_freq), rotary, decays.data_ptr(), float(key_scale), state.data_ptr(),
                                       query_starts.data_ptr(), state_slots.data_ptr(), positions.data_ptr(),
                                       out.data_ptr(), _ptr(prepared), tokens, rows, heads, dim, value_dim, _stream()))


# --------------------------------------------------------------------------- routed experts
def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], has_gate: bool, ids: torch.Tensor,
              weights: torch.Tensor, shared_gate: Optional[torch.Tensor], experts: int, top: int, groups: int, keep: int,
              scale: float, score: str = "sigmoid", group_score: str = "top2") -> None:
    """Per token, from the router's 32-bit logits [tokens, >= experts (+ 1)]: scores = sigmoid(logits), or with
    `score` "softmax" the softmax over the `experts` logits; the `top` experts with the largest score + correction
    among the experts of the `keep` best of `groups` groups of neighbours (a group's score: the sum of its two largest
    score + correction, or with `group_score` "max" the largest) -> ids [tokens, top]; weights [tokens, top] = their
    scores / their sum * scale; with has_gate, shared_gate[t] = sigmoid(logits[t, experts])."""
    _require(score in ("sigmoid", "softmax") and group_score in ("top2", "max"), "moe_route: unknown score rule")
    _cuda(logits, correction, ids, weights, shared_gate)
    tokens = logits.shape[0]
    _require(logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= experts + int(has_gate)
             and (correction is None or (correction.dtype == torch.float32 and correction.numel() == experts))
             and ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (tokens, top)
             and weights.dtype == torch.float32 and weights.is_contiguous() and weights.shape == (tokens, top)
             and (not has_gate or (shared_gate is not None and shared_gate.dtype == torch.float32
                                   and shared_gate.numel() >= tokens)), "moe_route: shapes or dtypes do not fit")
    lib = library("core")
    _check(lib, lib.mir_moe_route(logits.data_ptr(), logits.stride(0), _ptr(correction), int(has_gate), ids.data_ptr(),
                                  weights.data_ptr(), _ptr(shared_gate), tokens, experts, top, groups, keep, float(scale),
                                  int(score == "softmax"), int(group_score == "max"), _stream()))


class ExpertOrder:
    """The pairs (token, chosen expert) of a step ordered by expert, on the device: order [pairs] (sorted place ->
    pair), offsets [experts + 1], tiles [2 * slots] and tile_count [1] for the grouped products."""

    def __init__(self, alloc, pairs: int, experts: int, tile_pairs: int = 8):
        lib = library("core")
        slots = int(lib.mir_moe_tile_slots(pairs, experts, tile_pairs))
        self.pairs, self.experts, self.tile_pairs = pairs, experts, tile_pairs
        self.order = alloc((pairs,), torch.int32)
        self.offsets = alloc((experts + 1,), torch.int32)
        self.tiles = alloc((2 * slots,), torch.int32)
        self.tile_count = alloc((1,), torch.int32)
        self.scratch = alloc((2, experts), torch.int32)            # counts and first tiles while sorting


EXPERT_TENSOR_CORES = True       # False: the grouped products of routed experts always run as 32-bit multiply-adds


def expert_tile_pairs(dtype: torch.dtype, width: int, inter: int) -> int:
    """The tile the grouped products of routed experts work on.  bfloat16 rows of 16-byte pieces: tiles of 128 pairs
    through the tcgen05 product (TMA, accumulators in tensor memory; it beats a kernel that streams an expert's weights
    for a tile of few pairs at every size measured, 49 against 82 us at 8 tokens).  Everything else: tiles of 8 pairs
    with 32-bit multiply-adds."""
    return 128 if (EXPERT_TENSOR_CORES and dtype == torch.bfloat16 and width % 8 == 0 and inter % 8 == 0) else 8


def moe_sort(ids: torch.Tensor, experts: int, alloc, tile_pairs: int = 8) -> ExpertOrder:
    """Order the pairs of ids [tokens, top] by expert (a pair's place among its expert's pairs follows its index) and
    cut each expert's run into tiles of tile_pairs (8 or 128) pairs."""
    _cuda(ids)
    _require(ids.dtype == torch.int32 and ids.is_contiguous(), "moe_sort: contiguous int32 ids are needed")
    found = ExpertOrder(alloc, ids.numel(), experts, tile_pairs)
    lib = library("core")
    _check(lib, lib.mir_moe_sort(ids.data_ptr(), ids.numel(), experts, tile_pairs, found.order.data_ptr(),
                                 found.offsets.data_ptr(), found.tiles.data_ptr(), found.tile_count.data_ptr(),
                                 found.scratch[0].data_ptr(), found.scratch[1].data_ptr(), _stream()))
    return found


def moe_gate_up(h: torch.Tensor, found: ExpertOrder, top: int, w_gate: torch.Tensor, w_up: torch.Tensor,
                hidden: torch.Tensor, alloc=None) -> None:
    """hidden[i] = silu(w_gate[e] x) * (w_up[e] x) for the i-th pair in expert order, x its token's row of h and e its
    expert; w_gate, w_up [experts, inter, width]; hidden [pairs, inter].  With tiles of 128 pairs (the tcgen05 product)
    the tokens' rows are first brought into the pairs' order (scratch from `alloc`), and w_up must lie right behind
    w_gate in memory (the two halves of one tensor)."""
    _cuda(h, w_gate, w_up, hidden)
    tokens, width = h.shape
    experts, inter = w_gate.shape[0], w_gate.shape[1]
    _require(h.stride(1) == 1 and w_gate.shape == (experts, inter, width) and w_up.shape == w_gate.shape
             and w_gate.is_contiguous() and w_up.is_contiguous() and hidden.is_contiguous()
             and hidden.shape == (found.pairs, inter) and found.pairs == tokens * top and found.experts == experts
             and h.dtype == w_gate.dtype == w_up.dtype == hidden.dtype, "moe_gate_up: shapes or dtypes do not fit")
    if found.tile_pairs == 128:
        _require(h.dtype == torch.bfloat16 and alloc is not None
                 and w_up.data_ptr() == w_gate.data_ptr() + w_gate.numel() * 2,
                 "moe_gate_up: the tcgen05 product takes bfloat16, scratch memory and w_up right behind w_gate")
        ordered = alloc((found.pairs, width), torch.bfloat16)
        core = library("core")
        _check(core, core.mir_moe_gather_rows(h.data_ptr(), h.stride(0), found.order.data_ptr(), top, ordered.data_ptr(),
                                              found.pairs, width, found.offsets[experts:].data_ptr(), _stream()))
        lib = library("bf16")
        _check(lib, lib.mir_gemm_tc_grouped_bf16(MODE_SWIGLU, ordered.data_ptr(), width, found.pairs, w_gate.data_ptr(),
                                                 experts, hidden.data_ptr(), inter, inter, width, found.tiles.data_ptr(),
                                                 found.tile_count.data_ptr(), found.offsets.data_ptr(), None,
                                                 found.pairs // 128 + experts, _stream()))
        return
    lib = library("core")
    _check(lib, lib.mir_moe_gate_up(_is_bf16(h), h.data_ptr(), h.stride(0), found.order.data_ptr(), top,
                                    w_gate.data_ptr(), w_up.data_ptr(), hidden.data_ptr(), found.tiles.data_ptr(),
                                    found.tile_count.data_ptr(), found.offsets.data_ptr(), found.pairs, experts, width,
                                    inter, found.tile_pairs, _stream()))


def moe_down(hidden: torch.Tensor, found: ExpertOrder, w_down: torch.Tensor, pair_rows: torch.Tensor) -> None:
    """pair_rows[pair] = w_down[e] hidden[i] (32-bit [pairs, width]) for the i-th pair in expert order."""
    _cuda(hidden, w_down, pair_rows)
    experts, width, inter = w_down.shape
    _require(hidden.is_contiguous() and hidden.shape == (found.pairs, inter) and w_down.is_contiguous()
             and hidden.dtype == w_down.dtype and pair_rows.dtype == torch.float32 and pair_rows.is_contiguous()
             and pair_rows.shape == (found.pairs, width) and found.experts == experts,
             "moe_down: shapes or dtypes do not fit")
    if found.tile_pairs == 128:
        _require(hidden.dtype == torch.bfloat16, "moe_down: the tcgen05 product takes bfloat16")
        lib = library("bf16")
        _check(lib, lib.mir_gemm_tc_grouped_bf16(MODE_F32, hidden.data_ptr(), inter, found.pairs, w_down.data_ptr(), experts,
                                                 pair_rows.data_ptr(), width, width, inter, found.tiles.data_ptr(),
                                                 found.tile_count.data_ptr(), found.offsets.data_ptr(),
                                                 found.order.data_ptr(), found.pairs // 128 + experts, _stream()))
        return
    lib = library("core")
    _check(lib, lib.mir_moe_down(_is_bf16(hidden), hidden.data_ptr(), found.order.data_ptr(), w_down.data_ptr(),
                                 pair_rows.data_ptr(), found.tiles.data_ptr(), found.tile_count.data_ptr(),
                                 found.offsets.data_ptr(), found.pairs, experts, width, inter, found.tile_pairs, _stream()))


def moe_combine(residual: torch.Tensor, pair_rows: torch.Tensor, weights: torch.Tensor,
                shared_rows: Optional[torch.Tensor], shared_gate: Optional[torch.Tensor], overwrite: bool = False,
                ids: Optional[torch.Tensor] = None, real_experts: int = 0,
                identity_rows: Optional[torch.Tensor] = None) -> None:
    """residual[t] += sum_s weights[t, s] * pair_rows[t * top + s] + shared_gate[t] * shared_rows[t] (the gate 1 if
    None; nothing of it without shared_rows); all 32-bit.  `overwrite`: the sum replaces residual[t].  With `ids`
    ([tokens, top] int32), a slot whose id is >= real_experts is an identity expert: it adds its weight times the
    token's row of `identity_rows` (the experts' input, bfloat16 or float32) and has no row in pair_rows."""
    _cuda(residual, pair_rows, weights, shared_rows, shared_gate, ids, identity_rows)
    _require(ids is None or (ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == weights.shape
                             and identity_rows is not None and identity_rows.stride(1) == 1
                             and identity_rows.shape == residual.shape
                             and identity_rows.dtype in (torch.bfloat16, torch.float32)),
             "moe_combine: identity experts need int32 ids and the tokens' input rows")
    tokens, width = residual.shape
    top = weights.shape[1]
    _require(residual.dtype == torch.float32 and residual.is_contiguous() and pair_rows.dtype == torch.float32
             and pair_rows.is_contiguous() and pair_rows.shape == (tokens * top, width) and weights.dtype == torch.float32
             and weights.is_contiguous() and weights.shape[0] == tokens
             and (shared_rows is None or (shared_rows.dtype == torch.float32 and shared_rows.is_contiguous()
                                          and shared_rows.shape == residual.shape))
             and (shared_gate is None or (shared_gate.dtype == torch.float32 and shared_gate.numel() >= tokens)),
             "moe_combine: shapes or dtypes do not fit")
    lib = library("core")
    _check(lib, lib.mir_moe_combine(residual.data_ptr(), pair_rows.data_ptr(), weights.data_ptr(), _ptr(shared_rows),
                                    _ptr(shared_gate), tokens, width, top, int(overwrite), _ptr(ids), int(real_experts),
                                    int(identity_rows is not None and identity_rows.dtype == torch.bfloat16),
                                    _ptr(identity_rows) if ids is not None else None,
                                    identity_rows.stride(0) if ids is not None else 0, _stream()))


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
               rows: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None) -> None:
    """out[r] = (u - mean(u)) / sqrt(var(u) + eps) * weight + bias, var the mean of the squared deviations, everything
    32-bit.  u is row rows[r] (or r) of x [tokens, width]; with `read` ([S] float32), x is a residual of S streams
    [tokens, S, width] and u = sum_s read[s] x[token, s]."""
    _cuda(x, weight, bias, out, rows, read)
    n_rows, width = out.shape
    _require(x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == width
             and (bias is None or (bias.dtype == torch.float32 and bias.numel() == width)) and out.is_contiguous()
             and out.dtype in (torch.bfloat16, torch.float32), "layer_norm: bad arguments")
    streams = 0
    if read is not None:
        _require(x.dim() == 3 and x.shape[2] == width and read.dtype == torch.float32 and read.numel() == x.shape[1],
                 "layer_norm: a mix of streams needs x [tokens, streams, width] and float32 [streams] factors")
        streams = x.shape[1]
    else:
        _require(x.dim() == 2 and x.shape[1] == width, "layer_norm: x must be [tokens, width]")
    if rows is not None:
        _require(rows.dtype == torch.int32 and rows.numel() == n_rows, "layer_norm: bad row index")
    else:
        _require(x.shape[0] >= n_rows, "layer_norm: fewer input rows than output rows")
    lib = library("core")
    _check(lib, lib.mir_layer_norm(_is_bf16(out), x.data_ptr(), streams, _ptr(read), weight.data_ptr(), _ptr(bias),
                                   out.data_ptr(), _ptr(rows), n_rows, width, eps, _stream()))


def streams_write(streams: torch.Tensor, branch: torch.Tensor, mix: torch.Tensor, write: torch.Tensor) -> None:
    """A residual of S streams [tokens, S, width] takes a sublayer's result `branch` [tokens, width], in place and all
    streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + write[t] * branch.  All 32-bit."""
    _cuda(streams, branch, mix, write)
    tokens, count, width = streams.shape
    _require(streams.dtype == torch.float32 and streams.is_contiguous() and branch.dtype == torch.float32
             and branch.is_contiguous() and branch.shape == (tokens, width) and mix.dtype == torch.float32
             and mix.is_contiguous() and mix.shape == (count, count) and write.dtype == torch.float32
             and write.numel() == count, "streams_write: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_streams_write(streams.data_ptr(), branch.data_ptr(), mix.data_ptr(), write.data_ptr(), tokens,
                                      count, width, _stream()))


def streams_write_norm(streams: torch.Tensor, branch: torch.Tensor, mix: torch.Tensor, write: torch.Tensor,
                       read: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
                       out: torch.Tensor) -> None:
    """streams_write, and in the same pass over a token out = layer_norm(sum_s read[s] x_s) of the streams as the update
    leaves them (what layer_norm with `read` would give for them): the next sublayer's input without a second trip of
    the streams through memory.  Without `weight`, out is the mix itself (with `read` of ones: the sum of the streams
    that the model ends with)."""
    _cuda(streams, branch, mix, write, read, weight, bias, out)
    tokens, count, width = streams.shape
    _require(streams.dtype == torch.float32 and streams.is_contiguous() and branch.dtype == torch.float32
             and branch.is_contiguous() and branch.shape == (tokens, width) and mix.dtype == torch.float32
             and mix.is_contiguous() and mix.shape == (count, count) and write.dtype == torch.float32
             and write.numel() == count and read.dtype == torch.float32 and read.numel() == count
             and (weight is None or (weight.dtype == torch.float32 and weight.numel() == width))
             and (bias is None or (weight is not None and bias.dtype == torch.float32 and bias.numel() == width))
             and out.is_contiguous()
             and out.shape == (tokens, width) and out.dtype in (torch.bfloat16, torch.float32),
             "streams_write_norm: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_streams_write_norm(_is_bf16(out), streams.data_ptr(), branch.data_ptr(), mix.data_ptr(),
                                           write.data_ptr(), read.data_ptr(), _ptr(weight), _ptr(bias), out.data_ptr(),
                                           tokens, count, width, eps, _stream()))


def streams_spread(x: torch.Tensor, streams: torch.Tensor) -> None:
    """Every stream of streams [tokens, S, width] becomes a copy of x [tokens, width] (32-bit)."""
    _cuda(x, streams)
    tokens, count, width = streams.shape
    _require(x.dtype == torch.float32 and streams.dtype == torch.float32 and x.is_contiguous()
             and streams.is_contiguous() and x.shape == (tokens, width), "streams_spread: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_streams_spread(x.data_ptr(), streams.data_ptr(), tokens, count, width, _stream()))


def streams_sum(streams: torch.Tensor, out: torch.Tensor) -> None:
    """out [tokens, width] = the sum of the streams [tokens, S, width], streams in ascending order (32-bit)."""
    _cuda(streams, out)
    tokens, count, width = streams.shape
    _require(out.dtype == torch.float32 and streams.dtype == torch.float32 and out.is_contiguous()
             and streams.is_contiguous() and out.shape == (tokens, width), "streams_sum: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_streams_sum(streams.data_ptr(), out.data_ptr(), tokens, count, width, _stream()))


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r] if rows else r]) * weight; x and weight are 32-bit."""
    _cuda(x, weight, out, rows)
    n_rows, hidden = out.shape
    _require(x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
             and x.shape[1] == hidden and weight.numel() == hidden, "rms_norm: bad arguments")
    if rows is not None:
        _require(rows.dtype == torch.int32 and rows.numel() == n_rows, "rms_norm: bad row index")
    else:
        _require(x.shape[0] >= n_rows, "rms_norm: fewer input rows than output rows")
    lib = library("core")
    _check(lib, lib.mir_rms_norm(_is_bf16(out), x.data_ptr(), weight.data_ptr(), out.data_ptr(), _ptr(rows), n_rows,
                                 hidden, eps, _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, I + c]."""
    _cuda(gate_up, out)
    rows, inter = out.shape
    _require(gate_up.shape == (rows, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous()
             and gate_up.dtype == out.dtype, "silu_mul: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_silu_mul(_is_bf16(out), gate_up.data_ptr(), out.data_ptr(), rows, inter, _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    _cuda(x, bias)
    rows, cols = x.shape
    _require(x.dtype == torch.float32 and x.is_contiguous() and bias.numel() == cols, "add_bias: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_add_bias(_is_bf16(bias), x.data_ptr(), bias.data_ptr(), rows, cols, _stream()))


CAST_KINDS = {(torch.float32, torch.bfloat16): 0, (torch.bfloat16, torch.float32): 1, (torch.float16, torch.bfloat16): 2,
              (torch.float16, torch.float32): 3}


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """Copy of equal shapes between what a checkpoint stores and what the engine keeps: float32 <-> bfloat16,
    float16 -> bfloat16 or float32 (load-time casts, libmir dense_cast.cu)."""
    _cuda(src, dst)
    _require(src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel(), "cast: bad arguments")
    kind = CAST_KINDS.get((src.dtype, dst.dtype))
    _require(kind is not None, f"cast: {src.dtype} -> {dst.dtype} is not supported")
    lib = library("core")
    _check(lib, lib.mir_cast(kind, src.data_ptr(), dst.data_ptr(), src.numel(), _stream()))


def random_normal(out: torch.Tensor, seed: int, deviation: float) -> None:
    """out (contiguous float32 or bfloat16, on the device) = deviation x normal deviates that depend on `seed` and
    the element's index only."""
    _cuda(out)
    _require(out.is_contiguous() and out.dtype in (torch.float32, torch.bfloat16), "random_normal: bad arguments")
    lib = library("core")
    lib.mir_random_normal.argtypes = [c_int, c_void_p, c_size_t, ctypes.c_ulonglong, c_float, c_void_p]
    lib.mir_random_normal.restype = c_int
    _check(lib, lib.mir_random_normal(int(out.dtype == torch.bfloat16), out.data_ptr(), out.numel(),
                                      seed & ((1 << 64) - 1), float(deviation), _stream()))


def decode_prepare(positions, block_table, page_size, slot_mapping, context_lens) -> None:
    """slot_mapping[r] and context_lens[r] of a decode batch from positions and block tables (on the device)."""
    rows = positions.numel()
    lib = library("core")
    _check(lib, lib.mir_decode_prepare(positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
                                       slot_mapping.data_ptr(), context_lens.data_ptr(), rows, _stream()))


def decode_advance(sampled, tokens, positions, token_log, step_counter, previous=None) -> None:
    """tokens <- sampled, positions += 1, token_log[step] <- sampled, step += 1 (on the device); with `previous`,
    previous <- tokens first (for an embedding that looks at pairs of tokens)."""
    rows = tokens.numel()
    lib = library("core")
    _check(lib, lib.mir_decode_advance(sampled.data_ptr(), tokens.data_ptr(), positions.data_ptr(),
                                       token_log.data_ptr(), token_log.shape[0], step_counter.data_ptr(), rows,
                                       _ptr(previous), _stream()))


# --------------------------------------------------------------------------- attention
def qk_rope_store(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                  k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int, rotary_dim: int, eps: float, write_kv: bool = True,
                  keys_in_place: bool = False, value_dim: Optional[int] = None, interleaved: bool = False,
                  queries_only: bool = False) -> None:
    """q/k-norm + rotary on the packed qkv rows in place for q, k and v into their pages.  `keys_in_place`:
    the keys are normed and rotated in place like the queries and nothing is written to the pages.  `interleaved`:
    the rotation pairs dims 2i and 2i + 1.  The rows may be wider than q, k and v (what lies behind them is left
    alone); `queries_only`: they start with the query heads and hold no keys or values."""
    write_kv = write_kv and not keys_in_place and not queries_only
    _cuda(qkv, positions, slot_mapping, inv_freq, q_norm, k_norm, k_pages, v_pages)
    tokens = qkv.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    packed = heads * head_dim if queries_only else (heads + kv_heads) * head_dim + kv_heads * value_dim
    _require(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= packed and qkv.stride(0) >= qkv.shape[1]
             and not (keys_in_place and queries_only), "qk_rope_store: bad qkv")
    _require(positions.dtype == torch.int32 and positions.numel() >= tokens, "qk_rope_store: bad positions")
    if rotary_dim:
        _require(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
                 "qk_rope_store: the angle table must hold rotary_dim / 2 float32 values")
    for norm in (q_norm, k_norm):
        _require(norm is None or (norm.dtype == torch.float32 and norm.numel() == head_dim),
                 "qk_rope_store: q/k norm weights must be float32 [head_dim]")
    if write_kv:
        _require(slot_mapping is not None and slot_mapping.dtype == torch.int32 and k_pages is not None
                 and v_pages is not None and k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype,
                 "qk_rope_store: cache pages of the activations' dtype and a slot mapping are needed")
    lib = library("core")
    _check(lib, lib.mir_qk_rope_store(_is_bf16(qkv), qkv.data_ptr(), positions.data_ptr(), _ptr(slot_mapping),
                                      _ptr(inv_freq), _ptr(q_norm), _ptr(k_norm), _ptr(k_pages), _ptr(v_pages),
                                      tokens, heads, kv_heads, head_dim, value_dim, rotary_dim, eps,
                                      2 if keys_in_place else int(write_kv), int(interleaved), qkv.stride(0),
                                      int(queries_only), _stream()))


QK_NORM_SPANS = {None: 0, "head": 1, "projection": 2}


def qk_prepare(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
               inv_freq: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
               k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int,
               value_dim: int, rotary_dim: int, eps: float, span: Optional[str], after_rotation: bool = False,
               write_kv: bool = True) -> None:
    """The q/k treatments that qk_rope_store does not know, on the packed rows in place for q, k and v into their
    pages: an RMS norm of q and of k with `span` "head" (every head by itself; the weights, if any, are float32
    [head_dim]), "projection" (q as a whole and k as a whole over all their heads; weights float32 [heads * head_dim]
    and [kv_heads * head_dim]) or None; the half-split rotation of the first rotary_dim channels of every head;
    `after_rotation`: the per-head norm follows the rotation.  The rows may be wider than q, k and v."""
    _cuda(qkv, positions, slot_mapping, inv_freq, q_weight, k_weight, k_pages, v_pages)
    _require(span in QK_NORM_SPANS, f"qk_prepare: unknown span {span!r}")
    tokens = qkv.shape[0]
    packed = (heads + kv_heads) * head_dim + kv_heads * value_dim
    _require(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= packed and qkv.stride(0) >= qkv.shape[1],
             "qk_prepare: bad qkv")
    _require(positions.dtype == torch.int32 and positions.numel() >= tokens, "qk_prepare: bad positions")
    if rotary_dim:
        _require(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
                 "qk_prepare: the angle table must hold rotary_dim / 2 float32 values")
    per = head_dim if span == "head" else 0
    for weight, count in ((q_weight, heads), (k_weight, kv_heads)):
        _require(weight is None or (span is not None and weight.dtype == torch.float32 and weight.is_contiguous()
                                    and weight.numel() == (per or count * head_dim)),
                 "qk_prepare: norm weights are float32, [head_dim] per head or [heads * head_dim] over the projection")
    if write_kv:
        _require(slot_mapping is not None and slot_mapping.dtype == torch.int32 and k_pages is not None
                 and v_pages is not None and k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype,
                 "qk_prepare: cache pages of the activations' dtype and a slot mapping are needed")
    lib = library("core")
    _check(lib, lib.mir_qk_prepare(_is_bf16(qkv), qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _ptr(slot_mapping),
                                   _ptr(inv_freq), _ptr(q_weight), _ptr(k_weight), _ptr(k_pages), _ptr(v_pages), tokens,
                                   heads, kv_heads, head_dim, value_dim, rotary_dim, eps, QK_NORM_SPANS[span],
                                   int(after_rotation), int(write_kv), _stream()))


def set_qk_prepare_resident_warps(warps: int) -> None:
    """For measurements: up to how many warps a CTA of qk_prepare may have to hold all heads of a token in registers
    for the norm over a projection (0: the row is always summed in a pass of its own)."""
    lib = library("core")
    lib.mir_qk_prepare_set_resident_warps.argtypes = [c_int]
    lib.mir_qk_prepare_set_resident_warps.restype = c_int
    _check(lib, lib.mir_qk_prepare_set_resident_warps(int(warps)))


def paged_attention_generic(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, row_of_token: torch.Tensor, positions: torch.Tensor,
                            page_size: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                            window: Optional[int], value_dim: Optional[int] = None, keep_first: int = 0,
                            values_in_keys: bool = False, sinks: Optional[torch.Tensor] = None,
                            gate: Optional[torch.Tensor] = None, gate_per_head: bool = False,
                            softcap: Optional[float] = None, distance_bias: Optional[torch.Tensor] = None) -> None:
    """out[t, h] = softmax over the visible cached keys of token t's request; q is read from the packed qkv rows.
    `value_dim`: width of a value head (head_dim if None); `keep_first`: with a window, the request's first keys
    that stay visible to every query; `values_in_keys`: a value is the first value_dim elements of its key (a cached
    latent that is read both ways) and v_pages is not looked at.  `sinks` (float32 [heads]): exp(sink_h) joins the
    denominator of head h's softmax.  `gate` ([tokens, heads * value_dim] view, unit column stride, out's dtype): the
    result is multiplied by its sigmoid; with `gate_per_head` it is [tokens, heads], one number per head.  `softcap`:
    score <- softcap * tanh(score / softcap) after the scale.  `distance_bias` (float32 [heads, rows]): row
    min(query position - key position, rows - 1) is added to the scores after the cap."""
    if values_in_keys:
        v_pages = k_pages
    _cuda(qkv, out, k_pages, v_pages, block_table, row_of_token, positions, sinks, gate, distance_bias)
    _require(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads and sinks.is_contiguous()),
             "paged_attention: sinks are float32 [heads]")
    _require(gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1
                              and gate.shape == ((out.shape[0], heads) if gate_per_head else out.shape)),
             "paged_attention: the gate has out's dtype and out's shape, or one column per head")
    _require(distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.is_contiguous()
                                       and distance_bias.dim() == 2 and distance_bias.shape[0] == heads
                                       and distance_bias.shape[1] > 0),
             "paged_attention: the bias by distance is float32 [heads, rows]")
    tokens = out.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    _require(out.is_contiguous() and out.shape[1] == heads * value_dim and qkv.dtype == out.dtype
             and k_pages.dtype == out.dtype and v_pages.dtype == out.dtype, "paged_attention: bad tensors")
    _require(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
             and row_of_token.dtype == torch.int32 and positions.dtype == torch.int32, "paged_attention: bad metadata")
    lib = library("core")
    _check(lib, lib.mir_paged_attention_generic(
        _is_bf16(out), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], row_of_token.data_ptr(), positions.data_ptr(), tokens,
        page_size, heads, kv_heads, head_dim, value_dim, scale, int(window or 0), int(keep_first or 0),
        head_dim if values_in_keys else 0, _ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0,
        int(gate_per_head), float(softcap or 0.0), _ptr(distance_bias),
        distance_bias.shape[1] if distance_bias is not None else 0, _stream()))


def _check_extras(what: str, sinks, gate, out: torch.Tensor, heads: int, gate_per_head: bool = False,
                  distance_bias=None) -> None:
    _require(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads and sinks.is_contiguous()),
             f"{what}: sinks are float32 [heads]")
    _require(gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1
                              and gate.shape == ((out.shape[0], heads) if gate_per_head else out.shape)),
             f"{what}: the gate has out's dtype and out's shape, or one column per head")
    _require(distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.is_contiguous()
                                       and distance_bias.dim() == 2 and distance_bias.shape[0] == heads
                                       and distance_bias.shape[1] > 0),
             f"{what}: the bias by distance is float32 [heads, rows]")


FAST_HEAD_DIMS = (64, 128)      # what the tensor-core attention kernels take; other sizes use the reference kernel


def decode_attention_plan(rows: int, heads: int, kv_heads: int, head_dim: int, page_size: int, max_context: int) -> tuple:
    """(keys per partition, partitions, floats of scratch) for the attention of `rows` single tokens whose longest
    context (or block-table width) is max_context keys.  The plan is native (csrc/ops_bf16.cu:
    mir_decode_attention_plan), the same for the Python launcher and the layer executor: the tcgen05 kernel where
    it takes the sizes (partitions chosen by the cost of its waves, or decode_tc_partition_keys), else the mma.sync
    kernel with partitions of decode_partition_keys."""
    partition, count, floats = ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    lib = library("bf16")
    _check(lib, lib.mir_decode_attention_plan(rows, heads, kv_heads, head_dim, page_size, max_context,
                                              ctypes.byref(partition), ctypes.byref(count), ctypes.byref(floats)))
    return partition.value, count.value, floats.value


def decode_attention_scratch_floats(rows: int, heads: int, head_dim: int, num_partitions: int) -> int:
    """What the kernels that take one partition per CTA want (decode_attention_plan says what a call will use)."""
    return 0 if num_partitions <= 1 else rows * heads * num_partitions * (head_dim + 2)


def decode_attention_kept_plan(rows: int, heads: int, head_dim: int, max_context: int) -> tuple:
    """(keys per partition, partitions, floats of scratch) for decode_attention with kept first keys, which runs the
    mma.sync kernel with partitions of decode_partition_keys."""
    partition = get_option("decode_partition_keys")
    count = max(1, -(-max_context // partition))
    return partition, count, decode_attention_scratch_floats(rows, heads, head_dim, count)


def decode_attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor, page_size: int, heads: int, kv_heads: int,
                     head_dim: int, scale: float, window: Optional[int], partition: int, num_partitions: int,
                     scratch: Optional[torch.Tensor], keep_first: int = 0,
                     numbering: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, gate_per_head: bool = False, softcap: Optional[float] = None,
                     distance_bias: Optional[torch.Tensor] = None) -> None:
    """bf16 split-KV attention for a batch of single tokens (row r of qkv belongs to request row r).  `keep_first`:
    with a window, the request's first keys that stay visible; the mma.sync kernel then walks over the kept keys and
    the window's as one run, and `numbering` (int32 [rows]) is scratch for the merge.  `sinks`, `gate`: as
    paged_attention_generic takes them (the kernel that writes a row's final result, the attention kernel or the
    merge of its partitions, adds the sink's term and applies the gate).  `gate_per_head`, `softcap`, `distance_bias`:
    as paged_attention_generic takes them: the scores are capped and biased in 32-bit before the softmax, by the
    tcgen05 kernel where it takes the sizes and the partition (decode_attention_plan), else by the mma.sync kernel."""
    _cuda(qkv, out, k_pages, v_pages, block_table, positions, scratch, sinks, gate, distance_bias)
    rows = out.shape[0]
    _check_extras("decode_attention", sinks, gate, out, heads, gate_per_head, distance_bias)
    gate_args = (_ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0)
    _require(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
             and v_pages.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == heads * head_dim,
             "decode_attention: bfloat16 tensors are needed")
    _require(block_table.dtype == torch.int32 and block_table.is_contiguous() and positions.dtype == torch.int32
             and positions.numel() >= rows and block_table.shape[0] >= rows, "decode_attention: bad metadata")
    _require(scratch is None or scratch.dtype == torch.float32, "decode_attention: scratch must be float32")
    lib = library("bf16")
    _require(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[0] == v_pages.shape[0],
             "decode_attention: the cache tensors must be contiguous [token rows, kv_heads, head_dim]")
    if gate_per_head or softcap or distance_bias is not None:
        _require(not (keep_first and window), "decode_attention: capped or biased scores do not go with kept first keys")
        _check(lib, lib.mir_decode_attention_paged_scored_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
            block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), rows, page_size, heads, kv_heads,
            head_dim, scale, int(window or 0), partition, num_partitions, _ptr(scratch),
            0 if scratch is None else scratch.numel(), _stream(), *gate_args, int(gate_per_head), float(softcap or 0.0),
            _ptr(distance_bias), distance_bias.shape[1] if distance_bias is not None else 0))
        return
    if keep_first and window:
        _cuda(numbering)
        _require(numbering is not None and numbering.dtype == torch.int32 and numbering.numel() >= rows,
                 "decode_attention: kept first keys need int32 scratch of one number per row")
        _check(lib, lib.mir_decode_attention_extra_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), rows, page_size, heads, kv_heads,
            head_dim, scale, int(window), partition, num_partitions, _ptr(scratch),
            0 if scratch is None else scratch.numel(), _stream(), int(keep_first), numbering.data_ptr(), *gate_args))
        return
    _check(lib, lib.mir_decode_attention_paged_extra_bf16(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), rows, page_size, heads, kv_heads, head_dim,
        scale,
        int(window or 0), partition, num_partitions, _ptr(scratch), 0 if scratch is None else scratch.numel(),
        _stream(), *gate_args))


# Whether prompt portions run the tcgen05 attention kernel where it takes the sizes (head_dim 128, pages of 8 to
# 128 keys that divide 128) and the portions average at least PREFILL_TENSOR_CORE_MIN_PORTION tokens.
PREFILL_TENSOR_CORES = True
PREFILL_TENSOR_CORE_MIN_PORTION = 32


def prefill_attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, query_starts: torch.Tensor, context_lens: torch.Tensor,
                      page_size: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                      window: Optional[int], tensor_cores: Optional[bool] = None,
                      portion_tokens: Optional[int] = None, keep_first: int = 0,
                      sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      gate_per_head: bool = False, softcap: Optional[float] = None,
                      distance_bias: Optional[torch.Tensor] = None) -> None:
    """bf16 tensor-core attention for any mix of portions (row r owns tokens query_starts[r]..query_starts[r+1]
    of the packed qkv and out; the rows may be a part of the batch, `portion_tokens` then says how many tokens
    they have together).  `tensor_cores`: True runs the tcgen05 kernel, False the mma.sync kernel, None chooses.
    `keep_first`: with a window, the first keys of a request that every later query still sees.  `sinks`, `gate`: as
    paged_attention_generic takes them, in the kernels' epilogues (the gate's rows are those of the whole batch, as
    out's are).  `gate_per_head`, `softcap`, `distance_bias`: as paged_attention_generic takes them; both tile kernels
    cap and bias the scores in 32-bit before the softmax."""
    _cuda(qkv, out, k_pages, v_pages, block_table, query_starts, context_lens, sinks, gate, distance_bias)
    tokens = out.shape[0]
    _check_extras("prefill_attention", sinks, gate, out, heads, gate_per_head, distance_bias)
    gate_args = (_ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0)
    rows = context_lens.numel()
    _require(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
             and v_pages.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == heads * head_dim,
             "prefill_attention: bfloat16 tensors are needed")
    _require(block_table.dtype == torch.int32 and block_table.is_contiguous() and query_starts.dtype == torch.int32
             and context_lens.dtype == torch.int32 and query_starts.numel() == rows + 1
             and block_table.shape[0] >= rows, "prefill_attention: bad metadata")
    lib = library("bf16")
    keep_first = int(keep_first or 0) if window else 0
    if gate_per_head or softcap or distance_bias is not None:
        _require(not keep_first, "prefill_attention: capped or biased scores do not go with kept first keys")
        scored_args = (*gate_args, int(gate_per_head), float(softcap or 0.0), _ptr(distance_bias),
                       distance_bias.shape[1] if distance_bias is not None else 0)
        if tensor_cores is None:
            portion_tokens = tokens if portion_tokens is None else portion_tokens
            tensor_cores = (PREFILL_TENSOR_CORES and portion_tokens >= PREFILL_TENSOR_CORE_MIN_PORTION * rows
                            and bool(lib.mir_prefill_attention_tc_takes(head_dim, page_size))
                            and k_pages.is_contiguous() and v_pages.is_contiguous() and scale > 0
                            and (gate is None or gate_per_head or (gate.data_ptr() % 16 == 0 and gate.stride(0) % 8 == 0)))
        if tensor_cores:
            _require(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape,
                     "prefill_attention: the tcgen05 kernel reads contiguous [rows, kv_heads, head_dim] pages")
            _check(lib, lib.mir_prefill_attention_tc_scored_bf16(
                qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
                block_table.data_ptr(), block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows,
                tokens, page_size, heads, kv_heads, head_dim, scale, int(window or 0), _stream(), *scored_args))
            return
        _check(lib, lib.mir_prefill_attention_scored_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows, tokens, page_size, heads,
            kv_heads, head_dim, scale, int(window or 0), _stream(), *scored_args))
        return
    if tensor_cores is None:
        portion_tokens = tokens if portion_tokens is None else portion_tokens
        tensor_cores = (PREFILL_TENSOR_CORES and portion_tokens >= PREFILL_TENSOR_CORE_MIN_PORTION * rows
                        and bool(lib.mir_prefill_attention_tc_takes(head_dim, page_size))
                        and k_pages.is_contiguous() and v_pages.is_contiguous() and scale > 0
                        and (gate is None or (gate.data_ptr() % 16 == 0 and gate.stride(0) % 8 == 0)))
    if tensor_cores:
        _require(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape,
                 "prefill_attention: the tcgen05 kernel reads contiguous [rows, kv_heads, head_dim] pages")
        _check(lib, lib.mir_prefill_attention_tc_extra_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
            block_table.data_ptr(), block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows, tokens,
            page_size, heads, kv_heads, head_dim, scale, int(window or 0), keep_first, _stream(), *gate_args))
        return
    _check(lib, lib.mir_prefill_attention_extra_bf16(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], query_starts.data_ptr(), context_lens.data_ptr(), rows, tokens, page_size, heads,
        kv_heads, head_dim, scale, int(window or 0), keep_first, _stream(), *gate_args))


def set_prefill_softmax_streams(streams: int) -> None:
    """For measurements: over how many softmax streams the tcgen05 attention splits a row's key tiles, 1 or 2."""
    lib = library("bf16")
    _check(lib, lib.mir_prefill_attention_tc_set_streams(int(streams)))


def set_prefill_shared_reference(shared: bool) -> None:
    """For measurements: whether the two softmax streams of the tcgen05 prompt attention share a row's reference and
    one output accumulator (the default) or keep a softmax each over their tiles."""
    lib = library("bf16")
    _check(lib, lib.mir_prefill_attention_tc_set_shared(1 if shared else 0))


def decode_attention_error() -> int:
    """0 unless a bounded wait of the tcgen05 decode attention kernel ran out (synchronises the device)."""
    return int(library("bf16").mir_decode_attention_tc_error())


def decode_attention_takes_tensor_cores(head_dim: int, page_size: int, partition: int) -> bool:
    """Whether single decoded tokens of these sizes run the tcgen05 kernel (and the option decode_tensor_cores is on)."""
    lib = library("bf16")
    return bool(lib.mir_get_option(b"decode_tensor_cores")) and \
        bool(lib.mir_decode_attention_tc_takes(head_dim, page_size, partition))


def prefill_attention_error() -> int:
    """0, or which role of the tcgen05 attention gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_prefill_attention_tc_error())


# --------------------------------------------------------------------------- matrix products
_LT_WORKSPACE: dict = {}
LT_WORKSPACE_BYTES = 64 * 1024 * 1024


def _lt_workspace(device) -> torch.Tensor:
    key = (device.type, device.index)
    buffer = _LT_WORKSPACE.get(key)
    if buffer is None:
        buffer = torch.empty(LT_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _LT_WORKSPACE[key] = buffer
    return buffer


class NormedResidual:
    """An RMSNorm of the 32-bit residual stream that is folded into the few-rows products around it.
    `weighted` holds bf16(residual * norm weight) and `sumsq`, per 16-column tile of the residual and per token,
    the sum of squares; both were written by the product that last updated the residual.  The product that takes
    this as its x multiplies each token's results by rsqrt(mean of squares + eps).  Anything else that needs the
    normed rows calls `materialize`."""

    def __init__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, sumsq: torch.Tensor, tiles: int,
                 dtype: torch.dtype, weighted: torch.Tensor):
        self.residual, self.weight, self.eps, self.sumsq, self.tiles, self.dtype = residual, weight, eps, sumsq, tiles, dtype
        self.weighted = weighted
        self.shape = residual.shape

    def materialize(self, alloc) -> torch.Tensor:
        out = alloc(tuple(self.residual.shape), self.dtype)
        rms_norm(self.residual, self.weight, self.eps, out)
        return out


def sumsq_tiles(columns: int) -> int:
    """How many 16-column tiles the accumulate epilogue writes sums of squares for."""
    return -(-columns // 16)


def linear(x, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           accumulate: bool = False, sumsq_out: Optional[torch.Tensor] = None, alloc=None,
           weighted_out: Optional[tuple] = None) -> bool:
    """out = (out if accumulate) + x . weight^T (+ bias).

    float32 tensors: the 32-bit FMA kernel.  bfloat16 x and weight: the native dispatch (csrc/ops_bf16.cu) runs up
    to few_rows_max (32) rows on the weight-streaming kernel and more on cuBLASLt, both with 32-bit accumulation;
    out is bfloat16 or float32.  x and out may be row-strided views; weight is [out_features, in_features].  x may
    be a NormedResidual (then `alloc` must be given in case it has to be materialised).  With `sumsq_out` (float32
    [ceil(N / 16), NORM_STAT_STRIDE]) and `weighted_out` = (bfloat16 [M, N], float32 norm weight [N]) an
    accumulating few-rows product also writes the sums of squares of the rows it updates and those rows times the
    weight; the return value says whether it did."""
    lazy = x if isinstance(x, NormedResidual) else None
    rows = lazy.weighted if lazy is not None else x
    _cuda(rows, weight, out, bias)
    m, k = rows.shape
    n = weight.shape[0]
    _require(weight.shape[1] == k and out.shape == (m, n) and rows.stride(1) == 1 and out.stride(1) == 1
             and weight.is_contiguous(), "linear: shapes or strides do not fit")
    if rows.dtype == torch.float32:
        _require(weight.dtype == torch.float32 and out.dtype == torch.float32
                 and (bias is None or bias.dtype == torch.float32), "linear: float32 takes float32 everywhere")
        lib = library("core")
        _check(lib, lib.mir_gemm_f32(x.data_ptr(), x.stride(0), weight.data_ptr(), k, _ptr(bias), out.data_ptr(),
                                     out.stride(0), m, n, k, 1.0 if accumulate else 0.0, _stream()))
        return False
    _require(rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16, "linear: x and weight must share a dtype")
    _require(out.dtype == torch.float32 or not accumulate, "linear: only a float32 output accumulates")
    late_bias = None
    if bias is not None and bias.dtype != out.dtype:
        _require(out.dtype == torch.float32 and (accumulate or out.is_contiguous()), "linear: bias dtype must match out")
        if accumulate:
            add_bias(out, bias)
        else:
            late_bias = bias           # a 32-bit result that replaces `out`: the bias is added behind the product
        bias = None
    stats, weighted, next_weight = None, None, None
    if sumsq_out is not None and weighted_out is not None and sumsq_out.numel() >= sumsq_tiles(n) * NORM_STAT_STRIDE:
        stats, (weighted, next_weight) = sumsq_out, weighted_out
        _cuda(stats, weighted, next_weight)
        _require(stats.dtype == torch.float32 and weighted.dtype == torch.bfloat16 and weighted.shape == (m, n)
                 and weighted.stride(1) == 1 and next_weight.dtype == torch.float32 and next_weight.numel() == n
                 and next_weight.is_contiguous(), "linear: weighted rows are bfloat16 [M, N], the weight float32 [N]")
    lib = library("bf16")
    workspace = _lt_workspace(rows.device)
    wrote = c_int(0)

    def call(source, folded):
        return lib.mir_linear_bf16(
            source.data_ptr(), source.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0),
            int(out.dtype == torch.float32), int(accumulate), m, n, k,
            folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
            folded.eps if folded is not None else 0.0, _ptr(stats), _ptr(next_weight), _ptr(weighted),
            weighted.stride(0) if weighted is not None else 0, workspace.data_ptr(), workspace.numel(), _stream(),
            ctypes.addressof(wrote))

    status = call(rows, lazy)
    if status == MIR_CANNOT_FOLD and lazy is not None:
        status = call(lazy.materialize(alloc), None)
    _check(lib, status)
    if late_bias is not None:
        add_bias(out, late_bias)
    return bool(wrote.value)


ACTIVATIONS = ("gelu_tanh", "gelu_erf", "relu2")      # what linear_act applies to a product's result


def linear_act(x, weight: torch.Tensor, out: torch.Tensor, activation: str, alloc=None) -> None:
    """out = act(x . weight^T) in the activations' dtype, act one of ACTIVATIONS: the tanh GELU, the exact GELU
    0.5 z (1 + erf(z / sqrt 2)) (computed with erff, in the epilogue too) or the square of relu.  bfloat16: one kernel
    with the activation in its epilogue where our tcgen05 products take the rows (up to few_rows_max on the
    weight-streaming kernel, where x may be a NormedResidual, a norm folded into this product; from
    tensor_core_min_rows on the many-rows kernel; the tanh form uses the approximate hardware tanh, whose error is below
    bfloat16's rounding), else the library product and the activation kernel.  float32: the 32-bit product and that
    kernel."""
    _require(activation in ACTIVATIONS, f"linear_act: unknown activation {activation!r}")
    lazy = x if isinstance(x, NormedResidual) else None
    rows = lazy.weighted if lazy is not None else x
    _cuda(rows, weight, out)
    m, k = rows.shape
    n = weight.shape[0]
    if (rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k % 8 == 0
            and rows.stride(0) % 8 == 0 and rows.data_ptr() % 16 == 0 and rows.stride(1) == 1 and out.stride(1) == 1
            and weight.is_contiguous() and out.shape == (m, n) and FUSE_GELU_INTO_PRODUCT):
        lib = library("bf16")
        mode = {"gelu_tanh": MODE_GELU, "gelu_erf": MODE_GELU_ERF, "relu2": MODE_RELU2}[activation]
        if 0 < m <= min(get_option("few_rows_max"), STREAM_MAX_ROWS) and (lazy is None or m <= NORM_STAT_STRIDE):
            _check(lib, lib.mir_gemm_tc_stream_bf16(
                mode, rows.data_ptr(), rows.stride(0), weight.data_ptr(), None, out.data_ptr(), out.stride(0), m, n,
                k, 0, lazy.sumsq.data_ptr() if lazy is not None else None, lazy.tiles if lazy is not None else 0,
                lazy.eps if lazy is not None else 0.0, None, None, None, 0, _stream()))
            return
        if lazy is None and m >= get_option("tensor_core_min_rows"):
            _check(lib, lib.mir_gemm_tc_bf16(mode, rows.data_ptr(), rows.stride(0), weight.data_ptr(), None,
                                             out.data_ptr(), out.stride(0), m, n, k, 0, _stream()))
            return
    if lazy is not None:
        x = lazy.materialize(alloc)
    linear(x, weight, out, alloc=alloc)
    _require(out.is_contiguous(), "linear_act: a contiguous result is needed")
    {"gelu_tanh": gelu_tanh, "gelu_erf": gelu_erf, "relu2": relu_squared}[activation](out)


def linear_gelu(x, weight: torch.Tensor, out: torch.Tensor, alloc=None, exact: bool = False) -> None:
    """out = gelu(x . weight^T): linear_act with the tanh form, or with `exact` the erf form."""
    linear_act(x, weight, out, "gelu_erf" if exact else "gelu_tanh", alloc=alloc)


def tensor_core_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                       bias: Optional[torch.Tensor] = None, accumulate: bool = False, swiglu: bool = False) -> None:
    """The tcgen05 product for many bfloat16 rows: out = x . weight^T (+ bias) as bfloat16, or as float32
    (added to out if `accumulate`); with `swiglu`, weight is [gate rows; up rows] and
    out[M, I] = silu(x w_gate^T) * (x w_up^T) in one kernel."""
    _cuda(x, weight, out, bias)
    m, k = x.shape
    _require(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
             and weight.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == m,
             "tensor_core_linear: bfloat16 x [M, K] and weight [N, K] are needed")
    lib = library("bf16")
    if swiglu:
        inter = out.shape[1]
        _require(weight.shape[0] == 2 * inter and out.dtype == torch.bfloat16 and bias is None and not accumulate,
                 "tensor_core_linear: the SwiGLU epilogue takes [2 I, K] weights, no bias, and writes bfloat16")
        mode, n, up_offset = MODE_SWIGLU, inter, inter
    else:
        n, up_offset = weight.shape[0], 0
        _require(out.shape[1] == n and (bias is None or bias.dtype == out.dtype)
                 and (out.dtype == torch.float32 or not accumulate),
                 "tensor_core_linear: out must be [M, N]; bias shares its dtype; only float32 accumulates")
        mode = MODE_STORE if out.dtype == torch.bfloat16 else (MODE_ACCUM if accumulate else MODE_F32)
    _check(lib, lib.mir_gemm_tc_bf16(mode, x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(),
                                     out.stride(0), m, n, k, up_offset, _stream()))


def stream_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  accumulate: bool = False, swiglu: bool = False, folded: Optional["NormedResidual"] = None,
                  sumsq_out: Optional[torch.Tensor] = None, weighted_out: Optional[tuple] = None) -> None:
    """The tcgen05 weight-streaming product for 1 to 128 bfloat16 rows (see tensor_core_linear for the modes).
    `folded`: x is folded.weighted and each token's results are scaled by the folded norm; `sumsq_out`,
    `weighted_out` as in linear (accumulate, up to 32 rows)."""
    if folded is not None:
        x = folded.weighted
    _cuda(x, weight, out, bias)
    m, k = x.shape
    _require(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
             and weight.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == m
             and 0 < m <= STREAM_MAX_ROWS, "stream_linear: 1..128 bfloat16 rows x [M, K] and weight [N, K] are needed")
    lib = library("bf16")
    if swiglu:
        inter = out.shape[1]
        _require(weight.shape[0] == 2 * inter and out.dtype == torch.bfloat16 and bias is None and not accumulate,
                 "stream_linear: the SwiGLU epilogue takes [2 I, K] weights, no bias, and writes bfloat16")
        mode, n, up_offset = MODE_SWIGLU, inter, inter
    else:
        n, up_offset = weight.shape[0], 0
        _require(out.shape[1] == n and (bias is None or bias.dtype == out.dtype)
                 and (out.dtype == torch.float32 or not accumulate),
                 "stream_linear: out must be [M, N]; bias shares its dtype; only float32 accumulates")
        mode = MODE_STORE if out.dtype == torch.bfloat16 else (MODE_ACCUM if accumulate else MODE_F32)
    rows, next_weight = weighted_out if weighted_out is not None else (None, None)
    if rows is not None:
        _cuda(rows, next_weight)
        _require(rows.dtype == torch.bfloat16 and rows.shape == (m, n) and rows.stride(1) == 1
                 and next_weight.dtype == torch.float32 and next_weight.numel() == n and next_weight.is_contiguous(),
                 "stream_linear: weighted rows are bfloat16 [M, N], the norm weight float32 [N]")
    _check(lib, lib.mir_gemm_tc_stream_bf16(
        mode, x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), m, n, k,
        up_offset, folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
        folded.eps if folded is not None else 0.0, _ptr(sumsq_out), _ptr(next_weight), _ptr(rows),
        rows.stride(0) if rows is not None else 0, _stream()))


STREAM_MAX_ROWS = 128


def stream_linear_error() -> int:
    """0, or which role of the weight-streaming product gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_gemm_tc_stream_error())


def tensor_core_linear_error() -> int:
    """0, or which role of the tcgen05 product gave up a bounded wait (synchronises the device)."""
    return int(library("bf16").mir_gemm_tc_error())


NORM_STAT_STRIDE = 32        # tokens per row of the sums-of-squares arrays (kNormStatStride of the kernels)
MODE_STORE, MODE_ACCUM, MODE_F32, MODE_SWIGLU, MODE_GELU, MODE_GELU_ERF, MODE_RELU2 = 0, 1, 2, 3, 4, 5, 6


def few_rows_max() -> int:
    """Up to how many rows products run the weight-streaming kernel, which can also take over RMSNorms."""
    return min(get_option("few_rows_max"), get_option("folded_norm_max_rows"), STREAM_MAX_ROWS)


def gate_up_silu(x, w_gate_up: torch.Tensor, out: torch.Tensor, scratch_alloc) -> None:
    """out[M, I] = silu(x w_gate^T) * (x w_up^T) with w_gate_up = [w_gate; w_up] of shape [2 I, K].

    bfloat16: the native dispatch (csrc/ops_bf16.cu) runs up to few_rows_max (32) rows on the weight-streaming
    kernel (x may be a NormedResidual, a norm folded into this product) and from tensor_core_min_rows (128) rows on
    the tcgen05 many-rows kernel, one kernel each, the [M, 2 I] intermediate never written; between them the library
    product followed by the SiLU-multiply kernel.  float32: the 32-bit product and that kernel.
    `scratch_alloc(shape, dtype)` provides the intermediate where one is needed."""
    lazy = x if isinstance(x, NormedResidual) else None
    rows = lazy.weighted if lazy is not None else x
    m, k = rows.shape
    inter = out.shape[1]
    _cuda(rows, w_gate_up, out)
    _require(w_gate_up.shape == (2 * inter, k) and out.shape[0] == m and out.is_contiguous()
             and w_gate_up.is_contiguous() and rows.stride(1) == 1, "gate_up_silu: shapes do not fit")
    if rows.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        gate_up = scratch_alloc((m, 2 * inter), rows.dtype)
        linear(x, w_gate_up, gate_up)
        silu_mul(gate_up, out)
        return
    _require(out.dtype == torch.bfloat16, "gate_up_silu: bfloat16 rows give a bfloat16 result")
    lib = library("bf16")
    workspace = _lt_workspace(rows.device)
    needs_scratch = get_option("few_rows_max") < m < get_option("tensor_core_min_rows") or k % 8 != 0 \
        or rows.stride(0) % 8 != 0 or rows.data_ptr() % 16 != 0

    def call(source, folded):
        scratch = scratch_alloc((m, 2 * inter), torch.bfloat16) if needs_scratch else None
        return lib.mir_gate_up_silu_bf16(
            source.data_ptr(), source.stride(0), w_gate_up.data_ptr(), out.data_ptr(), m, inter, k,
            folded.sumsq.data_ptr() if folded is not None else None, folded.tiles if folded is not None else 0,
            folded.eps if folded is not None else 0.0, _ptr(scratch), workspace.data_ptr(), workspace.numel(), _stream())

    status = call(rows, lazy)
    if status == MIR_CANNOT_FOLD and lazy is not None:
        status = call(lazy.materialize(scratch_alloc), None)
    _check(lib, status)


# --------------------------------------------------------------------------- sampling
SAMPLE_OPTIONS = np.dtype([("draw", "<f8"), ("temperature", "<f4"), ("top_p", "<f4"), ("top_k", "<i4"),
                           ("pad", "<i4")])


def ranked_scratch_keys(rows: int, vocab: int) -> int:
    """How many 64-bit keys of scratch top-k / top-p sampling needs for `rows` rows."""
    padded = 1
    while padded < vocab:
        padded <<= 1
    return rows * padded


class HeadCandidates:
    """What the output head's kernel can leave beside the logits (head_logits): per row the largest finite logit of
    every 32 columns and its column.  `valid` says whether the last product that was given these buffers filled
    them; sample() then finds each row's largest logit among them instead of among the whole vocabulary."""

    def __init__(self, values: torch.Tensor, indices: torch.Tensor):
        self.values, self.indices, self.valid = values, indices, False

    @staticmethod
    def count(vocab: int) -> int:
        return -(-vocab // 128) * 4

    @classmethod
    def allocate(cls, alloc, rows: int, vocab: int) -> "HeadCandidates":
        return cls(alloc((rows, cls.count(vocab)), torch.float32), alloc((rows, cls.count(vocab)), torch.int32))


def head_logits(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                candidates: Optional[HeadCandidates] = None) -> None:
    """out[M, V] (float32) = x . weight^T, the output head.  bfloat16 rows up to few_rows_max go through the
    weight-streaming kernel, whose epilogue also fills `candidates` (and sets candidates.valid); every other case is
    linear() and leaves candidates.valid False."""
    if candidates is not None:
        candidates.valid = False
    if candidates is None or x.dtype != torch.bfloat16:
        linear(x, weight, out)
        return
    _cuda(x, weight, out, candidates.values, candidates.indices)
    m, k = x.shape
    n = weight.shape[0]
    _require(weight.dtype == torch.bfloat16 and weight.shape[1] == k and weight.is_contiguous()
             and out.dtype == torch.float32 and out.shape == (m, n) and x.stride(1) == 1 and out.stride(1) == 1,
             "head_logits: bfloat16 x [M, K] and weight [V, K], float32 out [M, V]")
    _require(candidates.values.shape == candidates.indices.shape and candidates.values.shape[0] >= m
             and candidates.values.is_contiguous() and candidates.indices.is_contiguous()
             and candidates.values.dtype == torch.float32 and candidates.indices.dtype == torch.int32,
             "head_logits: candidates are float32 values and int32 indices of one shape [rows, count]")
    lib = library("bf16")
    workspace = _lt_workspace(x.device)
    wrote = c_int(0)
    _check(lib, lib.mir_head_logits_bf16(x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), m, n,
                                         k, candidates.values.data_ptr(), candidates.indices.data_ptr(),
                                         candidates.values.shape[1], workspace.data_ptr(), workspace.numel(), _stream(),
                                         ctypes.addressof(wrote)))
    candidates.valid = bool(wrote.value)


def sample(logits: torch.Tensor, options: torch.Tensor, tokens: torch.Tensor,
           sort_keys: Optional[torch.Tensor] = None, needs_ranked: bool = False,
           candidates: Optional[HeadCandidates] = None) -> None:
    """tokens[r] = one token from row r of the 32-bit logits; options is a uint8 view of SAMPLE_OPTIONS records.
    `candidates` (valid, from the product that wrote these very logits): where each row's largest logit is found."""
    _cuda(logits, options, tokens, sort_keys)
    rows, vocab = logits.shape
    _require(logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.dtype == torch.int32
             and tokens.numel() >= rows and options.numel() * options.element_size() >= rows * SAMPLE_OPTIONS.itemsize,
             "sample: bad arguments")
    capacity = 0 if sort_keys is None else sort_keys.numel() * sort_keys.element_size() // 8
    use = candidates is not None and candidates.valid and candidates.values.shape[0] >= rows
    lib = library("core")
    _check(lib, lib.mir_sample(logits.data_ptr(), logits.stride(0), rows, vocab, options.data_ptr(), _ptr(sort_keys),
                               capacity, int(needs_ranked), tokens.data_ptr(),
                               candidates.values.data_ptr() if use else None,
                               candidates.indices.data_ptr() if use else None,
                               candidates.values.shape[1] if use else 0, _stream()))


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, id_rows: torch.Tensor,
                       penalties: torch.Tensor) -> None:
    _cuda(logits, ids, id_rows, penalties)
    rows, vocab = logits.shape
    _require(logits.dtype == torch.float32 and ids.dtype == torch.int32 and id_rows.dtype == torch.int32
             and penalties.dtype == torch.float32 and penalties.numel() >= rows and ids.numel() == id_rows.numel(),
             "repetition_penalty: bad arguments")
    lib = library("core")
    _check(lib, lib.mir_repetition_penalty(logits.data_ptr(), logits.stride(0), vocab, ids.data_ptr(),
                                           id_rows.data_ptr(), penalties.data_ptr(), ids.numel(), _stream()))
