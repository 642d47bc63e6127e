"""Python entry points of the sm_100a kernels (``pylon_b200/csrc``).

Each function checks its tensors (device, dtype, contiguity, sizes), launches on torch's
current CUDA stream and returns without synchronising.  There is no CPU path: a tensor that
is not on a CUDA device, or a kernel library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence

import torch

from pylon_b200.kernels import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels run in float32 or bfloat16, not {dtype}")


# The raw handle of torch's current stream, without building a Stream object (that costs some
# 15 us of host time, and an eager step asks some 300 times).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The address for a ``c_void_p`` parameter (ctypes takes an int, or None for null)."""
    return None if tensor is None else tensor.data_ptr()


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("pylon_b200 kernels need CUDA tensors; there is no CPU path")


def _need(condition: bool, text: str) -> None:
    if not condition:
        raise KernelError(text)


# Kernels of this package launched so far in this process (library matrix products are
# not counted).  Benchmarks read it before and after a timed region.
launches = [0]


def _check(library: ctypes.CDLL, code: int) -> None:
    launches[0] += 1
    if code != 0:
        raise KernelError(library.pylon_last_error().decode(errors="replace") or f"kernel call failed ({code})")


# Kernels that wait on mbarriers (TMA copies, tensor-core completion) bound every wait; one that
# runs out sets its word here instead of hanging, and the result of that launch is void.  One
# tensor per device: [tcgen05 product, attention, TMA-fed decode product, unused].
_error_word_storage: dict[int, torch.Tensor] = {}
_ERROR_WORD_NAMES = ("tcgen05 product", "attention", "TMA-fed decode product", "cache write")
BAD_PAGE_CODE = 5   # PYLON_ERROR_BAD_PAGE of csrc/common.cuh: a block table named a page that the pool does not have


def _device_index(device: torch.device | str) -> int:
    """``cuda`` and ``cuda:N`` name the same device when N is the current one: buffers kept per device go by the number."""
    device = torch.device(device)
    return torch.cuda.current_device() if device.index is None else device.index


def _multiprocessors(device: torch.device | str) -> int:
    """How many multiprocessors ``device`` has (asked once): grids, splits and tile choices are sized by it."""
    index = _device_index(device)
    if index not in _multiprocessor_counts:
        _multiprocessor_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _multiprocessor_counts[index]


_multiprocessor_counts: dict[int, int] = {}


def _error_words(device: torch.device) -> torch.Tensor:
    key = _device_index(device)
    if key not in _error_word_storage:
        _error_word_storage[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _error_word_storage[key]


def cache_write_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the kernel that writes new keys and values into their pages sets when the block
    table names a page the pool does not have (nothing is written there).  Zero in every healthy run."""
    return _error_words(device)[3:4]


_error_word_copies: dict[int, torch.Tensor] = {}   # pinned host copies, filled by queue_error_word_read


def queue_error_word_read(device: torch.device) -> None:
    """Enqueues a copy of the error words into pinned host memory behind the work queued so far, without waiting.  A
    caller that is about to wait for the stream anyway (to read a step's tokens back) queues this first and looks at
    the words with ``raise_on_kernel_errors(device, queued=True)`` afterwards: one trip to the device instead of two."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return
    if key not in _error_word_copies:
        _error_word_copies[key] = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    _error_word_copies[key].copy_(_error_word_storage[key], non_blocking=True)


def queue_error_word_copy(device: torch.device) -> Optional[torch.Tensor]:
    """Like :func:`queue_error_word_read`, into a pinned buffer of the caller's own (returned; ``None`` if no kernel that
    can set the words has run): for callers that have more than one step in flight and look at each step's words when
    they come to it, with ``raise_on_kernel_errors(device, words=...)``."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return None
    words = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    words.copy_(_error_word_storage[key], non_blocking=True)
    return words


def raise_on_kernel_errors(device: torch.device, queued: bool = False, words: Optional[torch.Tensor] = None) -> None:
    """Reads the error words of ``device`` (a 16-byte copy that waits for the work queued so
    far; with ``queued`` the copy :func:`queue_error_word_read` enqueued, with ``words`` the one
    :func:`queue_error_word_copy` returned, which the caller has
    waited for since) and raises if, since the last call, a kernel gave up one of its bounded
    waits or met a block table that names a page outside the pool.  The words are cleared, so
    the next call reports only what happens from now on; and the counters by which the blocks
    of a decode attention find the last of them are put back to zero, since a block that gave
    up never took part in the count of the rows it shared, and the next launch must find zeros."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return   # no kernel that can set them has run
    if words is not None:
        words = words.tolist()
    elif queued and key in _error_word_copies:
        words = _error_word_copies[key].tolist()
    else:
        words = _error_word_storage[key].cpu().tolist()
    if any(words):
        _error_word_storage[key].zero_()
        for (index, _purpose), buffer in _counter_buffers.items():
            if index == key:
                buffer.zero_()
        what = ", ".join(
            f"{name} ({'a block table names a page outside the pool' if code == BAD_PAGE_CODE else 'a bounded wait ran out'}, code {code})"
            for name, code in zip(_ERROR_WORD_NAMES, words) if code)
        raise KernelError(f"kernel error in: {what}; the results of that step are void")


_SIGNATURES = {
    "elementwise.cu": {
        "pylon_embed_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "pylon_take_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "pylon_logit_transform": [c_void_p, c_longlong, c_float, c_float, c_void_p],
        "pylon_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "pylon_residual_add": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
        "pylon_add_parts_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "pylon_qk_norm_rope_kv_write": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_qk_norm_rope_kv_write_parts": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_void_p],
        "pylon_qk_norm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
        "pylon_qk_norm_mix_kv_write": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_qk_whole_norm_kv_write": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    },
    "streams.cu": {
        "pylon_streams_update_norm": [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p],
    },
    "delta_rule.cu": {
        "pylon_gated_delta_rule": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_float, c_float, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p],
    },
    "state_space.cu": {
        "pylon_state_space": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                              c_int, c_void_p],
    },
    "linear_recurrence.cu": {
        "pylon_linear_recurrence_conv": [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "pylon_linear_recurrence_scan": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                         c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                         c_int, c_void_p, c_int, c_void_p],
    },
    "matrix_memory.cu": {
        "pylon_matrix_memory_scan": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_matrix_memory_out": [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "combine.cu": {
        "pylon_side_by_side": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "pylon_gated_unit": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_add_bias": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
        "pylon_mean_of_normed": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "pylon_weighted_sum": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
        "pylon_activation": [c_void_p, c_longlong, c_int, c_int, c_void_p],
    },
    "experts.cu": {
        "pylon_experts_row_tile": [],
        "pylon_experts_route": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                c_float, c_int, c_void_p, c_void_p],
        "pylon_experts_plan": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_experts_product": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p],
        "pylon_experts_sort_rows": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_experts_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    },
    "gemm_f32.cu": {
        "pylon_gemm_f32_nt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
        "pylon_gemm_f32_nt_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_longlong,
                                      c_longlong, c_longlong, c_void_p],
    },
    "attention_latent.cu": {
        "pylon_latent_attention": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_latent_attention_scratch_floats": [c_int, c_int, c_int],
    },
    "lightning.cu": {
        "pylon_lightning_attention": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int,
                                      c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_lightning_work_floats": [c_int, c_int, c_int, c_int, c_int, c_int, c_int],
    },
    "rotary.cu": {
        "pylon_qkv_rotate_write": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_latent_norm_rotate_write": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_rotate_heads": [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                               c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_skinny.cu": {
        "pylon_gemm_skinny_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    },
    "gemm_stream.cu": {
        "pylon_gemm_stream_partial": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p],
        "pylon_gemm_stream_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
        "pylon_gemm_stream_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
        "pylon_gemm_stream_glu_clamped": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_float, c_float, c_void_p, c_void_p],
    },
    "gemm_tcgen05.cu": {
        "pylon_gemm_tcgen05_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                                    c_void_p, c_int, c_void_p],
        "pylon_gemm_tcgen05_glu_clamped": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_float, c_float,
                                           c_void_p, c_int, c_void_p],
        "pylon_gemm_tcgen05_force_tile": [c_int],
        "pylon_gemm_tcgen05_grouped": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_void_p, c_int,
                                       c_void_p, c_int, c_void_p],
        "pylon_gemm_tcgen05_qkv_rotate": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_float,
                                          c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_int, c_void_p, c_void_p, c_int, c_void_p],
    },
    "attention_simple.cu": {
        "pylon_paged_attention_simple": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                         c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    },
    "attention_window.cu": {
        "pylon_window_attention": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        "pylon_window_attention_max_group": [],
        "pylon_window_attention_scratch_floats": [c_int, c_int, c_int],
    },
    "attention_mma.cu": {
        "pylon_paged_attention_mma": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_paged_attention_mma_masked": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_attention_scratch_floats": [c_int, c_int, c_int, c_int, c_int, c_int],
        "pylon_attention_decode_blocks": [],
    },
    "attention_tcgen05.cu": {
        "pylon_paged_attention_tcgen05": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_paged_attention_tcgen05_masked": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                 c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    },
    "sampling.cu": {
        "pylon_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
}


_typed_libraries: dict[tuple, ctypes.CDLL] = {}


def _library(source: str, defines: Optional[dict[str, int]] = None) -> ctypes.CDLL:
    key = (source, tuple(sorted(defines.items())) if defines else ())
    library = _typed_libraries.get(key)
    if library is not None:
        return library
    library = build.load(source, defines)
    if not getattr(library, "_pylon_typed", False):
        for name, argtypes in _SIGNATURES.get(source, {}).items():
            function = getattr(library, name)
            function.argtypes = argtypes
            function.restype = c_longlong if name.endswith("_floats") else c_int
        library._pylon_typed = True
    _typed_libraries[key] = library
    return library


def build_all() -> list[str]:
    """Every library with its default sizes (the tensor-core attention for head size 128)."""
    names = []
    for source in _SIGNATURES:
        defines = {"PYLON_HEAD_DIM": 128} if source in ("attention_mma.cu", "attention_tcgen05.cu") else None
        _library(source, defines)
        names.append(build.library_name(source, defines))
    return names


# ---------------------------------------------------------------------------------------
# embedding, norms, residual
# ---------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0, copies: int = 1,
                 accumulate: bool = False) -> torch.Tensor:
    """float32 ``[T, width]`` rows of ``table`` (``[vocab, width]``) picked by int32 ``ids``, times ``scale``.  With
    ``copies`` > 1 the result is ``[T, copies, width]``, every copy the same row (a model with several residual streams).
    ``accumulate``: the rows are added to what ``out`` holds instead of replacing it."""
    _need(not accumulate or out is not None, "embed_gather: accumulating needs the tensor to add to")
    _need_cuda(ids, table, out)
    _need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "embed_gather: ids must be contiguous int32 [T]")
    _need(table.dim() == 2 and table.is_contiguous(), "embed_gather: table must be contiguous [vocab, width]")
    tokens, (vocab, width) = ids.shape[0], table.shape
    shape = (tokens, width) if copies == 1 else (tokens, int(copies), width)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=table.device)
    _need(out.dtype == torch.float32 and out.shape == shape and out.is_contiguous(), "embed_gather: out must be contiguous float32 [T, width] or [T, copies, width]")
    library = _library("elementwise.cu")
    _check(library, library.pylon_embed_gather(_ptr(ids), _ptr(table), _ptr(out), tokens, width, vocab, _dtype_code(table.dtype), float(scale), int(copies), int(bool(accumulate)), _stream()))
    return out


def take_tokens(ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor) -> torch.Tensor:
    """In place on int32 ``ids [T]``: ``ids[t] = sampled[source[t]]`` wherever ``source[t] >= 0``.  How a step gets tokens
    that the sampling kernel chose in the step before and the host has not read yet."""
    _need_cuda(ids, source, sampled)
    for name, tensor in (("ids", ids), ("source", source), ("sampled", sampled)):
        _need(tensor.dtype == torch.int32 and tensor.dim() == 1 and tensor.is_contiguous(), f"take_tokens: {name} must be contiguous int32")
    _need(source.shape[0] >= ids.shape[0], "take_tokens: a source for every token")
    library = _library("elementwise.cu")
    _check(library, library.pylon_take_tokens(_ptr(ids), _ptr(source), _ptr(sampled), sampled.shape[0], ids.shape[0], _stream()))
    return ids


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 ``logits``: ``y = x * scale``, then with a ``softcap`` c: ``y = c * tanh(y / c)``."""
    _need_cuda(logits)
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logit_transform: logits must be contiguous float32")
    _need(softcap is None or softcap > 0, "logit_transform: a soft cap must be positive")
    library = _library("elementwise.cu")
    _check(library, library.pylon_logit_transform(_ptr(logits), logits.numel(), float(scale), float(softcap or 0.0), _stream()))
    return logits


def add_rmsnorm(
    residual: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    out_dtype: torch.dtype,
    rows: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``residual += delta`` (float32, in place, skipped when ``rows`` selects rows), then
    RMSNorm of the selected rows with the float32 ``weight``; returns ``out_dtype [n, width]``.
    ``delta`` may also be float32 partial sums ``[parts, T, width]`` (see
    :func:`linear_for_residual`): their sum is the delta."""
    _need_cuda(residual, delta, weight, rows, out)
    if delta is not None and delta.dim() == 3:
        if out is None and out_dtype == torch.bfloat16 and delta.dtype == torch.float32 and delta.is_contiguous() \
                and delta.shape[1:] == residual.shape and residual.is_contiguous() and residual.shape[1] % 4 == 0 and residual.shape[1] <= 8192 \
                and (rows is None or (rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous())):
            n_rows = residual.shape[0] if rows is None else rows.shape[0]
            normed = torch.empty((n_rows, residual.shape[1]), dtype=torch.bfloat16, device=residual.device)
            library = _library("elementwise.cu")
            _check(library, library.pylon_add_parts_rmsnorm(_ptr(residual), _ptr(delta), delta.shape[0], _ptr(weight), _ptr(rows), _ptr(normed),
                                                            n_rows, residual.shape[0], residual.shape[1], float(eps), _stream()))
            return normed
        delta = delta.sum(dim=0).to(out_dtype)
    _need(residual.dtype == torch.float32 and residual.dim() == 2 and residual.is_contiguous(), "add_rmsnorm: residual must be contiguous float32 [T, width]")
    tokens, width = residual.shape
    _need(weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(), "add_rmsnorm: weight must be float32 [width]")
    if delta is not None:
        _need(delta.shape == residual.shape and delta.is_contiguous() and delta.dtype == out_dtype, "add_rmsnorm: delta must be contiguous [T, width] in the activation dtype")
    n_rows = tokens
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "add_rmsnorm: rows must be contiguous int32")
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, width), dtype=out_dtype, device=residual.device)
    _need(out.shape == (n_rows, width) and out.dtype == out_dtype and out.is_contiguous(), "add_rmsnorm: out has the wrong shape or dtype")
    library = _library("elementwise.cu")
    _check(library, library.pylon_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(rows), _ptr(out), n_rows, width,
                                              float(eps), 0 if rows is not None else 1, _dtype_code(out_dtype), _stream()))
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    if delta.dim() == 3:   # partial sums
        for part in delta:
            residual_add(residual, part)
        return
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and delta.is_contiguous() and delta.shape == residual.shape, "residual_add: shapes differ or tensors are not contiguous")
    library = _library("elementwise.cu")
    _check(library, library.pylon_residual_add(_ptr(residual), _ptr(delta), residual.numel(), _dtype_code(delta.dtype), _stream()))


def qk_norm_rope_kv_write(
    qkv: torch.Tensor,
    q_weight: Optional[torch.Tensor],
    k_weight: Optional[torch.Tensor],
    eps: float,
    cos: Optional[torch.Tensor],
    sin: Optional[torch.Tensor],
    rotary_dim: int,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
) -> torch.Tensor:
    """On ``qkv [T, (nq + 2 nkv) * d]``: RMSNorm each q and k head (when weights are given),
    rotate them by the float32 ``cos``/``sin [positions, rotary_dim / 2]`` tables, write q
    back in place and k, v into ``[pages, nkv, page_size, d]`` pages at each token's slot.
    Returns the tensor whose first ``nq * d`` columns now hold q: ``qkv`` itself.

    ``qkv`` may also be float32 partial sums ``[parts, T, (nq + 2 nkv) * d]`` (see
    :func:`linear_for_rotation`): they are added up on the way, and q is returned in a tensor
    of its own, ``[T, nq * d]`` in the pages' dtype."""
    _need_cuda(qkv, q_weight, k_weight, cos, sin, positions, token_row, block_table, k_pages, v_pages)
    partial = qkv.dim() == 3
    tokens = qkv.shape[-2]
    _need(qkv.dim() in (2, 3) and qkv.is_contiguous() and qkv.shape[-1] == (nq + 2 * nkv) * head_dim, "qk_norm_rope_kv_write: qkv must be contiguous [T, (nq + 2 nkv) * d]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "qk_norm_rope_kv_write: norm weights must be float32 [d]")
    table_positions = 0
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape
              and cos.dim() == 2 and cos.shape[1] * 2 == rotary_dim and cos.is_contiguous() and sin.is_contiguous(),
              "qk_norm_rope_kv_write: cos/sin must be float32 [positions, rotary_dim / 2]")
        table_positions = cos.shape[0]
    else:
        rotary_dim = 0
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "qk_norm_rope_kv_write: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "qk_norm_rope_kv_write: block_table must be contiguous int32 [rows, width]")
    activation = k_pages.dtype if partial else qkv.dtype
    for pages in (k_pages, v_pages):
        _need(pages.dtype == activation and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, head_dim),
              "qk_norm_rope_kv_write: pages must be contiguous [pages, nkv, page_size, d] in the activation dtype")
    library = _library("elementwise.cu")
    if partial:
        _need(qkv.dtype == torch.float32 and activation == torch.bfloat16 and head_dim in (64, 128, 256) and rotary_dim in (0, head_dim),
              "qk_norm_rope_kv_write: partial sums are float32, for bfloat16 pages, head size 64, 128 or 256 and rotation over the whole head")
        q = torch.empty((tokens, nq * head_dim), dtype=torch.bfloat16, device=qkv.device)
        _check(library, library.pylon_qk_norm_rope_kv_write_parts(
            _ptr(qkv), qkv.shape[0], _ptr(q), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim, table_positions,
            _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
            k_pages.shape[0], nq, nkv, head_dim, tokens, _ptr(cache_write_error_word(k_pages.device)), _stream()))
        return q
    _check(library, library.pylon_qk_norm_rope_kv_write(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim, table_positions,
        _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        k_pages.shape[0], nq, nkv, head_dim, tokens, _dtype_code(qkv.dtype), _ptr(cache_write_error_word(k_pages.device)), _stream()))
    return qkv


def qk_norm(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, nq: int, nkv: int, head_dim: int) -> torch.Tensor:
    """RMSNorm of every q and k head of ``qkv [T, (nq + 2 nkv) * d]`` in place, without rotation or
    cache write: for position encodings that run as a step of their own between the norms and
    :func:`qk_norm_rope_kv_write` (called without weights and tables, it then only writes the cache)."""
    _need_cuda(qkv, q_weight, k_weight)
    _need(qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (nq + 2 * nkv) * head_dim, "qk_norm: qkv must be contiguous [T, (nq + 2 nkv) * d]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "qk_norm: norm weights must be float32 [d]")
    library = _library("elementwise.cu")
    _check(library, library.pylon_qk_norm(_ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), nq, nkv, head_dim, qkv.shape[0],
                                          _dtype_code(qkv.dtype), _stream()))
    return qkv


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleaved: bool = False,
           limit: Optional[float] = None, alpha: float = 1.0) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` of shape ``[T, 2 * inter]``: ``[gate | up]`` in two
    halves, or with ``interleaved`` in alternating groups of 8 columns
    (``[g0..g7 u0..u7 g8..g15 u8..u15 ...]``, the layout :func:`interleave_gate_up` gives the
    weights).  With a ``limit`` the gated unit is the clamped one: ``g = min(gate, limit)``,
    ``u = clamp(up, -limit, limit)``, result ``g * sigmoid(alpha * g) * (u + 1)``."""
    _need(limit is None or limit > 0, "swiglu: a limit must be positive")
    _need_cuda(gate_up, out)
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0, "swiglu: gate_up must be contiguous [T, 2 * inter]")
    tokens, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out.shape == (tokens, inter) and out.dtype == gate_up.dtype and out.is_contiguous(), "swiglu: out has the wrong shape or dtype")
    library = _library("elementwise.cu")
    _check(library, library.pylon_swiglu(_ptr(gate_up), _ptr(out), tokens, inter, int(interleaved), _dtype_code(gate_up.dtype),
                                         float(limit or 0.0), float(alpha), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# matrix products: y = x @ w.T
# ---------------------------------------------------------------------------------------
SKINNY_MAX_ROWS = 8   # up to this many rows the weight-streaming kernel runs (it takes up to 64); above, the library


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K].T`` with float32 accumulation.

    float32 operands use the plain-FMA kernel (true 32-bit, no tensor cores).  bfloat16
    operands with up to ``SKINNY_MAX_ROWS`` rows use the weight-streaming kernel; many rows
    whose 128 x 256 tiles fill whole rounds over the SMs use our tcgen05 kernel; the rest go to
    the library matrix product, as raun6k/Pylon's ``nn.Linear`` layers do
    (src/pylon/model/layers.py:17-23,95-106).  ``out_dtype=torch.float32`` keeps the 32-bit
    accumulator (used for logits).
    """
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype, f"linear: activations are {x.dtype} but weights are {w.dtype}")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear: the reduced dimension must be contiguous")
    out_dtype = out_dtype or x.dtype
    m, k = x.shape
    n = w.shape[0]
    if x.dtype == torch.float32:
        _need(out_dtype == torch.float32, "linear: float32 operands give float32 results")
        y = torch.empty((m, n), dtype=torch.float32, device=x.device)
        library = _library("gemm_f32.cu")
        _check(library, library.pylon_gemm_f32_nt(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), n, _stream()))
        return y
    _need(x.dtype == torch.bfloat16, f"linear: unsupported dtype {x.dtype}")
    _need(out_dtype in (torch.bfloat16, torch.float32), f"linear: unsupported result dtype {out_dtype}")
    if m <= SKINNY_MAX_ROWS and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 \
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
        return linear_skinny(x, w, out_dtype)   # few rows (decode): our weight-streaming kernel
    if out_dtype == torch.bfloat16:
        if (m <= STREAM_MAX_ROWS and k >= 1024 and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return linear_stream(x, w)   # 9 to 32 rows over a long k: the TMA-fed kernel is ahead of the library there
        if _tcgen05_fills_the_sms(m, n, _multiprocessors(x.device)) and k % 8 == 0 and n % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 \
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            return linear_tcgen05(x, w)
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=torch.float32)


def _tcgen05_fills_the_sms(m: int, n: int, sms: int) -> bool:
    """Whether a persistent block per SM over 128 x 256 tiles wastes under a fifth of its
    rounds: there our kernel is level with the library's, elsewhere the library is ahead.  (The
    output and down projections of 2,048 rows are 160 such tiles on 148 SMs.  With tiles of 288
    columns, one round, our kernel takes 31.7 and 78.7 us for them, the library 29.6 and 71.7 us.)"""
    if m < TCGEN05_MIN_ROWS:
        return False
    tiles = -(-m // 128) * -(-n // 256)
    rounds = -(-tiles // sms)
    return tiles >= 0.8 * rounds * sms


STREAM_MAX_ROWS = 32   # up to this many rows the TMA-fed kernel beats the library (it takes up to 64)
STREAM_MAX_PARTS = 4


def linear_for_residual(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for a result that goes straight into the residual stream: either the
    product ``[M, N]`` in the activation dtype, or - for the few rows of a decode step -
    float32 partial sums ``[parts, M, N]`` over slices of k, which the stream's next norm adds
    up (no extra kernel, no atomics).  The slices make enough blocks to fill the GPU however
    few rows the matrix has."""
    m, k = x.shape
    n = w.shape[0]
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and m <= STREAM_MAX_ROWS and k >= 1024 and k % 8 == 0
            and n % 4 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return linear_stream_partial(x, w)
    return linear(x, w)


def linear_for_rotation(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """The fused QKV product for :func:`qk_norm_rope_kv_write`: the product ``[M, N]`` in the
    activation dtype, or - for the few rows of a decode step, where the TMA-fed kernel with
    its slices of k is the fastest way to read the weights - float32 partial sums
    ``[parts, M, N]``, which the rotation kernel adds up as it reads them."""
    m, k = x.shape
    n = w.shape[0]
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and m <= STREAM_MAX_ROWS and k >= 1024 and k % 8 == 0
            and head_dim in (64, 128, 256) and rotary_dim in (0, head_dim) and n % 4 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return linear_stream_partial(x, w)
    return linear(x, w)


def stream_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the TMA-fed decode product sets when one of its bounded waits ran out
    (its result is then void).  Zero in every healthy run."""
    return _error_words(device)[2:3]


def linear_stream_partial(x: torch.Tensor, w: torch.Tensor, parts: Optional[int] = None) -> torch.Tensor:
    """bfloat16 ``x [M <= 64, K] @ w [N, K].T`` as float32 partial sums ``[parts, M, N]`` over
    slices of k, the weights streamed by TMA through a shared-memory ring.  ``parts`` defaults
    to what gives every SM up to three blocks (64 weight rows x one slice each), at most
    ``STREAM_MAX_PARTS``: more parts cost the reader more than they save here (the norm that adds
    them up took 3.0 us with 4 parts and 5.1 us with 11)."""
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16,
          "linear_stream_partial: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_stream_partial: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    slabs, k_boxes = -(-n // 64), -(-k // 64)
    if parts is None:
        parts = max(1, min(STREAM_MAX_PARTS, k_boxes, (3 * _multiprocessors(x.device)) // slabs))
    y = torch.empty((parts, m, n), dtype=torch.float32, device=x.device)
    library = _library("gemm_stream.cu")
    _check(library, library.pylon_gemm_stream_partial(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), parts,
                                                      _ptr(stream_error_word(x.device)), _stream()))
    return y


def linear_stream(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False, limit: Optional[float] = None, alpha: float = 1.0) -> torch.Tensor:
    """bfloat16 ``x [M <= 64, K] @ w [N, K].T`` on the TMA-fed kernel, one block per 64 weight rows
    over the whole of k; with ``swiglu`` the rows of ``w`` are interleaved gate/up groups (see
    :func:`interleave_gate_up`) and the result is ``silu(gate) * up``, ``[M, N / 2]`` - or, with a
    ``limit``, the clamped gated unit of :func:`swiglu`."""
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16,
          "linear_stream: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_stream: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_stream.cu")
    if swiglu and limit is not None:
        _check(library, library.pylon_gemm_stream_glu_clamped(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), float(limit),
                                                              float(alpha), _ptr(stream_error_word(x.device)), _stream()))
        return y
    entry = library.pylon_gemm_stream_swiglu if swiglu else library.pylon_gemm_stream_bf16
    _check(library, entry(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), _ptr(stream_error_word(x.device)), _stream()))
    return y


def linear_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The weight-streaming kernel itself: bfloat16 ``x [M <= 64, K] @ w [N, K].T`` with ``K``
    and the row strides multiples of 8 and 16-byte aligned operands; anything else is refused."""
    _need_cuda(x, w)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1],
          "linear_skinny: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_skinny: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    library = _library("gemm_skinny.cu")
    _check(library, library.pylon_gemm_skinny_bf16(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), n, _dtype_code(out_dtype), _stream()))
    return y


TCGEN05_MIN_ROWS = 128   # from this many rows the gate/up product runs on our tcgen05 kernel, SwiGLU in its epilogue

def tcgen05_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the tcgen05 kernels set when one of their bounded waits ran out
    (the result of that launch is then void).  Zero in every healthy run."""
    return _error_words(device)[0:1]


def tcgen05_force_tile(columns: int = 0) -> None:
    """For measurements: later ``linear_tcgen05`` calls use ``128 x columns`` output tiles
    (288, 256, 192, 160 or 128); 0 restores the choice by size."""
    _library("gemm_tcgen05.cu").pylon_gemm_tcgen05_force_tile(columns)


def linear_tcgen05(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False, limit: Optional[float] = None, alpha: float = 1.0) -> torch.Tensor:
    """bfloat16 ``x [M, K] @ w [N, K].T`` on the tcgen05 tensor cores (TMA-fed, accumulators in
    tensor memory).  With ``swiglu`` the rows of ``w`` are interleaved by
    :func:`interleave_gate_up` and the result is ``silu(gate) * up``, ``[M, N / 2]`` - or, with a
    ``limit``, the clamped gated unit of :func:`swiglu`."""
    _need_cuda(x, w)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1],
          "linear_tcgen05: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_tcgen05: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_tcgen05.cu")
    if swiglu and limit is not None:
        _check(library, library.pylon_gemm_tcgen05_glu_clamped(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), float(limit),
                                                               float(alpha), _ptr(tcgen05_error_word(x.device)), _multiprocessors(x.device), _stream()))
        return y
    _check(library, library.pylon_gemm_tcgen05_bf16(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), int(swiglu),
                                                    _ptr(tcgen05_error_word(x.device)), _multiprocessors(x.device), _stream()))
    return y

QKV_ROTATION_MIN_ROWS = 3_072


def qkv_rotation_fuses(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int, k_pages: torch.Tensor) -> bool:
    """Whether :func:`linear_qkv_rotated` takes this step's QKV product: a long prompt portion, in bfloat16, heads of 64
    or 128 rotated as a whole.  The last tile's longer epilogue has nothing to hide behind, so the fusion pays from some
    3,000 rows on (Qwen3-4B widths: 108 us against 115 us for product and rotation kernel at 4,096 rows, 204 against 239
    at 8,192; 61 against 59 at 2,048)."""
    m, k = x.shape
    return (m >= QKV_ROTATION_MIN_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and x.is_cuda and head_dim in (64, 128)
            and rotary_dim == head_dim and k % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and _tcgen05_fills_the_sms(m, w.shape[0], _multiprocessors(x.device)))


def linear_qkv_rotated(
    x: torch.Tensor, w: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, cos: torch.Tensor,
    sin: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor, block_table: torch.Tensor, page_size: int, k_pages: torch.Tensor,
    v_pages: torch.Tensor, nq: int, nkv: int, head_dim: int,
) -> torch.Tensor:
    """The fused QKV product ``x [T, K] @ w [(nq + 2 nkv) * d, K].T`` on the tcgen05 kernel with
    :func:`qk_norm_rope_kv_write` in its epilogue: the heads are normalised and rotated from the float32 accumulators, k
    and v go straight into their pages and q, ``[T, nq * d]`` in bfloat16, is returned; the product never goes to memory."""
    _need_cuda(x, w, q_weight, k_weight, cos, sin, positions, token_row, block_table, k_pages, v_pages)
    tokens, k = x.shape
    _need(x.dim() == 2 and w.dim() == 2 and w.shape == ((nq + 2 * nkv) * head_dim, k) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
          and x.stride(1) == 1 and w.stride(1) == 1, "linear_qkv_rotated: bfloat16 x [T, K] and w [(nq + 2 nkv) * d, K]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "linear_qkv_rotated: norm weights must be float32 [d]")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] * 2 == head_dim
          and cos.is_contiguous() and sin.is_contiguous(), "linear_qkv_rotated: cos/sin must be float32 [positions, d / 2]")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "linear_qkv_rotated: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "linear_qkv_rotated: block_table must be contiguous int32 [rows, width]")
    for pages in (k_pages, v_pages):
        _need(pages.dtype == torch.bfloat16 and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, head_dim),
              "linear_qkv_rotated: pages must be contiguous bfloat16 [pages, nkv, page_size, d]")
    q = torch.empty((tokens, nq * head_dim), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_tcgen05.cu")
    _check(library, library.pylon_gemm_tcgen05_qkv_rotate(
        _ptr(x), _ptr(w), _ptr(q), tokens, k, x.stride(0), w.stride(0), q.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin),
        cos.shape[0], _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        k_pages.shape[0], nq, nkv, head_dim, _ptr(cache_write_error_word(k_pages.device)), _ptr(tcgen05_error_word(x.device)),
        _multiprocessors(x.device), _stream()))
    return q


# Small integer buffers kernels use to find out which of their blocks finishes last.  They
# are zero between launches (a kernel leaves its counters as it found them) and launches on
# one stream follow each other, so one buffer per device and purpose is enough.
_counter_buffers: dict[tuple, torch.Tensor] = {}


def _zeroed_counters(device: torch.device, purpose: str, count: int) -> torch.Tensor:
    key = (_device_index(device), purpose)
    buffer = _counter_buffers.get(key)
    if buffer is None or buffer.numel() < count:
        if buffer is not None:
            _retired_counter_buffers.append(buffer)   # a captured graph may still hold its address
        buffer = torch.zeros(max(count, 1 << 16), dtype=torch.int32, device=device)
        _counter_buffers[key] = buffer
    return buffer


_retired_counter_buffers: list[torch.Tensor] = []


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stacks the ``[inter, K]`` gate and up matrices in alternating groups of 8 rows (8 gate
    rows, their 8 up rows, ...), so that one block of 16 weight rows holds both halves of 8
    outputs.  ``inter`` must be a multiple of 8."""
    inter, k = gate.shape
    _need(up.shape == gate.shape and inter % 8 == 0, "interleave_gate_up: equal shapes with a row count that is a multiple of 8")
    return torch.stack((gate.reshape(inter // 8, 8, k), up.reshape(inter // 8, 8, k)), dim=1).reshape(2 * inter, k).contiguous()


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, limit: Optional[float] = None, alpha: float = 1.0) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` for weights stacked by :func:`interleave_gate_up`:
    one kernel for few rows (the TMA-fed decode kernel) and for many (the tcgen05 kernel), the
    library product and the SwiGLU kernel in between.  With a ``limit`` the gated unit is the clamped
    one of :func:`swiglu`, in the same kernels."""
    _need_cuda(x, w_interleaved)
    n, k = w_interleaved.shape
    m = x.shape[0]
    if (x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and x.dim() == 2 and m <= STREAM_MAX_ROWS and x.shape[1] == k
            and k % 8 == 0 and n % 16 == 0 and x.stride(1) == 1 and w_interleaved.stride(1) == 1 and x.stride(0) % 8 == 0
            and w_interleaved.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0):
        return linear_stream(x, w_interleaved, swiglu=True, limit=limit, alpha=alpha)
    if (x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and k % 8 == 0
            and n % 16 == 0 and x.stride(1) == 1 and w_interleaved.stride(1) == 1 and x.stride(0) % 8 == 0 and w_interleaved.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0):
        return linear_tcgen05(x, w_interleaved, swiglu=True, limit=limit, alpha=alpha)   # many rows: our tcgen05 kernel with the gated unit in its epilogue
    return swiglu(linear(x, w_interleaved), interleaved=True, limit=limit, alpha=alpha)


# ---------------------------------------------------------------------------------------
# attention over the paged cache
# ---------------------------------------------------------------------------------------
def attention_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the attention kernels set when a bounded wait for one of their TMA copies
    ran out (the output of that launch is then void).  Zero in every healthy run."""
    return _error_words(device)[1:2]


def attention_splits(num_rows: int, nkv: int, group: int, max_q: int, max_kv: int, sms: int) -> int:
    """How many key/value splits the tiled attention kernel uses for rows with more than 16
    packed query rows (tokens x group), on a device with ``sms`` multiprocessors.

    Steps with long rows (prefill) have enough query tiles to fill the GPU and use one; a few
    short portions over a long context are split so that two blocks per SM have work.  Rows
    of decoded tokens do not use this: their kernel cuts all rows' tiles into equal runs.
    """
    if max_q * group <= 16:
        return 1
    kv_tiles = max(1, -(-max_kv // 64))
    blocks = num_rows * nkv * -(-max_q * group // 64)
    if blocks >= sms or kv_tiles == 1:
        return 1
    return int(max(1, min(kv_tiles, 64, 2 * sms // blocks)))


def paged_attention(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    block_table: torch.Tensor,
    nq: int,
    max_q: int,
    max_kv: int,
    window: Optional[int] = None,
    scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    force_simple: bool = False,
    decode_blocks: Optional[int] = None,
    prefill_kernel: Optional[str] = None,
    row_tokens: Optional[Sequence[int]] = None,
    rows_alike: bool = False,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
    sinks: Optional[torch.Tensor] = None,
    values_in_keys: Optional[int] = None,
    keep_first: int = 0,
    distance_bias: Optional[torch.Tensor] = None,
    split_weights: bool = False,
) -> torch.Tensor:
    """Causal attention of every token of a step over its request's pages.

    ``split_weights`` (latent rows on the tensor cores): a softmax weight enters the weighted sum as two bfloat16 numbers, the rounded
    weight and what the rounding dropped, so that it counts with 16 bits instead of 8, at twice the products over the values.

    ``keep_first`` n: a window never hides the keys at positions below n (a token sees ``j <= p`` with ``p - j < window`` or
    ``j < n``).  ``distance_bias``: float32 ``[rows, nq]``; the scaled score of the key ``p - j`` positions back gets
    ``distance_bias[min(p - j, rows - 1), h]`` added.  These, sinks and values of another width than the keys run in bfloat16 on a
    tensor-core kernel of their own (``csrc/attention_window.cu``, built per pair of sizes on first use: keys of a multiple of 16 and
    values of a multiple of 8 up to 256, at most 8 query heads to a KV head), else on the plain kernel.

    ``sinks``: float32 ``[nq]``; the softmax's denominator of head h also holds ``exp(sinks[h])``, a key without a
    value whose score is taken as it stands.  ``values_in_keys`` n (with ``v_pages=None``): the values are the first n
    columns of the key rows themselves - one latent row per token that every head reads (``nkv`` = 1 then).

    ``chunk``: a token sees only the keys of its own chunk of positions (``j // chunk == p // chunk``,
    counted from position 0 of the request).  ``softcap`` c: a scaled score s becomes ``c * tanh(s / c)``.
    The value pages may have another row width than the key pages; the result is ``[T, nq * value width]``.

    ``q``: ``[T, >= nq * d]`` (only the first ``nq * d`` columns of each row are read, so
    the fused qkv buffer can be passed as it is); pages ``[P, nkv, page_size, d]``;
    ``positions``/``token_row`` int32 ``[T]``; ``q_start`` int32 ``[rows + 1]``; ``kv_len``
    int32 ``[rows]`` (tokens each row holds after this step, so a row's first new token is
    at position ``kv_len - (q_start[r + 1] - q_start[r])``); ``block_table`` int32
    ``[rows, width]``; ``max_q``/``max_kv``: longest row and longest context (upper bounds
    are fine).  ``num_splits`` and ``decode_blocks`` override the split of long rows' keys and
    the number of blocks that share the decoded rows' tiles, ``prefill_kernel`` (``"tcgen05"`` or
    ``"mma"``) the kernel for rows of more than 16 packed query rows (for tests).
    ``row_tokens``: the rows' token counts on the host, if the caller has them: the kernel
    for prompt portions then launches blocks only for the rows that are its own (a step that
    mixes one portion with 63 decoded rows would otherwise start 63 rows of blocks that find
    nothing to do).  ``rows_alike``: the caller knows that the rows hold about equally many tokens;
    a step of a few decoded rows then gives every (row, KV head) pair a thread-block cluster of
    its own, whose blocks combine their results through distributed shared memory (right for any
    lengths, but slow if they differ much).  Returns ``[T, nq * d]``.

    bfloat16 with a head size that is a multiple of 16 up to 256 runs on the tensor cores
    (built per head size on first use): prompt portions on ``tcgen05.mma`` with the accumulators
    in tensor memory where the head size is 64 or 128 and a page holds a multiple of 64 keys,
    else on ``mma.sync``; decoded tokens on their own kernel.  float32, and other head sizes up
    to 512, take the plain kernel.
    """
    _need_cuda(q, k_pages, v_pages, positions, token_row, q_start, kv_len, block_table, out, sinks, distance_bias)
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous()), "paged_attention: sinks must be float32 [nq]")
    _need(distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.dim() == 2 and distance_bias.shape[0] >= 1 and distance_bias.shape[1] == nq
                                    and distance_bias.is_contiguous()), "paged_attention: distance_bias must be contiguous float32 [rows, nq]")
    _need(keep_first >= 0 and (keep_first == 0 or (chunk is None and values_in_keys is None)), "paged_attention: kept first keys go with a window only")
    _need(distance_bias is None or values_in_keys is None, "paged_attention: no bias by distance over latent rows")
    plain_only = keep_first > 0 or distance_bias is not None
    if values_in_keys is not None:
        _need(v_pages is None and k_pages.dim() == 4 and k_pages.is_contiguous() and 1 <= values_in_keys <= k_pages.shape[3],
              "paged_attention: values inside the key rows are their first columns, and there are no value pages then")
        return _latent_attention(q, k_pages, int(values_in_keys), positions, token_row, q_start, kv_len, block_table, nq, max_q, max_kv, window, scale,
                                 sinks, out, force_simple, num_splits, split_weights)
    _need(k_pages.dim() == 4 and v_pages.dim() == 4 and k_pages.shape[:3] == v_pages.shape[:3] and k_pages.is_contiguous() and v_pages.is_contiguous()
          and k_pages.dtype == v_pages.dtype, "paged_attention: pages must be contiguous [P, nkv, page_size, d] and [P, nkv, page_size, value width]")
    num_pages, nkv, page_size, d = k_pages.shape
    dv = v_pages.shape[3]
    _need(chunk is None or chunk >= 1, "paged_attention: a chunk holds at least one position")
    _need(softcap is None or softcap > 0, "paged_attention: a soft cap must be positive")
    same_width = dv == d   # the tensor-core kernels are built for values as wide as the keys
    tokens = q.shape[0]
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= nq * d and q.dtype == k_pages.dtype, "paged_attention: q must be [T, >= nq * d] in the cache dtype")
    _need(nq % nkv == 0, f"paged_attention: {nq} query heads over {nkv} KV heads")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "paged_attention: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "paged_attention: block_table must be contiguous int32 [rows, width]")
    rows = block_table.shape[0]
    _need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.shape[0] >= rows + 1, "paged_attention: q_start must be int32 [rows + 1]")
    _need(kv_len.dtype == torch.int32 and kv_len.is_contiguous() and kv_len.shape[0] >= rows, "paged_attention: kv_len must be int32 [rows]")
    if out is None:
        out = torch.empty((tokens, nq * dv), dtype=q.dtype, device=q.device)
    _need(out.shape == (tokens, nq * dv) and out.dtype == q.dtype and out.is_contiguous(), "paged_attention: out has the wrong shape or dtype")
    scale = 1.0 / math.sqrt(d) if scale is None else float(scale)
    _need(scale > 0, "paged_attention: the softmax scale must be positive")
    if q.dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and not force_simple and same_width and sinks is None and not plain_only:
        library = _library("attention_mma.cu", {"PYLON_HEAD_DIM": d})
        group = nq // nkv
        any_large = max_q * group > 16
        # Rows of decoded tokens can occur unless the step is one long row.
        maybe_small = not any_large or rows > 1
        if row_tokens is not None and len(row_tokens) == rows and all(count * group > 16 for count in row_tokens):
            maybe_small = False   # the host knows that every row is a prompt portion: no launch of the decode kernel
        # Prompt portions go to the tcgen05 kernel where it exists: head size 64 or 128, pages of a multiple of 64 keys.
        if prefill_kernel is None:
            prefill_kernel = "tcgen05" if d in (64, 128) and page_size % 64 == 0 and num_splits in (None, 1) else "mma"
        _need(prefill_kernel in ("tcgen05", "mma"), f"paged_attention: unknown prefill kernel {prefill_kernel!r}")
        use_tcgen05 = any_large and prefill_kernel == "tcgen05"
        if use_tcgen05:
            _need(d in (64, 128) and page_size % 64 == 0, "paged_attention: the tcgen05 kernel needs head size 64 or 128 and pages of a multiple of 64 keys")
            fast = _library("attention_tcgen05.cu", {"PYLON_HEAD_DIM": d})
            first_row, row_count = 0, rows
            if row_tokens is not None and len(row_tokens) == rows:
                large = [index for index, count in enumerate(row_tokens) if count * group > 16]
                if large and large[-1] - large[0] + 1 == len(large):   # one run of rows: the scheduler puts decoded rows first
                    first_row, row_count = large[0], len(large)
            _check(fast, fast.pylon_paged_attention_tcgen05_masked(
                _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(q_start), _ptr(kv_len), _ptr(block_table),
                block_table.shape[1], page_size, num_pages, nq, nkv, int(window or 0), int(chunk or 0), float(softcap or 0.0), scale,
                first_row, row_count, int(max_q), int(maybe_small),
                _ptr(attention_error_word(q.device)), _stream()))
            if not maybe_small:
                return out
        splits = 1 if use_tcgen05 else (attention_splits(rows, nkv, group, max_q, max_kv, _multiprocessors(q.device)) if num_splits is None else int(num_splits))
        blocks = 0
        if maybe_small:
            blocks = library.pylon_attention_decode_blocks() if decode_blocks is None else int(decode_blocks)
            _need(blocks >= 1, "paged_attention: the decode kernel does not fit on this device")
        scratch = counters = None
        floats = library.pylon_attention_scratch_floats(splits, tokens, nq, rows, nkv, blocks)
        if floats:
            scratch = torch.empty((floats,), dtype=torch.float32, device=q.device)
        if blocks:
            counters = _zeroed_counters(q.device, "attention", rows * nkv)
        _check(library, library.pylon_paged_attention_mma_masked(
            _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(counters), _ptr(q_start), _ptr(kv_len),
            _ptr(block_table), block_table.shape[1], page_size, num_pages, nq, nkv, int(window or 0), int(chunk or 0), float(softcap or 0.0),
            scale, rows, tokens,
            int(max_q), splits, blocks, int(use_tcgen05), int(bool(rows_alike)), _ptr(attention_error_word(q.device)), _stream()))
        return out
    if ((plain_only or sinks is not None) and q.dtype == torch.bfloat16 and not force_simple and chunk is None and softcap is None and d % 16 == 0 and d <= 256 and dv % 8 == 0 and dv <= 256
            and nq // nkv <= 8 and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0):
        library = _library("attention_window.cu", {"PYLON_HEAD_DIM": d, "PYLON_VALUE_DIM": dv})
        splits = window_attention_splits(rows, nkv, max_q, max_kv, window, keep_first, _multiprocessors(q.device)) if num_splits is None else int(num_splits)
        scratch = None
        if splits > 1:
            scratch = torch.empty((library.pylon_window_attention_scratch_floats(splits, tokens, nq),), dtype=torch.float32, device=q.device)
        _check(library, library.pylon_window_attention(
            _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.shape[1], page_size,
            num_pages, nq, nkv, int(window or 0), int(keep_first), scale, _ptr(distance_bias), 0 if distance_bias is None else distance_bias.shape[0],
            _ptr(sinks), rows, int(max_q), splits, _ptr(scratch), _ptr(token_row), tokens, _ptr(attention_error_word(q.device)), _stream()))
        if splits > 1:
            launches[0] += 1   # the parts' sum is a kernel of its own
        return out
    _need(d <= 2048 and dv <= 512, f"paged_attention: head sizes {d} / {dv}: at most 2048 / 512")
    library = _library("attention_simple.cu")
    _check(library, library.pylon_paged_attention_simple(
        _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(positions), _ptr(token_row), _ptr(block_table),
        block_table.shape[1], page_size, num_pages, nq, nkv, d, dv, int(window or 0), int(chunk or 0), float(softcap or 0.0), scale,
        _ptr(sinks), 0, 0, tokens, _dtype_code(q.dtype), int(keep_first), _ptr(distance_bias), 0 if distance_bias is None else distance_bias.shape[0], _stream()))
    return out


def window_attention_splits(rows: int, nkv: int, max_q: int, max_kv: int, window: Optional[int], keep_first: int, sms: int) -> int:
    """Over how many blocks the kernel for windows with kept first keys deals out the key tiles of 16 tokens of one KV head: one for steps
    with enough blocks to fill the device (prompt portions); for a few decoded tokens as many as give every SM two blocks, each with
    at least two key tiles of 32."""
    blocks = rows * nkv * -(-max_q // 16)
    key_tiles = -(-min(max_kv, (window or max_kv) + keep_first + 16) // 32)
    if blocks >= sms or key_tiles < 4:
        return 1
    return int(max(1, min(key_tiles // 2, 2 * sms // blocks, 32)))


def latent_attention_splits(rows: int, nq: int, max_q: int, max_kv: int, window: Optional[int], sms: int) -> int:
    """Over how many blocks the tensor-core kernel for latent rows cuts the keys of a tile of 64 packed query rows: one for steps
    with enough tiles to fill the device (prompt portions); for a few decoded tokens as many as give every SM two blocks, each
    with at least two key tiles of 32."""
    tiles = rows * -(-max_q * nq // 64)
    key_tiles = -(-min(max_kv, (window or max_kv) + max_q) // 32)
    if max_q * nq > 64 or tiles >= sms or key_tiles < 4:
        return 1
    return int(max(1, min(key_tiles // 2, 2 * sms // tiles, 64)))


def _latent_attention(q, pages, dv, positions, token_row, q_start, kv_len, block_table, nq, max_q, max_kv, window, scale, sinks, out, force_simple, num_splits,
                      split_weights=False):
    """Attention of ``nq`` heads over one shared row per token: keys are the whole rows ``[d]``, values their first ``dv`` columns.
    bfloat16 rows of a multiple of 16 numbers (up to 832) with values of a multiple of 32 (up to 512) run on the tensor cores
    (``csrc/attention_latent.cu``, built per pair of sizes on first use); float32 and other sizes take the plain kernel."""
    num_pages, nkv, page_size, d = pages.shape
    tokens = q.shape[0]
    _need(nkv == 1, "paged_attention: a latent row per token is shared by all heads (one KV head)")
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= nq * d and q.dtype == pages.dtype, "paged_attention: q must be [T, >= nq * d] in the cache dtype")
    _need(scale is not None and scale > 0, "paged_attention: latent rows need the softmax scale spelled out")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "paged_attention: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "paged_attention: block_table must be contiguous int32 [rows, width]")
    if out is None:
        out = torch.empty((tokens, nq * dv), dtype=q.dtype, device=q.device)
    _need(out.shape == (tokens, nq * dv) and out.dtype == q.dtype and out.is_contiguous(), "paged_attention: out has the wrong shape or dtype")
    _need(d <= 2048 and dv <= 512, f"paged_attention: latent rows of {d} with values of {dv}: at most 2048 / 512")
    rows = block_table.shape[0]
    _need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.shape[0] >= rows + 1, "paged_attention: q_start must be int32 [rows + 1]")
    _need(kv_len.dtype == torch.int32 and kv_len.is_contiguous() and kv_len.shape[0] >= rows, "paged_attention: kv_len must be int32 [rows]")
    if q.dtype == torch.bfloat16 and d % 16 == 0 and d <= 832 and dv % 32 == 0 and not force_simple and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
        defines = {"PYLON_LATENT_DIM": d, "PYLON_LATENT_VALUE_DIM": dv}
        if split_weights:   # the weights with 16 bits in the second product (a library of its own)
            defines["PYLON_LATENT_SPLIT_WEIGHTS"] = 1
        library = _library("attention_latent.cu", defines)
        splits = latent_attention_splits(rows, nq, max_q, max_kv, window, _multiprocessors(q.device)) if num_splits is None else int(num_splits)
        scratch = None
        if splits > 1:
            scratch = torch.empty((library.pylon_latent_attention_scratch_floats(splits, tokens, nq),), dtype=torch.float32, device=q.device)
        _check(library, library.pylon_latent_attention(
            _ptr(q), q.stride(0), _ptr(pages), _ptr(out), _ptr(scratch), _ptr(q_start), _ptr(kv_len), _ptr(token_row), _ptr(block_table),
            block_table.shape[1], page_size, num_pages, nq, int(window or 0), float(scale), _ptr(sinks), rows, tokens, int(max_q), splits, _stream()))
        return out
    library = _library("attention_simple.cu")
    _check(library, library.pylon_paged_attention_simple(
        _ptr(q), q.stride(0), _ptr(pages), _ptr(pages), _ptr(out), _ptr(positions), _ptr(token_row), _ptr(block_table),
        block_table.shape[1], page_size, num_pages, nq, 1, d, dv, int(window or 0), 0, 0.0, float(scale),
        _ptr(sinks), d, d, tokens, _dtype_code(q.dtype), 0, None, 0, _stream()))
    return out


def qk_norm_mix_kv_write(
    qkv: torch.Tensor,
    q_weight: Optional[torch.Tensor],
    k_weight: Optional[torch.Tensor],
    eps: float,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
    value_dim: int,
    other_values: Optional[torch.Tensor] = None,
    mix_weight: Optional[torch.Tensor] = None,
    other_head_width: Optional[int] = None,
    whole_rows: bool = False,
) -> torch.Tensor:
    """For attention without rotation, on ``qkv [T, nq * d + nkv * d + nkv * dv]``: RMSNorm each q and k head (when
    weights are given), q back in place, k into its page slot; every v head, mixed first with another layer's values
    of the same token when ``other_values [T, >= nkv * dv]`` (any row stride) and ``mix_weight`` (one float32 on the
    device, the share of the other values) are given - ``v = (1 - w) v + w other`` -, back in place and into its page
    slot.  ``other_head_width``: how far apart the heads of ``other_values`` lie (default ``dv``; another width when the
    other layer keeps its values padded: only the columns that both have are mixed).  Returns ``qkv``: its first ``nq * d``
    columns hold q, its last ``nkv * dv`` the values that were kept."""
    _need_cuda(qkv, q_weight, k_weight, positions, token_row, block_table, k_pages, v_pages, other_values, mix_weight)
    tokens = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (nq + nkv) * head_dim + nkv * value_dim, "qk_norm_mix_kv_write: qkv must be contiguous [T, nq d + nkv d + nkv dv]")
    for weight, heads in ((q_weight, nq), (k_weight, nkv)):
        if weight is not None or whole_rows:
            size = heads * head_dim if whole_rows else head_dim
            _need(weight is not None and weight.dtype == torch.float32 and weight.shape == (size,) and weight.is_contiguous(),
                  f"qk_norm_mix_kv_write: norm weights must be float32 [{size}]")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "qk_norm_mix_kv_write: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "qk_norm_mix_kv_write: block_table must be contiguous int32 [rows, width]")
    for pages, width in ((k_pages, head_dim), (v_pages, value_dim)):
        _need(pages.dtype == qkv.dtype and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, width),
              "qk_norm_mix_kv_write: pages must be contiguous [pages, nkv, page_size, width] in the activation dtype")
    _need((other_values is None) == (mix_weight is None), "qk_norm_mix_kv_write: other values and their weight go together")
    other_stride = 0
    other_head_width = value_dim if other_head_width is None else int(other_head_width)
    if other_values is not None:
        _need(other_head_width >= 1 and other_values.dim() == 2 and other_values.shape == (tokens, nkv * other_head_width)
              and other_values.stride(1) == 1 and other_values.dtype == qkv.dtype,
              "qk_norm_mix_kv_write: other values must be [T, nkv * other_head_width] in the activation dtype")
        _need(mix_weight.dtype == torch.float32 and mix_weight.numel() == 1, "qk_norm_mix_kv_write: the mixing weight is one float32")
        other_stride = other_values.stride(0)
    library = _library("elementwise.cu")
    if whole_rows:
        _need(other_values is None, "qk_norm_mix_kv_write: no value mixing beside norms over whole rows")
        _check(library, library.pylon_qk_whole_norm_kv_write(
            _ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size,
            _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], nq, nkv, head_dim, value_dim, tokens, _dtype_code(qkv.dtype),
            _ptr(cache_write_error_word(k_pages.device)), _stream()))
        return qkv
    _check(library, library.pylon_qk_norm_mix_kv_write(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(other_values), other_stride, other_head_width, _ptr(mix_weight), _ptr(positions),
        _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], nq, nkv,
        head_dim, value_dim, tokens, _dtype_code(qkv.dtype), _ptr(cache_write_error_word(k_pages.device)), _stream()))
    return qkv


# ---------------------------------------------------------------------------------------
# residual streams (one or several) and the norms that read them
# ---------------------------------------------------------------------------------------
NORM_KINDS = {"layernorm": 0, "rmsnorm": 1, "dynamic_tanh": 2}


def streams_update_norm(
    streams: torch.Tensor,
    delta: Optional[torch.Tensor],
    scale: float = 1.0,
    mix: Optional[torch.Tensor] = None,
    out_weights: Optional[torch.Tensor] = None,
    read_weights: Optional[torch.Tensor] = None,
    norm_weight: Optional[torch.Tensor] = None,
    eps: float = 0.0,
    kind: str = "layernorm",
    out_dtype: Optional[torch.dtype] = None,
    rows: Optional[torch.Tensor] = None,
    norm_bias: Optional[torch.Tensor] = None,
    norm_alpha: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """The residual stream kept as ``S`` copies, float32 ``[T, S, width]`` (``[T, width]`` is one copy).

    First, if anything is pending (``delta``, the sublayer output ``[T, width]`` in the activation dtype or float32
    partial sums ``[parts, T, width]``; or a ``mix``), all streams at once from the old ones:
    ``x_t = sum_s mix[s, t] x_s + scale * out_weights[t] * delta`` (``mix`` float32 ``[S, S]``, ``None`` = identity;
    ``out_weights`` float32 ``[S]``, ``None`` = ones), in place.  Then, with a ``norm_weight``, the combination
    ``u = sum_s read_weights[s] x_s`` (``None`` = the plain sum) goes through the norm (``layernorm``: mean subtracted,
    variance the mean of squared deviations, no bias; ``rmsnorm``; ``dynamic_tanh``: ``tanh(norm_alpha * u) * norm_weight + norm_bias``
    with ``norm_alpha`` float32 ``[1]`` and ``norm_bias`` float32 ``[width]``, no statistics and no eps) and comes back ``[T, width]`` in ``out_dtype``.
    With ``rows`` (int32) only those tokens are normalised, from updated values computed on the fly; the streams stay
    as they are."""
    _need_cuda(streams, delta, mix, out_weights, read_weights, norm_weight, rows)
    _need(streams.dtype == torch.float32 and streams.is_contiguous() and streams.dim() in (2, 3), "streams_update_norm: streams must be contiguous float32 [T, S, width] or [T, width]")
    tokens, width = streams.shape[0], streams.shape[-1]
    count = 1 if streams.dim() == 2 else streams.shape[1]
    parts, delta_code = 1, F32
    if delta is not None:
        _need(delta.is_contiguous() and delta.shape[-2:] == (tokens, width) and delta.dim() in (2, 3), "streams_update_norm: delta must be contiguous [T, width] or [parts, T, width]")
        parts = delta.shape[0] if delta.dim() == 3 else 1
        delta_code = _dtype_code(delta.dtype)
    for name, tensor, shape in (("mix", mix, (count, count)), ("out_weights", out_weights, (count,)), ("read_weights", read_weights, (count,)),
                                ("norm_weight", norm_weight, (width,))):
        if tensor is not None:
            _need(tensor.dtype == torch.float32 and tuple(tensor.shape) == shape and tensor.is_contiguous(), f"streams_update_norm: {name} must be contiguous float32 {shape}")
    _need(kind in NORM_KINDS, f"streams_update_norm: unknown norm kind {kind!r}")
    if kind == "dynamic_tanh" and norm_weight is not None:
        _need_cuda(norm_bias, norm_alpha)
        _need(norm_bias is not None and norm_bias.dtype == torch.float32 and norm_bias.shape == (width,) and norm_bias.is_contiguous()
              and norm_alpha is not None and norm_alpha.dtype == torch.float32 and norm_alpha.numel() == 1,
              "streams_update_norm: a dynamic tanh needs a float32 bias [width] and one float32 alpha")
    n_rows = tokens
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "streams_update_norm: rows must be contiguous int32")
        _need(norm_weight is not None, "streams_update_norm: a row selection needs a norm")
        n_rows = rows.shape[0]
    out = None
    if norm_weight is not None:
        _need(out_dtype is not None, "streams_update_norm: a norm needs an output dtype")
        out = torch.empty((n_rows, width), dtype=out_dtype, device=streams.device)
    elif delta is None and mix is None:
        return None
    library = _library("streams.cu")
    _check(library, library.pylon_streams_update_norm(
        _ptr(streams), _ptr(delta), parts, delta_code, float(scale), _ptr(mix), _ptr(out_weights), _ptr(read_weights), _ptr(norm_weight),
        _ptr(rows), _ptr(out), _dtype_code(out_dtype) if out is not None else F32, n_rows, tokens, count, width, float(eps), NORM_KINDS[kind],
        _ptr(norm_bias), _ptr(norm_alpha), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# gated delta rule
# ---------------------------------------------------------------------------------------
def gated_delta_rule(
    proj: torch.Tensor,
    conv_weight: torch.Tensor,
    state: torch.Tensor,
    token_row: torch.Tensor,
    q_start: torch.Tensor,
    slots: torch.Tensor,
    a_log: torch.Tensor,
    dt_bias: torch.Tensor,
    norm_weight: torch.Tensor,
    heads: int,
    kv_heads: int,
    dim: int,
    vdim: int,
    num_rows: int,
    norm_eps: float,
    unit_eps: float = 1e-6,
    decay_in: Optional[torch.Tensor] = None,
    gate_in: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """The gated delta rule over the tokens of a step (see ``csrc/delta_rule.cu`` for the equations).

    ``decay_in`` float32 ``[T, heads * dim]``: a decay per head and key channel, from this input (``dt_bias`` is then ``[heads * dim]``
    and ``proj`` has no ``a`` columns).  ``gate_in`` float32 ``[T, heads * vdim]``: the output gate is its sigmoid (``proj`` then
    has no ``gate`` columns).

    ``proj [T, 2 kv_heads dim + 2 heads vdim + 2 heads]``: the projections of the layer's input with columns
    ``[q | k | v | gate | a | b]``; ``conv_weight`` float32 ``[taps, channels]`` over the q, k, v columns (the last tap weighs the current token); ``state`` float32
    ``[slots, heads * dim * vdim + (taps - 1) * channels]``: per request the heads' matrices and the convolution's last
    inputs, read at ``state[slots[row]]`` and advanced in place by the row's tokens; ``a_log``, ``dt_bias`` float32
    ``[heads]``; ``norm_weight`` float32 ``[vdim]``.  Returns ``[T, heads * vdim]`` in ``proj``'s dtype: the read-out,
    normalised per head and gated, ready for the output projection."""
    _need_cuda(proj, conv_weight, state, token_row, q_start, slots, a_log, dt_bias, norm_weight)
    channels = 2 * kv_heads * dim + heads * vdim
    col_gate = channels
    col_a = col_gate + (0 if gate_in is not None else heads * vdim)
    col_b = col_a + (0 if decay_in is not None else heads)
    columns = col_b + heads
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] >= columns, f"gated_delta_rule: proj must be [T, {columns}] (or wider)")
    tokens = proj.shape[0]
    for name, tensor, size in (("decay_in", decay_in, heads * dim), ("gate_in", gate_in, heads * vdim)):
        _need(tensor is None or (tensor.is_cuda and tensor.dtype == torch.float32 and tensor.dim() == 2 and tensor.shape[0] == tokens
                                 and tensor.shape[1] >= size and tensor.stride(1) == 1), f"gated_delta_rule: {name} must be float32 [T, {size}]")
    _need(conv_weight.dtype == torch.float32 and conv_weight.dim() == 2 and conv_weight.shape[1] == channels and conv_weight.is_contiguous(),
          "gated_delta_rule: conv_weight must be contiguous float32 [taps, channels]")
    taps = conv_weight.shape[0]
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous(), "gated_delta_rule: state must be contiguous float32 [slots, floats]")
    for name, tensor, size in (("a_log", a_log, heads), ("dt_bias", dt_bias, heads * dim if decay_in is not None else heads), ("norm_weight", norm_weight, vdim)):
        _need(tensor.dtype == torch.float32 and tensor.shape == (size,) and tensor.is_contiguous(), f"gated_delta_rule: {name} must be float32 [{size}]")
    for name, tensor, size in (("token_row", token_row, tokens), ("q_start", q_start, num_rows + 1), ("slots", slots, num_rows)):
        _need(tensor.dtype == torch.int32 and tensor.is_contiguous() and tensor.shape[0] >= size, f"gated_delta_rule: {name} must be int32 [{size}]")
    qkv = torch.empty((tokens, channels), dtype=torch.float32, device=proj.device)
    gates = torch.empty((tokens, 2 * heads), dtype=torch.float32, device=proj.device)
    read = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    out = torch.empty((tokens, heads * vdim), dtype=proj.dtype, device=proj.device)
    decays = None if decay_in is None else torch.empty((tokens, heads * dim), dtype=torch.float32, device=proj.device)
    library = _library("delta_rule.cu")
    _check(library, library.pylon_gated_delta_rule(
        _ptr(proj), proj.stride(0), _ptr(conv_weight), taps, _ptr(state), state.shape[1], _ptr(token_row), _ptr(q_start), _ptr(slots),
        _ptr(qkv), _ptr(gates), _ptr(read), _ptr(out), _ptr(a_log), _ptr(dt_bias), _ptr(norm_weight), col_a, col_b, col_gate,
        heads, kv_heads, dim, vdim, float(unit_eps), float(norm_eps), tokens, num_rows,
        _dtype_code(proj.dtype), _ptr(decay_in), 0 if decay_in is None else decay_in.stride(0), _ptr(decays), _ptr(gate_in),
        0 if gate_in is None else gate_in.stride(0), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# state-space mixer
# ---------------------------------------------------------------------------------------
def state_space(
    proj: torch.Tensor,
    conv_weight: torch.Tensor,
    conv_bias: torch.Tensor,
    state: torch.Tensor,
    token_row: torch.Tensor,
    q_start: torch.Tensor,
    slots: torch.Tensor,
    a_log: torch.Tensor,
    dt_bias: torch.Tensor,
    skip: torch.Tensor,
    norm_weight: torch.Tensor,
    heads: int,
    groups: int,
    state_dim: int,
    vdim: int,
    norm_groups: int,
    num_rows: int,
    norm_eps: float,
) -> torch.Tensor:
    """A state-space layer with one decay per head and step over the tokens of a step (``csrc/state_space.cu`` has the equations).

    ``proj [T, 2 heads vdim + 2 groups N + heads]``: the projection of the layer's input with columns ``[z | x | B | C | dt]``;
    ``conv_weight`` float32 ``[taps, channels]`` and ``conv_bias`` float32 ``[channels]`` over the x, B, C columns (the last tap weighs
    the current token); ``state`` float32 ``[slots, heads * N * vdim + (taps - 1) * channels]``: per request the heads' matrices and
    the convolution's last inputs, read at ``state[slots[row]]`` and advanced in place by the row's tokens; ``a_log``, ``dt_bias``,
    ``skip`` float32 ``[heads]``; ``norm_weight`` float32 ``[heads * vdim]``.  Returns ``[T, heads * vdim]`` in ``proj``'s dtype: the
    read-out, gated and normed in ``norm_groups`` parts, ready for the output projection."""
    _need_cuda(proj, conv_weight, conv_bias, state, token_row, q_start, slots, a_log, dt_bias, skip, norm_weight)
    inner = heads * vdim
    channels = inner + 2 * groups * state_dim
    columns = inner + channels + heads
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] == columns, f"state_space: proj must be [T, {columns}]")
    tokens = proj.shape[0]
    _need(conv_weight.dtype == torch.float32 and conv_weight.dim() == 2 and conv_weight.shape[1] == channels and conv_weight.is_contiguous(),
          "state_space: conv_weight must be contiguous float32 [taps, channels]")
    taps = conv_weight.shape[0]
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous(), "state_space: state must be contiguous float32 [slots, floats]")
    for name, tensor, size in (("a_log", a_log, heads), ("dt_bias", dt_bias, heads), ("skip", skip, heads), ("norm_weight", norm_weight, inner),
                               ("conv_bias", conv_bias, channels)):
        _need(tensor.dtype == torch.float32 and tensor.shape == (size,) and tensor.is_contiguous(), f"state_space: {name} must be float32 [{size}]")
    for name, tensor, size in (("token_row", token_row, tokens), ("q_start", q_start, num_rows + 1), ("slots", slots, num_rows)):
        _need(tensor.dtype == torch.int32 and tensor.is_contiguous() and tensor.shape[0] >= size, f"state_space: {name} must be int32 [{size}]")
    xbc = torch.empty((tokens, channels), dtype=torch.float32, device=proj.device)
    gates = torch.empty((tokens, 2 * heads), dtype=torch.float32, device=proj.device)
    read = torch.empty((tokens, inner), dtype=torch.float32, device=proj.device)
    out = torch.empty((tokens, inner), dtype=proj.dtype, device=proj.device)
    library = _library("state_space.cu")
    _check(library, library.pylon_state_space(
        _ptr(proj), proj.stride(0), _ptr(conv_weight), _ptr(conv_bias), taps, _ptr(state), state.shape[1], _ptr(token_row), _ptr(q_start),
        _ptr(slots), _ptr(xbc), _ptr(gates), _ptr(read), _ptr(out), _ptr(a_log), _ptr(dt_bias), _ptr(skip), _ptr(norm_weight), heads, groups,
        state_dim, vdim, norm_groups, float(norm_eps), tokens, num_rows, _dtype_code(proj.dtype), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# gated linear recurrence over channels; matrix memory
# ---------------------------------------------------------------------------------------
def _rows_meta(what: str, tokens: int, num_rows: int, **tensors: torch.Tensor) -> None:
    sizes = {"token_row": tokens, "q_start": num_rows + 1, "slots": num_rows}
    for name, tensor in tensors.items():
        _need(tensor.dtype == torch.int32 and tensor.is_contiguous() and tensor.shape[0] >= sizes[name], f"{what}: {name} must be int32 [{sizes[name]}]")


def linear_recurrence(proj: torch.Tensor, bias: torch.Tensor, conv_weight: torch.Tensor, conv_bias: torch.Tensor, w_gates: torch.Tensor,
                      gate_bias: torch.Tensor, lam: torch.Tensor, factor: float, state: torch.Tensor, token_row: torch.Tensor, q_start: torch.Tensor,
                      slots: torch.Tensor, num_rows: int, max_q: Optional[int] = None) -> torch.Tensor:
    """A gated linear recurrence per channel over the tokens of a step (``csrc/linear_recurrence.cu`` has the equations).

    ``proj [T, 2 C]``: the projection of the layer's input, columns ``[y | x]``, and ``bias`` float32 ``[2 C]`` to match; ``conv_weight``
    float32 ``[C, taps]`` (the last tap weighs the current token) and ``conv_bias`` float32 ``[C]``; ``w_gates [blocks, 2 C / blocks, C / blocks]``
    in ``proj``'s dtype: per block of channels the rows of the recurrence gate's map, then those of the input gate's; ``gate_bias`` float32
    ``[2, C]`` (recurrence gate, input gate); ``lam`` float32 ``[C]``; ``state`` float32 ``[slots, C + (taps - 1) * C]``: per request the
    recurrence's state and the convolution's last inputs, read at ``state[slots[row]]`` and advanced in place by the row's tokens.
    ``max_q``: the most tokens a row brings (an upper bound is fine): rows of 256 tokens and more are walked in segments side by side.  Returns
    ``[T, C]`` in ``proj``'s dtype: state times ``gelu_tanh(y)``, ready for the output projection."""
    _need_cuda(proj, bias, conv_weight, conv_bias, w_gates, gate_bias, lam, state, token_row, q_start, slots)
    tokens, channels = proj.shape[0], proj.shape[1] // 2
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] == 2 * channels, "linear_recurrence: proj must be [T, 2 C]")
    blocks = w_gates.shape[0]
    _need(channels % blocks == 0 and w_gates.shape == (blocks, 2 * channels // blocks, channels // blocks) and w_gates.is_contiguous() and w_gates.dtype == proj.dtype,
          "linear_recurrence: w_gates must be [blocks, 2 C / blocks, C / blocks] in proj's dtype")
    _need(conv_weight.dtype == torch.float32 and conv_weight.dim() == 2 and conv_weight.shape[0] == channels and conv_weight.is_contiguous(),
          "linear_recurrence: conv_weight must be contiguous float32 [C, taps]")
    taps = conv_weight.shape[1]
    for name, tensor, shape in (("bias", bias, (2 * channels,)), ("conv_bias", conv_bias, (channels,)), ("gate_bias", gate_bias, (2, channels)), ("lam", lam, (channels,))):
        _need(tensor.dtype == torch.float32 and tuple(tensor.shape) == shape and tensor.is_contiguous(), f"linear_recurrence: {name} must be float32 {shape}")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == channels * taps, "linear_recurrence: state must be contiguous float32 [slots, C * taps]")
    _rows_meta("linear_recurrence", tokens, num_rows, token_row=token_row, q_start=q_start, slots=slots)
    device, code = proj.device, _dtype_code(proj.dtype)
    u32 = torch.empty((tokens, channels), dtype=torch.float32, device=device)
    u16 = torch.empty((tokens, channels), dtype=proj.dtype, device=device) if proj.dtype != torch.float32 else None
    library = _library("linear_recurrence.cu")
    _check(library, library.pylon_linear_recurrence_conv(
        _ptr(proj), proj.stride(0), channels, _ptr(bias[channels:]), _ptr(conv_weight), _ptr(conv_bias), taps, _ptr(state), state.shape[1], _ptr(token_row),
        _ptr(q_start), _ptr(slots), _ptr(u32), _ptr(u16), channels, tokens, code, _stream()))
    operand = (u32 if u16 is None else u16).view(tokens, blocks, channels // blocks)
    gates = linear_heads(operand, w_gates, out_dtype=torch.float32)   # [T, blocks, 2 C / blocks], float32 sums whatever the operands
    out = torch.empty((tokens, channels), dtype=proj.dtype, device=device)
    scratch = torch.empty((2, tokens, channels), dtype=torch.float32, device=device)   # a - 1 and the gelu branch of every token
    longest = tokens if max_q is None else min(tokens, int(max_q))
    segments = 1 if longest < 256 else min(64, longest // 64)   # by the step's size alone: the same launches whatever the rows hold
    segment_scratch = torch.empty((3, num_rows, segments, channels), dtype=torch.float32, device=device) if segments > 1 else None
    _check(library, library.pylon_linear_recurrence_scan(
        _ptr(proj), proj.stride(0), 0, channels, _ptr(bias), _ptr(bias[channels:]), _ptr(u32), _ptr(gates), _ptr(gate_bias), _ptr(gate_bias[1]), _ptr(lam),
        float(factor), taps, _ptr(state), state.shape[1], _ptr(token_row), _ptr(q_start), _ptr(slots), _ptr(scratch[0]), _ptr(scratch[1]), _ptr(out),
        channels, blocks, num_rows, tokens, segments, _ptr(segment_scratch), code, _stream()))
    launches[0] += 1 if segments == 1 else 3   # what a token needs besides the state, then the walk (in segments: three kernels)
    return out


def matrix_memory(proj: torch.Tensor, gate_logits: torch.Tensor, gate_bias: torch.Tensor, norm_weight: torch.Tensor, state: torch.Tensor,
                  q_start: torch.Tensor, slots: torch.Tensor, heads: int, dim: int, vdim: int, cap: float, norm_eps: float, read_eps: float,
                  num_rows: int) -> torch.Tensor:
    """A matrix of memory per head with exponential gates over the tokens of a step (``csrc/matrix_memory.cu`` has the equations).

    ``proj [T, 2 heads dim + 2 heads vdim]``: the projection of the layer's input, columns ``[q | k | v | g]``; ``gate_logits`` float32
    ``[T, 2 heads]``: the input gates', then the forget gates' (replaced by the gates' logarithms); ``gate_bias`` float32 ``[2, heads]`` to match; ``norm_weight`` float32
    ``[heads * vdim]``; ``state`` float32 ``[slots, heads * (dim * vdim + dim + 1)]``: per request and head the matrix, the normaliser
    and the running maximum, read at ``state[slots[row]]`` and advanced in place by the row's tokens.  Returns ``[T, heads * vdim]`` in
    ``proj``'s dtype: the read-out, normed per head, times the weight and ``sigmoid(g)``, ready for the output projection."""
    _need_cuda(proj, gate_logits, gate_bias, norm_weight, state, q_start, slots)
    tokens = proj.shape[0]
    columns = 2 * heads * (dim + vdim)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] == columns, f"matrix_memory: proj must be [T, {columns}]")
    _need(gate_logits.dtype == torch.float32 and gate_logits.shape == (tokens, 2 * heads) and gate_logits.is_contiguous(), "matrix_memory: gate_logits must be float32 [T, 2 heads]")
    _need(gate_bias.dtype == torch.float32 and gate_bias.shape == (2, heads) and gate_bias.is_contiguous(), "matrix_memory: gate_bias must be float32 [2, heads]")
    _need(norm_weight.dtype == torch.float32 and norm_weight.shape == (heads * vdim,) and norm_weight.is_contiguous(), "matrix_memory: norm_weight must be float32 [heads * vdim]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous() and state.shape[1] == heads * (dim * vdim + dim + 1),
          "matrix_memory: state must be contiguous float32 [slots, heads * (dim * vdim + dim + 1)]")
    _need(dim <= 256, f"matrix_memory: heads of {dim} query/key elements (at most 256)")
    _rows_meta("matrix_memory", tokens, num_rows, q_start=q_start, slots=slots)
    device, code = proj.device, _dtype_code(proj.dtype)
    read = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=device)
    fresh = torch.empty((num_rows, heads, dim + 1), dtype=torch.float32, device=device)
    library = _library("matrix_memory.cu")
    _check(library, library.pylon_matrix_memory_scan(
        _ptr(proj), proj.stride(0), _ptr(gate_logits), _ptr(gate_bias), _ptr(gate_bias[1]), float(cap), float(read_eps), _ptr(state), state.shape[1],
        _ptr(q_start), _ptr(slots), _ptr(read), _ptr(fresh), heads, dim, vdim, num_rows, tokens, code, _stream()))
    launches[0] += 2   # three kernels: the gates' logarithms, the walk, the normaliser and the maximum into the slots
    out = torch.empty((tokens, heads * vdim), dtype=proj.dtype, device=device)
    _check(library, library.pylon_matrix_memory_out(_ptr(read), _ptr(proj), proj.stride(0), 2 * heads * dim + heads * vdim, _ptr(norm_weight), float(norm_eps),
                                                    _ptr(out), heads, vdim, tokens, code, _stream()))
    return out


# ---------------------------------------------------------------------------------------
# small kernels between products
# ---------------------------------------------------------------------------------------
ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "gelu": 3}   # "gelu": the exact form, with erf


def concat_cast(a: torch.Tensor, b: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``[a | b]`` row by row in ``dtype`` from two float32 blocks ``[T, width]``."""
    _need_cuda(a, b)
    _need(a.dtype == torch.float32 and b.dtype == torch.float32 and a.dim() == 2 and a.shape == b.shape and a.is_contiguous() and b.is_contiguous(),
          "concat_cast: two contiguous float32 blocks of one shape")
    tokens, width = a.shape
    out = torch.empty((tokens, 2 * width), dtype=dtype, device=a.device)
    library = _library("combine.cu")
    _check(library, library.pylon_side_by_side(_ptr(a), _ptr(b), _ptr(out), tokens, width, _dtype_code(dtype), _stream()))
    return out


def gated_unit(gate_up: torch.Tensor, bias: Optional[torch.Tensor], activation: str) -> torch.Tensor:
    """``act(gate + b_gate) * (up + b_up)`` from ``gate_up [T, 2 F]`` with columns ``[gate | up]`` and an optional float32 bias ``[2 F]``."""
    _need_cuda(gate_up, bias)
    _need(activation in ACTIVATIONS, f"gated_unit: activation {activation!r} (known: {', '.join(ACTIVATIONS)})")
    _need(gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.shape[1] % 2 == 0, "gated_unit: gate_up must be [T, 2 F]")
    tokens, inner = gate_up.shape[0], gate_up.shape[1] // 2
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (2 * inner,) and bias.is_contiguous()), "gated_unit: bias must be float32 [2 F]")
    out = torch.empty((tokens, inner), dtype=gate_up.dtype, device=gate_up.device)
    library = _library("combine.cu")
    _check(library, library.pylon_gated_unit(_ptr(gate_up), gate_up.stride(0), _ptr(bias), _ptr(out), tokens, inner, ACTIVATIONS[activation],
                                             _dtype_code(gate_up.dtype), _stream()))
    return out


def add_bias(rows: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """In place on float32 ``rows [..., width]``: every row plus float32 ``bias [width]``."""
    _need_cuda(rows, bias)
    width = bias.shape[0]
    _need(rows.dtype == torch.float32 and rows.is_contiguous() and rows.shape[-1] == width and bias.dtype == torch.float32 and bias.is_contiguous(),
          "add_bias: contiguous float32 rows and a float32 bias of their width")
    library = _library("combine.cu")
    _check(library, library.pylon_add_bias(_ptr(rows), _ptr(bias), rows.numel() // width, width, _stream()))
    return rows


def mean_of_normed(outputs: Sequence[torch.Tensor], weights: Sequence[torch.Tensor], eps: float, dtype: torch.dtype) -> torch.Tensor:
    """``(1 / n) sum_i rmsnorm(y_i) * w_i`` over the width, row by row, in float32.  Each ``y_i`` is ``[T, width]`` in ``dtype`` or
    float32 partial sums ``[parts, T, width]`` whose sum is the output (what :func:`linear_for_residual` returns); ``w_i`` float32
    ``[width]``.  Returns float32 ``[1, T, width]``: in the form of partial sums, so that the residual stream takes it in 32-bit."""
    _need(1 <= len(outputs) == len(weights) <= 4, "mean_of_normed: one to four outputs, a weight for each")
    _need_cuda(*outputs, *weights)
    tokens, width = outputs[0].shape[-2:]
    parts, floats = [], []
    for y, w in zip(outputs, weights):
        _need(y.is_contiguous() and y.shape[-2:] == (tokens, width) and ((y.dim() == 3 and y.dtype == torch.float32) or (y.dim() == 2 and y.dtype == dtype)),
              "mean_of_normed: an output is [T, width] in the compute dtype or float32 [parts, T, width]")
        _need(w.dtype == torch.float32 and w.shape == (width,) and w.is_contiguous(), "mean_of_normed: a weight is float32 [width]")
        parts.append(y.shape[0] if y.dim() == 3 else 1)
        floats.append(1 if y.dtype == torch.float32 else 0)
    count = len(outputs)
    out = torch.empty((1, tokens, width), dtype=torch.float32, device=outputs[0].device)
    library = _library("combine.cu")
    _check(library, library.pylon_mean_of_normed(
        (c_void_p * count)(*[y.data_ptr() for y in outputs]), (c_void_p * count)(*[w.data_ptr() for w in weights]), (c_int * count)(*parts),
        (c_int * count)(*floats), count, _ptr(out), tokens, width, float(eps), _dtype_code(dtype), _stream()))
    return out


def weighted_sum(outputs: Sequence[torch.Tensor], scales: Sequence[float], dtype: torch.dtype) -> torch.Tensor:
    """``sum_i scales[i] * y_i`` in float32.  Each ``y_i`` is ``[T, width]`` in ``dtype`` or float32 partial sums ``[parts, T, width]``
    whose sum is the output.  Returns float32 ``[1, T, width]``: in the form of partial sums, so that the residual stream takes it
    in 32-bit."""
    _need(1 <= len(outputs) == len(scales) <= 4, "weighted_sum: one to four outputs, a factor for each")
    _need_cuda(*outputs)
    tokens, width = outputs[0].shape[-2:]
    parts, floats = [], []
    for y in outputs:
        _need(y.is_contiguous() and y.shape[-2:] == (tokens, width) and ((y.dim() == 3 and y.dtype == torch.float32) or (y.dim() == 2 and y.dtype == dtype)),
              "weighted_sum: an output is [T, width] in the compute dtype or float32 [parts, T, width]")
        parts.append(y.shape[0] if y.dim() == 3 else 1)
        floats.append(1 if y.dim() == 3 or y.dtype == torch.float32 else 0)
    count = len(outputs)
    out = torch.empty((1, tokens, width), dtype=torch.float32, device=outputs[0].device)
    library = _library("combine.cu")
    _check(library, library.pylon_weighted_sum(
        (c_void_p * count)(*[y.data_ptr() for y in outputs]), (c_int * count)(*parts), (c_int * count)(*floats),
        (c_float * count)(*[float(scale) for scale in scales]), count, _ptr(out), tokens * width, _dtype_code(dtype), _stream()))
    return out


def activation_in_place(x: torch.Tensor, kind: str) -> torch.Tensor:
    """In place: ``x <- act(x)`` element by element on a contiguous tensor."""
    _need_cuda(x)
    _need(kind in ACTIVATIONS and x.is_contiguous(), f"activation: {kind!r} on a contiguous tensor")
    library = _library("combine.cu")
    _check(library, library.pylon_activation(_ptr(x), x.numel(), ACTIVATIONS[kind], _dtype_code(x.dtype), _stream()))
    return x


# ---------------------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------------------
EXPERT_TILE_ROWS = 128   # the row tile of the grouped tcgen05 product


def expert_mixture(h: torch.Tensor, router: torch.Tensor, router_bias: Optional[torch.Tensor], w_gate_up: torch.Tensor, w_down: torch.Tensor,
                   top: int, activation: str = "silu", interleaved: bool = False, gated: bool = True, routing: str = "softmax",
                   correction: Optional[torch.Tensor] = None, groups: int = 0, groups_keep: int = 0, share_eps: float = 0.0,
                   common_up: Optional[torch.Tensor] = None, common_down: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sum over a token's top experts e of share_e * W_down,e (act(W_gate,e h) * (W_up,e h))`` (``csrc/experts.cu``).

    ``h [T, width]``; ``router`` float32 ``[experts, width]`` and ``router_bias`` float32 ``[experts]`` (or None): the logits are
    float32 whatever ``h`` is; ``w_gate_up [experts, 2 F, width]`` (an expert's gate rows, then its up rows; with ``interleaved``
    every expert's rows stacked by :func:`interleave_gate_up`) and ``w_down [experts, width, F]`` in ``h``'s dtype.  Returns float32
    ``[1, T, width]`` (the form of partial sums: the residual stream takes it in 32-bit).

    ``gated=False``: an expert is ``W_down act(W_up h)`` and ``w_gate_up`` holds the up rows only, ``[experts, F, width]``.
    ``routing="sigmoid"``: the scores are ``sigmoid(z)``; the choice goes by score plus ``correction`` (float32 ``[experts]`` or None), with
    ``groups`` > 0 only among the experts of the ``groups_keep`` groups of neighbours whose two largest choice scores add up to most; the
    shares are the chosen experts' scores divided by their sum plus ``share_eps``.  ``common_up [G, width]`` / ``common_down [width, G]``:
    an ungated expert that every token goes through, added times ``sigmoid(w h)`` with ``w`` the row that ``router`` then holds behind
    the experts' rows (``[experts + 1, width]``).

    The tokens are sorted by expert on the device.  A step of few tokens runs the experts' products from row tiles of 32 slots that
    gather their rows themselves (``mma.sync``, bound by the matrices coming from memory); a bfloat16 step with about half a
    128-row tile or more per expert (gated: interleaved weights and ``silu``) copies the rows into their sorted order and runs both
    products on the grouped form of the tcgen05 kernel (the gated unit in the first one's epilogue; an ungated expert's activation
    is a pass of its own between the two)."""
    _need_cuda(h, router, router_bias, w_gate_up, w_down, correction, common_up, common_down)
    _need(activation in ACTIVATIONS, f"expert_mixture: activation {activation!r}")
    _need(routing in ("softmax", "sigmoid"), f"expert_mixture: routing {routing!r}")
    _need(h.dim() == 2 and h.stride(1) == 1, "expert_mixture: h must be [T, width]")
    tokens, width = h.shape
    halves = 2 if gated else 1
    experts, inner = w_gate_up.shape[0], w_gate_up.shape[1] // halves
    _need(w_gate_up.shape == (experts, halves * inner, width) and w_down.shape == (experts, width, inner) and w_gate_up.is_contiguous() and w_down.is_contiguous()
          and w_gate_up.dtype == h.dtype and w_down.dtype == h.dtype, "expert_mixture: w_gate_up [experts, 2 F, width] (ungated: [experts, F, width]) and w_down [experts, width, F] in h's dtype")
    scored = routing == "sigmoid"
    extra = 1 if common_up is not None else 0
    _need(scored or (correction is None and not groups and not extra), "expert_mixture: a correction, groups and a common expert go with sigmoid routing")
    _need(router.dtype == torch.float32 and router.shape == (experts + extra, width) and router.is_contiguous(), "expert_mixture: router must be float32 [experts (+ 1), width]")
    _need(router_bias is None or (router_bias.dtype == torch.float32 and router_bias.shape == (experts,)), "expert_mixture: router_bias must be float32 [experts]")
    _need(correction is None or (correction.dtype == torch.float32 and correction.shape == (experts,) and correction.is_contiguous()), "expert_mixture: correction must be float32 [experts]")
    _need(1 <= top <= experts, f"expert_mixture: top {top} of {experts} experts")
    _need(not interleaved or (gated and inner % 8 == 0), "expert_mixture: interleaved rows need a gated unit of an inner width that is a multiple of 8")
    _need((common_up is None) == (common_down is None), "expert_mixture: a common expert has both its matrices")
    library = _library("experts.cu")
    pairs = tokens * top
    grouped = ((not gated or (interleaved and activation == "silu")) and h.dtype == torch.bfloat16 and pairs * 2 >= EXPERT_TILE_ROWS * experts and width % 8 == 0
               and inner % 8 == 0 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0)
    tile = EXPERT_TILE_ROWS if grouped else library.pylon_experts_row_tile()
    max_tiles = min(pairs, experts) + pairs // tile    # every expert with tokens ends in at most one partly filled tile
    max_slots = max_tiles * tile
    device = h.device
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=device)
    share = torch.empty((tokens, top), dtype=torch.float32, device=device)
    slot_of = torch.empty((pairs,), dtype=torch.int32, device=device)
    source = torch.empty((max_slots,), dtype=torch.int32, device=device)
    tile_expert = torch.empty((max_tiles,), dtype=torch.int32, device=device)
    common_gate = torch.empty((tokens,), dtype=torch.float32, device=device) if extra else None
    code, kind = _dtype_code(h.dtype), ACTIVATIONS[activation]
    _check(library, library.pylon_experts_route(_ptr(h), h.stride(0), _ptr(router), _ptr(router_bias), _ptr(chosen), _ptr(share), width, experts, top,
                                                tokens, code, int(scored), _ptr(correction), int(groups or 0), int(groups_keep or 0), float(share_eps), extra,
                                                _ptr(common_gate), _stream()))
    _check(library, library.pylon_experts_plan(_ptr(chosen), _ptr(slot_of), _ptr(source), _ptr(tile_expert), pairs, experts, max_slots, max_tiles, tile, _stream()))
    common, common_code = None, F32
    if extra:   # the expert of every token: two plain products around the activation
        common = linear(activation_in_place(linear(h, common_up), activation), common_down)
        common_code = _dtype_code(common.dtype)
    out = torch.empty((1, tokens, width), dtype=torch.float32, device=device)
    if grouped:
        product = _library("gemm_tcgen05.cu")
        error, sms = _ptr(tcgen05_error_word(device)), _multiprocessors(device)
        rows = torch.empty((max_slots, width), dtype=h.dtype, device=device)
        _check(library, library.pylon_experts_sort_rows(_ptr(h), h.stride(0), _ptr(source), _ptr(rows), width, top, max_slots, code, _stream()))
        act = torch.empty((max_slots, inner), dtype=h.dtype, device=device)
        _check(product, product.pylon_gemm_tcgen05_grouped(_ptr(rows), _ptr(w_gate_up), _ptr(act), max_slots, halves * inner, width, width, width, inner,
                                                           1 if gated else 0, _ptr(tile_expert), experts, error, sms, _stream()))
        if not gated:
            activation_in_place(act, activation)   # (rows of empty slots hold act(0) of zeros: they are never gathered)
        y = torch.empty((max_slots, width), dtype=h.dtype, device=device)
        _check(product, product.pylon_gemm_tcgen05_grouped(_ptr(act), _ptr(w_down), _ptr(y), max_slots, width, inner, inner, inner, width, 0,
                                                           _ptr(tile_expert), experts, error, sms, _stream()))
        _check(library, library.pylon_experts_gather(_ptr(y), _ptr(slot_of), _ptr(share), _ptr(out), tokens, width, top, code, _ptr(common), _ptr(common_gate),
                                                     common_code, _stream()))
        return out
    act = torch.empty((max_slots, inner), dtype=h.dtype, device=device)
    _check(library, library.pylon_experts_product(_ptr(h), h.stride(0), _ptr(w_gate_up), _ptr(source), _ptr(tile_expert), 1, top, _ptr(act), inner, width,
                                                  max_tiles, 1 if gated else 2, kind, int(interleaved), code, _stream()))
    y = torch.empty((max_slots, width), dtype=torch.float32, device=device)
    _check(library, library.pylon_experts_product(_ptr(act), inner, _ptr(w_down), _ptr(source), _ptr(tile_expert), 0, 1, _ptr(y), width, inner,
                                                  max_tiles, 0, kind, 0, code, _stream()))
    _check(library, library.pylon_experts_gather(_ptr(y), _ptr(slot_of), _ptr(share), _ptr(out), tokens, width, top, _dtype_code(torch.float32), _ptr(common),
                                                 _ptr(common_gate), common_code, _stream()))
    return out


# ---------------------------------------------------------------------------------------
# products per head
# ---------------------------------------------------------------------------------------
def linear_heads(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """One product per head: ``y[t, h] = w[h] @ x[t, h]`` for ``x [T, H, K]``, ``w [H, N, K]`` -> ``[T, H, N]``.
    ``out_dtype=torch.float32`` keeps the 32-bit sums of a bfloat16 product (logits of gates, say).

    ``x`` and ``out`` may be views whose heads are slices of wider rows (any token and head strides; the last dimension
    contiguous).  float32 runs the plain-FMA kernel, one grid layer per head; bfloat16 goes to the library's batched
    product with float32 accumulation, as the large plain products do."""
    _need_cuda(x, w, out)
    _need(x.dim() == 3 and w.dim() == 3 and x.shape[1] == w.shape[0] and x.shape[2] == w.shape[2], f"linear_heads: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype and x.stride(2) == 1 and w.is_contiguous(), "linear_heads: one dtype, the reduced dimension contiguous, the weights contiguous")
    tokens, heads, k = x.shape
    n = w.shape[1]
    if out_dtype is not None and out_dtype != x.dtype:
        _need(out is None and x.dtype == torch.bfloat16 and out_dtype == torch.float32, "linear_heads: only a bfloat16 product can keep its float32 sums")
        if tokens == 0:
            return torch.empty((tokens, heads, n), dtype=torch.float32, device=x.device)
        return torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32).transpose(0, 1).contiguous()
    if out is None:
        out = torch.empty((tokens, heads, n), dtype=x.dtype, device=x.device)
    _need(out.shape == (tokens, heads, n) and out.dtype == x.dtype and out.stride(2) == 1, "linear_heads: out must be [T, H, N] with its last dimension contiguous")
    if tokens == 0:
        return out
    if x.dtype == torch.float32:
        library = _library("gemm_f32.cu")
        _check(library, library.pylon_gemm_f32_nt_batched(_ptr(x), _ptr(w), _ptr(out), tokens, n, k, x.stride(0), k, out.stride(0), heads,
                                                          x.stride(1), n * k, out.stride(1), _stream()))
        return out
    _need(x.dtype == torch.bfloat16, f"linear_heads: unsupported dtype {x.dtype}")
    torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    return out


# ---------------------------------------------------------------------------------------
# rotations, norms and cache writes between an attention mixer's projections and its attention
# ---------------------------------------------------------------------------------------
ROTARY_LAYOUTS = {"halves": 0, "neighbours": 1}


def _rotary_tables(cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, what: str) -> int:
    if cos is None:
        return 0
    _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape and cos.dim() == 2
          and cos.shape[1] * 2 == rotary_dim and cos.is_contiguous() and sin.is_contiguous(), f"{what}: cos/sin must be float32 [positions, rotary_dim / 2]")
    return cos.shape[0]


def qkv_rotate_write(
    qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, layout: str,
    norm: Optional[str], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
    token_row: torch.Tensor, block_table: torch.Tensor, page_size: int, k_pages: torch.Tensor, v_pages: torch.Tensor, nq: int, nkv: int,
    head_dim: int, value_dim: int,
) -> torch.Tensor:
    """On ``qkv [T, nq * d + nkv * d + nkv * dv]``: add ``bias`` (float32, one number per column), rotate the first
    ``rotary_dim`` elements of every q and k head by the tables (``layout``: ``"halves"`` pairs element i with i + rotary_dim / 2,
    ``"neighbours"`` element 2 i with 2 i + 1), divide every q and k head by its root mean square (``norm``: ``"before"`` or
    ``"after"`` the rotation, ``None``: not at all; times ``q_weight`` / ``k_weight [d]`` where given), write q back in place and
    k, v into the token's slot of its pages ``[pages, nkv, page_size, d]`` and ``[pages, nkv, page_size, dv]``.  Returns ``qkv``."""
    _need_cuda(qkv, bias, cos, sin, q_weight, k_weight, positions, token_row, block_table, k_pages, v_pages)
    tokens, columns = qkv.shape[0], nq * head_dim + nkv * head_dim + nkv * value_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == columns, "qkv_rotate_write: qkv must be [T, nq * d + nkv * d + nkv * dv]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (columns,) and bias.is_contiguous()), "qkv_rotate_write: bias must be float32, one per column")
    _need(layout in ROTARY_LAYOUTS and norm in (None, "before", "after"), f"qkv_rotate_write: layout {layout!r}, norm {norm!r}")
    table_positions = _rotary_tables(cos, sin, rotary_dim, "qkv_rotate_write")
    for weight in (q_weight, k_weight):
        _need(weight is None or (weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous()), "qkv_rotate_write: norm weights must be float32 [d]")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "qkv_rotate_write: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "qkv_rotate_write: block_table must be contiguous int32 [rows, width]")
    for pages, width in ((k_pages, head_dim), (v_pages, value_dim)):
        _need(pages.dtype == qkv.dtype and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, width),
              "qkv_rotate_write: pages must be contiguous [pages, nkv, page_size, width] in the activation dtype")
    library = _library("rotary.cu")
    _check(library, library.pylon_qkv_rotate_write(
        _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0, ROTARY_LAYOUTS[layout], table_positions,
        {None: 0, "before": 1, "after": 2}[norm], _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(positions), _ptr(token_row), _ptr(block_table),
        block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], nq, nkv, head_dim, value_dim, tokens, _dtype_code(qkv.dtype),
        _ptr(cache_write_error_word(k_pages.device)), _stream()))
    return qkv


def latent_norm_rotate_write(
    down: torch.Tensor, q_weight: Optional[torch.Tensor], kv_weight: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
    rotary_dim: int, layout: str, positions: torch.Tensor, token_row: torch.Tensor, block_table: torch.Tensor, page_size: int, pages: torch.Tensor,
    q_rank: int, kv_rank: int, rot_dim: int,
) -> torch.Tensor:
    """``down [T, q_rank + kv_rank + rot_dim]``: the query latent, the key/value latent and the rotated key part that all heads
    share.  Returns the query latent after its RMS norm (times ``q_weight``), ``[T, q_rank]``; the token's one cache row
    ``[kv_rank + rot_dim]`` in ``pages [pages, 1, page_size, kv_rank + rot_dim]`` receives the key/value latent after its RMS norm
    (times ``kv_weight``) and the key part with its first ``rotary_dim`` elements rotated (not normed)."""
    _need_cuda(down, q_weight, kv_weight, cos, sin, positions, token_row, block_table, pages)
    tokens = down.shape[0]
    _need(down.dim() == 2 and down.stride(1) == 1 and down.shape[1] == q_rank + kv_rank + rot_dim, "latent_norm_rotate_write: down must be [T, q_rank + kv_rank + rot_dim]")
    _need(layout in ROTARY_LAYOUTS, f"latent_norm_rotate_write: layout {layout!r}")
    table_positions = _rotary_tables(cos, sin, rotary_dim, "latent_norm_rotate_write")
    _need(q_rank == 0 or (q_weight is not None and q_weight.dtype == torch.float32 and q_weight.shape == (q_rank,) and q_weight.is_contiguous()), "latent_norm_rotate_write: q_weight must be float32 [q_rank]")
    _need(kv_weight.dtype == torch.float32 and kv_weight.shape == (kv_rank,) and kv_weight.is_contiguous(), "latent_norm_rotate_write: kv_weight must be float32 [kv_rank]")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "latent_norm_rotate_write: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "latent_norm_rotate_write: block_table must be contiguous int32 [rows, width]")
    _need(pages.dtype == down.dtype and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (1, page_size, kv_rank + rot_dim),
          "latent_norm_rotate_write: pages must be contiguous [pages, 1, page_size, kv_rank + rot_dim] in the activation dtype")
    cq = torch.empty((tokens, q_rank), dtype=down.dtype, device=down.device)
    library = _library("rotary.cu")
    _check(library, library.pylon_latent_norm_rotate_write(
        _ptr(down), down.stride(0), _ptr(cq), _ptr(q_weight), _ptr(kv_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        ROTARY_LAYOUTS[layout], table_positions, _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(pages),
        pages.shape[0], q_rank, kv_rank, rot_dim, tokens, _dtype_code(down.dtype), _ptr(cache_write_error_word(pages.device)), _stream()))
    return cq


def rotate_heads(src: torch.Tensor, dst: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, layout: str,
                 positions: torch.Tensor) -> torch.Tensor:
    """``dst[t, h] = src[t, h]`` with the first ``rotary_dim`` elements of every head rotated by the token's position.  ``src`` and ``dst``
    are ``[T, H, width]`` views (any token and head strides, the last dimension contiguous): a slice of each head of a wider row, say."""
    _need_cuda(src, dst, cos, sin, positions)
    _need(src.dim() == 3 and src.shape == dst.shape and src.dtype == dst.dtype and src.stride(2) == 1 and dst.stride(2) == 1, "rotate_heads: src and dst must be [T, H, width] views of one dtype")
    _need(layout in ROTARY_LAYOUTS, f"rotate_heads: layout {layout!r}")
    table_positions = _rotary_tables(cos, sin, rotary_dim, "rotate_heads")
    tokens, heads, width = src.shape
    _need(positions.dtype == torch.int32 and positions.is_contiguous() and positions.shape[0] >= tokens, "rotate_heads: positions must be int32 [T]")
    library = _library("rotary.cu")
    _check(library, library.pylon_rotate_heads(
        _ptr(src), src.stride(0), src.stride(1), _ptr(dst), dst.stride(0), dst.stride(1), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        ROTARY_LAYOUTS[layout], table_positions, _ptr(positions), heads, width, tokens, _dtype_code(src.dtype), _stream()))
    return dst


# ---------------------------------------------------------------------------------------
# linear attention with a fixed decay per head
# ---------------------------------------------------------------------------------------
def lightning_attention(
    proj: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, decay: torch.Tensor, norm_weight: torch.Tensor,
    heads: int, dim: int, vdim: int, rows: int, eps: float, max_q: Optional[int] = None,
) -> torch.Tensor:
    """``proj [T, 2 * heads * dim + 2 * heads * vdim]`` holds the projections ``[q | k | v | gate]`` of a step's tokens.  Per head and
    request, in token order, in float32: ``S = decay * S + silu(k) silu(v)^T``, ``o = S^T silu(q)``, with S ``[dim, vdim]`` in
    ``state[slots[row]]`` (``state [slots, heads * vdim * dim]`` float32, a head's matrix stored column by column: entry (d, j) at ``j * dim + d``; a row's tokens are ``q_start[row] .. q_start[row + 1]``).
    Returns ``o / rms(o) * norm_weight * sigmoid(gate)`` over a token's concatenated heads, ``[T, heads * vdim]`` in the activation dtype.
    ``max_q``: the most tokens a row brings (an upper bound is fine; default: all of them).  In bfloat16 a row of 1,024 tokens or more is
    walked in segments of 256 side by side, whose states a scan chains and whose tokens a second walk corrects."""
    _need_cuda(proj, state, q_start, slots, decay, norm_weight)
    tokens, qk, width = proj.shape[0], heads * dim, heads * vdim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] == 2 * qk + 2 * width, "lightning_attention: proj must be [T, 2 * heads * dim + 2 * heads * vdim]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == qk * vdim and state.is_contiguous(), "lightning_attention: state must be contiguous float32 [slots, heads * dim * vdim]")
    _need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.shape[0] >= rows + 1, "lightning_attention: q_start must be int32 [rows + 1]")
    _need(slots.dtype == torch.int32 and slots.is_contiguous() and slots.shape[0] >= rows, "lightning_attention: slots must be int32 [rows]")
    _need(decay.dtype == torch.float32 and decay.shape == (heads,) and decay.is_contiguous(), "lightning_attention: decay must be float32 [heads]")
    _need(norm_weight.dtype == torch.float32 and norm_weight.shape == (width,) and norm_weight.is_contiguous(), "lightning_attention: norm_weight must be float32 [heads * vdim]")
    read_out = torch.empty((tokens, width), dtype=torch.float32, device=proj.device)
    out = torch.empty((tokens, width), dtype=proj.dtype, device=proj.device)
    library = _library("lightning.cu")
    max_q = tokens if max_q is None else int(max_q)
    work = torch.empty((library.pylon_lightning_work_floats(tokens, rows, max_q, heads, dim, vdim, _dtype_code(proj.dtype)),), dtype=torch.float32, device=proj.device)
    _check(library, library.pylon_lightning_attention(
        _ptr(proj), proj.stride(0), 0, qk, 2 * qk, 2 * qk + width, _ptr(state), state.stride(0), state.shape[0], _ptr(q_start), _ptr(slots), rows,
        _ptr(decay), _ptr(norm_weight), float(eps), _ptr(read_out), _ptr(work), _ptr(out), tokens, max_q, heads, dim, vdim, _dtype_code(proj.dtype), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
def sample(
    logits: torch.Tensor,
    temperature: Optional[torch.Tensor] = None,
    top_p: Optional[torch.Tensor] = None,
    uniform: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    host_copy: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One token per row of float32 ``logits [R, vocab]``: arg-max where a row's temperature
    is 0 (or none is given), else a draw from ``softmax(logits / T)`` cut to the ``top_p``
    nucleus, using the row's number from ``uniform`` (float32 in [0, 1)).  The per-row parameters may lie in pinned
    host memory, which the kernel then reads where it is.  ``host_copy``: int32 ``[R + 4]`` in pinned host memory, into
    which the kernel also writes the tokens and, behind them, the kernels' four error words as they stand: whoever
    waits for the launch can read both there, and no copy has to follow it."""
    _need_cuda(logits, out)
    _need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be float32 [R, vocab]")
    rows, vocab = logits.shape
    for per_row in (temperature, top_p, uniform):
        if per_row is not None:
            _need(per_row.dtype == torch.float32 and per_row.is_contiguous() and per_row.shape[0] >= rows
                  and (per_row.is_cuda or per_row.is_pinned()), "sample: per-row parameters must be float32 [R] on the device or in pinned memory")
    words = None
    if host_copy is not None:
        _need(host_copy.dtype == torch.int32 and host_copy.is_contiguous() and host_copy.shape == (rows + 4,) and host_copy.is_pinned(),
              "sample: host_copy must be int32 [R + 4] in pinned memory")
        words = _error_words(logits.device)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _need(out.dtype == torch.int32 and out.is_contiguous() and out.shape[0] >= rows, "sample: out must be int32 [R]")
    library = _library("sampling.cu")
    _check(library, library.pylon_sample(
        _ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_p), _ptr(uniform), _ptr(out),
        None if host_copy is None else host_copy.data_ptr(), _ptr(words), None if host_copy is None else host_copy.data_ptr() + 4 * rows, _stream()))
    return out
