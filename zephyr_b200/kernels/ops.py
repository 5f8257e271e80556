"""Python faces of the hand-written kernels.

Each function checks what the kernel cannot check for itself (device, types, contiguity, sizes),
launches on the current CUDA stream and returns without synchronising.  There is no fallback of
any kind: if the library cannot be built or loaded, or a kernel refuses a shape, the call raises.
"""

from __future__ import annotations

import contextlib
import ctypes
import gc
import math
import os
import struct
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Sequence

import torch

from ..config.errors import InvalidArgumentError, ZephyrError
from .build import BuildError, build_library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
DECODE_SPLIT_SIZE = 256     # the shortest context a captured decode graph is sized for

_RC_TEXT = {1: "an argument outside the kernel's contract", 2: "the CUDA launch failed",
            3: "a configuration this kernel does not support"}
STATUS_TEXT = {
    1: "a token id outside the vocabulary",
    2: "a position outside the position table",
    3: "a page id outside the cache pool (or the null page) where a real page was expected",
    4: "a request row or block index outside the step's tables",
    5: "NaN or +inf among the logits",
    6: "an asynchronous copy into shared memory that did not complete within the wait limit",
    7: "an address or size that failed a kernel's own check (a bug in this package)",
    8: "a barrier across the grid that did not complete within the wait limit",
}


class KernelError(ZephyrError):
    pass


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

_SIGNATURES = {
    "zb_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_longlong, c_longlong, c_int,
                   c_void_p],
    "zb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "zb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_act_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "zb_head_linear": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_int, c_int, c_int,
                       c_int, c_int, c_int, c_int, c_void_p],
    "zb_head_linear_strided": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "zb_route_grouped": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_float, c_void_p],
    "zb_pair_embedding": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p,
                          c_void_p],
    "zb_store_last_token": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "zb_sum_rms_norm": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p,
                        c_void_p, c_int, c_float, c_int, c_int, c_void_p],
    "zb_clamped_gate": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float,
                        c_void_p],
    "zb_scale_rows": [c_void_p, c_longlong, c_float, c_void_p],
    "zb_latent_rope": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_void_p, c_float, c_void_p,
                       c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                       c_int, c_int, c_void_p, c_void_p],
    "zb_route_max_outputs": [],
    "zb_expert_tile_rows": [c_int],
    "zb_route": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    "zb_route_align": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_expert_product": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_void_p],
    "zb_route_align_padded": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_gather_places": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    "zb_gemm_tc_grouped": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_int, c_int,
                           c_void_p, c_void_p],
    "zb_route_combine": [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                         c_int, c_int, c_int, c_void_p],
    "zb_add_bias": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "zb_qk_norm_rope_cache": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p,
                              c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_rope": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                c_void_p],
    "zb_kv_write": [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_attention_simt_tile_tokens": [c_int],
    "zb_paged_attention_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_qkv_halves": [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float,
                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_pool_blocks": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_head_mix": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "zb_sigmoid_gate": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "zb_delta_max_channels": [],
    "zb_delta_gates": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                       c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                       c_void_p],
    "zb_delta_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong,
                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p, c_void_p],
    "zb_residual_rms_norm": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_float, c_float, c_int,
                             c_int, c_int, c_void_p],
    "zb_route_biased": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_float, c_void_p, c_void_p],
    "zb_qkv_pairs": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p,
                     c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_layer_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p],
    "zb_residual_layer_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int,
                               c_float, c_float, c_int, c_int, c_int, c_void_p],
    "zb_embedding_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_causal_conv_silu": [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                            c_void_p],
    "zb_state_scan_max_channels": [],
    "zb_decayed_state_scan": [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                              c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                              c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "zb_gated_group_rms_norm": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_float, c_int, c_int, c_void_p],
    "zb_scaled_sum": [c_void_p, c_void_p, c_void_p, c_float, c_float, c_longlong, c_int, c_int, c_void_p],
    "zb_paged_decode_supported": [c_int, c_int, c_int, c_int],
    "zb_paged_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                        c_void_p, c_void_p],
    "zb_paged_decode_masked": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p,
                               c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "zb_paged_prefill_masked": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_float, c_int, c_void_p, c_void_p, c_void_p],
    "zb_paged_prefill_windowed": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_void_p],
    "zb_paged_decode_fused": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_longlong, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p],
    "zb_paged_decode_set_trace": [c_void_p],
    "zb_paged_prefill_tile_tokens": [],
    "zb_paged_prefill_supported": [c_int, c_int, c_int, c_int],
    "zb_paged_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "zb_paged_prefill_tc_supported": [c_int, c_int, c_int, c_int, c_int],
    "zb_paged_prefill_tc_set_trace": [c_void_p],
    "zb_paged_prefill_tc_masked": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                   c_void_p, c_void_p, c_void_p],
    "zb_paged_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "zb_gemm_small_supported": [c_int, c_int, c_int],
    "zb_gemm_small": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                      c_int, c_void_p],
    "zb_fill_normal": [c_void_p, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_int, c_void_p],
    "zb_gemm_tc_supported": [c_int, c_int, c_int, c_longlong, c_int, c_int],
    "zb_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p],
    "zb_gemm_tc_bounded": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_int, c_int, c_int, c_longlong,
                           c_int, c_int, c_void_p, c_void_p],
    "zb_gemm_small_bounded": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_int, c_int, c_int,
                              c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    "zb_gemm_nt_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                        c_int, c_int, c_void_p],
    "zb_fused_chain_stage_supported": [c_int, c_int, c_int, c_int, c_int],
    "zb_fused_chain_max_stages": [],
    "zb_fused_chain_grid": [],
    "zb_set_sm_share": [c_int],
    "zb_fused_chain_set_flip_bytes": [c_longlong],
    "zb_set_dependent_launch": [c_int],
    "zb_fused_chain": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "zb_sample_chunks": [c_int],
    "zb_sample": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
}


def library() -> ctypes.CDLL:
    """The compiled kernels, built at the first call.  Raises if they cannot be had."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            try:
                path = build_library()
            except BuildError as error:
                raise KernelError(f"the CUDA kernels of zephyr_b200 are unavailable: {error}") from error
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as error:
                raise KernelError(f"cannot load {path}: {error}") from error
            for name, argtypes in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            lib.zb_last_cuda_error.argtypes = []
            lib.zb_last_cuda_error.restype = ctypes.c_char_p
            lib.zb_paged_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
            lib.zb_paged_decode_scratch_floats.restype = c_longlong
            lib.zb_paged_decode_balanced_scratch_floats.argtypes = [c_int, c_int, c_int]
            lib.zb_paged_decode_balanced_scratch_floats.restype = c_longlong
            if os.environ.get("ZEPHYR_B200_DEPENDENT_LAUNCH", "1") == "0":
                lib.zb_set_dependent_launch(0)
            _lib = lib
    return _lib


def library_path() -> str:
    return library()._name


LAUNCHES = 0      # kernels of this package launched so far (the bench reports the count of a timed region)
LAUNCH_COUNTS: dict[str, int] = {}      # the same by entry point


def _check(rc: int, name: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    LAUNCH_COUNTS[name] = LAUNCH_COUNTS.get(name, 0) + kernels
    if rc != 0:
        detail = ""
        if rc == 2:
            said = library().zb_last_cuda_error()
            detail = (f": {said.decode() if said else 'unknown'} ({torch.cuda.get_device_name()}; "
                      "the library holds sm_100a code only)")
        raise KernelError(f"{name}: {_RC_TEXT.get(rc, f'error {rc}')}{detail}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise InvalidArgumentError(message)


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("zephyr_b200 kernels run on CUDA tensors only; there is no CPU path")


def _i32(*tensors: torch.Tensor) -> None:
    for t in tensors:
        _require(t.dtype == torch.int32 and t.is_contiguous(), "index tensors must be contiguous int32")


@contextlib.contextmanager
def capture(graph: "torch.cuda.CUDAGraph", **kwargs):
    """``torch.cuda.graph`` with the garbage collector held still.  A collection that happens to run
    inside a capture may destroy an older CUDA graph (one of a runner that was dropped, kept alive
    until then by a reference cycle); the runtime forbids that while any stream captures and the
    capture is lost ("operation failed due to a previous error during capture").  Such objects wait
    for the first collection after the capture."""
    enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **kwargs):
            yield
    finally:
        if enabled:
            gc.enable()


def new_status(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device status word kernels report into: [code, detail, index, unused]."""
    return torch.zeros(4, dtype=torch.int32, device=device)


_device_status: dict = {}


def device_status(device: torch.device | str) -> torch.Tensor:
    """The one status word of a device: kernels that are called without a status word report into it,
    and a model runner takes it as its own, so that what a product deep inside a part reports
    (a wait that ran out) is seen by the check after the step."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device(device.type, torch.cuda.current_device())
    word = _device_status.get(device)
    if word is None:
        word = _device_status[device] = new_status(device)
    return word


def check_status(status: torch.Tensor, where: str = "step") -> None:
    """Read the status word (this synchronises) and raise if a kernel reported an error."""
    code, detail, index, _ = status.tolist()
    if code != 0:
        status.zero_()
        for pool in _decode_buffers.values():       # a kernel that gave up may have left counters behind
            for _, count in pool:
                count.zero_()
        for buffer in list(_chain_sync.values()) + [b for (_, name), b in _sample_buffers.items() if name == "counters"]:
            buffer.zero_()
        raise KernelError(f"{where}: a kernel reported {STATUS_TEXT.get(code, f'error {code}')} "
                          f"(value {detail}, at element {index})")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> torch.Tensor:
    """Fills a contiguous bfloat16 or float32 tensor with mean + std * z, z standard normal: element i
    is a function of (key, i) alone (a counter-based generator; see random_fill.cu)."""
    _cuda(out)
    _require(out.is_contiguous() and out.dtype in DTYPE_CODE, "a contiguous bfloat16 or float32 tensor")
    _check(library().zb_fill_normal(_ptr(out), out.numel(), int(key) & (2**64 - 1), float(mean), float(std),
                                    DTYPE_CODE[out.dtype], _stream()), "fill_normal")
    return out


# --------------------------------------------------------------------------- elementwise
def embedding(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, out: torch.Tensor | None = None):
    _cuda(table, ids, status)
    _i32(ids)
    _require(table.dim() == 2 and table.is_contiguous() and table.dtype in DTYPE_CODE, "table must be [V, H]")
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _require(out.shape == (T, H) and out.dtype == table.dtype and out.is_contiguous(), "out must be [T, H]")
    _check(library().zb_embedding(_ptr(out), _ptr(table), _ptr(ids), T, H, V, DTYPE_CODE[table.dtype],
                                  _ptr(status), _stream()), "embedding")
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    _cuda(x, rows, status)
    _i32(rows)
    _require(x.dim() == 2 and x.is_contiguous() and x.dtype in DTYPE_CODE, "x must be a contiguous [T, H]")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(library().zb_gather_rows(_ptr(out), _ptr(x), _ptr(rows), rows.numel(), x.shape[1], x.shape[0],
                                    DTYPE_CODE[x.dtype], _ptr(status), _stream()), "gather_rows")
    return out


def _scale_code(w: torch.Tensor, size: int) -> int:
    _require(w.dim() == 1 and w.numel() == size and w.is_contiguous() and w.dtype in DTYPE_CODE,
             f"a norm scale must be a contiguous vector of {size} float32 or bfloat16 values")
    return DTYPE_CODE[w.dtype]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm over the last dimension of a contiguous tensor (any leading shape)."""
    _cuda(x, w)
    _require(x.is_contiguous() and x.dtype in DTYPE_CODE, "x must be contiguous float32 or bfloat16")
    H = x.shape[-1]
    rows = x.numel() // H if H else 0
    if out is None:
        out = torch.empty_like(x)
    _require(out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous(), "out must match x")
    _check(library().zb_rmsnorm(_ptr(out), _ptr(x), _ptr(w), _scale_code(w, H), float(eps), rows, H, H, H,
                                DTYPE_CODE[x.dtype], _stream()), "rmsnorm")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (in place), then return rmsnorm(residual) * w."""
    _cuda(residual, delta, w)
    _require(residual.dim() == 2 and residual.is_contiguous() and residual.dtype in DTYPE_CODE
             and delta.shape == residual.shape and delta.dtype == residual.dtype and delta.is_contiguous(),
             "residual and delta must be matching contiguous [T, H] tensors")
    rows, H = residual.shape
    if out is None:
        out = torch.empty_like(residual)
    _require(out.shape == residual.shape and out.dtype == residual.dtype and out.is_contiguous(), "out must match")
    _check(library().zb_add_rmsnorm(_ptr(out), _ptr(residual), _ptr(delta), _ptr(w), _scale_code(w, H), float(eps),
                                    rows, H, DTYPE_CODE[residual.dtype], _stream()), "add_rmsnorm")
    return out


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y [T, N] += bias [N] in place (rows of y may be strided; the bias bfloat16 or float32)."""
    _cuda(y, bias)
    _require(y.dim() == 2 and y.stride(1) == 1 and y.dtype in DTYPE_CODE, "y must be [T, N] with unit inner stride")
    _require(bias.dim() == 1 and bias.numel() == y.shape[1] and bias.is_contiguous() and bias.dtype in DTYPE_CODE,
             "one bias value per column")
    _check(library().zb_add_bias(_ptr(y), y.stride(0), _ptr(bias), DTYPE_CODE[bias.dtype], y.shape[0], y.shape[1],
                                 DTYPE_CODE[y.dtype], _stream()), "add_bias")
    return y


ACTIVATIONS = {"silu": 0, "relu": 1}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, blocked: bool = False,
             act: str = "silu") -> torch.Tensor:
    """act(gate_up[:, :I]) * gate_up[:, I:] for a contiguous [T, 2I] tensor, ``act`` being "silu" or "relu".
    With ``blocked`` the gate and up columns alternate in blocks of 8 (the layout
    ``gemm_small(..., swiglu=True)`` reads)."""
    _require(act in ACTIVATIONS, f"the gate's activation is one of {sorted(ACTIVATIONS)}")
    _cuda(gate_up)
    _require(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.dtype in DTYPE_CODE
             and gate_up.shape[1] % 2 == 0, "gate_up must be a contiguous [T, 2I] tensor")
    T, two_i = gate_up.shape
    if out is None:
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _require(out.shape == (T, two_i // 2) and out.dtype == gate_up.dtype and out.is_contiguous(), "out must be [T, I]")
    _require(not blocked or (two_i // 2) % 8 == 0, "the blocked layout needs I to be a multiple of 8")
    _check(library().zb_act_mul(_ptr(out), _ptr(gate_up), T, two_i // 2, DTYPE_CODE[gate_up.dtype], int(blocked),
                                ACTIVATIONS[act], _stream()), "silu_mul")
    return out


# ------------------------------------------------------- layer norm, recurrences and their norms
def _f32_vector(v: torch.Tensor | None, size: int, what: str) -> None:
    _require(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == size),
             f"{what} must be a contiguous float32 tensor of {size} values")


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float,
               out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w + b over the last dimension of a contiguous [rows, H]; x float32 or
    bfloat16, the result in ``out_dtype`` (default: x's type); w and b float32; ``b`` None: no shift."""
    _cuda(x, w, b)
    _require(x.dim() == 2 and x.is_contiguous() and x.dtype in DTYPE_CODE, "x must be a contiguous [rows, H]")
    rows, H = x.shape
    _f32_vector(w, H, "the scale")
    _f32_vector(b, H, "the shift")
    out = torch.empty((rows, H), dtype=out_dtype or x.dtype, device=x.device)
    _check(library().zb_layer_norm(_ptr(out), _ptr(x), _ptr(w), _ptr(b), 0, float(eps), rows, H, DTYPE_CODE[x.dtype],
                                   DTYPE_CODE[out.dtype], _stream()), "layer_norm")
    return out


def residual_layer_norm(residual: torch.Tensor, delta: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor | None,
                        eps1: float, mult: float, w2: torch.Tensor | None = None, b2: torch.Tensor | None = None,
                        eps2: float = 0.0, rounded_sum: bool = False) -> torch.Tensor | None:
    """residual (float32, in place) += mult * LN(delta; w1, b1); with w2 (and b2, if that norm has a shift)
    also returns LN(residual; w2, b2) in delta's type: the sum and the next norm in one pass over the row.
    With ``rounded_sum`` and no w2 it returns the sum itself in delta's type, for a part that reads the
    stream as it is.  ``b1`` None: the first norm has no shift."""
    _cuda(residual, delta, w1, b1, w2, b2)
    _require(residual.dim() == 2 and residual.is_contiguous() and residual.dtype == torch.float32
             and delta.shape == residual.shape and delta.is_contiguous() and delta.dtype in DTYPE_CODE,
             "a float32 residual [rows, H] and a summand of the same shape")
    rows, H = residual.shape
    for vector in (w1, b1, w2, b2):
        _f32_vector(vector, H, "scales and shifts")
    _require(b2 is None or w2 is not None, "a shift comes with a scale")
    out = torch.empty_like(delta) if (w2 is not None or rounded_sum) else None
    _check(library().zb_residual_layer_norm(_ptr(residual), _ptr(delta), _ptr(w1), _ptr(b1), float(mult), _ptr(out),
                                            _ptr(w2), _ptr(b2), 0, float(eps1), float(eps2), rows, H,
                                            DTYPE_CODE[delta.dtype], _stream()), "residual_layer_norm")
    return out


def residual_rms_norm(residual: torch.Tensor, delta: torch.Tensor, w1: torch.Tensor, eps1: float, mult: float,
                      w2: torch.Tensor | None = None, eps2: float = 0.0, rounded_sum: bool = False) -> torch.Tensor | None:
    """residual (float32, in place) += mult * RMSnorm(delta; w1); with w2 also returns RMSnorm(residual; w2) in
    delta's type; with ``rounded_sum`` and no w2 the sum itself in delta's type.  Scales are float32."""
    _cuda(residual, delta, w1, w2)
    _require(residual.dim() == 2 and residual.is_contiguous() and residual.dtype == torch.float32
             and delta.shape == residual.shape and delta.is_contiguous() and delta.dtype in DTYPE_CODE,
             "a float32 residual [rows, H] and a summand of the same shape")
    rows, H = residual.shape
    for vector in (w1, w2):
        _f32_vector(vector, H, "scales")
    out = torch.empty_like(delta) if (w2 is not None or rounded_sum) else None
    _check(library().zb_residual_rms_norm(_ptr(residual), _ptr(delta), _ptr(w1), float(mult), _ptr(out), _ptr(w2), 0,
                                          float(eps1), float(eps2), rows, H, DTYPE_CODE[delta.dtype], _stream()),
           "residual_rms_norm")
    return out


def embedding_f32(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, scale: float = 1.0,
                  rounded: bool = False):
    """``scale`` times the rows of the table as float32 [T, H]: the start of a float32 residual stream.
    With ``rounded`` returns (float32 rows, the same rows in the table's type)."""
    _cuda(table, ids, status)
    _i32(ids)
    _require(table.dim() == 2 and table.is_contiguous() and table.dtype in DTYPE_CODE, "table must be [V, H]")
    V, H = table.shape
    out = torch.empty((ids.numel(), H), dtype=torch.float32, device=table.device)
    copy = torch.empty((ids.numel(), H), dtype=table.dtype, device=table.device) if rounded else None
    _check(library().zb_embedding_f32(_ptr(out), _ptr(copy), _ptr(table), _ptr(ids), float(scale), ids.numel(), H, V,
                                      DTYPE_CODE[table.dtype], _ptr(status), _stream()), "embedding_f32")
    return (out, copy) if rounded else out


def pair_embedding(table: torch.Tensor, pair_table: torch.Tensor, ctx_ids: torch.Tensor, positions: torch.Tensor,
                   token_row: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
                   state_slots: torch.Tensor, last_token: torch.Tensor, mul_prev: int, mul_cur: int,
                   status: torch.Tensor, rounded: bool = False):
    """Rows of ``table`` plus rows of ``pair_table`` ([buckets + 1, H]) chosen by a hash of the token and the
    token before it, (prev * mul_prev + id * mul_cur) mod buckets, as a float32 stream [T, H]; a sequence's
    first token (position 0) takes the pair table's last row.  The token before a row's first new token is
    ``last_token[state_slots[row]]`` (int32 [slots]); after the lookup the slots take the rows' last new
    tokens.  With ``rounded`` returns (float32 rows, the same rows in the tables' type)."""
    _cuda(table, pair_table, ctx_ids, positions, token_row, row_q_start, row_q_len, state_slots, last_token, status)
    _i32(ctx_ids, positions, token_row, row_q_start, row_q_len, state_slots, last_token)
    _require(table.dim() == 2 and table.is_contiguous() and table.dtype in DTYPE_CODE and pair_table.dim() == 2
             and pair_table.is_contiguous() and pair_table.dtype == table.dtype and pair_table.shape[1] == table.shape[1]
             and pair_table.shape[0] >= 2, "table [V, H] and pair table [buckets + 1, H] of one type")
    _require(last_token.is_contiguous() and positions.numel() == ctx_ids.numel() == token_row.numel()
             and row_q_start.numel() == row_q_len.numel() == state_slots.numel(), "one position and row per token")
    V, H = table.shape
    T, R = ctx_ids.numel(), row_q_start.numel()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    copy = torch.empty((T, H), dtype=table.dtype, device=table.device) if rounded else None
    lib = library()
    _check(lib.zb_pair_embedding(_ptr(out), _ptr(copy), _ptr(table), _ptr(pair_table), _ptr(ctx_ids), _ptr(positions),
                                 _ptr(token_row), _ptr(row_q_start), _ptr(state_slots), _ptr(last_token), T, H, V,
                                 pair_table.shape[0] - 1, int(mul_prev), int(mul_cur), R, last_token.numel(),
                                 DTYPE_CODE[table.dtype], _ptr(status), _stream()), "pair_embedding")
    _check(lib.zb_store_last_token(_ptr(last_token), _ptr(ctx_ids), _ptr(row_q_start), _ptr(row_q_len),
                                   _ptr(state_slots), R, last_token.numel(), _stream()), "store_last_token")
    return (out, copy) if rounded else out


def sum_rms_norm(x: torch.Tensor, a: torch.Tensor | None, b: torch.Tensor | None, w: torch.Tensor | None,
                 eps: float, out_dtype: torch.dtype | None = None, bias: torch.Tensor | None = None) -> torch.Tensor | None:
    """x (float32 [rows, H], unit inner stride, rows may be slices of wider rows) += (a + b + bias) in place,
    where a and b are contiguous [rows, H] summands of either type or None and ``bias`` is a float32 [H] shift
    of one of them (added to every row), or None; then, with a scale ``w``, returns
    x / sqrt(mean(x^2) + eps) * w in ``out_dtype``.  Statistics and sums are float32."""
    _cuda(x, a, b, w, bias)
    _f32_vector(bias, x.shape[-1], "the shift")
    _require(bias is None or a is not None or b is not None, "a shift comes with a summand")
    _require(x.dim() == 2 and x.dtype == torch.float32 and x.stride(1) == 1, "a float32 stream [rows, H]")
    rows, H = x.shape
    for summand in (a, b):
        _require(summand is None or (summand.shape == x.shape and summand.is_contiguous() and summand.dtype in DTYPE_CODE),
                 "summands are contiguous [rows, H]")
    out = None
    if w is not None:
        out = torch.empty((rows, H), dtype=out_dtype or torch.float32, device=x.device)
    _check(library().zb_sum_rms_norm(_ptr(out), H, DTYPE_CODE[out.dtype] if out is not None else 0, _ptr(x), x.stride(0),
                                     _ptr(a), DTYPE_CODE[a.dtype] if a is not None else 0, _ptr(b),
                                     DTYPE_CODE[b.dtype] if b is not None else 0, _ptr(bias), _ptr(w),
                                     _scale_code(w, H) if w is not None else 0, float(eps), rows, H, _stream()),
           "sum_rms_norm")
    return out


def clamped_gate(gate_up: torch.Tensor, bias: torch.Tensor | None, limit: float, alpha: float, shift: float,
                 out_dtype: torch.dtype, blocked: bool = False) -> torch.Tensor:
    """g * sigmoid(alpha * g) * (u + shift) with g = min(G + b_g, limit) and u = clamp(U + b_u, -limit, limit),
    for a contiguous product [T, 2I] (float32 or bfloat16) that holds G then U, or with ``blocked`` blocks
    of 8 gate columns each followed by its 8 up columns; ``bias`` float32 [2I] in the same column order, or
    None.  Returns [T, I] in ``out_dtype``."""
    _cuda(gate_up, bias)
    _require(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.dtype in DTYPE_CODE and gate_up.shape[1] % 2 == 0,
             "gate_up must be a contiguous [T, 2I] tensor")
    T, two_i = gate_up.shape
    _f32_vector(bias, two_i, "the bias")
    out = torch.empty((T, two_i // 2), dtype=out_dtype, device=gate_up.device)
    _check(library().zb_clamped_gate(_ptr(out), DTYPE_CODE[out_dtype], _ptr(gate_up), DTYPE_CODE[gate_up.dtype], _ptr(bias),
                                     T, two_i // 2, int(blocked), float(limit), float(alpha), float(shift), _stream()),
           "clamped_gate")
    return out


def scale_rows(y: torch.Tensor, scale: float) -> torch.Tensor:
    """y *= scale in place, for a contiguous float32 tensor."""
    _cuda(y)
    _require(y.dtype == torch.float32 and y.is_contiguous(), "a contiguous float32 tensor")
    _check(library().zb_scale_rows(_ptr(y), y.numel(), float(scale), _stream()), "scale_rows")
    return y


def latent_rope(q: torch.Tensor | None, nh: int, q_head_stride: int, q_rot_offset: int, q_out: torch.Tensor | None,
                kv: torch.Tensor | None, rank: int, rot: int, norm_w: torch.Tensor | None, eps: float,
                freqs: torch.Tensor | None, mult: float, positions: torch.Tensor, token_row: torch.Tensor,
                kv_cache: torch.Tensor | None, block_table: torch.Tensor, status: torch.Tensor,
                dtype: torch.dtype) -> None:
    """What latent attention with a rotated part keeps of a position, and the rotated part of its queries.
    ``kv`` (float32 [T, >= rank + rot], unit inner stride): the first ``rank`` values are RMS-normed with
    ``norm_w`` and the last ``rot`` rotated by the position's angles; the row of rank + rot values goes into
    the keys-only pages of ``kv_cache``.  ``q`` (float32, heads ``q_head_stride`` apart, the rotated part at
    ``q_rot_offset`` of a head): rotated the same way into the last ``rot`` values of every head of
    ``q_out`` [T, nh * (rank + rot)].  Rotation of halves: value i pairs with value i + rot / 2; angle =
    position * freqs[i] in float32; cosine and sine are multiplied by ``mult``."""
    _cuda(q, q_out, kv, norm_w, freqs, positions, token_row, kv_cache, block_table, status)
    _i32(positions, token_row, block_table)
    T = positions.numel()
    width = rank + rot
    for vector, size in ((norm_w, rank), (freqs, rot // 2)):
        _require(vector is None or (vector.dtype == torch.float32 and vector.is_contiguous() and vector.numel() == size),
                 f"a float32 vector of {size} values")
    if nh > 0:
        _require(q is not None and q.dtype == torch.float32 and q.dim() == 2 and q.stride(1) == 1 and q.shape[0] == T
                 and q.shape[1] >= (nh - 1) * q_head_stride + q_rot_offset + rot, "float32 queries [T, heads * head stride]")
        _require(q_out is not None and q_out.is_contiguous() and q_out.shape == (T, nh * width) and q_out.dtype == dtype,
                 "q_out [T, heads * (rank + rot)] in the model's type")
    pages, page_size = (0, 1)
    if kv_cache is not None:
        _require(kv is not None and kv.dtype == torch.float32 and kv.dim() == 2 and kv.stride(1) == 1
                 and kv.shape[0] == T and kv.shape[1] >= width, "float32 latent rows [T, rank + rot]")
        pages, page_size = _cache_geometry(kv_cache, 1, width, 0, dtype)
    _check(library().zb_latent_rope(
        _ptr(q_out), _ptr(q), q.stride(0) if q is not None else 0, int(q_head_stride), int(q_rot_offset), _ptr(kv),
        kv.stride(0) if kv is not None else 0, _ptr(norm_w), float(eps), _ptr(freqs), float(mult), _ptr(positions),
        _ptr(token_row), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages, block_table.shape[0],
        T, int(nh), int(rank), int(rot), DTYPE_CODE[dtype], _ptr(status), _stream()), "latent_rope")


CONV_MAX_TAPS = 8


def causal_conv_silu(x: torch.Tensor, channels: int, w: torch.Tensor, bias: torch.Tensor, state: torch.Tensor,
                     slots: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor, token_row: torch.Tensor,
                     status: torch.Tensor, write_state: bool = True) -> torch.Tensor:
    """silu(conv(x) + bias) per channel over each row's new tokens (``token_row``: the row of every token); ``x`` [T, >= channels] (rows may be
    strided), ``w`` float32 [channels, taps] whose last column weighs the current token.  ``state``
    [slots, (taps - 1) * channels] float32 (rows may be strided) holds every request's last taps - 1
    inputs, oldest first, and is brought up to date."""
    _cuda(x, w, bias, state, slots, row_q_start, row_q_len, token_row, status)
    _i32(slots, row_q_start, row_q_len, token_row)
    _require(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= channels and x.dtype in DTYPE_CODE
             and token_row.numel() == x.shape[0], "x shape")
    _require(w.dim() == 2 and w.shape[0] == channels and w.dtype == torch.float32 and w.is_contiguous(), "w must be float32 [channels, taps]")
    taps = w.shape[1]
    _f32_vector(bias, channels, "the bias")
    _require(state.dim() == 2 and state.dtype == torch.float32 and state.stride(1) == 1
             and state.shape[1] == (taps - 1) * channels, "state must be float32 [slots, (taps - 1) * channels]")
    out = torch.empty((x.shape[0], channels), dtype=x.dtype, device=x.device)
    _check(library().zb_causal_conv_silu(
        _ptr(out), _ptr(x), x.stride(0), _ptr(state), state.stride(0), _ptr(slots), _ptr(row_q_start), _ptr(row_q_len),
        _ptr(token_row), x.shape[0], slots.numel(), _ptr(w), _ptr(bias), 0, channels, taps, state.shape[0],
        int(write_state), DTYPE_CODE[x.dtype], _ptr(status), _stream()), "causal_conv_silu",
        kernels=2 if write_state and taps > 1 else 1)
    return out


SCAN_SEGMENT = 128     # tokens of a segment when long requests are cut into segments that run side by side


def state_scan_max_channels() -> int:
    return library().zb_state_scan_max_channels()


def decayed_state_scan(mode: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, key_dim: int,
                       value_dim: int, state: torch.Tensor, slots: torch.Tensor, row_q_start: torch.Tensor,
                       row_q_len: torch.Tensor, status: torch.Tensor, *, decay_logits: torch.Tensor | None = None,
                       decay_bias: torch.Tensor | None = None, inv_tau: float = 1.0, q_scale: float = 1.0,
                       dt: torch.Tensor | None = None, dt_bias: torch.Tensor | None = None,
                       a_log: torch.Tensor | None = None, skip: torch.Tensor | None = None, heads_per_group: int = 1,
                       write_state: bool = True, segment: int | None = None) -> torch.Tensor:
    """S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head over each row's new tokens, from and
    to ``state`` [slots, heads * key_dim * value_dim] float32 (rows may be strided); returns o as float32
    [T, heads * value_dim].  q, k, v: [T, .] with unit inner stride, head h at column h * width.
    ``mode`` "gated": a = sigmoid(decay_logits + decay_bias)^inv_tau per key channel (logits float32
    [T, heads * key_dim], overwritten with the decays), q times ``q_scale``.  ``mode`` "state_space": step = softplus(dt + dt_bias),
    a = exp(-exp(a_log) step) per head, k times step, o += skip * v; q and k belong to the head's group
    (head // heads_per_group at column group * key_dim).
    ``segment``: long requests are cut into segments of this many tokens that run side by side (a pass
    from zero states, a carry of the state from segment to segment, a pass with the outputs: twice the
    arithmetic on many times the threads); 0: never; None: chosen, for steps whose requests bring 256
    tokens and more on average and whose requests x heads x columns / 64 do not fill the SMs (measured,
    one request of 2048 tokens: 8 heads of 128 x 256: 712 -> 270 us; 16 heads: 720 -> 482 us)."""
    _cuda(q, k, v, state, slots, row_q_start, row_q_len, status, decay_logits, decay_bias, dt, dt_bias, a_log, skip)
    _i32(slots, row_q_start, row_q_len)
    T = v.shape[0]
    for t in (q, k, v):
        _require(t.dim() == 2 and t.stride(1) == 1 and t.shape[0] == T and t.dtype == v.dtype and t.dtype in DTYPE_CODE,
                 "q, k and v must be [T, .] of one type with unit inner stride")
    _require(state.dim() == 2 and state.dtype == torch.float32 and state.stride(1) == 1
             and state.shape[1] == heads * key_dim * value_dim, "state must be float32 [slots, heads * key_dim * value_dim]")
    gated = mode == "gated"
    _require(gated or mode == "state_space", "mode is 'gated' or 'state_space'")
    if gated:
        _require(decay_logits is not None and decay_logits.dtype == torch.float32 and decay_logits.dim() == 2
                 and decay_logits.stride(1) == 1 and decay_logits.shape == (T, heads * key_dim), "decay logits: float32 [T, heads * key_dim]")
        _f32_vector(decay_bias, heads * key_dim, "the decay bias")
        _require(decay_bias is not None, "the gated mode needs a decay bias")
    else:
        _require(dt is not None and dt.dim() == 2 and dt.stride(1) == 1 and dt.shape[0] == T and dt.shape[1] >= heads
                 and dt.dtype == v.dtype, "dt must be [T, heads] of the model's type")
        for vector in (dt_bias, a_log, skip):
            _require(vector is not None, "the state-space mode needs dt_bias, a_log and skip")
            _f32_vector(vector, heads, "a per-head constant")
    out = torch.empty((T, heads * value_dim), dtype=torch.float32, device=v.device)
    rows = slots.numel()
    if segment is None:
        few = rows * heads * -(-value_dim // 64) <= _sm_count()
        segment = (max(SCAN_SEGMENT, -(-T // (64 * 16)) * 16)
                   if few and T >= 4 * SCAN_SEGMENT and T >= 2 * SCAN_SEGMENT * rows else 0)
    ws_state = ws_decay = None
    if segment:
        pieces = rows * -(-T // segment)
        ws_state = torch.empty((pieces, heads * key_dim * value_dim), dtype=torch.float32, device=v.device)
        ws_decay = torch.empty((pieces, heads * key_dim), dtype=torch.float32, device=v.device)
    _check(library().zb_decayed_state_scan(
        _ptr(out), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(decay_logits),
        decay_logits.stride(0) if gated else 0, _ptr(decay_bias), _ptr(dt), dt.stride(0) if not gated else 0,
        _ptr(dt_bias), _ptr(a_log), _ptr(skip), 0, _ptr(state), state.stride(0), _ptr(slots), _ptr(row_q_start),
        _ptr(row_q_len), slots.numel(), T, heads, key_dim, value_dim, int(heads_per_group), state.shape[0],
        int(write_state), float(q_scale), float(inv_tau), 0 if gated else 1, DTYPE_CODE[v.dtype], int(segment),
        _ptr(ws_state), _ptr(ws_decay), _ptr(status), _stream()), "decayed_state_scan",
        kernels=(2 if gated else 1) + (2 if segment else 0))
    return out


def gated_group_rms_norm(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group: int, eps: float,
                         gate_first: bool) -> torch.Tensor:
    """RMS norm of a float32 [T, W] over groups of ``group`` columns with a SiLU gate ([T, >= W], rows may
    be strided) multiplied in before the norm (``gate_first``) or after it; ``w`` float32, used
    periodically (W values, or one group's).  The result has the gate's type."""
    _cuda(o, gate, w)
    _require(o.dim() == 2 and o.is_contiguous() and o.dtype == torch.float32, "o must be a contiguous float32 [T, W]")
    T, W = o.shape
    _require(gate.dim() == 2 and gate.stride(1) == 1 and gate.shape[0] == T and gate.shape[1] >= W
             and gate.dtype in DTYPE_CODE, "the gate must be [T, W] with unit inner stride")
    _require(w.dtype == torch.float32 and w.is_contiguous() and w.numel() in (W, group), "w: float32, W or group values")
    out = torch.empty((T, W), dtype=gate.dtype, device=o.device)
    _check(library().zb_gated_group_rms_norm(_ptr(out), _ptr(o), _ptr(gate), gate.stride(0), _ptr(w), 0, w.numel(), T, W,
                                             int(group), float(eps), int(gate_first), DTYPE_CODE[gate.dtype],
                                             _stream()), "gated_group_rms_norm")
    return out


def scaled_sum(a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float,
               out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """scale_a * a + scale_b * b in float32 with one rounding; a and b may be float32 whatever the result is."""
    _cuda(a, b)
    _require(a.shape == b.shape and a.dtype == b.dtype and a.dtype in DTYPE_CODE and a.is_contiguous()
             and b.is_contiguous(), "two contiguous tensors of one shape and type")
    out = torch.empty(a.shape, dtype=out_dtype or a.dtype, device=a.device)
    _check(library().zb_scaled_sum(_ptr(out), _ptr(a), _ptr(b), float(scale_a), float(scale_b), a.numel(),
                                   DTYPE_CODE[a.dtype], DTYPE_CODE[out.dtype], _stream()), "scaled_sum")
    return out


# ------------------------------------------------------------------ position and cache
def kv_swizzle(pos: int, chunks: int) -> int:
    """By how much the 16-byte chunks of the cache row at position ``pos`` are permuted: logical chunk
    c lives at chunk ``c ^ kv_swizzle(pos, chunks)``, with ``chunks`` = row bytes / 16.  (The same
    function as in csrc/common.cuh; tools and tests that read or fill a cache by hand need it.)"""
    step = chunks & 7
    if step == 0:
        return pos & 7
    if step == 4:
        return (pos >> 1) & 3
    if step in (2, 6):
        return (pos >> 2) & 1
    return 0


def kv_row_permutation(pos: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """``perm`` with ``stored_row[perm[i]] == logical_row[i]`` for the cache row at position ``pos``."""
    size = torch.empty((), dtype=dtype).element_size()
    per_chunk = 16 // size
    chunks = head_dim * size // 16
    index = torch.arange(head_dim)
    return ((index // per_chunk) ^ kv_swizzle(pos, chunks)) * per_chunk + index % per_chunk



def _check_cache(kv_cache: torch.Tensor, nkv: int, hd: int, dtype: torch.dtype) -> tuple[int, int]:
    _require(kv_cache.dim() == 5 and kv_cache.is_contiguous() and kv_cache.shape[1] == 2
             and kv_cache.shape[2] == nkv and kv_cache.shape[4] == hd and kv_cache.dtype == dtype,
             "a cache must be a contiguous [pages, 2, kv_heads, page_size, head_dim] tensor of the model's type")
    return kv_cache.shape[0], kv_cache.shape[3]


def qk_norm_rope_cache(qkv: torch.Tensor, nh: int, nkv: int, hd: int, q_norm_w: torch.Tensor | None,
                       k_norm_w: torch.Tensor | None, eps: float, cos: torch.Tensor | None,
                       sin: torch.Tensor | None, positions: torch.Tensor, token_row: torch.Tensor,
                       kv_cache: torch.Tensor | None, block_table: torch.Tensor, status: torch.Tensor,
                       q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused per-head norm of q and k, rotation, and the cache write; returns q as [T, nh*hd]."""
    _cuda(qkv, positions, token_row, block_table, status, kv_cache)
    _i32(positions, token_row, block_table)
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * hd if kv_cache is not None else nh * hd
    _require(qkv.dim() == 2 and qkv.shape[1] >= width and qkv.stride(1) == 1 and qkv.dtype in DTYPE_CODE,
             "qkv must be [T, (heads + 2*kv_heads)*head_dim] with unit inner stride")
    _require(hd % 2 == 0 and positions.numel() == T and token_row.numel() == T, "one position and row per token")
    _require(block_table.dim() == 2, "block_table must be [rows, blocks]")
    w_code = 0
    if q_norm_w is not None or k_norm_w is not None:
        _require(q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype,
                 "q and k norm scales come together and share a type")
        w_code = _scale_code(q_norm_w, hd)
        _scale_code(k_norm_w, hd)
    max_positions = 0
    if cos is not None:
        _require(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
                 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == hd // 2
                 and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
        max_positions = cos.shape[0]
    pages, page_size = (0, 1)
    if kv_cache is not None:
        pages, page_size = _check_cache(kv_cache, nkv, hd, qkv.dtype)
    if q_out is None:
        q_out = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    _require(q_out.shape == (T, nh * hd) and q_out.is_contiguous() and q_out.dtype == qkv.dtype, "q_out shape")
    _check(library().zb_qk_norm_rope_cache(
        _ptr(q_out), _ptr(qkv), qkv.stride(0), _ptr(q_norm_w), _ptr(k_norm_w), w_code, float(eps), _ptr(cos),
        _ptr(sin), max_positions, _ptr(positions), _ptr(token_row), _ptr(kv_cache), _ptr(block_table),
        block_table.shape[1], page_size, pages, block_table.shape[0], T, nh, nkv, hd, DTYPE_CODE[qkv.dtype],
        _ptr(status), _stream()), "qk_norm_rope_cache")
    return q_out


def rope(x: torch.Tensor, heads: int, hd: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
         status: torch.Tensor) -> torch.Tensor:
    """Rotate x [T, >= heads*hd] in place (rows may be strided)."""
    _cuda(x, cos, sin, positions, status)
    _i32(positions)
    _require(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= heads * hd and x.dtype in DTYPE_CODE, "x shape")
    _require(cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[1] == hd // 2
             and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
    _check(library().zb_rope(_ptr(x), x.stride(0), x.shape[0], heads, hd, _ptr(cos), _ptr(sin), cos.shape[0],
                             _ptr(positions), DTYPE_CODE[x.dtype], _ptr(status), _stream()), "rope")
    return x


def kv_write(k: torch.Tensor, v: torch.Tensor, nkv: int, hd: int, positions: torch.Tensor, token_row: torch.Tensor,
             kv_cache: torch.Tensor, block_table: torch.Tensor, status: torch.Tensor) -> None:
    _cuda(k, v, positions, token_row, kv_cache, block_table, status)
    _i32(positions, token_row, block_table)
    _require(k.dim() == 2 and v.dim() == 2 and k.stride(1) == 1 and v.stride(1) == 1 and k.dtype == v.dtype
             and k.shape[0] == v.shape[0] and k.shape[1] >= nkv * hd and v.shape[1] >= nkv * hd, "k/v shapes")
    pages, page_size = _check_cache(kv_cache, nkv, hd, k.dtype)
    _check(library().zb_kv_write(_ptr(k), _ptr(v), k.stride(0), v.stride(0), _ptr(positions), _ptr(token_row),
                                 _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
                                 block_table.shape[0], k.shape[0], nkv, hd, DTYPE_CODE[k.dtype], _ptr(status),
                                 _stream()), "kv_write")


# ----------------------------------------------------------------------------- attention
def attention_tile_tokens(group: int) -> int:
    """New tokens of one request per tile of the general attention kernel, for this group size."""
    return library().zb_attention_simt_tile_tokens(int(group))


def _cache_geometry(kv_cache: torch.Tensor, nkv: int, kd: int, vd: int, dtype: torch.dtype) -> tuple[int, int]:
    """(pages, page size) of a cache whose pages hold [nkv][page][kd] keys and then [nkv][page][vd] values:
    the five-dimensional form for equal widths, or flat pages (``vd`` 0: pages of keys alone)."""
    _require(kv_cache.is_contiguous() and kv_cache.dtype == dtype, "a cache must be contiguous and of the model's type")
    if kv_cache.dim() == 5:
        _require(kd == vd, "a [pages, 2, kv_heads, page_size, head_dim] cache has one width")
        return _check_cache(kv_cache, nkv, kd, dtype)
    _require(kv_cache.dim() == 2 and kv_cache.shape[1] % (nkv * (kd + vd)) == 0,
             "a cache of two widths must be [pages, kv_heads * page_size * (key_dim + value_dim)]")
    page_size = kv_cache.shape[1] // (nkv * (kd + vd))
    _require(page_size * kv_cache.element_size() % 16 == 0, "a page must hold a multiple of 16 bytes per element column")
    return kv_cache.shape[0], page_size


def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, tile_row: torch.Tensor,
                    tile_q0: torch.Tensor, tile_tokens: int, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
                    row_ctx: torch.Tensor, nh: int, nkv: int, hd: int, window: int, scale: float,
                    status: torch.Tensor, out: torch.Tensor | None = None,
                    head_slopes: torch.Tensor | None = None, value_dim: int | None = None, chunk: int = 0,
                    sinks: torch.Tensor | None = None, softcap: float = 0.0, shared_kv: bool = False,
                    keep_first: int = 0, pool: int = 0, pool_cache: torch.Tensor | None = None,
                    pool_table: torch.Tensor | None = None, cross_values: bool = False,
                    out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The general kernel: causal attention of every new token over its request's pages.
    ``head_slopes`` (float32 [nh]): query head h adds head_slopes[h] * (key position - query position)
    to its scores, a position encoding that is a bias on the scores.  ``value_dim``: the width of the
    values where it differs from the keys' ``hd``.  ``chunk`` > 0: a query sees only the keys of its own
    run of ``chunk`` positions, runs counted from position 0.  ``sinks`` (float32 [nh]): exp(sinks[h])
    joins the denominator of head h's softmax.  ``softcap`` > 0: scaled scores become
    softcap * tanh(score / softcap).  ``shared_kv``: the cache keeps keys only (flat pages
    [kv_heads * page_size * hd]) and they are the values too.  ``keep_first`` = n (with a window): keys at
    positions below n stay visible to every later query.  ``pool`` = P (with a window), ``pool_cache`` and
    ``pool_table``: a second store of one entry per block of P positions; a query at position i also sees
    the first floor((i - window + 1) / P) entries, in the same softmax.  ``cross_values``: every query
    head's weights applied to every key/value head's values; the result is [T, nh, nkv, value_dim].
    ``out_dtype``: float32 for a result that is not rounded to the cache's type."""
    _cuda(q, kv_cache, block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx, status, head_slopes, sinks,
          pool_cache, pool_table)
    for per_head in (head_slopes, sinks):
        _require(per_head is None or (per_head.dtype == torch.float32 and per_head.is_contiguous()
                                      and per_head.numel() == nh), "one float32 value per query head")
    _i32(block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx)
    vd = hd if value_dim is None else int(value_dim)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype in DTYPE_CODE, "q shape")
    _require(not shared_kv or vd == hd, "keys that serve as values have the values' width")
    pages, page_size = _cache_geometry(kv_cache, nkv, hd, 0 if shared_kv else vd, q.dtype)
    out_dtype = out_dtype or q.dtype
    _require(out_dtype in (q.dtype, torch.float32), "the result has the queries' type or float32")
    width = nh * vd * (nkv if cross_values else 1)
    if out is None:
        out = torch.empty((q.shape[0], width), dtype=out_dtype, device=q.device)
    _require(out.shape == (q.shape[0], width) and out.dtype == out_dtype and out.is_contiguous(), "out must be [T, heads * value_dim]")
    pool_pages, pool_blocks = 0, 0
    if pool:
        _require(window > 0 and pool_cache is not None and pool_table is not None and pool_table.dtype == torch.int32
                 and pool_table.dim() == 2 and pool_table.shape[0] == block_table.shape[0]
                 and pool_cache.shape[1:] == kv_cache.shape[1:] and pool_cache.dtype == kv_cache.dtype
                 and pool_cache.is_contiguous(), "a pooled store has the pages' shape and a table row per request")
        pool_pages, pool_blocks = pool_cache.shape[0], pool_table.shape[1]
    _check(library().zb_paged_attention_simt(
        _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
        block_table.shape[0], _ptr(tile_row), _ptr(tile_q0), tile_row.numel(), int(tile_tokens), _ptr(row_q_start),
        _ptr(row_q_len), _ptr(row_ctx), nh, nkv, hd, vd, int(window), int(chunk), float(scale), float(softcap),
        int(shared_kv), _ptr(head_slopes), _ptr(sinks), int(keep_first), int(pool), _ptr(pool_cache),
        _ptr(pool_table), pool_blocks, pool_pages, int(cross_values), int(out_dtype == torch.float32 and q.dtype != torch.float32),
        DTYPE_CODE[q.dtype], _ptr(status), _stream()), "paged_attention")
    return out


QK_NORMS = {"none": 0, "per_head": 1, "whole": 2}


def qkv_halves(qkv: torch.Tensor, nh: int, nkv: int, kd: int, vd: int, norm: str, q_norm_w: torch.Tensor | None,
               k_norm_w: torch.Tensor | None, eps: float, freqs: torch.Tensor | None, rot_dims: int, rot_mult: float,
               value_unit_norm: bool, positions: torch.Tensor, token_row: torch.Tensor, kv_cache: torch.Tensor | None,
               block_table: torch.Tensor, status: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """From a fused q/k/v projection to queries and cache entries, for a rotation of halves: an RMS norm of q
    and of k (``norm`` "per_head": per head, scales [kd] shared by the heads; "whole": one statistic over all
    heads of q and one over all heads of k, scales [nh * kd] and [nkv * kd]; "none"; scales may be None),
    the rotation of value i with value i + rot_dims / 2 by position * freqs[i] on the first ``rot_dims``
    values of every q and k head (cosine and sine times ``rot_mult``), every value head divided by its root
    mean square (``value_unit_norm``), and the cache write of k and v.  Returns the queries [T, nh * kd] in
    ``dtype``; ``qkv`` may be float32 whatever ``dtype`` is.  Without ``kv_cache`` only the queries are made."""
    _cuda(qkv, q_norm_w, k_norm_w, freqs, positions, token_row, kv_cache, block_table, status)
    _i32(positions, token_row, block_table)
    T = qkv.shape[0]
    width = nh * kd + (nkv * (kd + vd) if kv_cache is not None else 0)
    _require(qkv.dim() == 2 and qkv.shape[1] >= width and qkv.stride(1) == 1 and qkv.dtype in DTYPE_CODE,
             "qkv must be [T, heads*key_dim + kv_heads*(key_dim + value_dim)] with unit inner stride")
    _require(norm in QK_NORMS, f"the norm of q and k is one of {sorted(QK_NORMS)}")
    sizes = (nh * kd, nkv * kd) if norm == "whole" else (kd, kd)
    for vector, size in ((q_norm_w, sizes[0]), (k_norm_w, sizes[1]), (freqs, rot_dims // 2)):
        _require(vector is None or (vector.dtype == torch.float32 and vector.is_contiguous() and vector.numel() == size),
                 f"a float32 vector of {size} values")
    _require(positions.numel() == T and token_row.numel() == T and block_table.dim() == 2, "one position and row per token")
    pages, page_size = (0, 1)
    if kv_cache is not None:
        pages, page_size = _cache_geometry(kv_cache, nkv, kd, vd, dtype)
    q_out = torch.empty((T, nh * kd), dtype=dtype, device=qkv.device)
    _check(library().zb_qkv_halves(
        _ptr(q_out), _ptr(qkv), qkv.stride(0), QK_NORMS[norm], _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(freqs),
        int(rot_dims), float(rot_mult), int(value_unit_norm), _ptr(positions), _ptr(token_row), _ptr(kv_cache),
        _ptr(block_table), block_table.shape[1], page_size, pages, block_table.shape[0], T, nh, nkv, kd, vd,
        DTYPE_CODE[qkv.dtype], DTYPE_CODE[dtype], _ptr(status), _stream()), "qkv_halves")
    return q_out


def pool_blocks(kv_cache: torch.Tensor, block_table: torch.Tensor, pool_cache: torch.Tensor, pool_table: torch.Tensor,
                positions: torch.Tensor, token_row: torch.Tensor, nkv: int, kd: int, vd: int, pool: int,
                status: torch.Tensor) -> None:
    """For every new token that completes a block of ``pool`` positions (position p with (p + 1) % pool == 0),
    entry p // pool of the pooled store becomes the mean of the block's keys and values as the pages hold
    them (float32 sums in the order of the positions, one rounding)."""
    _cuda(kv_cache, block_table, pool_cache, pool_table, positions, token_row, status)
    _i32(block_table, pool_table, positions, token_row)
    pages, page_size = _cache_geometry(kv_cache, nkv, kd, vd, kv_cache.dtype)
    _require(pool_cache.shape[1:] == kv_cache.shape[1:] and pool_cache.dtype == kv_cache.dtype and pool_cache.is_contiguous()
             and pool_table.dim() == 2 and pool_table.shape[0] == block_table.shape[0], "a pooled store has the pages' shape")
    _check(library().zb_pool_blocks(
        _ptr(kv_cache), _ptr(block_table), block_table.shape[1], pages, _ptr(pool_cache), _ptr(pool_table),
        pool_table.shape[1], pool_cache.shape[0], _ptr(positions), _ptr(token_row), positions.numel(),
        block_table.shape[0], page_size, nkv, kd, vd, int(pool), DTYPE_CODE[kv_cache.dtype], _ptr(status), _stream()),
        "pool_blocks")


def head_mix(a: torch.Tensor, mix: torch.Tensor, nh: int, nkv: int, vd: int, out_dtype: torch.dtype) -> torch.Tensor:
    """out[t, h] = sum_g mix[h, g] * a[t, g, kv(h)]: ``a`` float32 [T, nh * nkv * vd] (what every head's softmax
    weights make of every key/value head's values), ``mix`` float32 [nh, nh]; the result [T, nh * vd]."""
    _cuda(a, mix)
    _require(a.dim() == 2 and a.is_contiguous() and a.dtype == torch.float32 and a.shape[1] == nh * nkv * vd, "a: float32 [T, nh * nkv * vd]")
    _require(mix.dtype == torch.float32 and mix.is_contiguous() and mix.shape == (nh, nh), "mix: float32 [nh, nh]")
    out = torch.empty((a.shape[0], nh * vd), dtype=out_dtype, device=a.device)
    _check(library().zb_head_mix(_ptr(out), _ptr(a), _ptr(mix), a.shape[0], nh, nkv, vd, DTYPE_CODE[out_dtype], _stream()),
           "head_mix")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x *= sigmoid(gate) in place and value by value; ``gate`` float32 [T, width], rows may be strided."""
    _cuda(x, gate)
    _require(x.dim() == 2 and x.is_contiguous() and x.dtype in DTYPE_CODE, "x: contiguous [T, width]")
    _require(gate.dtype == torch.float32 and gate.shape == x.shape and gate.stride(1) == 1, "gate: float32 [T, width]")
    _check(library().zb_sigmoid_gate(_ptr(x), _ptr(gate), gate.stride(0), x.shape[0], x.shape[1], DTYPE_CODE[x.dtype],
                                     _stream()), "sigmoid_gate")
    return x


def delta_max_channels() -> int:
    return library().zb_delta_max_channels()


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b: torch.Tensor, a: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, heads: int, qk_heads: int, key_dim: int, value_dim: int,
               state: torch.Tensor, slots: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
               status: torch.Tensor, q_scale: float, unit_eps: float = 1e-6, write_state: bool = True) -> torch.Tensor:
    """The gated delta rule per head over each row's new tokens, from and to ``state`` [slots, heads *
    value_dim * key_dim] float32 (rows may be strided; a head's state lies [value_dim][key_dim]):
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q and k [T, qk_heads * key_dim] (head h uses
    q/k head h // (heads / qk_heads)) are made unit vectors, x / sqrt(sum(x^2) + unit_eps), q times
    ``q_scale``; v [T, heads * value_dim]; beta = sigmoid(b), g = exp(-exp(a_log) softplus(a + dt_bias)) from
    float32 b and a [T, heads].  q, k, v share a type and may be strided slices.  Returns o float32
    [T, heads * value_dim]."""
    _cuda(q, k, v, b, a, a_log, dt_bias, state, slots, row_q_start, row_q_len, status)
    _i32(slots, row_q_start, row_q_len)
    T = v.shape[0]
    for t, width in ((q, qk_heads * key_dim), (k, qk_heads * key_dim), (v, heads * value_dim)):
        _require(t.dim() == 2 and t.stride(1) == 1 and t.shape == (T, width) and t.dtype == v.dtype and t.dtype in DTYPE_CODE,
                 "q, k and v must be [T, .] of one type with unit inner stride")
    for t in (b, a):
        _require(t.dim() == 2 and t.shape == (T, heads) and t.dtype == torch.float32 and t.stride(1) == 1
                 and t.stride(0) == b.stride(0), "b and a: float32 [T, heads] with one row stride")
    _f32_vector(a_log, heads, "A_log")
    _f32_vector(dt_bias, heads, "dt_bias")
    _require(heads % qk_heads == 0, "heads must be a multiple of the q/k heads")
    _require(state.dim() == 2 and state.dtype == torch.float32 and state.stride(1) == 1
             and state.shape[1] == heads * key_dim * value_dim, "state must be float32 [slots, heads * value_dim * key_dim]")
    dev = v.device
    qn = torch.empty((T, qk_heads * key_dim), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    beta = torch.empty((T, heads), dtype=torch.float32, device=dev)
    decay = torch.empty_like(beta)
    _check(library().zb_delta_gates(_ptr(qn), _ptr(kn), _ptr(beta), _ptr(decay), _ptr(q), q.stride(0), _ptr(k), k.stride(0),
                                    _ptr(b), _ptr(a), b.stride(0), _ptr(a_log), _ptr(dt_bias), T, qk_heads, heads, key_dim,
                                    float(q_scale), float(unit_eps), DTYPE_CODE[v.dtype], _stream()), "delta_gates")
    out = torch.empty((T, heads * value_dim), dtype=torch.float32, device=dev)
    _check(library().zb_delta_scan(_ptr(out), _ptr(qn), _ptr(kn), _ptr(v), v.stride(0), _ptr(beta), _ptr(decay), _ptr(state),
                                   state.stride(0), _ptr(slots), _ptr(row_q_start), _ptr(row_q_len), slots.numel(), T, heads,
                                   heads // qk_heads, key_dim, value_dim, state.shape[0], int(write_state),
                                   DTYPE_CODE[v.dtype], _ptr(status), _stream()), "delta_scan")
    return out


def qkv_pairs(qkv: torch.Tensor, nh: int, nkv: int, kd: int, vd: int, bias: torch.Tensor | None,
              q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, eps: float, freqs: torch.Tensor | None,
              rot_dims: int, positions: torch.Tensor, token_row: torch.Tensor, kv_cache: torch.Tensor | None,
              block_table: torch.Tensor, status: torch.Tensor, dtype: torch.dtype, unit_norm: bool = False,
              values_from_keys: bool = False, q_temp: tuple[float, int] | None = None) -> torch.Tensor | None:
    """Bias, per-head RMS norm of q and k, rotation of adjacent pairs by position * freqs on the first
    ``rot_dims`` dimensions, and the cache write of k and v (keys ``kd`` wide, values ``vd``); returns the
    queries [T, nh * kd] in ``dtype``.  ``qkv`` may be float32 whatever ``dtype`` is; bias, norm scales and
    frequencies are float32.  Without ``kv_cache`` only the queries are made.

    ``unit_norm``: q and k are divided by their root mean square and no scale follows.
    ``values_from_keys``: ``qkv`` has no value columns; the values are the keys as projected (before
    their norm).  ``q_temp`` = (coef, every): the normed queries are multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1) at position p.  ``vd`` 0: the cache keeps keys only.
    ``nh`` 0: there are no queries, only the cache is written (returns None)."""
    _cuda(qkv, bias, q_norm_w, k_norm_w, freqs, positions, token_row, kv_cache, block_table, status)
    _i32(positions, token_row, block_table)
    T = qkv.shape[0]
    width = nh * kd + (nkv * (kd + (0 if values_from_keys else vd)) if kv_cache is not None else 0)
    _require(qkv.dim() == 2 and qkv.shape[1] >= width and qkv.stride(1) == 1 and qkv.dtype in DTYPE_CODE,
             "qkv must be [T, heads*key_dim + kv_heads*(key_dim + value_dim)] with unit inner stride")
    for vector, size in ((bias, width), (q_norm_w, kd), (k_norm_w, kd), (freqs, rot_dims // 2)):
        _require(vector is None or (vector.dtype == torch.float32 and vector.is_contiguous() and vector.numel() == size),
                 f"a float32 vector of {size} values")
    _require(positions.numel() == T and token_row.numel() == T and block_table.dim() == 2, "one position and row per token")
    pages, page_size = (0, 1)
    if kv_cache is not None:
        pages, page_size = _cache_geometry(kv_cache, nkv, kd, vd, dtype)
    q_out = torch.empty((T, nh * kd), dtype=dtype, device=qkv.device) if nh > 0 else None
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 1)
    _check(library().zb_qkv_pairs(
        _ptr(q_out), _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(freqs),
        int(rot_dims), _ptr(positions), _ptr(token_row), _ptr(kv_cache), _ptr(block_table), block_table.shape[1],
        page_size, pages, block_table.shape[0], T, nh, nkv, kd, vd, int(unit_norm), int(values_from_keys), coef,
        every, DTYPE_CODE[qkv.dtype], DTYPE_CODE[dtype], _ptr(status), _stream()), "qkv_pairs")
    return q_out


def paged_decode_supported(nh: int, nkv: int, hd: int, dtype: torch.dtype) -> bool:
    return dtype in DTYPE_CODE and bool(library().zb_paged_decode_supported(nh, nkv, hd, DTYPE_CODE[dtype]))


def paged_decode_scratch_floats(n_rows: int, nh: int, hd: int, max_splits: int) -> int:
    return int(library().zb_paged_decode_scratch_floats(n_rows, nh, hd, max_splits))


# Buffers of the decode kernel, kept for the life of the process: the partial results of the splits
# (contents irrelevant between calls) and the arrival counters (zero between calls: the kernel
# leaves them as it found them).  Buffers are only ever added, never freed or moved, because
# captured graphs hold their addresses.
_decode_buffers: dict[tuple[torch.device, int], list[tuple[torch.Tensor, torch.Tensor]]] = {}

# Two halves of a batch may run side by side on two streams (``parts.Model``): each is a lane with
# workspaces of its own (the decode kernel's partial results and counters, the chain's barrier
# counters), and the persistent kernels take half the SMs each.
LANE = 0


class lane:
    """``with ops.lane(1, ctas): ...``: launches inside use lane 1's workspaces and at most ``ctas``
    CTAs per persistent kernel (0: one per SM)."""

    def __init__(self, index: int, ctas: int = 0):
        self.index, self.ctas = index, ctas

    def __enter__(self):
        global LANE
        self.before = (LANE, int(library().zb_set_sm_share(int(self.ctas))))
        LANE = self.index
        return self

    def __exit__(self, *exc):
        global LANE
        LANE = self.before[0]
        library().zb_set_sm_share(self.before[1])
        return False


def _decode_workspace(device: torch.device, floats: int, counters: int) -> tuple[torch.Tensor, torch.Tensor]:
    pool = _decode_buffers.setdefault((device, LANE), [])
    for scratch, count in pool:
        if scratch.numel() >= floats and count.numel() >= counters:
            return scratch, count
    scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
    count = torch.zeros(max(counters, 1 << 12), dtype=torch.int32, device=device)
    pool.append((scratch, count))
    return scratch, count


def decode_split_size(n_rows: int, nkv: int, max_context: int) -> int:
    """A size for fixed splits (``paged_decode(..., split_size=...)``): as many splits of a row's
    context as give every SM one item and none two (a second round of items would leave most SMs
    idle), and no split shorter than 128 positions.  ``paged_decode`` takes fixed splits for a
    handful of rows (4 * rows * key/value heads <= SMs); for more, the kernel spreads the tiles of
    all rows evenly over its CTAs.  Either way, where a row's context is cut, and with that the last
    bits of its result, depends on how many rows are decoded beside it."""
    per_pair = max(1, _sm_count() // max(1, n_rows * nkv))     # splits of a (row, key/value head) pair: one item per SM
    split = -(-max_context // per_pair)
    return max(128, -(-split // 32) * 32)


_SM_COUNT: dict[int, int] = {}


def _sm_count() -> int:
    """SMs a persistent kernel launched now may take (all, or the current lane's share)."""
    device = torch.cuda.current_device()
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    share = int(library().zb_set_sm_share(0))
    library().zb_set_sm_share(share)
    return min(_SM_COUNT[device], share) if share > 0 else _SM_COUNT[device]


def paged_decode(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, rows: torch.Tensor,
                 row_q_start: torch.Tensor, row_ctx: torch.Tensor, max_context: int, nh: int, nkv: int, hd: int,
                 window: int, scale: float, status: torch.Tensor, out: torch.Tensor,
                 scratch: torch.Tensor | None = None, split_size: int | None = None,
                 counters: torch.Tensor | None = None, chunk: int = 0,
                 sinks: torch.Tensor | None = None, softcap: float = 0.0, keys_only: bool = False) -> torch.Tensor:
    """Split-context attention for rows with one new token each; writes those tokens' rows of ``out``.
    ``chunk``, ``sinks`` and ``softcap`` as in ``paged_attention``; ``keys_only`` as its ``shared_kv``.

    ``max_context`` is at least the longest context of the rows, the new token included.  ``scratch``
    (float32, any contents) and ``counters`` (int32, zero) come from a process-wide workspace unless
    given.  ``split_size`` None or 0: balanced work items; a multiple of 32: fixed splits of that size."""
    _cuda(q, kv_cache, block_table, rows, row_q_start, row_ctx, status, out)
    _i32(block_table, rows, row_q_start, row_ctx)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype == torch.bfloat16, "q shape")
    _require(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    pages, page_size = _cache_geometry(kv_cache, nkv, hd, 0, q.dtype) if keys_only else _check_cache(kv_cache, nkv, hd, q.dtype)
    n_rows = rows.numel()
    if split_size is None and n_rows * nkv * 4 <= _sm_count():
        # A handful of long rows: fixed splits keep every item inside one row (a CTA whose share
        # straddles two rows pays for two merges, which shows when the shares are a few tiles).
        split_size = decode_split_size(n_rows, nkv, max_context)
    if split_size is None or split_size == 0:
        # Balanced items: the tiles of all rows spread evenly over the CTAs (see attention_decode.cu).
        split_size, max_splits = 0, max(1, math.ceil(max_context / 32))
        need = int(library().zb_paged_decode_balanced_scratch_floats(nh, nkv, hd))
    else:
        max_splits = max(1, math.ceil(max_context / split_size))
        need = paged_decode_scratch_floats(n_rows, nh, hd, max_splits)
    if scratch is None or counters is None:
        scratch, counters = _decode_workspace(q.device, need, n_rows * nkv)
    _require(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
             f"scratch must hold {need} floats")
    _require(counters.dtype == torch.int32 and counters.is_contiguous() and counters.numel() >= n_rows * nkv,
             f"counters must hold {n_rows * nkv} zeroed int32 values")
    if chunk or sinks is not None or softcap or keys_only:
        _cuda(sinks)
        _require(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == nh),
                 "one float32 sink per query head")
        _check(library().zb_paged_decode_masked(
            _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
            block_table.shape[0], _ptr(rows), n_rows, _ptr(row_q_start), _ptr(row_ctx), nh, nkv, hd, int(window),
            int(chunk), float(scale), float(softcap), int(keys_only), _ptr(sinks), int(split_size), max_splits,
            _ptr(scratch), _ptr(counters), _ptr(status), _stream()), "paged_decode")
        return out
    _check(library().zb_paged_decode(
        _ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
        block_table.shape[0], _ptr(rows), n_rows, _ptr(row_q_start), _ptr(row_ctx), nh, nkv, hd, int(window),
        float(scale), int(split_size), max_splits, _ptr(scratch), _ptr(counters), _ptr(status), _stream()),
        "paged_decode")
    return out


def paged_decode_fused(qkv: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, rows: torch.Tensor,
                       row_q_start: torch.Tensor, row_ctx: torch.Tensor, max_context: int, nh: int, nkv: int, hd: int,
                       window: int, scale: float, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, eps: float,
                       cos: torch.Tensor | None, sin: torch.Tensor | None, status: torch.Tensor, out: torch.Tensor,
                       split_size: int | None = None) -> torch.Tensor:
    """``qk_norm_rope_cache`` and ``paged_decode`` in one kernel, for steps in which every request
    has exactly one new token: ``qkv`` [T, >= (nh + 2 nkv) hd] holds the new tokens raw; the per-head
    norms, the rotation and the cache write of the new keys and values happen inside the attention
    kernel (a row's new position is its ``row_ctx``), and ``out`` [T, nh hd] gets the attention's
    result.  No kernel stands between the projection and the attention then."""
    _cuda(qkv, kv_cache, block_table, rows, row_q_start, row_ctx, status, out, q_norm_w, k_norm_w, cos, sin)
    _i32(block_table, rows, row_q_start, row_ctx)
    T = qkv.shape[0]
    _require(qkv.dim() == 2 and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= (nh + 2 * nkv) * hd
             and qkv.stride(0) % 2 == 0, "qkv must be bfloat16 [T, (heads + 2*kv_heads)*head_dim] with unit inner stride")
    _require(out.shape == (T, nh * hd) and out.dtype == torch.bfloat16 and out.is_contiguous(), "out must be [T, heads*head_dim]")
    pages, page_size = _check_cache(kv_cache, nkv, hd, qkv.dtype)
    w_code = 0
    if q_norm_w is not None or k_norm_w is not None:
        _require(q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype,
                 "q and k norm scales come together and share a type")
        w_code = _scale_code(q_norm_w, hd)
        _scale_code(k_norm_w, hd)
    max_positions = 0
    if cos is not None:
        _require(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32
                 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == hd // 2
                 and cos.is_contiguous() and sin.is_contiguous(), "cos/sin must be float32 [positions, head_dim/2]")
        max_positions = cos.shape[0]
    n_rows = rows.numel()
    if split_size is None and n_rows * nkv * 4 <= _sm_count():
        split_size = decode_split_size(n_rows, nkv, max_context)
    if split_size is None or split_size == 0:
        split_size, max_splits = 0, max(1, math.ceil(max_context / 32))
        need = int(library().zb_paged_decode_balanced_scratch_floats(nh, nkv, hd))
    else:
        max_splits = max(1, math.ceil(max_context / split_size))
        need = paged_decode_scratch_floats(n_rows, nh, hd, max_splits)
    scratch, counters = _decode_workspace(qkv.device, need, n_rows * nkv)
    _check(library().zb_paged_decode_fused(
        _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages, block_table.shape[0],
        _ptr(rows), n_rows, _ptr(row_q_start), _ptr(row_ctx), nh, nkv, hd, int(window), float(scale), int(split_size),
        max_splits, _ptr(scratch), _ptr(counters), _ptr(status), _ptr(qkv), qkv.stride(0), _ptr(q_norm_w), _ptr(k_norm_w),
        w_code, float(eps), _ptr(cos), _ptr(sin), max_positions, _stream()), "paged_decode_fused")
    return out


USE_TCGEN05_PREFILL = True      # off: the mma.sync kernel for every head size (for comparisons)


def paged_decode_trace(buffer: torch.Tensor | None) -> None:
    """Later ``paged_decode`` launches write every CTA's timeline into ``buffer`` (int32 [1024, 8] on the
    device: the global timer in ns at the CTA's start, after the wait for earlier kernels, when its
    first tile had landed, after its last tile, at its end; then its items and tiles); None turns it off."""
    if buffer is not None:
        _cuda(buffer)
        _require(buffer.dtype == torch.int32 and buffer.is_contiguous() and buffer.numel() >= 8 * 1024, "int32 [1024, 8]")
    _check(library().zb_paged_decode_set_trace(_ptr(buffer)), "paged_decode_trace", kernels=0)


def paged_prefill_trace(buffer: torch.Tensor | None) -> None:
    """Later tcgen05 prompt-attention launches write the timeline of their first CTA (the longest
    work of the launch) into ``buffer`` (int32 [2, 64, 4] on the device; per tile of keys, [0]: the
    global timer in ns when S was issued, when its softmax began, when its probabilities were written,
    when O += P V was issued; [1]: when the first loader thread began to issue its keys, its values,
    and when it had issued them); None turns it off."""
    if buffer is not None:
        _cuda(buffer)
        _require(buffer.dtype == torch.int32 and buffer.is_contiguous() and buffer.numel() >= 512, "int32 [2, 64, 4]")
    _check(library().zb_paged_prefill_tc_set_trace(_ptr(buffer)), "paged_prefill_trace", kernels=0)


def paged_prefill_tile_tokens() -> int:
    """New tokens of one request per tile of the tensor-core prompt attention kernel."""
    return library().zb_paged_prefill_tile_tokens()


def paged_prefill_supported(nh: int, nkv: int, hd: int, dtype: torch.dtype) -> bool:
    return dtype in DTYPE_CODE and bool(library().zb_paged_prefill_supported(nh, nkv, hd, DTYPE_CODE[dtype]))


def paged_prefill(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, tile_row: torch.Tensor,
                  tile_q0: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx: torch.Tensor,
                  nh: int, nkv: int, hd: int, window: int, scale: float, status: torch.Tensor,
                  out: torch.Tensor, chunk: int = 0, sinks: torch.Tensor | None = None, softcap: float = 0.0,
                  keys_only: bool = False, keep_first: int = 0, pool: int = 0, pool_cache: torch.Tensor | None = None,
                  pool_table: torch.Tensor | None = None, cross_values: bool = False,
                  by_group: bool = False) -> torch.Tensor:
    """Tensor-core attention for rows with several new tokens, cut into tiles of
    ``paged_prefill_tile_tokens()``; writes those tokens' rows of ``out``.  ``chunk``, ``sinks`` and
    ``softcap`` as in ``paged_attention``, ``keys_only`` as its ``shared_kv``.  Head size 128 runs on tcgen05
    with the accumulators in tensor memory (every form but the chunked mask), other sizes and chunked masks
    on mma.sync.  ``keep_first``, ``pool`` with its store, and ``cross_values`` (``out`` is then
    [T, nh * nkv * hd], bfloat16 or float32) as in ``paged_attention``: these run on mma.sync.  ``by_group``: every
    tile is one new token (the tiles of single-token rows), and a CTA's query rows are the heads that share a
    key/value head: a decoded token's keys and values stream once a group."""
    _cuda(q, kv_cache, block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx, status, out, pool_cache, pool_table)
    _i32(block_table, tile_row, tile_q0, row_q_start, row_q_len, row_ctx)
    _require(q.dim() == 2 and q.is_contiguous() and q.shape[1] == nh * hd and q.dtype == torch.bfloat16, "q shape")
    windowed = bool(keep_first or pool or cross_values or by_group)
    if windowed:
        _require(out.shape == (q.shape[0], nh * hd * (nkv if cross_values else 1)) and out.is_contiguous()
                 and out.dtype in ((torch.float32, q.dtype) if cross_values else (q.dtype,)), "out: [T, nh (* nkv) * hd]")
    else:
        _require(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    pages, page_size = _cache_geometry(kv_cache, nkv, hd, 0, q.dtype) if keys_only else _check_cache(kv_cache, nkv, hd, q.dtype)
    _cuda(sinks)
    _require(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == nh),
             "one float32 sink per query head")
    pool_pages, pool_blocks = 0, 0
    if pool:
        _require(window > 0 and not keys_only and pool_cache is not None and pool_table is not None
                 and pool_table.dtype == torch.int32 and pool_table.dim() == 2 and pool_table.shape[0] == block_table.shape[0]
                 and pool_cache.shape[1:] == kv_cache.shape[1:] and pool_cache.dtype == kv_cache.dtype
                 and pool_cache.is_contiguous(), "a pooled store has the pages' shape and a table row per request")
        pool_pages, pool_blocks = pool_cache.shape[0], pool_table.shape[1]
    tensor_memory = (USE_TCGEN05_PREFILL and not chunk and not windowed
                     and bool(library().zb_paged_prefill_tc_supported(nh, nkv, hd, DTYPE_CODE[q.dtype], page_size)))
    common = (_ptr(out), _ptr(q), _ptr(kv_cache), _ptr(block_table), block_table.shape[1], page_size, pages,
              block_table.shape[0], _ptr(tile_row), _ptr(tile_q0), tile_row.numel(), _ptr(row_q_start), _ptr(row_q_len),
              _ptr(row_ctx), nh, nkv, hd, int(window))
    if tensor_memory:
        _check(library().zb_paged_prefill_tc_masked(*common, float(scale), float(softcap), int(keys_only), _ptr(sinks),
                                                    _ptr(status), _stream()), "paged_prefill")
    elif windowed:
        _check(library().zb_paged_prefill_windowed(*common, int(chunk), float(scale), float(softcap), int(keys_only),
                                                   _ptr(sinks), int(keep_first), int(pool), _ptr(pool_cache),
                                                   _ptr(pool_table), pool_blocks, pool_pages, int(cross_values),
                                                   int(out.dtype == torch.float32), int(by_group), _ptr(status),
                                                   _stream()), "paged_prefill")
    else:
        _check(library().zb_paged_prefill_masked(*common, int(chunk), float(scale), float(softcap), int(keys_only),
                                                 _ptr(sinks), _ptr(status), _stream()), "paged_prefill")
    return out


# ------------------------------------------------------------------------ matrix products
def gemm_nt_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed, float32 multiply-adds on CUDA cores."""
    _cuda(x, w)
    _require(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == w.dtype
             and x.dtype in DTYPE_CODE and x.stride(1) == 1 and w.stride(1) == 1, "x [M, K] and w [N, K] of one type")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _require(out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1, "out must be [M, N]")
    _check(library().zb_gemm_nt_simt(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                     DTYPE_CODE[x.dtype], DTYPE_CODE[out_dtype], _stream()), "gemm_nt_simt")
    return out


SMALL_GEMM_MAX_ROWS = 64      # what the kernel takes
SMALL_GEMM_ROWS = 16          # up to here it beats the library product; beyond, activations are re-read too often


def gemm_small_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True if the weight-streaming kernel for few rows takes x [M, K] times w [N, K] transposed."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.shape[0] <= SMALL_GEMM_MAX_ROWS and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library().zb_gemm_small_supported(x.shape[0], w.shape[0], x.shape[1])))


@dataclass(frozen=True)
class BoundedGate:
    """The bounded gate as a product's epilogue: with g = min(G + b_g, limit) and u = clamp(U + b_u, -limit,
    limit), g * sigmoid(alpha * g) * (u + shift).  ``bias`` is float32, one value per row of the packed weight
    (b_g and b_u where their rows are), or None."""
    bias: torch.Tensor | None
    limit: float
    alpha: float
    shift: float


def _bounded_args(bounded: BoundedGate, rows: int) -> tuple:
    _require(bounded.limit > 0.0, "the bounded gate needs a positive limit")
    _f32_vector(bounded.bias, rows, "the gate's bias")
    return _ptr(bounded.bias), float(bounded.limit), float(bounded.alpha), float(bounded.shift)


def gemm_small(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
               swiglu: bool = False, act: str = "silu", bounded: BoundedGate | None = None) -> torch.Tensor:
    """x [M <= 64, K] times w [N, K] transposed, bfloat16, float32 accumulation, weights read once.
    With ``swiglu`` the rows of w are blocks of 8 gate rows each followed by its 8 up rows, and the
    result is silu(gate) * up, [M, N / 2]; with ``bounded`` as well, the bounded gate of those sums."""
    _cuda(x, w)
    _require(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], "x [M, K] and w [N, K]")
    _require(gemm_small_supported(x, w), "gemm_small takes bfloat16, M <= 64, K a multiple of 8, 16-byte aligned rows")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    _require(not swiglu or N % 16 == 0, "swiglu needs a multiple of 16 rows")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    if bounded is not None:
        _require(swiglu, "the bounded gate is a gated epilogue")
        _cuda(bounded.bias)
        _check(library().zb_gemm_small_bounded(_ptr(out), _ptr(x), _ptr(w), *_bounded_args(bounded, N), M, N, K, x.stride(0),
                                               w.stride(0), out.stride(0), DTYPE_CODE[out_dtype], _stream()), "gemm_small")
        return out
    _check(library().zb_gemm_small(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                   DTYPE_CODE[out_dtype], (2 if act == "relu" else 1) if swiglu else 0, _stream()),
           "gemm_small")
    return out


GEMM_TC_MIN_ROWS = 512        # from here on the product with the activation in its epilogue beats the library's
                              # product followed by the activation kernel (measured at widths 1024 to 5120)


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> bool:
    """True if the tcgen05 product takes x [M, K] times w [N, K] transposed (bfloat16, K a multiple of 8)."""
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.shape[1] == w.shape[1] and x.stride(1) == 1 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return False
    M, K = x.shape
    N = w.shape[0]
    ldy = (N // 2 if swiglu else N + 7) // 8 * 8
    return bool(library().zb_gemm_tc_supported(M, N, K, x.stride(0), ldy, int(swiglu)))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False, block_n: int = 0,
            status: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, act: str = "silu",
            bounded: BoundedGate | None = None) -> torch.Tensor:
    """x [M, K] times w [N, K] transposed on tcgen05 tensor cores, bfloat16 with float32 sums in
    tensor memory; the result in bfloat16, or with ``out_dtype=torch.float32`` the sums as they are.
    With ``swiglu`` the rows of w are blocks of 8 gate rows each followed by its 8 up
    rows, and the result is silu(gate) * up, [M, N / 2], taken from the float32 sums and rounded once
    (with ``bounded`` as well: the bounded gate of those sums and their biases).
    ``block_n`` is the width of an output tile (256, 128; 2: tiles of 256 x 256 on pairs of SMs; 0: chosen).  ``status`` (default: the
    device's status word) receives a report if a wait inside the kernel ran out."""
    _cuda(x, w)
    _require(gemm_tc_supported(x, w, swiglu), "gemm_tc takes bfloat16 x [M, K] and contiguous w [N, K], K a multiple of 8, "
             "16-byte aligned; with swiglu N a multiple of 16")
    wide = out_dtype == torch.float32
    _require(out_dtype in (None, torch.bfloat16, torch.float32) and not (wide and swiglu), "bfloat16 out, or float32 without the activation")
    M, K = x.shape
    N = w.shape[0]
    width = N // 2 if swiglu else N
    ldy = (width + 3) // 4 * 4 if wide else (width + 7) // 8 * 8
    out = torch.empty((M, ldy), dtype=torch.float32 if wide else torch.bfloat16, device=x.device)
    if status is None:
        status = device_status(x.device)
    if bounded is not None:
        _require(swiglu, "the bounded gate is a gated epilogue")
        _cuda(bounded.bias)
        _check(library().zb_gemm_tc_bounded(_ptr(out), _ptr(x), _ptr(w), *_bounded_args(bounded, N), M, N, K, x.stride(0), ldy,
                                            int(block_n), _ptr(status), _stream()), "gemm_tc")
        return out if ldy == width else out[:, :width].contiguous()
    _require(act in ACTIVATIONS, f"the gate's activation is one of {sorted(ACTIVATIONS)}")
    gated = 3 if act == "relu" else 1         # the kernel's codes for the two gated epilogues
    _check(library().zb_gemm_tc(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), ldy, 2 if wide else (gated if swiglu else 0),
                                int(block_n), _ptr(status), _stream()), "gemm_tc")
    return out if ldy == width else out[:, :width].contiguous()


# ------------------------------------------------------------------ chains of small products
PROLOGUE_NONE, PROLOGUE_NORM, PROLOGUE_ADD_NORM = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1
FUSED_CHAIN_MAX_TOKENS = 16


class _ChainStage(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("ldw", c_longlong), ("N", c_int), ("K", c_int), ("prologue", c_int),
                ("epilogue", c_int), ("x", c_void_p), ("ldx", c_longlong), ("residual_in", c_void_p),
                ("residual_out", c_void_p), ("delta", c_void_p), ("ldd", c_longlong), ("norm_w", c_void_p),
                ("norm_w_dtype", c_int), ("eps", c_float), ("y", c_void_p), ("ldy", c_longlong)]


@dataclass
class ChainStage:
    """One stage of ``fused_chain``: y = epilogue(prologue(...) w^T), bfloat16.

    The input is ``x`` [M, K] as given, or, with ``norm_w``, the RMS norm of ``residual_in`` [M, K]
    (after ``delta`` [M, K] has been added to it, if given; the sum goes to ``residual_out``).  With
    ``swiglu`` the rows of ``w`` are blocks of 8 gate rows and their 8 up rows and y is [M, N / 2]."""

    w: torch.Tensor
    y: torch.Tensor
    x: torch.Tensor | None = None
    residual_in: torch.Tensor | None = None
    residual_out: torch.Tensor | None = None
    delta: torch.Tensor | None = None
    norm_w: torch.Tensor | None = None
    eps: float = 0.0
    swiglu: bool = False

    @property
    def prologue(self) -> int:
        if self.norm_w is None:
            return PROLOGUE_NONE
        return PROLOGUE_ADD_NORM if self.delta is not None else PROLOGUE_NORM


def fused_chain_stage_supported(tokens: int, w: torch.Tensor, normed_input: bool, swiglu: bool) -> bool:
    """True if a product with ``w`` [N, K] can be a stage of a chain for this many tokens."""
    return (w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.data_ptr() % 16 == 0
            and bool(library().zb_fused_chain_stage_supported(int(tokens), w.shape[0], w.shape[1],
                                                              PROLOGUE_NORM if normed_input else PROLOGUE_NONE,
                                                              EPILOGUE_SWIGLU if swiglu else EPILOGUE_NONE)))


def fused_chain_max_stages() -> int:
    return int(library().zb_fused_chain_max_stages())


# The arrival counters of the chain kernel's barrier, per device: zero between launches.
_chain_sync: dict[tuple[torch.device, int], torch.Tensor] = {}
_chain_rows: dict[tuple[torch.device, int], torch.Tensor] = {}


def set_dependent_launch(enabled: bool) -> bool:
    """Launch the kernels of a decode step (position encoding with cache write, decode attention,
    chain) as programmatic dependents of the kernel before them: a kernel's CTAs then set themselves
    up while the one before is still finishing.  On by default; returns the previous setting."""
    return bool(library().zb_set_dependent_launch(int(bool(enabled))))


def fused_chain_grid() -> int:
    """CTAs of a chain launch (one per SM)."""
    return int(library().zb_fused_chain_grid())


def fused_chain(stages: Sequence[ChainStage], tokens: int, status: torch.Tensor,
                trace: torch.Tensor | None = None) -> None:
    """Run the stages one after the other in one cooperative launch (see csrc/fused_chain.cu).
    Every tensor is bfloat16 on the device (a norm weight may be float32); rows are contiguous.
    ``trace`` (int32 [fused_chain_grid(), stages, 4]) receives every CTA's timeline, nanoseconds of
    the device's global timer (low 32 bits): the stage's start, its input in place, its products
    done, the barrier passed."""
    _require(1 <= len(stages) <= fused_chain_max_stages(), "a chain has 1 to 8 stages")
    _require(1 <= tokens <= FUSED_CHAIN_MAX_TOKENS, "a chain takes 1 to 16 tokens")
    packed = (_ChainStage * len(stages))()
    for slot, st in zip(packed, stages):
        N, K = st.w.shape
        _cuda(st.w, st.y, st.x, st.residual_in, st.residual_out, st.delta, st.norm_w)
        for t in (st.w, st.y, st.x, st.residual_in, st.residual_out, st.delta):
            _require(t is None or (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1), "bfloat16 matrices")
        _require(st.y.shape == (tokens, N // 2 if st.swiglu else N), "y must be [tokens, N] ([tokens, N / 2] with swiglu)")
        slot.w, slot.ldw, slot.N, slot.K = st.w.data_ptr(), st.w.stride(0), N, K
        slot.prologue, slot.epilogue = st.prologue, EPILOGUE_SWIGLU if st.swiglu else EPILOGUE_NONE
        slot.y, slot.ldy = st.y.data_ptr(), st.y.stride(0)
        if st.norm_w is None:
            _require(st.x is not None and st.x.shape == (tokens, K), "x must be [tokens, K]")
            slot.x, slot.ldx = st.x.data_ptr(), st.x.stride(0)
        else:
            _require(st.residual_in is not None and st.residual_in.shape == (tokens, K) and st.residual_in.is_contiguous(),
                     "residual_in must be contiguous [tokens, K]")
            _require(st.norm_w.numel() == K and st.norm_w.dtype in DTYPE_CODE and st.norm_w.is_contiguous(), "norm weight [K]")
            slot.residual_in, slot.norm_w = st.residual_in.data_ptr(), st.norm_w.data_ptr()
            slot.norm_w_dtype, slot.eps = DTYPE_CODE[st.norm_w.dtype], float(st.eps)
            if st.delta is not None:
                _require(st.delta.shape == (tokens, K), "delta must be [tokens, K]")
                _require(st.residual_out is not None and st.residual_out.shape == (tokens, K)
                         and st.residual_out.is_contiguous() and st.residual_out.data_ptr() != st.residual_in.data_ptr(),
                         "residual_out must be a second contiguous [tokens, K] buffer")
                slot.delta, slot.ldd, slot.residual_out = st.delta.data_ptr(), st.delta.stride(0), st.residual_out.data_ptr()
    device = (stages[0].w.device, LANE)
    sync = _chain_sync.get(device)
    if sync is None:
        sync = _chain_sync[device] = torch.zeros(2, dtype=torch.int32, device=stages[0].w.device)
    if trace is not None:
        _cuda(trace)
        _require(trace.dtype == torch.int32 and trace.is_contiguous()
                 and trace.numel() >= 4 * len(stages) * fused_chain_grid(), "trace must be int32 [fused_chain_grid(), stages, 4]")
    # Room for the rows of a long normalised input, which the kernel normalises once for all CTAs.
    longest = max((st.w.shape[1] for st in stages if st.norm_w is not None), default=0)
    scratch = _chain_rows.get(device)
    if longest and (scratch is None or scratch.numel() < FUSED_CHAIN_MAX_TOKENS * longest):
        scratch = _chain_rows[device] = torch.empty(FUSED_CHAIN_MAX_TOKENS * longest, dtype=torch.bfloat16,
                                                    device=stages[0].w.device)
    _check(library().zb_fused_chain(ctypes.addressof(packed), len(stages), int(tokens), _ptr(sync), _ptr(status),
                                    _ptr(trace), _ptr(scratch) if longest else None, _stream()), "fused_chain")


USE_LIBRARY_PRODUCTS = True     # off: every bfloat16 product of more than a few rows runs on this package's tcgen05 kernel


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x w^T.  float32 runs on this package's CUDA-core kernel (no TF32 anywhere).  bfloat16
    with up to 64 rows (a decode step) runs on this package's weight-streaming kernel; larger
    bfloat16 products run on the vendor library's tensor-core product, as the reference's linear
    layers do (src/layer/linear.cpp:22-24 -> cuBLASLt), where that is the faster one; with
    ``USE_LIBRARY_PRODUCTS`` off they run on this package's tcgen05 kernel (``gemm_tc``), so that no
    library kernel is left on the path.  Accumulation is float32 everywhere.  A ``bias`` [N] is
    added to the product's (rounded) output by a kernel of its own."""
    if bias is not None:
        return add_bias(linear(x, w, out_dtype), bias)
    _cuda(x, w)
    if x.dtype == torch.float32:
        return gemm_nt_simt(x, w, out_dtype)
    if x.shape[0] <= SMALL_GEMM_ROWS and gemm_small_supported(x, w):
        return gemm_small(x, w, out_dtype)
    if not USE_LIBRARY_PRODUCTS and gemm_tc_supported(x, w):
        return gemm_tc(x, w, out_dtype=out_dtype)
    if out_dtype is None or out_dtype == x.dtype:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# ------------------------------------------------------------- products per head and per expert
def head_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                gate: torch.Tensor | None = None, x_head_stride: int | None = None,
                out: torch.Tensor | None = None, out_head_stride: int | None = None, walk: int = 0) -> torch.Tensor:
    """y[t, h, :] = w[h] x[t, h, :] for x [T, heads * K] (unit inner stride) and w [heads, N, K]: a product
    that is block-diagonal over heads; returns [T, heads * N] in ``out_dtype`` (default: w's type).  x may be
    float32 beside bfloat16 matrices.  ``gate`` (float32, unit inner stride): [T, >= heads] multiplies head
    h's output by sigmoid(gate[t, h]); [T, heads * N] multiplies every output value by the logistic function
    of its own gate value.  float32 sums in the order of k.

    ``x_head_stride``: head h's K inputs start at x[t, h * x_head_stride] (heads that are slices of wider
    ones; x is then [T, >= heads * x_head_stride]).  ``out`` with ``out_head_stride``: head h's N outputs go
    to out[t, h * out_head_stride ...] of a given [T, heads * out_head_stride] tensor, the rest of which is
    left as it is.  ``walk``: which bfloat16 kernel runs where rows start on 16-byte boundaries and K is a
    multiple of 16: 0 by the row count, 1 the walk along k in steps, 2 and 3 all of K at once with 32 and 64
    rows a CTA (the sums are the same to the bit)."""
    _cuda(x, w, gate, out)
    heads, N, K = w.shape
    xhs = K if x_head_stride is None else int(x_head_stride)
    _require(x.dim() == 2 and xhs >= K and x.shape[1] >= (heads - 1) * xhs + K and x.stride(1) == 1
             and w.is_contiguous() and x.dtype in (w.dtype, torch.float32) and w.dtype in DTYPE_CODE,
             "x [T, heads * K] in w's type or float32, and w [heads, N, K]")
    per_element = gate is not None and gate.shape[1] == heads * N and N > 1
    _require(gate is None or (gate.dtype == torch.float32 and gate.dim() == 2 and gate.shape[0] == x.shape[0]
                              and gate.shape[1] >= heads and gate.stride(1) == 1),
             "one float32 gate per token and head, or per token and output value")
    yhs = N if out_head_stride is None else int(out_head_stride)
    if out is None:
        _require(yhs == N, "a head stride of the output needs the output tensor")
        out = torch.empty((x.shape[0], heads * N), dtype=out_dtype or w.dtype, device=x.device)
    _require(out.dim() == 2 and out.shape[0] == x.shape[0] and out.stride(1) == 1 and yhs >= N
             and out.shape[1] >= (heads - 1) * yhs + N and out.dtype in DTYPE_CODE, "out [T, heads * out_head_stride]")
    _check(library().zb_head_linear_strided(_ptr(out), _ptr(x), _ptr(w), _ptr(gate), x.stride(0), out.stride(0),
                                            gate.stride(0) if gate is not None else 0, xhs, yhs, int(per_element),
                                            x.shape[0], heads, N, K, DTYPE_CODE[x.dtype], DTYPE_CODE[w.dtype],
                                            DTYPE_CODE[out.dtype], int(walk), _stream()), "head_linear")
    return out


def route_max_outputs() -> int:
    return library().zb_route_max_outputs()


ROUTE_SCORES = {"softmax": 0, "sigmoid": 1, "top_softmax": 2}


def route(logits: torch.Tensor, correction: torch.Tensor | None, top: int, scores: str = "softmax",
          groups: tuple[int, int, int] | None = None, weight_scale: float = 1.0,
          logit_bias: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Token-choice routing: s = softmax(logits) over all outputs (``scores`` "sigmoid": the logistic function
    of each logit on its own); the ``top`` outputs with the largest s + correction are taken (ties: the lower
    index), each with the weight s * ``weight_scale``.  ``groups`` = (count, keep, group_top): the outputs
    form ``count`` equal runs of neighbours, a run's mark is the sum of its ``group_top`` largest choice
    values, and only outputs of the ``keep`` runs with the largest marks can be taken.  ``logit_bias``
    (float32 [outputs]) is added to the logits before anything else.  ``scores`` "top_softmax": the ``top``
    largest logits are taken and weigh their outputs by the softmax over the taken logits only.  Returns
    (ids int32 [T, top], weights float32 [T, top]), in the order of choice."""
    _cuda(logits, correction, logit_bias)
    _f32_vector(logit_bias, logits.shape[1], "the logits' bias")
    _require(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1, "float32 logits [T, outputs]")
    _require(scores in ROUTE_SCORES, f"router scores are one of {sorted(ROUTE_SCORES)}")
    T, outputs = logits.shape
    _f32_vector(correction, outputs, "the correction")
    count, keep, group_top = (int(v) for v in groups) if groups is not None else (1, 1, 1)
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(library().zb_route_biased(_ptr(ids), _ptr(weights), _ptr(logits), logits.stride(0), _ptr(correction), T,
                                     outputs, int(top), ROUTE_SCORES[scores], count, keep, group_top,
                                     float(weight_scale), _ptr(logit_bias), _stream()), "route")
    return ids, weights


GROUPED_TILE_ROWS = 128        # rows of a tile of the tcgen05 product
GROUPED_MIN_ROWS_PER_EXPERT = 0    # the grouped tcgen05 products from this many choices per expert on (on average)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[E, ff, width] twice -> [E, 2 ff, width] in blocks of 8 gate rows each followed by its 8 up rows
    (ff a multiple of 8): the layout whose product can apply act(gate) * up where the sums leave the tensor
    cores."""
    E, ff, width = w_gate.shape
    return torch.stack([w_gate.view(E, ff // 8, 8, width), w_up.view(E, ff // 8, 8, width)], dim=2).reshape(E, 2 * ff, width).contiguous()


def routed_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate: torch.Tensor,
                   w_up: torch.Tensor | None, w_down: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """sum_j weights[t, j] * expert_{ids[t, j]}(x[t]) for x [T, width]: expert e < E is
    w_down[e] (act(w_gate[e] x) * (w_up[e] x)) with w_gate, w_up [E, ff, width] and w_down [E, width, ff]; an
    id >= E names an identity expert, whose output is x itself.  Without ``w_up``, ``w_gate`` holds both
    matrices as ``interleave_gate_up`` lays them out.  The tokens are sorted by expert on the device and
    nothing comes back to the host: alignment, the two products (gate/up with the activation, down) and the
    weighted sum.  bfloat16 with many tokens per expert and the interleaved layout: each product is ONE
    grouped launch of the tcgen05 kernel over runs padded to whole tiles; otherwise tiles on mma.sync
    (bfloat16) or CUDA cores (float32)."""
    _cuda(x, ids, weights, w_gate, w_up, w_down)
    T, width = x.shape
    top = ids.shape[1]
    interleaved = w_up is None
    E = w_gate.shape[0]
    ff = w_gate.shape[1] // 2 if interleaved else w_gate.shape[1]
    _require(x.stride(1) == 1 and x.dtype in DTYPE_CODE and all(w is None or (w.dtype == x.dtype and w.is_contiguous())
             for w in (w_gate, w_up, w_down)), "tokens and expert matrices of one type")
    _require(w_gate.shape == ((E, 2 * ff, width) if interleaved else (E, ff, width)) and (interleaved or w_up.shape == (E, ff, width))
             and w_down.shape == (E, width, ff) and (not interleaved or ff % 8 == 0),
             "expert matrices [E, ff, width] (or [E, 2 ff, width] interleaved), [E, width, ff]")
    _require(act in ACTIVATIONS, f"the gate's activation is one of {sorted(ACTIVATIONS)}")
    _i32(ids)
    _require(weights.dtype == torch.float32 and weights.is_contiguous() and weights.shape == ids.shape, "one weight per choice")
    lib, device = library(), x.device
    num_slots = T * top
    code = DTYPE_CODE[x.dtype]
    out = torch.empty((T, width), dtype=x.dtype, device=device)
    place = torch.empty(max(num_slots, 1), dtype=torch.int32, device=device)
    grouped = (USE_GROUPED_TCGEN05 and interleaved and x.dtype == torch.bfloat16 and width % 8 == 0 and x.stride(0) % 8 == 0
               and num_slots >= GROUPED_MIN_ROWS_PER_EXPERT * E)
    if grouped:
        tiles = -(-num_slots // GROUPED_TILE_ROWS) + E
        places = tiles * GROUPED_TILE_ROWS
        tile_group = torch.empty(tiles, dtype=torch.int32, device=device)
        slots = torch.empty(places, dtype=torch.int32, device=device)
        _check(lib.zb_route_align_padded(_ptr(tile_group), _ptr(slots), _ptr(place), _ptr(ids), num_slots, E, tiles,
                                         GROUPED_TILE_ROWS, _stream()), "route_align")
        rows = torch.empty((places, width), dtype=x.dtype, device=device)
        _check(lib.zb_gather_places(_ptr(rows), _ptr(x), x.stride(0), _ptr(slots), places, width, top, _stream()),
               "gather_places")
        status = device_status(device)
        hidden = torch.empty((places, ff), dtype=x.dtype, device=device)
        _check(lib.zb_gemm_tc_grouped(_ptr(hidden), _ptr(rows), _ptr(w_gate), _ptr(tile_group), tiles, E, 2 * ff, width, width,
                                      ff, 3 if act == "relu" else 1, _ptr(status), _stream()), "gemm_tc_grouped")
        # An expert's output takes the model's type before it is weighted on every path: here the product writes it so.
        ldy = width
        y = torch.empty((places, ldy), dtype=x.dtype, device=device)
        _check(lib.zb_gemm_tc_grouped(_ptr(y), _ptr(hidden), _ptr(w_down), _ptr(tile_group), tiles, E, width, ff, ff, ldy, 0,
                                      _ptr(status), _stream()), "gemm_tc_grouped")
    else:
        tile_rows = lib.zb_expert_tile_rows(code)          # CUDA-core tiles in float32, tensor-core tiles in bfloat16
        max_tiles = -(-num_slots // tile_rows) + E
        plan = torch.empty(1 + 3 * max_tiles, dtype=torch.int32, device=device)
        slots = torch.empty(max(num_slots, 1), dtype=torch.int32, device=device)
        _check(lib.zb_route_align(_ptr(plan), _ptr(slots), _ptr(place), _ptr(ids), num_slots, E, max_tiles, tile_rows,
                                  _stream()), "route_align")
        hidden = torch.empty((max(num_slots, 1), ff), dtype=x.dtype, device=device)
        ldy = width
        y = torch.empty((max(num_slots, 1), width), dtype=torch.float32, device=device)
        _check(lib.zb_expert_product(_ptr(hidden), _ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(plan), _ptr(slots),
                                     max_tiles, ff, width, top, ACTIVATIONS[act], 0, code, _stream()), "expert_product")
        _check(lib.zb_expert_product(_ptr(y), _ptr(hidden), ff, _ptr(w_down), None, _ptr(plan), _ptr(slots), max_tiles,
                                     width, ff, top, ACTIVATIONS[act], 1, code, _stream()), "expert_product")
    _check(lib.zb_route_combine(_ptr(out), _ptr(y), ldy, DTYPE_CODE[y.dtype], _ptr(x), x.stride(0), _ptr(ids), _ptr(weights),
                                _ptr(place), T, width, top, code, _stream()), "route_combine")
    return out


USE_GROUPED_TCGEN05 = True      # off: a routed layer's products stay on the mma.sync tiles whatever the token count


# ------------------------------------------------------------------------------ sampling
@dataclass(frozen=True)
class SampleRow:
    """How one row of logits is turned into a token (the kernel's record of a row).

    ``temperature`` below 1e-7 means greedy.  ``top_k`` 0, ``top_p`` 0 and ``min_p`` 0 switch those
    filters off.  ``num_logprobs`` -1 asks for no report; n >= 0 for the chosen token's
    log-probability and the n most probable tokens."""

    temperature: float = 0.0
    uniform: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    min_p: float = 0.0
    num_logprobs: int = -1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-7

    @property
    def ranked(self) -> bool:
        return not self.greedy and (self.top_k > 0 or self.top_p > 0.0)


@dataclass(frozen=True)
class TokenAdjustment:
    """What a row's history and biases do to one token's logit."""

    row: int
    token: int
    generated_count: int = 0
    seen: bool = False
    bias: float = 0.0


@dataclass
class SampleOutput:
    """Device results of ``sample_rows``: row r's chosen token is ``ids[offsets[r]]``, followed by its
    top tokens if it reports; ``logprobs`` runs parallel to ``ids`` (None if no row reports)."""

    ids: torch.Tensor
    logprobs: torch.Tensor | None
    offsets: list[int]


_ROW_FORMAT = struct.Struct("<dddffffiiiiii")
_ADJUSTMENT_FORMAT = struct.Struct("<iiiif")
_JOB_FORMAT = struct.Struct("<ii")
_PHASE_WEIGHTS, _PHASE_DRAW_INDEXED, _PHASE_DRAW_RANKED, _PHASE_REPORT = 1, 2, 4, 8

# Work buffers of the sampling kernels, kept per device and only ever grown.  The counters are zero
# between calls: the kernel leaves them as it found them.
_sample_buffers: dict[tuple[torch.device, str], torch.Tensor] = {}


def _sample_buffer(device: torch.device, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
    have = _sample_buffers.get((device, name))
    if have is None or have.numel() < numel:
        size = max(numel, 1024)
        have = (torch.zeros if zero else torch.empty)(size, dtype=dtype, device=device)
        _sample_buffers[(device, name)] = have
    return have


def sample_chunks(vocab: int) -> int:
    return int(library().zb_sample_chunks(int(vocab)))


def sample_rows(logits: torch.Tensor, rows: Sequence[SampleRow] | None, status: torch.Tensor,
                adjustments: Sequence[TokenAdjustment] = ()) -> SampleOutput:
    """One token per row of float32 logits [rows, V], chosen as each row's ``SampleRow`` says
    (``rows`` None: argmax everywhere).  Adjustments are applied to ``logits`` in place first."""
    _cuda(logits, status)
    _require(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
             "logits must be float32 [rows, V]")
    R, V = logits.shape
    device = logits.device
    chunks = sample_chunks(V)
    part_f = _sample_buffer(device, "part_f", 3 * R * chunks, torch.float32)
    part_i = _sample_buffer(device, "part_i", R * chunks, torch.int32)
    counters = _sample_buffer(device, "counters", R, torch.int32, zero=True)
    row_max = _sample_buffer(device, "row_max", R, torch.float32)
    row_arg = _sample_buffer(device, "row_arg", R, torch.int32)
    if rows is None:
        _require(not adjustments, "adjustments need row parameters")
        ids = torch.empty(R, dtype=torch.int32, device=device)
        _check(library().zb_sample(_ptr(ids), None, _ptr(logits), logits.stride(0), R, V, None, None, 0, None, 0, 0,
                                   _ptr(part_f), _ptr(part_i), _ptr(counters), _ptr(row_max), _ptr(row_arg), None,
                                   None, None, None, _ptr(status), _stream()), "sample")
        return SampleOutput(ids, None, list(range(R)))
    _require(len(rows) == R, "one SampleRow per row of logits")

    # Pack the rows, the sort jobs they need and the adjustments into one upload.
    jobs: list[tuple[int, int]] = []
    offsets: list[int] = []
    packed_rows = bytearray()
    results, phases = 0, 0
    for r, row in enumerate(rows):
        sort_slot = report_slot = -1
        if not row.greedy or row.num_logprobs >= 0:
            phases |= _PHASE_WEIGHTS
        if row.ranked:
            sort_slot = len(jobs)
            jobs.append((r, 0))
            phases |= _PHASE_DRAW_RANKED
        elif not row.greedy:
            phases |= _PHASE_DRAW_INDEXED
        num_logprobs = min(int(row.num_logprobs), V)
        if num_logprobs >= 0:
            phases |= _PHASE_REPORT
            if num_logprobs > 0:
                report_slot = len(jobs)
                jobs.append((r, 1))
        offsets.append(results)
        packed_rows += _ROW_FORMAT.pack(row.temperature, row.top_p, row.min_p, row.uniform, row.frequency_penalty,
                                        row.presence_penalty, row.repetition_penalty, min(int(row.top_k), V),
                                        num_logprobs, results, sort_slot, report_slot, 0)
        results += 1 + max(num_logprobs, 0)
    for a in adjustments:
        _require(0 <= a.row < R and 0 <= a.token < V, "an adjustment names a row and a token of the logits")
    packed_adjustments = b"".join(_ADJUSTMENT_FORMAT.pack(a.row, a.token, a.generated_count, int(a.seen), a.bias)
                                  for a in adjustments)
    packed_jobs = b"".join(_JOB_FORMAT.pack(*job) for job in jobs)
    at_adjustments = len(packed_rows)
    at_jobs = (at_adjustments + len(packed_adjustments) + 15) // 16 * 16
    blob = bytes(packed_rows) + packed_adjustments + bytes(at_jobs - at_adjustments - len(packed_adjustments)) + packed_jobs
    host = torch.frombuffer(bytearray(blob), dtype=torch.uint8).pin_memory()
    uploaded = host.to(device, non_blocking=True)
    base = uploaded.data_ptr()

    ids = torch.empty(results, dtype=torch.int32, device=device)
    logprobs = torch.zeros(results, dtype=torch.float32, device=device) if phases & _PHASE_REPORT else None
    weights = _sample_buffer(device, "weights", R * V, torch.float32) if phases else None
    sort_keys = _sample_buffer(device, "sort_keys", 2 * len(jobs) * V, torch.int32) if jobs else None
    sort_idx = _sample_buffer(device, "sort_idx", 2 * len(jobs) * V, torch.int32) if jobs else None
    job_state = _sample_buffer(device, "job_state", 4 * len(jobs), torch.int32) if jobs else None
    _check(library().zb_sample(
        _ptr(ids), _ptr(logprobs), _ptr(logits), logits.stride(0), R, V, base,
        base + at_adjustments if adjustments else None, len(adjustments), base + at_jobs if jobs else None, len(jobs),
        phases, _ptr(part_f), _ptr(part_i), _ptr(counters), _ptr(row_max), _ptr(row_arg), _ptr(weights),
        _ptr(sort_keys), _ptr(sort_idx), _ptr(job_state), _ptr(status), _stream()),
        "sample", kernels=1 + bool(adjustments) + 3 * bool(jobs) + bin(phases).count("1"))
    _sample_buffers[(device, "jobs_of_last_call")] = len(jobs)
    return SampleOutput(ids, logprobs, offsets)


def last_sample_job_state(device: torch.device | str | None = None) -> list[tuple[int, bool]]:
    """For every ranking of the last ``sample_rows`` call on ``device``, in the order of the rows (a
    row's draw before its report): how many ranks were sorted, and whether the head of the order was
    enough.  Reads from the device; for tests and timing."""
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    count = _sample_buffers.get((device, "jobs_of_last_call"), 0)
    if not count:
        return []
    state = _sample_buffers[(device, "job_state")][:4 * count].cpu().view(count, 4).tolist()
    return [(int(n), bool(done)) for n, done, _, _ in state]


def sample(logits: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """The argmax of every row of float32 logits, the lowest index among equal maxima."""
    return sample_rows(logits, None, status).ids
