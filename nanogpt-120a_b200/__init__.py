"""Host-side mirror of the reference's NVFP4 projection-path modules on top of the C ABI.

The product is `libnvfp4_b200.so` (hand-written sm_100a kernels behind `extern "C"`
entry points, declared in include/nvfp4_b200.h).  This package binds it with ctypes and
mirrors the reference's per-op module structs (`Nvfp4QuantModule`, `Nvfp4GemmModule`,
`Sm120ScalePackModule`, `Nvfp4DecodeModule`, `ProjectionPostOpModule`,
`LinearBackwardModule`, crates/cuda-kernels/src/lib.rs:80-92) with the same method names
and argument meaning.  PyTorch only provides device memory and streams: every method takes
torch CUDA tensors, passes raw pointers and enqueues on the current stream.

There is no CPU path: importing works anywhere, but every operation raises if the
library is missing or no CUDA device is present.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_size_t, c_uint8, c_uint32, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnvfp4_b200.so")

DTYPE_F32, DTYPE_BF16 = 0, 1
SCALES_LOGICAL, SCALES_PACKED = 0, 1
GS_NONE, GS_TENSOR, GS_ROWWISE_A = 0, 1, 2
EPI_NONE, EPI_BIAS, EPI_RELU2, EPI_RESIDUAL = 0, 1, 2, 3
SRC_F32_ROWS, SRC_F32_TRANSPOSED, SRC_NVFP4_TRANSPOSED, SRC_ROWWISE_NVFP4_TRANSPOSED = 0, 1, 2, 3

QUARTET_MS_EDEN_SCALE_OVERRIDE = float(torch.tensor(17.0 / 16.0, dtype=torch.float32) * torch.tensor(0.93, dtype=torch.float32))


class Nvfp4Error(RuntimeError):
    """A C-ABI call returned a non-zero CUDA error number (the reference's DriverError)."""

    def __init__(self, code: int, text: str):
        super().__init__(f"nvfp4 call failed with CUDA error {code}: {text}")
        self.code = code


class MsEdenArgs(Structure):
    _fields_ = [
        ("src_kind", c_int), ("src_dtype", c_int), ("x", c_void_p), ("src_bytes", c_void_p),
        ("src_scales", c_void_p), ("src_scale_layout", c_int), ("src_global", c_void_p), ("rows", c_uint32),
        ("cols", c_uint32),
        ("dst_row_len", c_uint32), ("global_scale", c_void_p), ("host_global_scale", c_float),
        ("host_global_scale_valid", c_int), ("scale_override", c_float), ("sign_seed", c_uint32),
        ("scale_seed", c_uint32), ("col_offset", c_uint32), ("group_offset", c_uint32), ("group_row_stride", c_uint32),
        ("out_fp4", c_void_p),
        ("out_scales", c_void_p), ("scale_layout", c_int), ("out_global_scales", c_void_p),
        ("out_chunk_amax", c_void_p),
    ]


class GemmArgs(Structure):
    _fields_ = [
        ("a_bytes", c_void_p), ("a_scales", c_void_p), ("a_global", c_void_p), ("b_bytes", c_void_p),
        ("b_scales", c_void_p), ("b_global", c_void_p), ("out", c_void_p), ("aux", c_void_p), ("bias", c_void_p),
        ("m", c_uint32), ("n", c_uint32), ("k", c_uint32), ("ldo", c_uint32), ("global_scale_mode", c_int),
        ("weight_global_scale", c_float), ("epilogue", c_int), ("out_dtype", c_int),
        ("bias_nvfp4_bytes", c_void_p), ("bias_nvfp4_scales", c_void_p), ("bias_nvfp4_global", c_void_p),
        ("relu2_row_amax", c_void_p),
    ]


class GemmPlan(Structure):
    """nvfp4_gemm_plan: what the library chooses for one GEMM (tile width, schedule, launch shape)."""
    _fields_ = [("block_m", c_uint32), ("block_n", c_uint32), ("acc_stages", c_uint32), ("k_splits", c_uint32), ("b_resident", c_uint32),
                ("resident_cpn", c_uint32), ("stages", c_uint32), ("grid", c_uint32), ("tma_store", c_uint32),
                ("smem_bytes", c_uint32)]


class ProjectionArgs(Structure):
    _fields_ = [
        ("input_bytes", c_void_p), ("input_scales", c_void_p), ("input_scale_layout", c_int),
        ("input_global_scales", c_void_p), ("weight_bytes", c_void_p), ("weight_scales", c_void_p),
        ("weight_scale_layout", c_int), ("weight_global_scale", c_void_p), ("bias_bytes", c_void_p),
        ("bias_scales", c_void_p), ("bias_global_scale", c_void_p), ("out", c_void_p), ("pre_activation", c_void_p),
        ("out_dtype", c_int), ("relu2_row_amax", c_void_p), ("token_count", c_uint32), ("input_dim", c_uint32),
        ("output_dim", c_uint32), ("input_scales_packed_scratch", c_void_p), ("weight_scales_packed_scratch", c_void_p),
    ]


class BackwardOperand(Structure):
    _fields_ = [("bytes", c_void_p), ("scales", c_void_p), ("scale_layout", c_int), ("global_scales", c_void_p),
                ("scales_packed_scratch", c_void_p)]


class LinearBackwardDeviceScaleArgs(Structure):
    _fields_ = [("e_h", BackwardOperand), ("weight_t_h", BackwardOperand), ("e_t_h", BackwardOperand),
                ("input_t_h", BackwardOperand), ("dinput", c_void_p), ("dinput_dtype", c_int), ("dweight", c_void_p),
                ("dweight_dtype", c_int), ("token_count", c_uint32), ("input_dim", c_uint32), ("output_dim", c_uint32)]


class MsEdenOperand(Structure):
    _fields_ = [("bytes", c_void_p), ("scales_packed", c_void_p), ("global_scales", c_void_p),
                ("global_scale", c_void_p), ("chunk_amax", c_void_p)]


class LinearBackwardArgs(Structure):
    _fields_ = [
        ("e", c_void_p), ("e_dtype", c_int), ("w_bytes", c_void_p), ("w_scales", c_void_p), ("w_scale_layout", c_int),
        ("w_global", c_void_p), ("x_bytes", c_void_p), ("x_scales", c_void_p), ("x_scale_layout", c_int),
        ("x_globals", c_void_p), ("e_h", MsEdenOperand),
        ("e_t_h", MsEdenOperand), ("weight_t_h", MsEdenOperand), ("input_t_h", MsEdenOperand), ("dinput", c_void_p),
        ("dinput_dtype", c_int), ("dweight", c_void_p), ("dweight_dtype", c_int), ("dbias", c_void_p), ("token_count", c_uint32),
        ("input_dim", c_uint32), ("output_dim", c_uint32), ("sign_seed", c_uint32), ("scale_seed", c_uint32),
        ("precomputed_e_amax_chunks", c_uint32), ("token_offset", c_uint32), ("e_global_scale_override", c_void_p),
        ("x_decoded_amax", c_void_p), ("side_stream", c_void_p), ("fork_event", c_void_p), ("join_event", c_void_p),
        ("total_token_count", c_uint32), ("weight_t_prepared", c_int),
    ]


class CheckpointTensorInfo(Structure):
    """`nvfp4_checkpoint_tensor_info`."""
    _fields_ = [("name", ctypes.c_char * 256), ("len", ctypes.c_uint64), ("byte_len", ctypes.c_uint64),
                ("scale_len", ctypes.c_uint64), ("global_scale", c_float)]


_P, _U, _F = c_void_p, c_uint32, c_float
# name -> argument ctypes (all return int unless listed in _SPECIAL_RESTYPE)
_SIGNATURES = {
    "nvfp4_read_device_status": [_P, POINTER(c_uint32)],
    "nvfp4_row_amax_f32": [_P, _P, _P, _U, _U],
    "nvfp4_row_amax_bf16": [_P, _P, _P, _U, _U],
    "nvfp4_tensor_amax_f32": [_P, _P, _P, _P, ctypes.c_uint64],
    "nvfp4_tensor_amax_bf16": [_P, _P, _P, _P, ctypes.c_uint64],
    "nvfp4_tensor_amax_from_chunks_f32": [_P, _P, _P, _U],
    "nvfp4_tensor_amax_f32_static_scratch": [_P, _P, _P, ctypes.c_uint64],
    "nvfp4_fp32_to_nvfp4_four_six": [_P, _P, _P, _P, _P, _P, _U],
    "nvfp4_fp32_to_nvfp4_four_six_rowwise": [_P, _P, _P, _P, _P, _P, _U, _U],
    "nvfp4_fp32_to_nvfp4_four_six_padded": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _U],
    "nvfp4_fp32_transpose_to_nvfp4_four_six_padded": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _U],
    "nvfp4_quantize_four_six": [_P, _P, c_int, _P, c_int, _U, _U, _P, _P, c_int, _P],
    "nvfp4_quantize_four_six_rowwise_fused": [_P, _P, c_int, _U, _U, _P, _P, c_int, _P, _P, _P],
    "nvfp4_quantize_relu2_four_six_rowwise": [_P, _P, c_int, _U, _U, _P, _P, _P, c_int, _P, _P, _P],
    "nvfp4_tc_matmul_ms_eden": [_P, _P, _P, _P, POINTER(MsEdenOperand), _F, POINTER(MsEdenOperand), _F, _U, _U, _U, _U, _U],
    "nvfp4_relu2_backward": [_P, _P, _P, _P, _U],
    "nvfp4_relu2_backward_f16": [_P, _P, _P, _P, _U],
    "nvfp4_relu2_backward_bf16": [_P, _P, _P, _P, ctypes.c_uint64],
    "nvfp4_relu2_backward_amax": [_P, _P, c_int, _P, _P, c_int, ctypes.c_uint64, _P, _U, POINTER(c_uint32)],
    "nvfp4_materialize_schedule_free": [_P, _P, _P, _P, _P, _P, _P, _P, _F, _U],
    "nvfp4_materialize_schedule_free_matrix": [_P, _P, _P, _P, _P, _P, _P, c_int, _P, _F, _U, _U],
    "nvfp4_ms_eden_quantize": [_P, POINTER(MsEdenArgs)],
    "nvfp4_fp32_to_nvfp4_ms_eden": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _F, _F, _U, _U],
    "nvfp4_fp32_to_nvfp4_ms_eden_device_scale": [_P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _F, _U, _U],
    "nvfp4_fp32_to_nvfp4_ms_eden_device_scale_no_chunk_amax": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _F, _U, _U],
    "nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale": [_P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _F, _U, _U],
    "nvfp4_fp32_transpose_to_nvfp4_ms_eden_device_scale_no_chunk_amax": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _F, _U, _U],
    "nvfp4_quartet_backward_ms_eden_global_scale_from_chunks": [_P, _P, _P, _U],
    "nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale": [_P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U],
    "nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax": [_P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U],
    "nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_with_global_scale": [_P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _F],
    "nvfp4_fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax":
        [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _U, _U, _U],
    "nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale": [_P] * 9 + [_U] * 5,
    "nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax": [_P] * 9 + [_U] * 5,
    "nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale": [_P] * 9 + [_U] * 5,
    "nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax": [_P] * 9 + [_U] * 5,
    "nvfp4_decode_transpose_f32": [_P, _P, _P, _P, _P, _U, _U],
    "nvfp4_decode_rowwise_transpose_f32": [_P, _P, _P, _P, _P, _U, _U],
    "nvfp4_decode_f32": [_P, _P, _P, _P, c_int, _P, _U, _U],
    "nvfp4_scale_pack": [_P, _P, _P, _U, _U],
    "nvfp4_pad_u4_rows": [_P, _P, _P, _U, _U, _U],
    "nvfp4_pad_f32": [_P, _P, _P, _U, _U, _U, _U],
    "nvfp4_transpose_pad_f32": [_P, _P, _P, _U, _U, _U, _U],
    "nvfp4_crop_f32": [_P, _P, _P, _U, _U, _U],
    "nvfp4_gemm": [_P, POINTER(GemmArgs)],
    "nvfp4_gemm_plan_query": [POINTER(GemmArgs), POINTER(GemmPlan)],
    "nvfp4_prepare_tma_nvfp4_device_scales": [_P, _P, _P, _P, _P, _U, _U, _U],
    "nvfp4_prepare_tma_nvfp4_device_scales_into": [_P, _P, _P, _P, _P, _U, _U, _U, _P],
    "nvfp4_tensor_map_cache_stats": [POINTER(ctypes.c_uint64), POINTER(ctypes.c_uint64)],
    "nvfp4_gemm_set_tile_override": [c_int, c_int],
    "nvfp4_gemm_set_wait_timeout_ns": [ctypes.c_uint64],
    "nvfp4_gemm_set_debug_flags": [_U],
    "nvfp4_qkv_projection": [_P, POINTER(ProjectionArgs)],
    "nvfp4_c_proj": [_P, POINTER(ProjectionArgs)],
    "nvfp4_mlp_up_relu2": [_P, POINTER(ProjectionArgs)],
    "nvfp4_mlp_down_residual": [_P, POINTER(ProjectionArgs)],
    "nvfp4_lm_head_logits": [_P, POINTER(ProjectionArgs)],
    "nvfp4_lm_head_logits_tma": [_P, POINTER(ProjectionArgs)],
    "nvfp4_nextlat_projection": [_P, POINTER(ProjectionArgs)],
    "nvfp4_linear_backward_device_scale_tma": [_P, POINTER(LinearBackwardDeviceScaleArgs)],
    "nvfp4_linear_backward_device_scale": [_P, POINTER(LinearBackwardDeviceScaleArgs)],
    "nvfp4_linear_backward_device_scale_cta": [_P, POINTER(LinearBackwardDeviceScaleArgs)],
    "nvfp4_linear_backward": [_P, POINTER(LinearBackwardDeviceScaleArgs)],
    "nvfp4_gemm_tma_nvfp4_device_scales_and_global_scale_buffers": [_P] * 6 + [_U] * 3 + [_P] * 2,
    "nvfp4_gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer": [_P] * 6 + [_U] * 3 + [_P] * 2,
    "nvfp4_gemm_tma_nvfp4_rowwise_a_scale_padded_output": [_P] * 6 + [_U] * 4 + [_P] * 2,
    "nvfp4_set_deterministic_reductions": [c_int],
    "nvfp4_gemm_timing_begin": [_U],
    "nvfp4_gemm_timing_end": [POINTER(c_uint32), POINTER(ctypes.c_double), POINTER(ctypes.c_double),
                              POINTER(c_float), POINTER(ctypes.c_double), _U],
    "nvfp4_projection_bias_inplace": [_P, _P, _P, _P, _P, _U, _U],
    "nvfp4_projection_residual_add": [_P, _P, _P, _P, _P, _P, _U, _U],
    "nvfp4_projection_relu2_inplace": [_P, _P, _P, _P, _P, _P, _U, _U],
    "nvfp4_linear_bias_grad": [_P, _P, _P, _U, _U],
    "nvfp4_linear_bias_grad_bf16": [_P, _P, _P, _U, _U],
    "nvfp4_linear_backward_ms_eden": [_P, POINTER(LinearBackwardArgs)],
    "nvfp4_linear_backward_prepare_weight_t": [_P, POINTER(LinearBackwardArgs)],
    "nvfp4_checkpoint_writer_open": [c_char_p, _U, POINTER(c_void_p)],
    "nvfp4_checkpoint_write_tensor": [_P, c_char_p, ctypes.c_uint64, _F, _P, ctypes.c_uint64, _P, ctypes.c_uint64],
    "nvfp4_checkpoint_write_tensor_device": [_P, _P, c_char_p, ctypes.c_uint64, _P, _P, ctypes.c_uint64, _P,
                                             ctypes.c_uint64],
    "nvfp4_checkpoint_writer_close": [_P],
    "nvfp4_checkpoint_reader_open": [c_char_p, POINTER(c_void_p), POINTER(c_uint32)],
    "nvfp4_checkpoint_next_tensor": [_P, POINTER(CheckpointTensorInfo)],
    "nvfp4_checkpoint_read_payload": [_P, _P, ctypes.c_uint64, _P, ctypes.c_uint64],
    "nvfp4_checkpoint_read_payload_device": [_P, _P, _P, _P, _P],
    "nvfp4_checkpoint_reader_close": [_P],
}
_SPECIAL = {
    "nvfp4_abi_version": (c_int, []),
    "nvfp4_get_deterministic_reductions": (c_int, []),
    "nvfp4_launch_count": (ctypes.c_uint64, []),
    "nvfp4_last_error": (c_char_p, []),
    "nvfp4_padded_k": (c_uint32, [_U]),
    "nvfp4_scale_padded_mn_extent": (c_uint32, [_U]),
    "nvfp4_scale_packed_len": (c_size_t, [_U, _U]),
    "nvfp4_tensor_amax_chunks": (c_uint32, [ctypes.c_uint64]),
    "nvfp4_relu2_backward_amax_chunks": (c_uint32, [ctypes.c_uint64]),
}
EXPORTED_SYMBOLS = sorted(list(_SIGNATURES) + list(_SPECIAL))

_lib = None


def library() -> ctypes.CDLL:
    """Loads libnvfp4_b200.so (built in-tree by build.py); raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python nanogpt-120a_b200/build.py` "
                "(there is no CPU or PyTorch fallback for the NVFP4 projection path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = c_int
            fn.argtypes = argtypes
        for name, (restype, argtypes) in _SPECIAL.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def _call(name: str, *args) -> None:
    lib = library()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise Nvfp4Error(rc, lib.nvfp4_last_error().decode())


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("the NVFP4 projection path needs a CUDA device (sm_100a); no fallback exists")


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(None)
    assert t.is_cuda and t.is_contiguous(), "tensors crossing the C ABI must be contiguous CUDA tensors"
    return c_void_p(t.data_ptr())


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DTYPE_F32
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    raise TypeError(f"unsupported dtype {t.dtype}; the path takes float32 or bfloat16")


def padded_k(k: int) -> int:
    return (k + 63) // 64 * 64


def scale_packed_len(mn: int, k: int) -> int:
    return (mn + 127) // 128 * (k // 64) * 512


def tensor_amax_chunks(n: int) -> int:
    return (n + 1023) // 1024


def launch_count() -> int:
    """Kernels launched by the library so far in this process."""
    return int(library().nvfp4_launch_count())


def set_deterministic_reductions(on: bool) -> None:
    """Caps split-K at two splits so that dW is bit-identical from run to run (small dW GEMMs then fill fewer
    SMs).  Off by default: more than two partial tiles are summed by TMA reduce-add in arrival order."""
    _call("nvfp4_set_deterministic_reductions", 1 if on else 0)


def deterministic_reductions() -> bool:
    return bool(library().nvfp4_get_deterministic_reductions())


def set_gemm_tile_override(block_n: int, block_m: int = 128) -> None:
    """Measurement aid: force the GEMM tile shape of every following launch (128 x {128, 192, 256} or
    256 x 192); block_n = 0 = automatic."""
    _call("nvfp4_gemm_set_tile_override", block_m, block_n)


def set_gemm_wait_timeout_ns(ns: int) -> None:
    """Limit of the GEMM kernel's bounded waits (default 2 s; 0 restores the default)."""
    _call("nvfp4_gemm_set_wait_timeout_ns", ns)


def set_gemm_debug_flags(flags: int) -> None:
    """Test aid: bit 0 makes CTA 0 of every following GEMM skip the loads of its first k-tile."""
    _call("nvfp4_gemm_set_debug_flags", flags)


def tensor_map_cache_stats():
    """(hits, misses) of the calling thread's tensor-map cache."""
    h, m = ctypes.c_uint64(0), ctypes.c_uint64(0)
    _call("nvfp4_tensor_map_cache_stats", ctypes.byref(h), ctypes.byref(m))
    return int(h.value), int(m.value)


def gemm_timing_begin(max_records: int) -> None:
    """Start bracketing every GEMM launch with CUDA events on its stream (measurement aid)."""
    _call("nvfp4_gemm_timing_begin", max_records)


def gemm_timing_end(capacity: int = 0):
    """Returns (launches, total_ms, total_flops, per_launch_ms list, per_launch_flops list)."""
    n, ms, fl = c_uint32(0), ctypes.c_double(0), ctypes.c_double(0)
    per_ms = (c_float * max(capacity, 1))()
    per_fl = (ctypes.c_double * max(capacity, 1))()
    _call("nvfp4_gemm_timing_end", ctypes.byref(n), ctypes.byref(ms), ctypes.byref(fl), per_ms, per_fl, capacity)
    k = min(int(n.value), capacity)
    return int(n.value), float(ms.value), float(fl.value), list(per_ms)[:k], list(per_fl)[:k]


def read_device_status() -> int:
    """Status word set by kernels whose bounded waits expired (0 = healthy); clears it."""
    _require_cuda()
    out = c_uint32(0)
    _call("nvfp4_read_device_status", _stream(), ctypes.byref(out))
    return int(out.value)


@dataclass
class Nvfp4Tensor:
    """The reference's (bytes, scales, global scale) triple, utils/nvfp4/tensor.rs:5-45."""
    bytes: torch.Tensor          # u8 [rows*cols/2]
    scales: torch.Tensor         # u8, logical [rows*cols/16] or packed layout
    global_scales: torch.Tensor  # f32 [1] (tensor scale) or [rows]
    rows: int
    cols: int
    packed: bool = False
    rowwise: bool = False
    decoded_amax: Optional[torch.Tensor] = None  # f32 [1]: max |decoded value|, when the quantizer emitted it


def _empty_u8(n: int, device) -> torch.Tensor:
    return torch.empty(n, dtype=torch.uint8, device=device)


# =============================================================================================
# Module mirrors
# =============================================================================================

class Nvfp4QuantModule:
    """utils/nvfp4/quant/launcher.rs:18-34 and the methods of utils/nvfp4/quant/*.rs."""

    # ---- amax ---------------------------------------------------------------------------
    def row_amax(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda()
        rows, cols = x.shape
        out = torch.empty(rows, dtype=torch.float32, device=x.device) if out is None else out
        name = "nvfp4_row_amax_f32" if x.dtype == torch.float32 else "nvfp4_row_amax_bf16"
        _dtype_code(x)
        _call(name, _stream(), _ptr(x), _ptr(out), rows, cols)
        return out

    row_amax_f32 = row_amax

    def tensor_amax(self, x: torch.Tensor, chunk_amax: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None):
        _require_cuda()
        n = x.numel()
        chunk_amax = torch.empty(tensor_amax_chunks(n), dtype=torch.float32, device=x.device) \
            if chunk_amax is None else chunk_amax
        out = torch.empty(1, dtype=torch.float32, device=x.device) if out is None else out
        name = "nvfp4_tensor_amax_f32" if x.dtype == torch.float32 else "nvfp4_tensor_amax_bf16"
        _dtype_code(x)
        _call(name, _stream(), _ptr(x), _ptr(chunk_amax), _ptr(out), n)
        return chunk_amax, out

    tensor_amax_f32 = tensor_amax

    def tensor_amax_f32_static_scratch(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Tensor amax of an f32 tensor into the caller's `out[0]`, with the chunk scratch held
        inside the library (no allocation anywhere; at most 2**26 values; calls on one device
        must not overlap in time; make the first call before any stream capture)."""
        _require_cuda()
        assert x.dtype == torch.float32 and out.dtype == torch.float32 and out.numel() >= 1
        _call("nvfp4_tensor_amax_f32_static_scratch", _stream(), _ptr(x), _ptr(out), x.numel())
        return out

    def tensor_amax_from_chunks_f32(self, chunk_amax: torch.Tensor, chunk_count: int,
                                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda()
        out = torch.empty(1, dtype=torch.float32, device=chunk_amax.device) if out is None else out
        _call("nvfp4_tensor_amax_from_chunks_f32", _stream(), _ptr(chunk_amax), _ptr(out), chunk_count)
        return out

    # ---- four-six -----------------------------------------------------------------------
    def fp32_to_nvfp4_four_six(self, x: torch.Tensor, amax: torch.Tensor) -> Nvfp4Tensor:
        _require_cuda()
        assert x.dtype == torch.float32 and x.numel() % 16 == 0
        n = x.numel()
        t = Nvfp4Tensor(_empty_u8(n // 2, x.device), _empty_u8(n // 16, x.device),
                        torch.empty(1, dtype=torch.float32, device=x.device), 1, n)
        _call("nvfp4_fp32_to_nvfp4_four_six", _stream(), _ptr(x), _ptr(amax), _ptr(t.bytes), _ptr(t.scales),
              _ptr(t.global_scales), n // 16)
        return t

    def fp32_to_nvfp4_four_six_rowwise(self, x: torch.Tensor, amax: torch.Tensor) -> Nvfp4Tensor:
        _require_cuda()
        assert x.dtype == torch.float32
        rows, cols = x.shape
        n = rows * cols
        t = Nvfp4Tensor(_empty_u8(n // 2, x.device), _empty_u8(n // 16, x.device),
                        torch.empty(rows, dtype=torch.float32, device=x.device), rows, cols, rowwise=True)
        _call("nvfp4_fp32_to_nvfp4_four_six_rowwise", _stream(), _ptr(x), _ptr(amax), _ptr(t.bytes), _ptr(t.scales),
              _ptr(t.global_scales), n // 16, cols)
        return t

    def fp32_to_nvfp4_four_six_padded(self, x, amax, padded_rows, padded_cols, transposed=False) -> Nvfp4Tensor:
        _require_cuda()
        assert x.dtype == torch.float32
        rows, cols = x.shape
        n = padded_rows * padded_cols
        t = Nvfp4Tensor(_empty_u8(n // 2, x.device), _empty_u8(n // 16, x.device),
                        torch.empty(1, dtype=torch.float32, device=x.device), padded_rows, padded_cols)
        name = "nvfp4_fp32_transpose_to_nvfp4_four_six_padded" if transposed else "nvfp4_fp32_to_nvfp4_four_six_padded"
        _call(name, _stream(), _ptr(x), _ptr(amax), _ptr(t.bytes), _ptr(t.scales), _ptr(t.global_scales), rows, cols,
              padded_rows, padded_cols)
        return t

    def fp32_transpose_to_nvfp4_four_six_padded(self, x, amax, padded_rows, padded_cols) -> Nvfp4Tensor:
        return self.fp32_to_nvfp4_four_six_padded(x, amax, padded_rows, padded_cols, transposed=True)

    def quantize_four_six(self, x: torch.Tensor, amax: Optional[torch.Tensor] = None, rowwise: bool = False,
                          packed: bool = True, out: Optional[Nvfp4Tensor] = None,
                          decoded_amax: bool = False) -> Nvfp4Tensor:
        """B200-native form: f32 / bf16 input, scales written in the layout the GEMM reads.
        decoded_amax (fused rowwise path only): also emit max |decoded value| of the result, which
        LinearBackwardModule.backward_ms_eden then uses instead of a pass over the saved tensor."""
        _require_cuda()
        rows, cols = x.shape
        fused = amax is None and rowwise
        if amax is None and not rowwise:
            amax = self.tensor_amax(x)[1]
        if out is None:
            n = rows * cols
            nsc = scale_packed_len(rows, cols) if packed else n // 16
            out = Nvfp4Tensor(_empty_u8(n // 2, x.device), _empty_u8(nsc, x.device),
                              torch.empty(rows if rowwise else 1, dtype=torch.float32, device=x.device), rows, cols,
                              packed=packed, rowwise=rowwise)
        if fused:  # row amax and quantization in one pass over x
            row_amax = torch.empty(rows, dtype=torch.float32, device=x.device) if cols > 4096 else None
            if decoded_amax and out.decoded_amax is None:
                out.decoded_amax = torch.empty(1, dtype=torch.float32, device=x.device)
            elif not decoded_amax:
                out.decoded_amax = None
            _call("nvfp4_quantize_four_six_rowwise_fused", _stream(), _ptr(x), _dtype_code(x), rows, cols,
                  _ptr(out.bytes), _ptr(out.scales), SCALES_PACKED if packed else SCALES_LOGICAL,
                  _ptr(out.global_scales), _ptr(row_amax), _ptr(out.decoded_amax))
            return out
        _call("nvfp4_quantize_four_six", _stream(), _ptr(x), _dtype_code(x), _ptr(amax), 1 if rowwise else 0, rows,
              cols, _ptr(out.bytes), _ptr(out.scales), SCALES_PACKED if packed else SCALES_LOGICAL,
              _ptr(out.global_scales))
        return out

    def quantize_relu2_four_six_rowwise(self, pre_activation: torch.Tensor, row_amax: Optional[torch.Tensor] = None,
                                        packed: bool = True, out: Optional[Nvfp4Tensor] = None,
                                        decoded_amax: bool = False) -> Nvfp4Tensor:
        """Rowwise four-six of relu(pre)^2 computed on load (the MLP activation is never stored).  `row_amax`:
        the row amax of relu(pre)^2 when the producing GEMM already wrote it (`relu2_row_amax`)."""
        _require_cuda()
        rows, cols = pre_activation.shape
        if out is None:
            n = rows * cols
            nsc = scale_packed_len(rows, cols) if packed else n // 16
            out = Nvfp4Tensor(_empty_u8(n // 2, pre_activation.device), _empty_u8(nsc, pre_activation.device),
                              torch.empty(rows, dtype=torch.float32, device=pre_activation.device), rows, cols,
                              packed=packed, rowwise=True)
        if decoded_amax and out.decoded_amax is None:
            out.decoded_amax = torch.empty(1, dtype=torch.float32, device=pre_activation.device)
        elif not decoded_amax:
            out.decoded_amax = None
        _call("nvfp4_quantize_relu2_four_six_rowwise", _stream(), _ptr(pre_activation), _dtype_code(pre_activation),
              rows, cols, _ptr(row_amax), _ptr(out.bytes), _ptr(out.scales),
              SCALES_PACKED if packed else SCALES_LOGICAL, _ptr(out.global_scales), c_void_p(None),
              _ptr(out.decoded_amax))
        return out

    # ---- MS-EDEN ------------------------------------------------------------------------
    def ms_eden_quantize(self, *, src_kind: int, x: Optional[torch.Tensor] = None, src: Optional[Nvfp4Tensor] = None,
                         rows: int, cols: int, dst_row_len: int, global_scale, sign_seed: int, scale_seed: int,
                         scale_override: float = QUARTET_MS_EDEN_SCALE_OVERRIDE, packed: bool = False,
                         want_chunk_amax: bool = False, col_offset: int = 0, group_offset: int = 0,
                         group_row_stride: int = 0) -> tuple:
        """Generic entry.  Returns (Nvfp4Tensor with per-row copies of the global scale, chunk_amax|None)."""
        _require_cuda()
        dev = x.device if x is not None else src.bytes.device
        out_rows = rows if src_kind == SRC_F32_ROWS else cols
        n = out_rows * dst_row_len
        nsc = scale_packed_len(out_rows, dst_row_len) if packed else n // 16
        out = Nvfp4Tensor(_empty_u8(n // 2, dev), _empty_u8(nsc, dev),
                          torch.empty(out_rows, dtype=torch.float32, device=dev), out_rows, dst_row_len,
                          packed=packed, rowwise=True)
        chunk_amax = torch.empty(n // 32, dtype=torch.float32, device=dev) if want_chunk_amax else None
        a = MsEdenArgs()
        a.src_kind = src_kind
        a.src_dtype = _dtype_code(x) if x is not None else DTYPE_F32
        a.x = _ptr(x)
        if src is not None:
            a.src_bytes, a.src_scales, a.src_global = _ptr(src.bytes), _ptr(src.scales), _ptr(src.global_scales)
            a.src_scale_layout = SCALES_PACKED if src.packed else SCALES_LOGICAL
        a.rows, a.cols, a.dst_row_len = rows, cols, dst_row_len
        if isinstance(global_scale, torch.Tensor):
            a.global_scale = _ptr(global_scale)
            a.host_global_scale_valid = 0
        else:
            a.host_global_scale = float(global_scale)
            a.host_global_scale_valid = 1
        a.scale_override = scale_override
        a.sign_seed, a.scale_seed = sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF
        a.col_offset, a.group_offset, a.group_row_stride = col_offset, group_offset, group_row_stride
        a.out_fp4, a.out_scales = _ptr(out.bytes), _ptr(out.scales)
        a.scale_layout = SCALES_PACKED if packed else SCALES_LOGICAL
        a.out_global_scales = _ptr(out.global_scales)
        a.out_chunk_amax = _ptr(chunk_amax)
        _call("nvfp4_ms_eden_quantize", _stream(), ctypes.byref(a))
        return out, chunk_amax

    def fp32_to_nvfp4_ms_eden(self, x, dst_row_len, global_scale: float, scale_override, sign_seed, scale_seed):
        rows, cols = x.shape
        return self.ms_eden_quantize(src_kind=SRC_F32_ROWS, x=x, rows=rows, cols=cols, dst_row_len=dst_row_len,
                                     global_scale=float(global_scale), sign_seed=sign_seed, scale_seed=scale_seed,
                                     scale_override=scale_override, want_chunk_amax=True)

    def quartet_backward_ms_eden_global_scale_from_chunks(self, chunk_amax, chunk_count, out=None):
        _require_cuda()
        out = torch.empty(1, dtype=torch.float32, device=chunk_amax.device) if out is None else out
        _call("nvfp4_quartet_backward_ms_eden_global_scale_from_chunks", _stream(), _ptr(chunk_amax), _ptr(out),
              chunk_count)
        return out

    def _named_rows(self, name, x, dst_row_len, sign_seed, scale_seed, want_chunk_amax):
        _require_cuda()
        assert x.dtype == torch.float32
        rows, cols = x.shape
        n = rows * dst_row_len
        out = Nvfp4Tensor(_empty_u8(n // 2, x.device), _empty_u8(n // 16, x.device),
                          torch.empty(rows, dtype=torch.float32, device=x.device), rows, dst_row_len, rowwise=True)
        chunk = torch.empty(max(tensor_amax_chunks(rows * cols), n // 32), dtype=torch.float32, device=x.device)
        gs = torch.empty(1, dtype=torch.float32, device=x.device)
        _call(name, _stream(), _ptr(x), _ptr(out.bytes), _ptr(out.scales), _ptr(out.global_scales), _ptr(chunk),
              _ptr(gs), rows, cols, dst_row_len, sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF)
        return out, gs, (chunk[: n // 32] if want_chunk_amax else None)

    def fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale(self, x, dst_row_len, sign_seed, scale_seed):
        return self._named_rows("nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale", x, dst_row_len,
                                sign_seed, scale_seed, True)

    def fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(self, x, dst_row_len, sign_seed,
                                                                                   scale_seed):
        return self._named_rows("nvfp4_fp32_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax", x,
                                dst_row_len, sign_seed, scale_seed, False)

    def fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax(
            self, x, dst_row_len, transpose_dst_row_len, sign_seed, scale_seed, transpose_scale_seed):
        """utils/nvfp4/quant/ms_eden_pair.rs:13-45.  Returns (rows, transposed, global_scale[1])."""
        _require_cuda()
        assert x.dtype == torch.float32
        rows, cols = x.shape
        dev = x.device
        n1, n2 = rows * dst_row_len, cols * transpose_dst_row_len
        o1 = Nvfp4Tensor(_empty_u8(n1 // 2, dev), _empty_u8(n1 // 16, dev),
                         torch.empty(rows, dtype=torch.float32, device=dev), rows, dst_row_len, rowwise=True)
        o2 = Nvfp4Tensor(_empty_u8(n2 // 2, dev), _empty_u8(n2 // 16, dev),
                         torch.empty(cols, dtype=torch.float32, device=dev), cols, transpose_dst_row_len, rowwise=True)
        chunk = torch.empty(tensor_amax_chunks(rows * cols), dtype=torch.float32, device=dev)
        gs = torch.empty(1, dtype=torch.float32, device=dev)
        _call("nvfp4_fp32_pair_to_nvfp4_quartet_backward_ms_eden_derived_device_scale_no_chunk_amax", _stream(),
              _ptr(x), _ptr(o1.bytes), _ptr(o1.scales), _ptr(o1.global_scales), _ptr(o2.bytes), _ptr(o2.scales),
              _ptr(o2.global_scales), _ptr(chunk), _ptr(gs), rows, cols, dst_row_len, transpose_dst_row_len,
              sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF, transpose_scale_seed & 0xFFFFFFFF, 0)
        return o1, o2, gs

    def _named_transpose(self, name, src: Nvfp4Tensor, dst_row_len, sign_seed, scale_seed):
        _require_cuda()
        dev = src.bytes.device
        n = src.cols * dst_row_len
        out = Nvfp4Tensor(_empty_u8(n // 2, dev), _empty_u8(n // 16, dev),
                          torch.empty(src.cols, dtype=torch.float32, device=dev), src.cols, dst_row_len, rowwise=True)
        chunk = torch.empty(max(tensor_amax_chunks(src.rows * src.cols), n // 32), dtype=torch.float32, device=dev)
        gs = torch.empty(1, dtype=torch.float32, device=dev)
        _call(name, _stream(), _ptr(src.bytes), _ptr(src.scales), _ptr(src.global_scales), _ptr(out.bytes),
              _ptr(out.scales), _ptr(out.global_scales), _ptr(chunk), _ptr(gs), src.rows, src.cols, dst_row_len,
              sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF)
        return out, gs, chunk[: n // 32]

    def nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(self, src, dst_row_len, sign_seed, scale_seed):
        return self._named_transpose("nvfp4_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale", src,
                                     dst_row_len, sign_seed, scale_seed)

    def rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale(self, src, dst_row_len, sign_seed,
                                                                                  scale_seed):
        return self._named_transpose("nvfp4_rowwise_nvfp4_transpose_to_quartet_backward_ms_eden_derived_device_scale",
                                     src, dst_row_len, sign_seed, scale_seed)


class Nvfp4TcMatmulModule:
    """utils/nvfp4_tc_matmul/launcher.rs:23-87."""

    def matmul_ms_eden(self, a: torch.Tensor, b_t: torch.Tensor, sign_seed: int, scale_seed: int,
                       a_global_scale: float = 1.0, b_global_scale: float = 1.0):
        """out[m, n] = a[m, k] . b_t[n, k]^T, both operands MS-EDEN quantized with the given global scales.
        Returns (out f32, a_quantized, b_quantized) with the operands as Nvfp4Tensor (packed scales)."""
        _require_cuda()
        assert a.dtype == torch.float32 and b_t.dtype == torch.float32 and a.shape[1] == b_t.shape[1]
        (m, k), n, dev = a.shape, b_t.shape[0], a.device
        pk = padded_k(k)

        def operand(rows):
            t = Nvfp4Tensor(_empty_u8(rows * pk // 2, dev), _empty_u8(scale_packed_len(rows, pk), dev),
                            torch.empty(rows, dtype=torch.float32, device=dev), rows, pk, packed=True, rowwise=True)
            chunk = torch.empty(max(1, rows * pk // 32), dtype=torch.float32, device=dev)
            return t, chunk, MsEdenOperand(_ptr(t.bytes), _ptr(t.scales), _ptr(t.global_scales), c_void_p(None), _ptr(chunk))

        ta, ca, oa = operand(m)
        tb, cb, ob = operand(n)
        out = torch.empty((m, n), dtype=torch.float32, device=dev)
        _call("nvfp4_tc_matmul_ms_eden", _stream(), _ptr(a), _ptr(b_t), _ptr(out), ctypes.byref(oa), a_global_scale,
              ctypes.byref(ob), b_global_scale, m, n, k, sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF)
        return out, ta, tb


class MlpModule:
    """gpt/mlp/launcher.rs:66-76: the element-wise step between the two MLP linears of the backward pass
    (the forward projections of that module are `projection_forward` with the ReLU^2 epilogue)."""

    def up_relu2(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Nvfp4Tensor, pre_activation=None, out=None,
                 out_dtype: torch.dtype = torch.float32, store_activation: bool = True, relu2_row_amax=None):
        """gpt/mlp/launcher.rs:53-59: pre = X . W^T + b, out = max(pre, 0)^2.  `store_activation=False` keeps only
        the pre-activation (relu^2 is then applied on load by `quantize_relu2_four_six_rowwise`).  Returns
        (pre_activation, out | None)."""
        _require_cuda()
        dev = input.bytes.device
        if pre_activation is None:
            pre_activation = torch.empty((input.rows, weight.rows), dtype=out_dtype, device=dev)
        if store_activation and out is None:
            out = torch.empty((input.rows, weight.rows), dtype=pre_activation.dtype, device=dev)
        a, keep = _projection_args(input, weight, bias, out if store_activation else None, pre_activation, relu2_row_amax)
        _call("nvfp4_mlp_up_relu2", _stream(), ctypes.byref(a))
        return pre_activation, (out if store_activation else None)

    def down_residual(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Nvfp4Tensor, residual: torch.Tensor):
        """gpt/mlp/launcher.rs:60-66: residual (f32, in place) += X . W^T + b."""
        _require_cuda()
        a, keep = _projection_args(input, weight, bias, residual)
        _call("nvfp4_mlp_down_residual", _stream(), ctypes.byref(a))
        return residual

    def relu2_backward(self, pre_activation: torch.Tensor, d_out: torch.Tensor,
                       d_pre_activation: Optional[torch.Tensor] = None) -> torch.Tensor:
        """d_pre = d_out * 2 * relu(pre).  (pre f32 | f16, gradients f32) as in the reference, or all bf16."""
        _require_cuda()
        n = pre_activation.numel()
        assert d_out.numel() == n
        if pre_activation.dtype == torch.bfloat16:
            assert d_out.dtype == torch.bfloat16
            out = torch.empty_like(d_out) if d_pre_activation is None else d_pre_activation
            _call("nvfp4_relu2_backward_bf16", _stream(), _ptr(pre_activation), _ptr(d_out), _ptr(out), n)
            return out
        assert d_out.dtype == torch.float32
        out = torch.empty_like(d_out) if d_pre_activation is None else d_pre_activation
        name = "nvfp4_relu2_backward" if pre_activation.dtype == torch.float32 else "nvfp4_relu2_backward_f16"
        assert pre_activation.dtype in (torch.float32, torch.float16)
        _call(name, _stream(), _ptr(pre_activation), _ptr(d_out), _ptr(out), n)
        return out

    relu2_backward_f16 = relu2_backward

    def relu2_backward_amax(self, pre_activation: torch.Tensor, d_out: torch.Tensor, chunk_amax: torch.Tensor,
                            d_pre_activation: Optional[torch.Tensor] = None) -> tuple:
        """`relu2_backward` that also writes the amax of the gradient it stores as a chunk list into
        `chunk_amax` (normally `LinearBackwardScratch.e_h["chunk_amax"]` of the fc linear's backward).  Returns
        (d_pre, chunk_count); pass chunk_count as `precomputed_e_amax_chunks` to `backward_ms_eden`, which then
        skips its own amax pass over the gradient (gpt/loss/kernels.rs:67-88 hands the loss gradient over the
        same way)."""
        _require_cuda()
        n = pre_activation.numel()
        assert d_out.numel() == n and d_out.dtype in (torch.float32, torch.bfloat16)
        pre_kind = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[pre_activation.dtype]
        out = torch.empty_like(d_out) if d_pre_activation is None else d_pre_activation
        assert out.dtype == d_out.dtype and chunk_amax.dtype == torch.float32
        chunks = c_uint32(0)
        _call("nvfp4_relu2_backward_amax", _stream(), _ptr(pre_activation), pre_kind, _ptr(d_out), _ptr(out),
              _dtype_code(d_out), n, _ptr(chunk_amax), chunk_amax.numel(), ctypes.byref(chunks))
        return out, chunks.value


class OptimizerModule:
    """The part of gpt/optimizer/launcher that feeds the projection path: weight materialisation."""

    def materialize_schedule_free(self, z_master: torch.Tensor, x_master: torch.Tensor, beta: float,
                                  packed: bool = False, out: Optional[Nvfp4Tensor] = None):
        """gpt/optimizer/launcher/update.rs:11-58.  z / x: f32 masters of one [rows, cols] weight.
        Returns (Nvfp4Tensor with a tensor scale, amax[1])."""
        _require_cuda()
        assert z_master.dtype == torch.float32 and x_master.dtype == torch.float32 and z_master.shape == x_master.shape
        rows, cols = z_master.shape
        dev, n = z_master.device, rows * cols
        if out is None:
            nsc = scale_packed_len(rows, cols) if packed else n // 16
            out = Nvfp4Tensor(_empty_u8(n // 2, dev), _empty_u8(nsc, dev),
                              torch.empty(1, dtype=torch.float32, device=dev), rows, cols, packed=packed, rowwise=False)
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        chunk = torch.empty(max(1, tensor_amax_chunks(n)), dtype=torch.float32, device=dev)
        if packed:
            _call("nvfp4_materialize_schedule_free_matrix", _stream(), _ptr(z_master), _ptr(x_master), _ptr(chunk),
                  _ptr(amax), _ptr(out.bytes), _ptr(out.scales), SCALES_PACKED, _ptr(out.global_scales), beta, rows, cols)
        else:
            _call("nvfp4_materialize_schedule_free", _stream(), _ptr(z_master), _ptr(x_master), _ptr(chunk), _ptr(amax),
                  _ptr(out.bytes), _ptr(out.scales), _ptr(out.global_scales), beta, n)
        return out, amax


class Nvfp4DecodeModule:
    """utils/nvfp4/decode/launcher.rs."""

    def decode(self, t: Nvfp4Tensor, transpose: bool = False) -> torch.Tensor:
        _require_cuda()
        assert not t.packed, "decode reads the logical scale layout"
        shape = (t.cols, t.rows) if transpose else (t.rows, t.cols)
        out = torch.empty(shape, dtype=torch.float32, device=t.bytes.device)
        if transpose:
            name = "nvfp4_decode_rowwise_transpose_f32" if t.rowwise else "nvfp4_decode_transpose_f32"
            _call(name, _stream(), _ptr(t.bytes), _ptr(t.scales), _ptr(t.global_scales), _ptr(out), t.rows, t.cols)
        else:
            _call("nvfp4_decode_f32", _stream(), _ptr(t.bytes), _ptr(t.scales), _ptr(t.global_scales),
                  1 if t.rowwise else 0, _ptr(out), t.rows, t.cols)
        return out

    def decode_transpose_f32(self, t: Nvfp4Tensor) -> torch.Tensor:
        return self.decode(t, transpose=True)

    decode_rowwise_transpose_f32 = decode_transpose_f32


class Sm120ScalePackModule:
    """utils/nvfp4_tma_matmul/scale_pack.rs:54-78 (name kept for drop-in; the layout is the
    tcgen05 128x4 scale-factor tile order)."""

    def pack(self, logical: torch.Tensor, mn_extent: int, k_dim: int, packed: Optional[torch.Tensor] = None):
        _require_cuda()
        packed = _empty_u8(scale_packed_len(mn_extent, k_dim), logical.device) if packed is None else packed
        _call("nvfp4_scale_pack", _stream(), _ptr(logical), _ptr(packed), mn_extent, k_dim)
        return packed


class TmaMatrixPadModule:
    """utils/nvfp4_tma_matmul/pad.rs:49-107."""

    def pad_u4_rows(self, src, rows, padded_rows, cols):
        _require_cuda()
        dst = _empty_u8(padded_rows * cols // 2, src.device)
        _call("nvfp4_pad_u4_rows", _stream(), _ptr(src), _ptr(dst), rows, padded_rows, cols)
        return dst

    def pad_f32(self, src, padded_rows, padded_cols, transpose=False):
        _require_cuda()
        rows, cols = src.shape
        dst = torch.empty((padded_rows, padded_cols), dtype=torch.float32, device=src.device)
        _call("nvfp4_transpose_pad_f32" if transpose else "nvfp4_pad_f32", _stream(), _ptr(src), _ptr(dst), rows, cols,
              padded_rows, padded_cols)
        return dst

    def transpose_pad_f32(self, src, padded_rows, padded_cols):
        return self.pad_f32(src, padded_rows, padded_cols, transpose=True)

    def crop_f32(self, src, dst_cols):
        _require_cuda()
        rows, cols = src.shape
        dst = torch.empty((rows, dst_cols), dtype=torch.float32, device=src.device)
        _call("nvfp4_crop_f32", _stream(), _ptr(src), _ptr(dst), rows, cols, dst_cols)
        return dst


def _packed_scales(t: Nvfp4Tensor) -> torch.Tensor:
    return t.scales if t.packed else Sm120ScalePackModule().pack(t.scales, t.rows, t.cols)


class Nvfp4GemmModule:
    """utils/nvfp4_tma_matmul/launcher.rs:23-328.  The tensor maps the reference prepares in a
    separate call are encoded inside each launch and passed as kernel parameters."""

    def _args(self, a: Nvfp4Tensor, b: Nvfp4Tensor, out, aux, bias, mode, epilogue, weight_global_scale, n, ldo,
              relu2_row_amax):
        g = GemmArgs()
        # keep the (possibly temporary) packed planes referenced until the launch is enqueued
        keep = (_packed_scales(a), _packed_scales(b))
        g.a_bytes, g.a_scales, g.a_global = _ptr(a.bytes), _ptr(keep[0]), _ptr(a.global_scales)
        g.b_bytes, g.b_scales, g.b_global = _ptr(b.bytes), _ptr(keep[1]), _ptr(b.global_scales)
        g.out, g.aux = _ptr(out), _ptr(aux)
        if isinstance(bias, Nvfp4Tensor):  # NVFP4-encoded bias, decoded in the epilogue
            assert not bias.packed and not bias.rowwise, "an NVFP4 bias carries logical scales and one global scale"
            g.bias_nvfp4_bytes, g.bias_nvfp4_scales = _ptr(bias.bytes), _ptr(bias.scales)
            g.bias_nvfp4_global = _ptr(bias.global_scales)
        else:
            g.bias = _ptr(bias)
        g.m, g.n, g.k, g.ldo = a.rows, n, a.cols, ldo
        g.global_scale_mode = mode
        g.weight_global_scale = weight_global_scale
        g.epilogue = epilogue
        g.out_dtype = _dtype_code(out)
        g.relu2_row_amax = _ptr(relu2_row_amax)
        return g, keep

    def gemm(self, a: Nvfp4Tensor, b: Nvfp4Tensor, *, mode: Optional[int] = None, bias=None,
             epilogue: int = EPI_NONE, out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None,
             aux: Optional[torch.Tensor] = None, weight_global_scale: float = 1.0, n: Optional[int] = None,
             ldo: Optional[int] = None, relu2_row_amax: Optional[torch.Tensor] = None,
             plan_only: bool = False):
        """out[m][n] = epilogue((A . B^T) * weight * ga * gb); A [m][k], B [n][k] NVFP4.  `bias` is an f32
        vector or an NVFP4-encoded `Nvfp4Tensor` [1, n]; `relu2_row_amax` (f32[m]) receives the row amax of
        relu(stored value)^2; `plan_only` returns the `GemmPlan` the library would choose instead of launching."""
        _require_cuda()
        assert a.cols == b.cols, "A and B must share K"
        m = a.rows
        n = b.rows if n is None else n
        ldo = n if ldo is None else ldo
        if mode is None:
            mode = GS_ROWWISE_A if a.rowwise else GS_TENSOR
        if out is None:
            out = torch.empty((m, ldo), dtype=out_dtype, device=a.bytes.device)
        g, keep = self._args(a, b, out, aux, bias, mode, epilogue, weight_global_scale, n, ldo, relu2_row_amax)
        if plan_only:
            plan = GemmPlan()
            _call("nvfp4_gemm_plan_query", ctypes.byref(g), ctypes.byref(plan))
            return plan
        _call("nvfp4_gemm", _stream(), ctypes.byref(g))
        del keep
        return out

    def plan(self, a: Nvfp4Tensor, b: Nvfp4Tensor, **kw) -> "GemmPlan":
        """The tile width / schedule `gemm(a, b, **kw)` takes on this device (nothing is launched)."""
        return self.gemm(a, b, plan_only=True, **kw)

    def prepare_tma_nvfp4_device_scales(self, a: Nvfp4Tensor, b: Nvfp4Tensor) -> None:
        """utils/nvfp4_tma_matmul/launcher.rs:39-166: validates the operands and encodes their tensor maps into
        the calling thread's cache ahead of the launches that use them."""
        _require_cuda()
        assert a.packed and b.packed
        _call("nvfp4_prepare_tma_nvfp4_device_scales", _stream(), _ptr(a.bytes), _ptr(a.scales), _ptr(b.bytes),
              _ptr(b.scales), a.rows, a.cols, b.rows)

    def _named(self, name, a, b, extra_dims=()):
        _require_cuda()
        out = torch.empty((a.rows, b.rows if not extra_dims else extra_dims[0]), dtype=torch.float32,
                          device=a.bytes.device)
        dims = [a.rows, a.cols, out.shape[1]] + ([b.rows] if extra_dims else [])
        a_packed, b_packed = _packed_scales(a), _packed_scales(b)
        _call(name, _stream(), _ptr(a.bytes), _ptr(a_packed), _ptr(b.bytes), _ptr(b_packed),
              _ptr(out), *dims, _ptr(a.global_scales), _ptr(b.global_scales))
        return out

    def gemm_tma_nvfp4_device_scales_and_global_scale_buffers(self, a, b):
        return self._named("nvfp4_gemm_tma_nvfp4_device_scales_and_global_scale_buffers", a, b)

    def gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer(self, a, b):
        return self._named("nvfp4_gemm_tma_nvfp4_rowwise_a_scale_and_global_scale_buffer", a, b)

    def gemm_tma_nvfp4_rowwise_a_scale_padded_output(self, a, b, output_dim):
        return self._named("nvfp4_gemm_tma_nvfp4_rowwise_a_scale_padded_output", a, b, extra_dims=(output_dim,))


def _projection_args(input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Optional[Nvfp4Tensor], out, pre_activation=None,
                     relu2_row_amax=None):
    assert input.rowwise and not weight.rowwise and input.cols == weight.cols
    a = ProjectionArgs()
    dev = input.bytes.device
    keep = []
    a.input_bytes, a.input_scales, a.input_global_scales = _ptr(input.bytes), _ptr(input.scales), _ptr(input.global_scales)
    a.input_scale_layout = SCALES_PACKED if input.packed else SCALES_LOGICAL
    a.weight_bytes, a.weight_scales, a.weight_global_scale = _ptr(weight.bytes), _ptr(weight.scales), _ptr(weight.global_scales)
    a.weight_scale_layout = SCALES_PACKED if weight.packed else SCALES_LOGICAL
    if not input.packed:
        keep.append(_empty_u8(scale_packed_len(input.rows, input.cols), dev))
        a.input_scales_packed_scratch = _ptr(keep[-1])
    if not weight.packed:
        keep.append(_empty_u8(scale_packed_len(weight.rows, weight.cols), dev))
        a.weight_scales_packed_scratch = _ptr(keep[-1])
    if bias is not None:
        assert not bias.packed and not bias.rowwise
        a.bias_bytes, a.bias_scales, a.bias_global_scale = _ptr(bias.bytes), _ptr(bias.scales), _ptr(bias.global_scales)
    ref = out if out is not None else pre_activation
    a.out, a.pre_activation = _ptr(out), _ptr(pre_activation)
    a.out_dtype = _dtype_code(ref)
    a.relu2_row_amax = _ptr(relu2_row_amax)
    a.token_count, a.input_dim, a.output_dim = input.rows, input.cols, weight.rows
    return a, keep


class AttentionModule:
    """gpt/attention/qkv_projection/launcher.rs:8-42 (the two projections of the attention block)."""

    def qkv_projection(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Nvfp4Tensor, out=None,
                       out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _require_cuda()
        out = torch.empty((input.rows, weight.rows), dtype=out_dtype, device=input.bytes.device) if out is None else out
        a, keep = _projection_args(input, weight, bias, out)
        _call("nvfp4_qkv_projection", _stream(), ctypes.byref(a))
        return out

    def c_proj(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Nvfp4Tensor, residual: torch.Tensor) -> torch.Tensor:
        """residual (f32, in place) = fma(1, X . W^T + b, residual)."""
        _require_cuda()
        a, keep = _projection_args(input, weight, bias, residual)
        _call("nvfp4_c_proj", _stream(), ctypes.byref(a))
        return residual


class LmHeadModule:
    """gpt/lm_head.rs:65-125."""

    def logits(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, logits=None, out_dtype: torch.dtype = torch.float32,
               tma: bool = False) -> torch.Tensor:
        _require_cuda()
        logits = torch.empty((input.rows, weight.rows), dtype=out_dtype, device=input.bytes.device) if logits is None else logits
        a, keep = _projection_args(input, weight, None, logits)
        _call("nvfp4_lm_head_logits_tma" if tma else "nvfp4_lm_head_logits", _stream(), ctypes.byref(a))
        return logits

    def logits_tma(self, input, weight, logits=None, out_dtype: torch.dtype = torch.float32):
        return self.logits(input, weight, logits, out_dtype, tma=True)


class NextLatModule:
    """gpt/next_latent/launch_projection.rs:10-29."""

    def projection(self, input: Nvfp4Tensor, weight: Nvfp4Tensor, bias: Nvfp4Tensor, out=None,
                   out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _require_cuda()
        out = torch.empty((input.rows, weight.rows), dtype=out_dtype, device=input.bytes.device) if out is None else out
        a, keep = _projection_args(input, weight, bias, out)
        _call("nvfp4_nextlat_projection", _stream(), ctypes.byref(a))
        return out


class ProjectionPostOpModule:
    """gpt/projection_postop.rs:50-162 (separate-pass post-ops; bias is NVFP4 encoded)."""

    def bias_inplace(self, raw, bias: Nvfp4Tensor):
        _require_cuda()
        rows, cols = raw.shape
        _call("nvfp4_projection_bias_inplace", _stream(), _ptr(raw), _ptr(bias.bytes), _ptr(bias.scales),
              _ptr(bias.global_scales), rows, cols)
        return raw

    def residual_add(self, raw, bias: Nvfp4Tensor, residual):
        _require_cuda()
        rows, cols = raw.shape
        _call("nvfp4_projection_residual_add", _stream(), _ptr(raw), _ptr(bias.bytes), _ptr(bias.scales),
              _ptr(bias.global_scales), _ptr(residual), rows, cols)
        return residual

    def relu2_inplace(self, pre_activation, bias: Nvfp4Tensor, out=None):
        _require_cuda()
        rows, cols = pre_activation.shape
        out = torch.empty_like(pre_activation) if out is None else out
        _call("nvfp4_projection_relu2_inplace", _stream(), _ptr(pre_activation), _ptr(out), _ptr(bias.bytes),
              _ptr(bias.scales), _ptr(bias.global_scales), rows, cols)
        return out


class LinearBackwardScratch:
    """Caller-owned scratch of one linear backward
    (gpt/linear_backward/args/ms_eden/scratch.rs:91-115), sized for (tokens, in, out)."""

    def __init__(self, token_count: int, input_dim: int, output_dim: int, device):
        ok, tk = padded_k(output_dim), padded_k(token_count)
        f32 = dict(dtype=torch.float32, device=device)

        def operand(rows, k, amax_elems):
            return dict(bytes=_empty_u8(rows * k // 2, device), scales_packed=_empty_u8(scale_packed_len(rows, k), device),
                        global_scales=torch.empty(rows, **f32), global_scale=torch.empty(1, **f32),
                        chunk_amax=torch.empty(max(1, tensor_amax_chunks(amax_elems)), **f32))

        self.e_h = operand(token_count, ok, token_count * output_dim)
        self.e_t_h = operand(output_dim, tk, 1)
        self.weight_t_h = operand(input_dim, ok, output_dim * input_dim)
        self.input_t_h = operand(input_dim, tk, token_count * input_dim)
        self.dims = (token_count, input_dim, output_dim)

    @staticmethod
    def _c(op) -> MsEdenOperand:
        return MsEdenOperand(_ptr(op["bytes"]), _ptr(op["scales_packed"]), _ptr(op["global_scales"]),
                             _ptr(op["global_scale"]), _ptr(op["chunk_amax"]))

    def as_tensor(self, name: str) -> Nvfp4Tensor:
        op = getattr(self, name)
        t, i, o = self.dims
        rows, k = {"e_h": (t, padded_k(o)), "e_t_h": (o, padded_k(t)), "weight_t_h": (i, padded_k(o)),
                   "input_t_h": (i, padded_k(t))}[name]
        return Nvfp4Tensor(op["bytes"], op["scales_packed"], op["global_scales"], rows, k, packed=True, rowwise=True)


class SideStream:
    """A caller-owned second stream with its fork / join events for `LinearBackwardModule.backward_ms_eden`
    (the library owns no stream: the transposers of a backward call run on this one beside the dY amax pass)."""

    def __init__(self, device):
        with torch.cuda.device(device):
            self.stream = torch.cuda.Stream(device=device)
            self.fork, self.join = torch.cuda.Event(), torch.cuda.Event()
            # torch creates the underlying cudaEvent_t lazily: one record materialises it
            self.fork.record(self.stream)
            self.join.record(self.stream)

    def handles(self):
        return (c_void_p(self.stream.cuda_stream), c_void_p(self.fork.cuda_event), c_void_p(self.join.cuda_event))


class LinearBackwardModule:
    """gpt/linear_backward.rs:31-67, gpt/linear_backward/ms_eden.rs:15-55."""

    def backward_device_scale(self, scratch: "LinearBackwardScratch", dinput: torch.Tensor, dweight: torch.Tensor,
                              variant: str = "tma") -> None:
        """gpt/linear_backward/device_scale.rs:38-187 / linear_backward.rs:40-67: the two gradient GEMMs over
        operands already quantized into `scratch` (variant: tma | plain | cta | backward)."""
        _require_cuda()
        t, i, o = scratch.dims
        a = LinearBackwardDeviceScaleArgs()
        for name, scalar in (("e_h", False), ("weight_t_h", True), ("e_t_h", False), ("input_t_h", True)):
            op = getattr(scratch, name)
            setattr(a, name, BackwardOperand(_ptr(op["bytes"]), _ptr(op["scales_packed"]), SCALES_PACKED,
                                             _ptr(op["global_scale"] if scalar else op["global_scales"]),
                                             c_void_p(None)))
        a.dinput, a.dinput_dtype = _ptr(dinput), _dtype_code(dinput)
        a.dweight, a.dweight_dtype = _ptr(dweight), _dtype_code(dweight)
        a.token_count, a.input_dim, a.output_dim = t, i, o
        name = {"tma": "nvfp4_linear_backward_device_scale_tma", "plain": "nvfp4_linear_backward_device_scale",
                "cta": "nvfp4_linear_backward_device_scale_cta", "backward": "nvfp4_linear_backward"}[variant]
        _call(name, _stream(), ctypes.byref(a))

    def linear_bias_grad(self, e: torch.Tensor, dbias: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda()
        tokens, n = e.shape
        dbias = torch.empty(n, dtype=torch.float32, device=e.device) if dbias is None else dbias
        name = "nvfp4_linear_bias_grad" if _dtype_code(e) == DTYPE_F32 else "nvfp4_linear_bias_grad_bf16"
        _call(name, _stream(), _ptr(e), _ptr(dbias), tokens, n)
        return dbias

    def backward_ms_eden(self, *, e: torch.Tensor, weight: Nvfp4Tensor, input: Nvfp4Tensor,
                         scratch: LinearBackwardScratch, sign_seed: int, scale_seed: int, want_dbias: bool = True,
                         grad_dtype: torch.dtype = torch.float32, dinput=None, dweight=None, dbias=None,
                         token_offset: int = 0, e_global_scale: Optional[torch.Tensor] = None,
                         precomputed_e_amax_chunks: int = 0, side: Optional["SideStream"] = None,
                         total_token_count: int = 0, x_decoded_amax: Optional[torch.Tensor] = None,
                         weight_t_prepared: bool = False, prepare_weight_t_only: bool = False):
        """dbias, dX = dY.W, dW = dY^T.X with MS-EDEN quantized operands.  `weight` is the NVFP4
        tensor-scale W[out][in], `input` the rowwise NVFP4 X[tokens][in] saved by the forward."""
        _require_cuda()
        tokens, out_dim = e.shape
        in_dim = weight.cols
        assert weight.rows == out_dim and input.rows == tokens and input.cols == in_dim
        assert scratch.dims == (tokens, in_dim, out_dim)
        dev = e.device
        dinput = torch.empty((tokens, in_dim), dtype=grad_dtype, device=dev) if dinput is None else dinput
        dweight = torch.empty((out_dim, in_dim), dtype=grad_dtype, device=dev) if dweight is None else dweight
        if want_dbias and dbias is None:
            dbias = torch.empty(out_dim, dtype=torch.float32, device=dev)
        a = LinearBackwardArgs()
        a.e, a.e_dtype = _ptr(e), _dtype_code(e)
        a.w_bytes, a.w_scales, a.w_global = _ptr(weight.bytes), _ptr(weight.scales), _ptr(weight.global_scales)
        a.w_scale_layout = SCALES_PACKED if weight.packed else SCALES_LOGICAL
        a.x_bytes, a.x_scales, a.x_globals = _ptr(input.bytes), _ptr(input.scales), _ptr(input.global_scales)
        a.x_scale_layout = SCALES_PACKED if input.packed else SCALES_LOGICAL
        a.e_h, a.e_t_h = scratch._c(scratch.e_h), scratch._c(scratch.e_t_h)
        a.weight_t_h, a.input_t_h = scratch._c(scratch.weight_t_h), scratch._c(scratch.input_t_h)
        a.dinput, a.dinput_dtype = _ptr(dinput), _dtype_code(dinput)
        a.dweight, a.dweight_dtype = _ptr(dweight), _dtype_code(dweight)
        a.dbias = _ptr(dbias if want_dbias else None)
        a.token_count, a.input_dim, a.output_dim = tokens, in_dim, out_dim
        a.sign_seed, a.scale_seed = sign_seed & 0xFFFFFFFF, scale_seed & 0xFFFFFFFF
        a.precomputed_e_amax_chunks = precomputed_e_amax_chunks
        a.token_offset = token_offset
        a.e_global_scale_override = _ptr(e_global_scale)
        a.x_decoded_amax = _ptr(x_decoded_amax if x_decoded_amax is not None else input.decoded_amax)
        a.total_token_count = total_token_count
        a.weight_t_prepared = 1 if weight_t_prepared else 0
        if prepare_weight_t_only:  # the W^T step alone (it reads only the weight and the seeds)
            _call("nvfp4_linear_backward_prepare_weight_t", _stream(), ctypes.byref(a))
            return None
        if side is not None:
            a.side_stream, a.fork_event, a.join_event = side.handles()
        _call("nvfp4_linear_backward_ms_eden", _stream(), ctypes.byref(a))
        return dinput, dweight, (dbias if want_dbias else None)


# =============================================================================================
# Convenience: one projection, forward, the way the model graph calls it
# (crates/gpt2-nvfp4/src/types/l3_mlp/forward.rs:15-67).
# =============================================================================================

class CheckpointWriter:
    """`CheckpointWriter` (src/checkpoint/format/writer.rs:11-38): header on construction, one `write_tensor` per
    NVFP4 triple, `finish` to flush.  Tensors may be host (`bytes`-like / CPU tensors) or device tensors."""

    def __init__(self, path: str, tensor_count: int):
        self._h = c_void_p()
        _call("nvfp4_checkpoint_writer_open", os.fsencode(path), tensor_count, ctypes.byref(self._h))

    def write_tensor(self, name: str, length: int, global_scale, fp4_bytes, scales) -> None:
        """Arguments in the reference's order: name, len (elements), global_scale, bytes, scales."""
        if isinstance(fp4_bytes, torch.Tensor) and fp4_bytes.is_cuda:
            gs = global_scale if isinstance(global_scale, torch.Tensor) else torch.tensor(
                [global_scale], dtype=torch.float32, device=fp4_bytes.device)
            _call("nvfp4_checkpoint_write_tensor_device", self._h, _stream(), name.encode(), length, _ptr(gs),
                  _ptr(fp4_bytes), fp4_bytes.numel(), _ptr(scales), scales.numel())
            return
        b, sc = _host_bytes(fp4_bytes), _host_bytes(scales)
        gs = float(global_scale.item() if isinstance(global_scale, torch.Tensor) else global_scale)
        _call("nvfp4_checkpoint_write_tensor", self._h, name.encode(), length, gs, b, len(b), sc, len(sc))

    def finish(self) -> None:
        h, self._h = self._h, c_void_p()
        if h:
            _call("nvfp4_checkpoint_writer_close", h)


class CheckpointTensor:
    """`CheckpointTensor` (src/checkpoint/format/reader.rs:10-16)."""

    def __init__(self, name, len, global_scale, bytes, scales):
        self.name, self.len, self.global_scale, self.bytes, self.scales = name, len, global_scale, bytes, scales


class CheckpointReader:
    """`CheckpointReader` (src/checkpoint/format/reader.rs:18-67): `read_header()` returns the tensor count,
    `read_tensor()` the next triple on the host, `read_tensor_device(device)` uploads it with the length checks
    of src/checkpoint/load/tensor.rs:27-39."""

    def __init__(self, path: str):
        self._h = c_void_p()
        count = c_uint32()
        _call("nvfp4_checkpoint_reader_open", os.fsencode(path), ctypes.byref(self._h), ctypes.byref(count))
        self._count = count.value

    def read_header(self) -> int:
        return self._count

    def _next(self) -> CheckpointTensorInfo:
        info = CheckpointTensorInfo()
        _call("nvfp4_checkpoint_next_tensor", self._h, ctypes.byref(info))
        return info

    def read_tensor(self) -> CheckpointTensor:
        info = self._next()
        b = ctypes.create_string_buffer(max(1, info.byte_len))
        sc = ctypes.create_string_buffer(max(1, info.scale_len))
        _call("nvfp4_checkpoint_read_payload", self._h, b, info.byte_len, sc, info.scale_len)
        return CheckpointTensor(info.name.decode(), info.len, info.global_scale, b.raw[:info.byte_len],
                                sc.raw[:info.scale_len])

    def read_tensor_device(self, device) -> CheckpointTensor:
        info = self._next()
        b = torch.empty(max(1, info.byte_len), dtype=torch.uint8, device=device)[:info.byte_len]
        sc = torch.empty(max(1, info.scale_len), dtype=torch.uint8, device=device)[:info.scale_len]
        gs = torch.empty(1, dtype=torch.float32, device=device)
        _call("nvfp4_checkpoint_read_payload_device", self._h, _stream(), _ptr(b), _ptr(sc), _ptr(gs))
        return CheckpointTensor(info.name.decode(), info.len, gs, b, sc)

    def close(self) -> None:
        h, self._h = self._h, c_void_p()
        if h:
            _call("nvfp4_checkpoint_reader_close", h)


def _host_bytes(x) -> bytes:
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().contiguous().numpy().tobytes()
    return x if isinstance(x, bytes) else memoryview(x).tobytes()


def projection_forward(x: torch.Tensor, weight: Nvfp4Tensor, bias: Optional[torch.Tensor] = None,
                       epilogue: Optional[int] = None, out_dtype: torch.dtype = torch.bfloat16,
                       rowwise: bool = True, out: Optional[torch.Tensor] = None, keep_logical: bool = False):
    """Y = X.W^T + b: quantize X (four-six, rowwise or tensor scale) then the block-scaled GEMM
    with the fused epilogue.  Returns (Y, quantized X) so the caller can keep X for backward."""
    q = Nvfp4QuantModule()
    xq = q.quantize_four_six(x, rowwise=rowwise, packed=not keep_logical)
    if epilogue is None:
        epilogue = EPI_BIAS if bias is not None else EPI_NONE
    y = Nvfp4GemmModule().gemm(xq, weight, bias=bias, epilogue=epilogue, out_dtype=out_dtype, out=out)
    return y, xq
