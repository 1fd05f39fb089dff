"""ctypes binding of libdynakv_b200.so (the C ABI declared in include/dynakv_b200.h).

Torch is used only for device memory and streams: every call passes raw device pointers,
element strides and the current CUDA stream handle.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdynakv_b200.so")

DKV_F32, DKV_F16, DKV_BF16 = 0, 1, 2
ST_OVERFLOW, ST_BAD_LENGTH, ST_EMPTY_ROW, ST_TIMEOUT = 1, 2, 4, 8

_DTYPES = {torch.float32: DKV_F32, torch.float16: DKV_F16, torch.bfloat16: DKV_BF16}

EXPORTS = (
    "dkv_version", "dkv_last_error", "dkv_fused_decode", "dkv_split_workspace_bytes", "dkv_split_decode",
    "dkv_split_combine", "dkv_two_stage_decode", "dkv_two_stage_decode_noalloc", "dkv_scores", "dkv_softmax_v", "dkv_append_decode",
    "dkv_pack_bulk", "dkv_decompress", "dkv_gate_lengths", "dkv_gate_workspace_bytes", "dkv_gate_lengths_pair", "dkv_project_bulk", "dkv_probe_tensor_pipe",
)


class Side(C.Structure):
    _fields_ = [
        ("flat", C.c_void_p), ("flat_stride", C.c_int64),
        ("lens", C.c_void_p), ("lens_stride_a", C.c_int64), ("lens_stride_s", C.c_int64),
        ("offs", C.c_void_p), ("offs_stride_a", C.c_int64), ("offs_stride_s", C.c_int64),
        ("ptr", C.c_void_p),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("n_q_heads", C.c_int32), ("n_basis_groups", C.c_int32),
        ("arenas_per_batch", C.c_int32), ("head_dim", C.c_int32), ("rank", C.c_int32), ("seq_len", C.c_int32),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_up", C.c_void_p), ("v_up", C.c_void_p),
        ("k", Side), ("v", Side),
        ("seq_lens", C.c_void_p), ("batch_index", C.c_void_p),
        ("k_norm_weight", C.c_void_p), ("k_norm_eps", C.c_float), ("theta", C.c_float),
        ("len_multiple", C.c_int32),
        ("out", C.c_void_p), ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p), ("n_sm", C.c_int32), ("stream", C.c_void_p),
        ("route_min_tokens", C.c_int32), ("route_max_tokens", C.c_int32),
    ]


class AppendArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("arenas_per_batch", C.c_int32), ("max_dim", C.c_int32),
        ("new_k", C.c_void_p), ("new_v", C.c_void_p), ("len_k", C.c_void_p), ("len_v", C.c_void_p),
        ("k_basis", C.c_void_p), ("v_basis", C.c_void_p),
        ("k", Side), ("v", Side),
        ("seq_pos", C.c_int32), ("seq_lens", C.c_void_p), ("seq_capacity", C.c_int32),
        ("len_multiple", C.c_int32), ("status", C.c_void_p), ("stream", C.c_void_p),
        ("tickets", C.c_void_p),
    ]


class PackArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("batch", C.c_int32), ("arenas_per_batch", C.c_int32), ("n_new", C.c_int32),
        ("max_dim", C.c_int32),
        ("states", C.c_void_p), ("stride_b", C.c_int64), ("stride_j", C.c_int64), ("stride_s", C.c_int64),
        ("new_lens", C.c_void_p), ("row_counts", C.c_void_p), ("seq_lens", C.c_void_p), ("side", Side),
        ("seq_pos", C.c_int32), ("seq_capacity", C.c_int32), ("len_multiple", C.c_int32),
        ("status", C.c_void_p), ("stream", C.c_void_p),
    ]


class ProjectArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("n_tokens", C.c_int32), ("n_heads", C.c_int32),
        ("x", C.c_void_p), ("x_stride", C.c_int64), ("basis", C.c_void_p), ("out", C.c_void_p), ("out_stride", C.c_int64),
        ("status", C.c_void_p), ("stream", C.c_void_p),
    ]


class GateArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("n_rows", C.c_int32), ("dim", C.c_int32), ("low_rank", C.c_int32),
        ("threshold", C.c_float),
        ("x", C.c_void_p), ("x_stride", C.c_int64), ("w", C.c_void_p), ("b", C.c_void_p),
        ("lengths", C.c_void_p), ("masked", C.c_void_p), ("masked_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("len_multiple", C.c_int32), ("native_rounding", C.c_int32),
    ]


_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the shared library; raise (never fall back) when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m dynakv_b200.build` "
            "(dynakv_b200 has no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.dkv_version.restype = C.c_int
    lib.dkv_last_error.restype = C.c_char_p
    for name in ("dkv_fused_decode", "dkv_split_decode", "dkv_split_combine", "dkv_two_stage_decode",
                 "dkv_two_stage_decode_noalloc", "dkv_scores"):
        fn = getattr(lib, name)
        fn.argtypes = [C.POINTER(AttnArgs)]
        fn.restype = C.c_int
    lib.dkv_split_workspace_bytes.argtypes = [C.POINTER(AttnArgs)]
    lib.dkv_split_workspace_bytes.restype = C.c_size_t
    lib.dkv_softmax_v.argtypes = [C.POINTER(AttnArgs), C.c_void_p, C.c_int64, C.c_int64]
    lib.dkv_softmax_v.restype = C.c_int
    lib.dkv_append_decode.argtypes = [C.POINTER(AppendArgs)]
    lib.dkv_append_decode.restype = C.c_int
    lib.dkv_pack_bulk.argtypes = [C.POINTER(PackArgs)]
    lib.dkv_pack_bulk.restype = C.c_int
    lib.dkv_decompress.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(Side), C.c_void_p, C.c_void_p]
    lib.dkv_decompress.restype = C.c_int
    lib.dkv_gate_lengths.argtypes = [C.POINTER(GateArgs)]
    lib.dkv_gate_lengths.restype = C.c_int
    lib.dkv_gate_workspace_bytes.argtypes = [C.POINTER(GateArgs)]
    lib.dkv_gate_workspace_bytes.restype = C.c_size_t
    lib.dkv_gate_lengths_pair.argtypes = [C.POINTER(GateArgs), C.POINTER(GateArgs)]
    lib.dkv_gate_lengths_pair.restype = C.c_int
    lib.dkv_project_bulk.argtypes = [C.POINTER(ProjectArgs)]
    lib.dkv_project_bulk.restype = C.c_int
    lib.dkv_probe_tensor_pipe.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.dkv_probe_tensor_pipe.restype = C.c_int
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().dkv_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected float32, float16 or bfloat16") from None


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("dynakv_b200 operators need CUDA tensors; there is no CPU path")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def make_side(flat: torch.Tensor, lens: torch.Tensor, offs: torch.Tensor,
              wptr: Optional[torch.Tensor] = None) -> Side:
    """flat [n_arena, cap]; lens/offs [n_arena, S] (any strides); wptr [n_arena] int32."""
    if flat.dim() != 2 or flat.stride(1) != 1:
        raise ValueError("flat buffer must be [n_arena, capacity] with contiguous rows")
    if lens.dtype != torch.int32 or offs.dtype != torch.int32:
        raise TypeError("lengths and offsets must be int32")
    s = Side()
    s.flat, s.flat_stride = flat.data_ptr(), flat.stride(0)
    s.lens, s.lens_stride_a, s.lens_stride_s = lens.data_ptr(), lens.stride(0), (lens.stride(1) if lens.shape[1] > 1 else 1)
    s.offs, s.offs_stride_a, s.offs_stride_s = offs.data_ptr(), offs.stride(0), (offs.stride(1) if offs.shape[1] > 1 else 1)
    s.ptr = ptr(wptr)
    return s
