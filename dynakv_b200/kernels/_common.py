"""Argument marshalling shared by the decode-attention entry points."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from .. import _lib

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_status: Dict[int, torch.Tensor] = {}
_n_sm: Dict[int, int] = {}


def n_sm(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _n_sm:
        _n_sm[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _n_sm[idx]


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels OR their DKV_ST_* conditions into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def read_status(device: torch.device, clear: bool = True) -> int:
    """Synchronising read of the device status word (0 = nothing to report)."""
    w = status_word(device)
    v = int(w.item())
    if clear and v:
        w.zero_()
    return v


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only scratch buffer per device, reused by every split-path call on the current stream."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, 0)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def arena_rows(t: torch.Tensor, what: str) -> torch.Tensor:
    """View [B, H, X] as [B*H, X] without copying; 2-D tensors pass through."""
    if t.dim() == 2:
        return t
    if t.dim() != 3:
        raise ValueError(f"{what}: expected a 2-D [rows, X] or 3-D [B, Hkv, X] tensor, got {tuple(t.shape)}")
    b, h, x = t.shape
    if b > 1 and t.stride(0) != h * t.stride(1):
        raise ValueError(f"{what}: batch and head axes cannot be folded without a copy")
    return t.as_strided((b * h, x), (t.stride(1), t.stride(2)))


def build_attn_args(q, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, *, out, seq_lens=None,
                    batch_index=None, k_norm_weight=None, k_norm_eps=1e-6, len_multiple=1, need_workspace=False,
                    route_min_tokens=0, route_max_tokens=0):
    """Fill a dkv_attn_args from torch tensors; returns (args, keepalive)."""
    lib = _lib.load()
    _lib.require_cuda(q, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, out)
    dev = out.device
    if q is not None and q.dim() == 4:
        q = q.squeeze(2)
    ref = q if q is not None else out
    B_total, Hq = ref.shape[0], ref.shape[1]
    D = k_up.shape[-1] if k_up is not None else v_up.shape[-1]
    basis = k_up if k_up is not None else v_up
    Hg, R = basis.shape[0], basis.shape[1]
    keep = [q, out]
    a = _lib.AttnArgs()
    a.dtype = _lib.dtype_code(out.dtype if q is None else q.dtype)
    a.n_q_heads, a.n_basis_groups, a.head_dim, a.rank = Hq, Hg, D, R
    if q is not None:
        if q.stride(-1) != 1:
            q = q.contiguous()
            keep.append(q)
        a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    for name, t in (("k_up", k_up), ("v_up", v_up)):
        if t is not None:
            if not t.is_contiguous():
                t = t.contiguous()
            keep.append(t)
            setattr(a, name, t.data_ptr())
    n_arena = None
    S = 0
    for side_name, flat, lens, offs in (("k", k_flat, l_k, o_k), ("v", v_flat, l_v, o_v)):
        if flat is None:
            continue
        flat2, lens2, offs2 = arena_rows(flat, side_name + "_flat"), arena_rows(lens, side_name + " lengths"), \
            arena_rows(offs, side_name + " offsets")
        if flat2.dtype != out.dtype and q is not None and flat2.dtype != q.dtype:
            raise TypeError("cache payload and query must share a dtype")
        setattr(a, side_name, _lib.make_side(flat2, lens2, offs2))
        keep += [flat2, lens2, offs2]
        n_arena, S = lens2.shape[0], lens2.shape[1]
    if n_arena is None:
        raise ValueError("at least one cache side is required")
    if n_arena % B_total != 0:
        raise ValueError(f"arena rows ({n_arena}) must be a multiple of the batch size ({B_total})")
    a.arenas_per_batch = n_arena // B_total
    a.seq_len = S
    if batch_index is not None:
        if batch_index.dtype != torch.int32:
            raise TypeError("batch_index must be int32")
        a.batch_index = batch_index.data_ptr()
        a.batch = batch_index.numel()
        keep.append(batch_index)
    else:
        a.batch = B_total
    if seq_lens is not None:
        if seq_lens.dtype != torch.int32 or seq_lens.numel() != B_total:
            raise TypeError("seq_lens must be an int32 tensor with one entry per batch row")
        a.seq_lens = seq_lens.data_ptr()
        keep.append(seq_lens)
    if k_norm_weight is not None:
        w = k_norm_weight.to(device=dev, dtype=torch.float32).contiguous()
        a.k_norm_weight = w.data_ptr()
        keep.append(w)
    a.k_norm_eps = float(k_norm_eps)
    a.theta = float(theta)
    a.len_multiple = int(len_multiple)
    a.route_min_tokens, a.route_max_tokens = int(route_min_tokens), int(route_max_tokens)
    if (a.route_min_tokens or a.route_max_tokens) and seq_lens is None:
        raise ValueError("device-side routing needs seq_lens (one cache length per batch row on the device)")
    a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    st = status_word(dev)
    a.status = st.data_ptr()
    a.n_sm = n_sm(dev)
    a.stream = _lib.stream_ptr(dev)
    if need_workspace:
        nbytes = lib.dkv_split_workspace_bytes(C.byref(a))
        if nbytes:
            ws = workspace(dev, nbytes)
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            keep.append(ws)
    return a, keep
