"""Long-cache decode attention (replaces src/dynakv/kernels/two_stage.py of the reference).

``two_stage_attention`` is what the router uses: a split-KV kernel writes per-split
(max, sum, latent accumulator) partials and a combine kernel merges them and applies the V
up-projection.  ``abx_sparse`` and ``avx`` keep the reference's stage-1 / stage-2 operators
(scores materialised in the query dtype, its masking constant) for callers that use them directly.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib
from ._common import build_attn_args


def two_stage_attention(q, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, *,
                        seq_lens: Optional[torch.Tensor] = None, batch_index: Optional[torch.Tensor] = None,
                        k_norm_weight: Optional[torch.Tensor] = None, k_norm_eps: float = 1e-6,
                        len_multiple: int = 1, out: Optional[torch.Tensor] = None,
                        route_min_tokens: int = 0, route_max_tokens: int = 0):
    """Same arguments and result as ``fused_attention_dispatch``; split-KV execution."""
    q3 = q.squeeze(2) if q.dim() == 4 else q
    if out is None:
        out = torch.empty((q3.shape[0], q3.shape[1], q3.shape[2]), dtype=q3.dtype, device=q3.device)
    args, keep = build_attn_args(q3, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, out=out,
                                 seq_lens=seq_lens, batch_index=batch_index, k_norm_weight=k_norm_weight,
                                 k_norm_eps=k_norm_eps, len_multiple=len_multiple, need_workspace=True,
                                 route_min_tokens=route_min_tokens, route_max_tokens=route_max_tokens)
    _lib.check(_lib.load().dkv_two_stage_decode(C.byref(args)), "dkv_two_stage_decode")
    del keep
    return out


def two_stage_attention_noalloc(q, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, *, out: torch.Tensor,
                                seq_lens: Optional[torch.Tensor] = None, batch_index: Optional[torch.Tensor] = None,
                                k_norm_weight: Optional[torch.Tensor] = None, k_norm_eps: float = 1e-6,
                                len_multiple: int = 8):
    """``two_stage_attention`` for processes that must not allocate device memory while serving: the
    caller passes the output tensor, and the split partials go to a fixed 2 MiB array inside the library
    instead of a torch workspace.  Raises when the call needs more scratch than that (large batches) or when
    the cache does not qualify for the split tensor-core path.  Calls on one device must not overlap.
    It is the library call that allocates nothing: this wrapper still creates the device status word with torch
    on its first use on a device (and small fp32 copies when ``k_norm_weight`` is not fp32 already), so call it
    once before the section that must not allocate."""
    q3 = q.squeeze(2) if q.dim() == 4 else q
    args, keep = build_attn_args(q3, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, out=out,
                                 seq_lens=seq_lens, batch_index=batch_index, k_norm_weight=k_norm_weight,
                                 k_norm_eps=k_norm_eps, len_multiple=len_multiple, need_workspace=False)
    _lib.check(_lib.load().dkv_two_stage_decode_noalloc(C.byref(args)), "dkv_two_stage_decode_noalloc")
    del keep
    return out


def abx_sparse(a: torch.Tensor, b: torch.Tensor, x_flat: torch.Tensor, l_vec: torch.Tensor,
               offsets: torch.Tensor = None, theta: float = 10000.0) -> torch.Tensor:
    """Scaled scores [B, Hq, S] in a's dtype; a = rotated queries [B,Hq,D], b = K basis [groups,R,D]."""
    if offsets is None:
        raise ValueError("offsets are required for the variable-length key cache")
    batch, heads, _ = a.shape
    seq_len = l_vec.shape[-1]
    out = torch.empty((batch, heads, seq_len), dtype=a.dtype, device=a.device)
    args, keep = build_attn_args(a, x_flat, b, None, None, l_vec, offsets, None, None, theta, out=out)
    _lib.check(_lib.load().dkv_scores(C.byref(args)), "dkv_scores")
    del keep
    return out


def avx(a: torch.Tensor, x_flat: torch.Tensor, v_up: torch.Tensor, l_vec: torch.Tensor,
        offsets: torch.Tensor = None) -> torch.Tensor:
    """softmax(a) applied to the compressed values; a = scores [B,Hq,S] or [B,Hq,1,S]."""
    if a.ndim == 4:
        a = a.squeeze(2)
    if offsets is None:
        raise ValueError("offsets are required for the variable-length value cache")
    if a.stride(-1) != 1:
        a = a.contiguous()
    batch, heads, _ = a.shape
    out = torch.empty((batch, heads, v_up.shape[-1]), dtype=a.dtype, device=a.device)
    args, keep = build_attn_args(None, None, None, x_flat, v_up, None, None, l_vec, offsets, 10000.0, out=out)
    _lib.check(_lib.load().dkv_softmax_v(C.byref(args), a.data_ptr(), a.stride(0), a.stride(1)), "dkv_softmax_v")
    del keep
    return out
