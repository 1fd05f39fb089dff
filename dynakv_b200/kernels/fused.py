"""Short-cache fused decode attention (replaces src/dynakv/kernels/fused.py of the reference).

One launch: gather the ragged coefficient rows, reconstruct K against the basis, rotate, QK,
online softmax, latent-space V accumulation and the V up-projection.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib
from ._common import build_attn_args


def fused_attention_dispatch(q, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, *,
                             seq_lens: Optional[torch.Tensor] = None,
                             batch_index: Optional[torch.Tensor] = None,
                             k_norm_weight: Optional[torch.Tensor] = None, k_norm_eps: float = 1e-6,
                             len_multiple: int = 1, out: Optional[torch.Tensor] = None,
                             route_min_tokens: int = 0, route_max_tokens: int = 0):
    """q [B,Hq,1,D] or [B,Hq,D] (already rotated); flat buffers [B,cap] (joint latent rows, as in the
    reference) or [B*Hkv,cap] / [B,Hkv,cap] (per-KV-head arenas); bases [Hkv or Hq, R, D];
    lengths/offsets int32 [rows, S] views.  Returns [B, Hq, D] in q's dtype.

    ``len_multiple=8`` declares gap-free rows whose lengths are all multiples of 8, which selects the
    tensor-core kernel; the default makes no assumption and uses the generic kernel.
    """
    q3 = q.squeeze(2) if q.dim() == 4 else q
    if out is None:
        out = torch.empty((q3.shape[0], q3.shape[1], q3.shape[2]), dtype=q3.dtype, device=q3.device)
    args, keep = build_attn_args(q3, k_flat, k_up, v_flat, v_up, l_k, o_k, l_v, o_v, theta, out=out,
                                 seq_lens=seq_lens, batch_index=batch_index, k_norm_weight=k_norm_weight,
                                 k_norm_eps=k_norm_eps, len_multiple=len_multiple, route_min_tokens=route_min_tokens,
                                 route_max_tokens=route_max_tokens)
    _lib.check(_lib.load().dkv_fused_decode(C.byref(args)), "dkv_fused_decode")
    del keep
    return out
