"""Runtime routing between the short (fused) and long (split two-stage) decode kernels.

Mirrors src/dynakv/kernels/router.py of the reference: ``KernelPolicy(switch_tokens=500)`` and the
keyword-only ``compressed_decode_attention``.  Extension: with ``seq_lens`` (one cache length per batch
row, on the device) every sequence is routed on its own length *by the kernels themselves*: both kernels
are launched over the whole batch with the policy's switch point as a bound, each skips the rows that
belong to the other, and nothing is copied to or from the host -- so a ragged batch that straddles the
switch point, or a row that crosses it between two steps of a captured graph, is handled without
re-partitioning.  ``seq_lens_host`` (the same lengths as python ints) only lets the call skip a kernel
that has no row to process.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass(frozen=True)
class KernelPolicy:
    """Select the fused kernel below ``switch_tokens`` and two-stage at or above it."""

    switch_tokens: int = 500

    def select(self, cache_length: int) -> str:
        if cache_length < 0:
            raise ValueError("cache_length must be non-negative")
        return "short_fused" if cache_length < self.switch_tokens else "long_two_stage"

    def partition(self, cache_lengths: Sequence[int]):
        """Split batch rows by route; returns (short_rows, long_rows) as lists of row indices."""
        short, long_ = [], []
        for i, n in enumerate(cache_lengths):
            (short if self.select(int(n)) == "short_fused" else long_).append(i)
        return short, long_


def compressed_decode_attention(
    *, q, k_flat, k_up, v_flat, v_up, key_lengths, key_offsets,
    value_lengths, value_offsets, theta: float, cache_length: int,
    policy: Optional[KernelPolicy] = None,
    seq_lens: Optional[torch.Tensor] = None,
    seq_lens_host: Optional[Sequence[int]] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    k_norm_eps: float = 1e-6,
    len_multiple: int = 1,
):
    """Run the kernel selected from the current physical cache length; returns [B, Hq, D]."""
    from .fused import fused_attention_dispatch
    from .two_stage import two_stage_attention

    policy = policy or KernelPolicy()
    common = dict(k_norm_weight=k_norm_weight, k_norm_eps=k_norm_eps, len_multiple=len_multiple, seq_lens=seq_lens)
    args = (q, k_flat, k_up, v_flat, v_up, key_lengths, key_offsets, value_lengths, value_offsets, theta)
    if seq_lens is None:
        if seq_lens_host is not None:
            raise ValueError("seq_lens_host needs the matching device tensor seq_lens")
        if policy.select(cache_length) == "short_fused":
            return fused_attention_dispatch(*args, **common)
        return two_stage_attention(*args, **common)

    # per-row routing on the device
    q3 = q.squeeze(2) if q.dim() == 4 else q
    out = torch.empty((q3.shape[0], q3.shape[1], q3.shape[2]), dtype=q3.dtype, device=q3.device)
    any_short, any_long = True, True
    if seq_lens_host is not None:
        short, long_ = policy.partition(seq_lens_host)
        any_short, any_long = bool(short), bool(long_)
    if any_short:
        fused_attention_dispatch(*args, out=out, route_max_tokens=policy.switch_tokens if any_long else 0, **common)
    if any_long:
        two_stage_attention(*args, out=out, route_min_tokens=policy.switch_tokens if any_short else 0, **common)
    return out
