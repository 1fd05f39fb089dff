"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

No dataset, tokenizer or checkpoint is involved: bases are orthonormal matrices from a seeded QR,
cached coefficients are N(0, sigma_i^2) with sigma_i = exp(-i/32), and per-token cutoffs r_t are drawn
from the distribution each configuration names (always multiples of 8 in [8, 128]).
Everything is generated with torch on the device it is asked for, so the same code builds the small
CPU inputs of the tests and the multi-GB device-resident caches of the benchmark.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

HEAD_DIM = 128
RANK = 128


def qr_bases(n: int, seed: int, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """[n, 128, 128]: row r of basis i is the r-th orthonormal direction (fp64 QR -> fp32 -> dtype)."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        m = torch.randn(HEAD_DIM, HEAD_DIM, generator=gen, dtype=torch.float64)
        q, _ = torch.linalg.qr(m)
        out.append(q.T.contiguous().to(torch.float32))
    return torch.stack(out).to(dtype).to(device)


def quantise_r(x: torch.Tensor) -> torch.Tensor:
    """Fraction in [0,1] -> multiple of 8 in [8,128]: r = 8*clip(rint(16x), 1, 16)."""
    return (8 * torch.clamp(torch.round(16.0 * x), 1, 16)).to(torch.int32)


def draw_lengths(shape, dist: str, gen: torch.Generator, device="cpu") -> torch.Tensor:
    """dist: 'uniform' (multiples of 8 in [8,128]) or 'beta:a,b' (Beta(a,b) fraction, quantised)."""
    if dist == "uniform":
        return (8 * torch.randint(1, 17, shape, generator=gen, device=device)).to(torch.int32)
    if dist.startswith("beta:"):
        a, b = (float(v) for v in dist[5:].split(","))
        # Beta(a,b) = Ga/(Ga+Gb); gamma variates from torch's seeded generator via _standard_gamma
        ga = torch._standard_gamma(torch.full(shape, a, device=device), generator=gen)
        gb = torch._standard_gamma(torch.full(shape, b, device=device), generator=gen)
        return quantise_r(ga / (ga + gb))
    raise ValueError(f"unknown length distribution {dist!r}")


@dataclass
class Side:
    flat: torch.Tensor   # [rows, capacity]
    lens: torch.Tensor   # [rows, seq_capacity] int32
    offs: torch.Tensor   # [rows, seq_capacity] int32
    ptr: torch.Tensor    # [rows] int32


def ragged_side(lens: torch.Tensor, gen: torch.Generator, dtype, flat_capacity: Optional[int] = None,
                seq_capacity: Optional[int] = None) -> Side:
    """Fill one side of a cache from lengths [rows, S]: coefficients N(0, exp(-i/32)^2), packed gap-free."""
    dev = lens.device
    rows, S = lens.shape
    lens64 = lens.to(torch.int64)
    incl = torch.cumsum(lens64, dim=1)
    offs = (incl - lens64)
    tot = incl[:, -1] if S > 0 else torch.zeros(rows, dtype=torch.int64, device=dev)
    cap = int(tot.max().item()) if rows and S else 0
    cap = max((max(cap, flat_capacity or 0) + 7) // 8 * 8, 8)
    scap = (max(seq_capacity or S, S, 1) + 3) // 4 * 4
    flat = torch.zeros((rows, cap), dtype=dtype, device=dev)
    sigma = torch.exp(-torch.arange(RANK, dtype=torch.float32, device=dev) / 32.0)
    tot_host = tot.cpu().tolist()
    n_all = int(sum(tot_host))
    if n_all:
        # all rows at once: element e of the concatenation belongs to token tok[e] and is its idx-th coefficient
        lens_flat = lens64.reshape(-1)
        starts = torch.cumsum(lens_flat, 0) - lens_flat
        tok = torch.repeat_interleave(torch.arange(rows * S, device=dev), lens_flat)
        idx = torch.arange(n_all, device=dev) - starts[tok]
        del tok
        vals = (torch.randn(n_all, generator=gen, device=dev) * sigma[idx]).to(dtype)
        del idx
        pos = 0
        for r in range(rows):
            n = tot_host[r]
            flat[r, :n] = vals[pos:pos + n]
            pos += n
    lens_buf = torch.zeros((rows, scap), dtype=torch.int32, device=dev)
    offs_buf = torch.zeros((rows, scap), dtype=torch.int32, device=dev)
    lens_buf[:, :S] = lens
    offs_buf[:, :S] = offs.to(torch.int32)
    return Side(flat, lens_buf, offs_buf, tot.to(torch.int32))


@dataclass
class LayerCase:
    """One attention layer's decode inputs in the per-KV-head layout."""
    q: torch.Tensor            # [B, Hq, D] rotated queries
    k_up: torch.Tensor         # [Hkv, R, D]
    v_up: torch.Tensor
    k: Side
    v: Side
    seq_lens: List[int]        # tokens per batch row
    S: int                     # max tokens (columns in use)
    theta: float
    n_q_heads: int
    n_kv_heads: int

    def views(self):
        S = self.S
        return (self.k.flat, self.v.flat, self.k.lens[:, :S], self.v.lens[:, :S], self.k.offs[:, :S], self.v.offs[:, :S])

    def compressed_bytes(self) -> int:
        es = self.k.flat.element_size()
        return int((self.k.ptr.sum().item() + self.v.ptr.sum().item()) * es)

    def retention(self) -> float:
        n_tok = sum(self.seq_lens) * self.n_kv_heads
        return float((self.k.ptr.sum().item() + self.v.ptr.sum().item()) / (2.0 * n_tok * RANK)) if n_tok else 0.0


def make_layer_case(seed: int, seq_lens: Sequence[int], dist: str, theta: float, dtype, device="cpu",
                    n_q_heads: int = 32, n_kv_heads: int = 8, extra_tokens: int = 0,
                    basis_seed: Optional[int] = None) -> LayerCase:
    """Ragged batch: row b holds seq_lens[b] tokens (right-padded with zero-length tokens up to the max)."""
    B = len(seq_lens)
    S = max(seq_lens) if B else 0
    gen_cpu = torch.Generator().manual_seed(seed)
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed) if dev.type == "cuda" else gen_cpu
    rows = B * n_kv_heads
    lk = draw_lengths((rows, S), dist, gen, dev)
    lv = draw_lengths((rows, S), dist, gen, dev)
    sl = torch.tensor(list(seq_lens), device=dev).repeat_interleave(n_kv_heads)
    pad = torch.arange(S, device=dev)[None, :] >= sl[:, None]
    lk = lk.masked_fill(pad, 0)
    lv = lv.masked_fill(pad, 0)
    cap_extra = extra_tokens * RANK
    k = ragged_side(lk, gen, dtype, flat_capacity=None, seq_capacity=S + extra_tokens)
    v = ragged_side(lv, gen, dtype, flat_capacity=None, seq_capacity=S + extra_tokens)
    if extra_tokens:
        for side in (k, v):
            grown = torch.zeros((rows, side.flat.shape[1] + cap_extra), dtype=dtype, device=dev)
            grown[:, : side.flat.shape[1]] = side.flat
            side.flat = grown
    bs = basis_seed if basis_seed is not None else seed + 7
    k_up = qr_bases(n_kv_heads, bs, dtype, dev)
    v_up = qr_bases(n_kv_heads, bs + 1, dtype, dev)
    q = torch.randn(B, n_q_heads, HEAD_DIM, generator=gen_cpu).to(dtype).to(dev)
    return LayerCase(q, k_up, v_up, k, v, list(seq_lens), S, theta, n_q_heads, n_kv_heads)


def cutoff_head_lengths(hidden: torch.Tensor, weight: torch.Tensor, bias: float) -> torch.Tensor:
    """Synthetic linear cutoff head of the long-cache configuration: score = sigmoid(h.w + bias) in fp32,
    r = 8*clip(ceil(16*score), 1, 16).  hidden [B, 4096], weight [n_out, 4096] -> int32 [B, n_out]."""
    score = torch.sigmoid(hidden.to(torch.float32) @ weight.to(torch.float32).T + bias)
    return (8 * torch.clamp(torch.ceil(16.0 * score), 1, 16)).to(torch.int32)


def log_uniform_lengths(n: int, lo: int, hi: int, seed: int) -> List[int]:
    gen = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=gen, dtype=torch.float64)
    return [int(math.floor(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo))))) for x in u]
