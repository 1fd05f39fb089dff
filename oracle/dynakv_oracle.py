"""CPU oracle for the DynaKV physical compressed-cache decode path.

TEST INFRASTRUCTURE ONLY.  This file restates, in plain torch-CPU / numpy fp32
code, the algorithm of the reference's decode path so that the CUDA kernels can
be checked against it.  It is imported by the test-suite, by the smoke check
and by the benchmark's CPU-baseline / reference arm, and by nothing else; the
product package never imports it and has no CPU fallback.

Parity status: PINNED.  Every function here is checked (tests/test_oracle_golden.py)
against fixtures under tests/golden/ that were produced by running the
reference's own code on CPU (research attention math, the Triton kernels under
the Triton interpreter, and the cache-update code); the generating script is
tests/golden/make_golden.py.  The reference ships no golden vectors of its own
for this path (its only hot-path tests pin the router boundary).

Reference locations restated (paths inside the reference project):
  * cache layout ............ src/dynakv/kernels/compressed_cache.py:7-34, 36-56, 182-209
  * fused decode math ....... src/dynakv/kernels/fused.py:28-142
  * scores / softmax-V ...... src/dynakv/kernels/two_stage.py:52-157, 211-281
  * research (compact) math . src/dynakv/custom_attn.py:21-25, 161-168, 237-255, 285-301
  * cutoff gate ............. src/dynakv/kernels/compressed_attention.py:84-119
  * router .................. src/dynakv/kernels/router.py:8-17
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

# --------------------------------------------------------------------------
# Router (src/dynakv/kernels/router.py:8-17)
# --------------------------------------------------------------------------


def select_path(cache_length: int, switch_tokens: int = 500) -> str:
    if cache_length < 0:
        raise ValueError("cache_length must be non-negative")
    return "short_fused" if cache_length < switch_tokens else "long_two_stage"


# --------------------------------------------------------------------------
# Cache layout (src/dynakv/kernels/compressed_cache.py)
# --------------------------------------------------------------------------


def pack_prefill(states: np.ndarray, lens: np.ndarray, start_ptr: Optional[np.ndarray] = None):
    """Pack rows of a prefill block.  compressed_cache.py:184-209.

    states [N, S, max_dim], lens [N, S] int.  Returns (flat list of 1-D arrays,
    offs [N, S] int32, new_ptr [N] int32): offs is the exclusive prefix sum of
    lens starting from start_ptr, flat[n] the kept coefficients back to back.
    """
    n_rows, s_new, max_dim = states.shape
    lens = lens.astype(np.int64)
    if start_ptr is None:
        start_ptr = np.zeros(n_rows, dtype=np.int64)
    offs = np.zeros((n_rows, s_new), dtype=np.int64)
    flats = []
    new_ptr = np.zeros(n_rows, dtype=np.int64)
    for n in range(n_rows):
        cum = np.cumsum(lens[n])
        offs[n] = start_ptr[n] + np.concatenate([[0], cum[:-1]]) if s_new else offs[n]
        mask = np.arange(max_dim)[None, :] < lens[n][:, None]
        flats.append(states[n][mask])
        new_ptr[n] = start_ptr[n] + (cum[-1] if s_new else 0)
    return flats, offs.astype(np.int32), new_ptr.astype(np.int32)


class LayoutOracle:
    """Growing ragged arena with the reference's invariants (one side, K or V).

    lens[n, s] = r_s ; offs[n, s] = sum_{t<s} lens[n, t] ; flat[n, offs:offs+len]
    = first len coefficients ; ptr[n] = sum_s lens[n, s] ; seq = tokens stored.
    Prefill = compressed_cache.py:184-209, decode append = :7-34.
    """

    def __init__(self, n_rows: int, dtype):
        self.n = n_rows
        self.flat = [np.zeros(0, dtype=dtype) for _ in range(n_rows)]
        self.lens = np.zeros((n_rows, 0), dtype=np.int32)
        self.offs = np.zeros((n_rows, 0), dtype=np.int32)
        self.ptr = np.zeros(n_rows, dtype=np.int32)
        self.seq = 0

    def update(self, states: np.ndarray, lens: np.ndarray):
        flats, offs, new_ptr = pack_prefill(states, lens, self.ptr.astype(np.int64))
        for n in range(self.n):
            self.flat[n] = np.concatenate([self.flat[n], flats[n].astype(self.flat[n].dtype)])
        self.lens = np.concatenate([self.lens, lens.astype(np.int32)], axis=1)
        self.offs = np.concatenate([self.offs, offs], axis=1)
        self.ptr = new_ptr
        self.seq += states.shape[1]

    def flat_padded(self, cap: Optional[int] = None) -> np.ndarray:
        cap = cap or max(1, int(self.ptr.max()))
        out = np.zeros((self.n, cap), dtype=self.flat[0].dtype)
        for n in range(self.n):
            out[n, : self.flat[n].size] = self.flat[n]
        return out


def decompress(flat: np.ndarray, lens: np.ndarray, max_dim: int, offs: Optional[np.ndarray] = None):
    """Ragged -> dense zero-padded [N, S, max_dim].  compressed_cache.py:36-56.

    Without offs the rows are assumed gap-free from element 0 (what the
    reference assumes); with offs each token is gathered from its own offset
    (what the reference kernels do: fused.py:86, two_stage.py:117).
    """
    n_rows, s = lens.shape
    out = np.zeros((n_rows, s, max_dim), dtype=flat.dtype)
    for n in range(n_rows):
        run = 0
        for t in range(s):
            ln = int(min(lens[n, t], max_dim))
            o = int(offs[n, t]) if offs is not None else run
            out[n, t, :ln] = flat[n, o : o + ln]
            run += int(lens[n, t])
    return out


def decompress_gather(flat: np.ndarray, lens: np.ndarray, offs: np.ndarray, max_dim: int) -> np.ndarray:
    """Same result as ``decompress(flat, lens, max_dim, offs)`` with whole-array numpy indexing, for caches of
    hundreds of thousands of tokens where the per-token loop above takes minutes (checked against it in
    tests/test_oracle_golden.py).  compressed_cache.py:36-56 / fused.py:86."""
    n_rows, s = lens.shape
    ln = np.minimum(lens.astype(np.int64), max_dim)
    idx = offs.astype(np.int64)[:, :, None] + np.arange(max_dim, dtype=np.int64)[None, None, :]
    keep = np.arange(max_dim)[None, None, :] < ln[:, :, None]
    idx = np.where(keep, idx, 0)
    rows = np.arange(n_rows)[:, None, None]
    return np.where(keep, flat[rows, idx], np.zeros((), dtype=flat.dtype))


# --------------------------------------------------------------------------
# RoPE (fused.py:65-66, 97-102; two_stage.py:28-46; custom_attn.py:21-25)
# --------------------------------------------------------------------------


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    j = torch.arange(0, head_dim // 2, dtype=torch.float32) * 2.0 / float(head_dim)
    return torch.exp(-j * math.log(theta))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    ang = positions.to(torch.float32)[..., None] * rope_inv_freq(head_dim, theta)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention: pairs (j, j + D/2).  x [..., S, D], cos/sin [S, D/2]."""
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Qwen3RMSNorm over the last axis: fp32 variance, weight multiplied after
    (custom_attn.py:285, 296 call the transformers module)."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return weight.to(torch.float32) * (xf * torch.rsqrt(var + eps))


# --------------------------------------------------------------------------
# Compact masked-dimension attention (the parity reference for outputs)
# --------------------------------------------------------------------------


def _dense_latents(flat, lens, offs, rank):
    f = flat.detach().to(torch.float32).cpu().numpy()
    dense = decompress(f, lens.cpu().numpy(), rank, offs.cpu().numpy())
    return torch.from_numpy(dense)


def compact_attention(
    q: torch.Tensor,
    k_flat: torch.Tensor,
    k_up: torch.Tensor,
    v_flat: torch.Tensor,
    v_up: torch.Tensor,
    l_k: torch.Tensor,
    o_k: torch.Tensor,
    l_v: torch.Tensor,
    o_v: torch.Tensor,
    theta: float,
    seq_lens: Optional[Sequence[int]] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    k_norm_eps: float = 1e-6,
) -> torch.Tensor:
    """Decode attention on a compressed cache in fp32.

    q [B, Hq, D] already rotated.  k_flat/v_flat [B*A, cap]; lens/offs
    [B*A, S] with A = arenas per batch row (1 = the reference's joint layout
    where all heads share one latent row, Hkv = one arena per KV head).
    k_up/v_up [Hg, R, D], Hg in {Hkv, Hq}.  Query head h uses basis h // (Hq/Hg)
    and arena b*A + h*A // Hq.

    Math: zero-masked dense latent -> up-projection (custom_attn.py:161-168) ->
    optional RMSNorm of K per head (custom_attn.py:296) -> RoPE of K at cache
    index (custom_attn.py:237-240, fused.py:97-102) -> scaled scores, fp32
    softmax (transformers eager attention) -> weighted V.  Tokens with
    key length 0 or index >= seq_lens[b] are excluded (fused.py:105-106).
    Returns [B, Hq, D] fp32.
    """
    q = q.detach().to(torch.float32).cpu()
    if q.dim() == 4:
        q = q.squeeze(2)
    B, Hq, D = q.shape
    Hg, R, _ = k_up.shape
    n_arena, S = l_k.shape
    A = n_arena // B
    ku = k_up.detach().to(torch.float32).cpu()
    vu = v_up.detach().to(torch.float32).cpu()
    xk = _dense_latents(k_flat, l_k, o_k, R)  # [B*A, S, R]
    xv = _dense_latents(v_flat, l_v, o_v, R)
    cos, sin = rope_cos_sin(torch.arange(S), D, theta)
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    lk = l_k.cpu()
    for b in range(B):
        sb = S if seq_lens is None else int(seq_lens[b])
        for h in range(Hq):
            g = h // (Hq // Hg)
            a = b * A + (h * A) // Hq
            k = xk[a] @ ku[g]  # [S, D]
            if k_norm_weight is not None:
                k = rms_norm(k, k_norm_weight.cpu(), k_norm_eps)
            k = apply_rope(k, cos, sin)
            s = (k @ q[b, h]) * scale
            valid = (lk[a] > 0) & (torch.arange(S) < sb)
            s = torch.where(valid, s, torch.full_like(s, float("-inf")))
            p = torch.softmax(s, dim=-1)
            p = torch.where(valid, p, torch.zeros_like(p))
            v = xv[a] @ vu[g]
            out[b, h] = p @ v
    return out


# --------------------------------------------------------------------------
# Two-stage compatibility semantics (two_stage.py)
# --------------------------------------------------------------------------


def scores_reference(q, k_up, k_flat, l_k, o_k, theta, out_dtype=torch.float32):
    """abx_sparse: [B, Hq, S] scaled scores; len-0 tokens get -1e4*scale
    (two_stage.py:153-155); result rounded to the query dtype (:157)."""
    q = q.detach().to(torch.float32).cpu()
    B, Hq, D = q.shape
    Hg, R, _ = k_up.shape
    n_arena, S = l_k.shape
    A = n_arena // B
    ku = k_up.detach().to(torch.float32).cpu()
    xk = _dense_latents(k_flat, l_k, o_k, R)
    cos, sin = rope_cos_sin(torch.arange(S), D, theta)
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq, S, dtype=torch.float32)
    for b in range(B):
        for h in range(Hq):
            g = h // (Hq // Hg)
            a = b * A + (h * A) // Hq
            k = apply_rope(xk[a] @ ku[g], cos, sin)
            s = k @ q[b, h]
            s = torch.where(l_k[a].cpu() > 0, s, torch.full_like(s, -1.0e4))
            out[b, h] = s * scale
    return out.to(out_dtype)


def softmax_v_reference(scores, v_flat, v_up, l_v, o_v):
    """avx: softmax over stored scores, accumulate p*x_v in latent space,
    divide by max(l, 1e-6), project through v_up[h // group] (two_stage.py:247-277)."""
    sc = scores.detach().to(torch.float32).cpu()
    if sc.dim() == 4:
        sc = sc.squeeze(2)
    B, Hq, S = sc.shape
    Hkv, R, D = v_up.shape
    n_arena = l_v.shape[0]
    A = n_arena // B
    vu = v_up.detach().to(torch.float32).cpu()
    xv = _dense_latents(v_flat, l_v, o_v, R)
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        for h in range(Hq):
            g = h // (Hq // Hkv)
            a = b * A + (h * A) // Hq
            m = sc[b, h].max()
            p = torch.exp(sc[b, h] - m)
            lat = (p[:, None] * xv[a]).sum(0) / torch.clamp(p.sum(), min=1e-6)
            out[b, h] = lat @ vu[g]
    return out


# --------------------------------------------------------------------------
# Cutoff gate (compressed_attention.py:84-119)
# --------------------------------------------------------------------------


def gate_lengths(x: torch.Tensor, W: torch.Tensor, b: torch.Tensor, low_rank: int) -> torch.Tensor:
    """len = #{i < low_rank : sum_{j <= R-1-i} softmax(xW+b)_j >= 0.1}, int32.

    x [N, d] spectral coefficient rows, W [d, d], b [d] or [1, d].
    """
    logits = torch.addmm(b.reshape(-1), x, W)
    m = torch.softmax(logits, dim=-1).cumsum(dim=-1).flip(dims=[-1])
    hard = m >= 0.1
    hard[..., int(low_rank):] = False
    return hard.sum(dim=-1, dtype=torch.int32)


def project_rows(x: torch.Tensor, basis: torch.Tensor) -> torch.Tensor:
    """Spectral coefficients of pre-RoPE rows: c[r] = sum_d x[d] * basis[r, d]
    (custom_attn.py:152 with the physical basis layout of
    compressed_attention.py:282).  x [N, Hkv, D], basis [Hkv, R, D] -> [N, Hkv, R] fp32."""
    return torch.einsum("nhd,hrd->nhr", x.to(torch.float32), basis.to(torch.float32))


def compact_attention_dense(q, xk, xv, k_up, v_up, theta, valid, k_norm_weight=None, k_norm_eps=1e-6):
    """The same compact attention as ``compact_attention`` on dense zero-masked latents, written with
    whole-tensor torch ops the way the research model runs it (custom_attn.py:161-168 einsum
    up-projection of the whole cache, :237-240 RoPE over 0..S-1, transformers eager attention with GQA
    head sharing).  Used as the timed CPU baseline.

    q [B,Hq,D]; xk/xv [B,Hkv,S,R]; k_up/v_up [Hkv,R,D]; valid [B,Hkv,S] bool.  Returns [B,Hq,D] fp32.
    """
    B, Hq, D = q.shape
    Hkv, S = xk.shape[1], xk.shape[2]
    G = Hq // Hkv
    k = torch.einsum("bhsr,hrd->bhsd", xk, k_up)
    if k_norm_weight is not None:
        k = rms_norm(k, k_norm_weight, k_norm_eps)
    cos, sin = rope_cos_sin(torch.arange(S), D, theta)
    k = apply_rope(k, cos, sin)
    v = torch.einsum("bhsr,hrd->bhsd", xv, v_up)
    scores = torch.einsum("bhgd,bhsd->bhgs", q.view(B, Hkv, G, D), k) * (D ** -0.5)
    scores = scores.masked_fill(~valid[:, :, None, :], float("-inf"))
    p = torch.softmax(scores, dim=-1, dtype=torch.float32)
    return torch.einsum("bhgs,bhsd->bhgd", p, v).reshape(B, Hq, D)
