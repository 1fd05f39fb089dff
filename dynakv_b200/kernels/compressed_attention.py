"""Decode-step caller of the physical path (the decode branch of the reference's attention module,
src/dynakv/kernels/compressed_attention.py:312-357, without the model plumbing around it).

``CompressedDecodeLayer.decode`` is the per-layer sequence the reference runs for every generated
token: append the new token's truncated K/V coefficient rows to the cache, then run the routed
compressed attention over the cache.  ``DecodeGraph`` captures that sequence for a stack of layers
in one CUDA graph with static input/output buffers (the reference replays its gate under a graph the
same way, compressed_attention.py:232-251), and offers ``step_from_host`` for callers whose per-step
inputs live in host memory.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _lib
from ._common import build_attn_args, status_word
from .compressed_cache import CustomDynamicCache
from .router import KernelPolicy


def merge_basis(up: torch.Tensor, n_kv_heads: int, head_dim: int, low_rank: Optional[int] = None) -> torch.Tensor:
    """Physical basis layout of the reference's one-time merge (compressed_attention.py:278-286):
    ``B[h, r, dd] = up[h*head_dim + dd, r]`` for a joint ``up`` of shape [n_kv_heads*head_dim, rank]."""
    rank = up.shape[1] if low_rank is None else int(low_rank)
    return up[:, :rank].reshape(n_kv_heads, head_dim, rank).transpose(1, 2).contiguous()


def project_bulk(x: torch.Tensor, basis: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Spectral coefficients of a block of pre-RoPE K (or V) rows for per-head bases, on the tensor core:
    ``out[..., h*128 + r] = sum_d x[..., h*128 + d] * basis[h, r, d]``.  ``x`` [..., Hkv*128] (the projection layer's
    output), ``basis`` [Hkv, 128, 128]; 16-bit types.  Stands in for the reference's one-time fold of the projection
    into ``k_proj`` / ``v_proj`` (kernels/compressed_attention.py:267-275); the result is what ``update_sp`` takes."""
    if not x.is_cuda:
        raise RuntimeError("dynakv_b200 has no CPU path: project_bulk needs CUDA tensors")
    n_heads = basis.shape[0]
    if basis.shape[1:] != (128, 128) or x.shape[-1] != n_heads * 128 or basis.dtype != x.dtype:
        raise ValueError("project_bulk takes x [..., Hkv*128] and basis [Hkv, 128, 128] of one 16-bit dtype")
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    o2 = out.view(-1, out.shape[-1])
    a = _lib.ProjectArgs()
    a.dtype, a.n_tokens, a.n_heads = _lib.dtype_code(x.dtype), x2.shape[0], n_heads
    a.x, a.x_stride, a.basis = x2.data_ptr(), x2.stride(0), basis.contiguous().data_ptr()
    a.out, a.out_stride = o2.data_ptr(), o2.stride(0)
    a.status, a.stream = status_word(x.device).data_ptr(), _lib.stream_ptr(x.device)
    _lib.check(_lib.load().dkv_project_bulk(C.byref(a)), "dkv_project_bulk")
    return out


_gate_scratch = {}


def _scratch(device, n_floats: int) -> torch.Tensor:
    """Grow-only fp32 scratch per device (reused by every gate call on the current stream)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _gate_scratch.get(key)
    if buf is None or buf.numel() < n_floats:
        buf = torch.empty(max(n_floats, 1 << 16), dtype=torch.float32, device=device)
        _gate_scratch[key] = buf
    return buf


def gate_lengths(states: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, low_rank: int,
                 threshold: float = 0.1, return_masked: bool = True, len_multiple: int = 1,
                 native_rounding: bool = True, out_lengths: Optional[torch.Tensor] = None):
    """Cutoff gate of one side (kernels/compressed_attention.py:84-119, one of the two halves of
    ``kv_process_fused``): ``states`` [..., d] spectral coefficient rows, ``weight`` [d, d], ``bias`` [d] or [1, d].

    Returns (masked states or None, lengths int32 [...]): lengths[t] = #{i < low_rank : cumsum(softmax(x W + b))
    [d-1-i] >= threshold}, masked = states with everything past the length zeroed.  fp32 sums; for 16-bit inputs
    ``native_rounding`` rounds the intermediates where the reference's torch ops do, so the lengths are the ones
    the reference computes in that dtype.  ``len_multiple=8`` rounds each length up to a multiple of 8 (a superset
    of the gate's choice), the form the tensor-core decode kernels take.
    """
    if not states.is_cuda:
        raise RuntimeError("dynakv_b200 has no CPU path: the gate needs CUDA tensors")
    d = states.shape[-1]
    if weight.shape != (d, d) or bias.numel() != d:
        raise ValueError(f"gate weight must be [{d}, {d}] and bias [{d}], got {tuple(weight.shape)} and {tuple(bias.shape)}")
    if weight.dtype != states.dtype or bias.dtype != states.dtype:
        raise ValueError("gate weight, bias and states must share a dtype")
    x = states.reshape(-1, d)
    if x.stride(-1) != 1:
        x = x.contiguous()
    w, b = weight.contiguous(), bias.reshape(-1).contiguous()
    if out_lengths is not None:     # caller-owned output (e.g. a static buffer of a captured graph): nothing is allocated
        if out_lengths.dtype != torch.int32 or out_lengths.numel() != x.shape[0] or not out_lengths.is_contiguous():
            raise ValueError("out_lengths must be a contiguous int32 tensor with one entry per row")
        lengths = out_lengths.view(-1)
    else:
        lengths = torch.empty(x.shape[0], dtype=torch.int32, device=states.device)
    masked = torch.empty((x.shape[0], d), dtype=states.dtype, device=states.device) if return_masked else None
    a = _lib.GateArgs()
    a.dtype, a.n_rows, a.dim, a.low_rank, a.threshold = _lib.dtype_code(states.dtype), x.shape[0], d, int(low_rank), threshold
    a.x, a.x_stride, a.w, a.b = x.data_ptr(), x.stride(0), w.data_ptr(), b.data_ptr()
    a.lengths = lengths.data_ptr()
    a.masked, a.masked_stride = (masked.data_ptr(), masked.stride(0)) if return_masked else (None, 0)
    lib = _lib.load()
    need = lib.dkv_gate_workspace_bytes(C.byref(a))
    scratch = _scratch(states.device, max(need, 4) // 4)
    a.workspace, a.workspace_bytes = scratch.data_ptr(), scratch.numel() * 4
    a.len_multiple, a.native_rounding = int(len_multiple), int(bool(native_rounding))
    a.stream = _lib.stream_ptr(states.device)
    _lib.check(lib.dkv_gate_lengths(C.byref(a)), "dkv_gate_lengths")
    lead = states.shape[:-1]
    return (masked.reshape(*lead, d) if return_masked else None), lengths.reshape(lead)


def gate_lengths_pair(k_rows: torch.Tensor, Wk: torch.Tensor, bk: torch.Tensor, v_rows: torch.Tensor, Wv: torch.Tensor,
                      bv: torch.Tensor, low_rank: int, out_len_k: torch.Tensor, out_len_v: torch.Tensor,
                      threshold: float = 0.1, len_multiple: int = 1, native_rounding: bool = True) -> None:
    """The cutoffs of the K rows and of the V rows in one launch, for rows of at most 128 coefficients (the decode
    shape of the per-head layout): the lengths ``gate_lengths`` gives for each side, written into the caller's int32
    tensors.  Nothing is allocated."""
    if not k_rows.is_cuda:
        raise RuntimeError("dynakv_b200 has no CPU path: the gate needs CUDA tensors")
    d = k_rows.shape[-1]
    if d > 128 or v_rows.shape != k_rows.shape:
        raise ValueError("gate_lengths_pair takes K and V rows of one shape with at most 128 coefficients")
    args = []
    keep = []
    for rows, w, b, out in ((k_rows, Wk, bk, out_len_k), (v_rows, Wv, bv, out_len_v)):
        if w.shape != (d, d) or b.numel() != d or w.dtype != rows.dtype or b.dtype != rows.dtype:
            raise ValueError(f"gate weight must be [{d}, {d}] and bias [{d}] in the rows' dtype")
        x = rows.reshape(-1, d)
        if x.stride(-1) != 1:
            x = x.contiguous()
        wc, bc = w.contiguous(), b.reshape(-1).contiguous()
        if out.dtype != torch.int32 or out.numel() != x.shape[0] or not out.is_contiguous():
            raise ValueError("the length outputs must be contiguous int32 tensors with one entry per row")
        a = _lib.GateArgs()
        a.dtype, a.n_rows, a.dim, a.low_rank, a.threshold = _lib.dtype_code(rows.dtype), x.shape[0], d, int(low_rank), threshold
        a.x, a.x_stride, a.w, a.b = x.data_ptr(), x.stride(0), wc.data_ptr(), bc.data_ptr()
        a.lengths, a.masked, a.masked_stride = out.data_ptr(), None, 0
        a.len_multiple, a.native_rounding = int(len_multiple), int(bool(native_rounding))
        a.stream = _lib.stream_ptr(rows.device)
        args.append(a)
        keep += [x, wc, bc]
    _lib.check(_lib.load().dkv_gate_lengths_pair(C.byref(args[0]), C.byref(args[1])), "dkv_gate_lengths_pair")
    del keep


def kv_process_fused(key_states: torch.Tensor, value_states: torch.Tensor, Wk, bk, Wv, bv, low_rank: int,
                     len_multiple: int = 1):
    """Drop-in for the reference module method of the same name (kernels/compressed_attention.py:84-119):
    returns (k_out, v_out, len_k, len_v, 1, 1) for key_states / value_states [B, S, d]."""
    k_out, len_k = gate_lengths(key_states, Wk, bk, low_rank, len_multiple=len_multiple)
    v_out, len_v = gate_lengths(value_states, Wv, bv, low_rank, len_multiple=len_multiple)
    return k_out, v_out, len_k, len_v, 1, 1


class CompressedDecodeLayer:
    """One attention layer's decode step on the compressed cache (per-KV-head arenas)."""

    def __init__(self, layer_idx: int, k_up: torch.Tensor, v_up: torch.Tensor, theta: float,
                 policy: Optional[KernelPolicy] = None, k_norm_weight: Optional[torch.Tensor] = None,
                 k_norm_eps: float = 1e-6, project_new_rows: bool = False, gate=None):
        """``gate`` = (Wk, bk, Wv, bv) with [R, R] weights: the step then computes the cutoffs of the new coefficient
        rows itself (kv_process_fused of the reference, one row per (sequence, KV head), lengths rounded up to the
        cache's ``len_multiple``) before it appends them; ``new_k`` / ``new_v`` must then be coefficient rows."""
        if gate is not None and project_new_rows:
            raise ValueError("the gate takes coefficient rows: project the new rows before the step")
        self.gate = gate
        self.layer_idx = layer_idx
        self.k_up, self.v_up = k_up.contiguous(), v_up.contiguous()
        self.theta = float(theta)
        self.policy = policy or KernelPolicy()
        if k_norm_weight is not None:   # fp32 on the device once, so no conversion happens per call
            k_norm_weight = k_norm_weight.to(device=k_up.device, dtype=torch.float32).contiguous()
        self.k_norm_weight, self.k_norm_eps = k_norm_weight, k_norm_eps
        self.project_new_rows = project_new_rows
        self._tickets: Optional[torch.Tensor] = None

    def prepare(self, batch: int, device) -> None:
        """Allocate what ``append`` needs on the device (before any graph capture)."""
        if self.project_new_rows and (self._tickets is None or self._tickets.numel() < batch):
            self._tickets = torch.zeros(max(batch, 1), dtype=torch.int32, device=device)

    def append(self, cache: CustomDynamicCache, new_k, new_v, len_k, len_v, row_counter: torch.Tensor,
               seq_capacity: int) -> None:
        """Append one token per arena at the position held by the device counter ``row_counter``.

        new_k/new_v [B, Hkv, 128]: coefficient rows, or pre-RoPE head vectors when
        ``project_new_rows`` (they are then projected onto the basis inside the kernel).
        """
        if self.gate is not None:
            Wk, bk, Wv, bv = self.gate
            R = new_k.shape[-1]
            if R <= 128:      # both sides in one launch
                gate_lengths_pair(new_k.view(-1, R), Wk, bk, new_v.view(-1, R), Wv, bv, R, len_k, len_v,
                                  len_multiple=cache.len_multiple)
            else:
                gate_lengths(new_k.view(-1, R), Wk, bk, R, return_masked=False, len_multiple=cache.len_multiple, out_lengths=len_k)
                gate_lengths(new_v.view(-1, R), Wv, bv, R, return_masked=False, len_multiple=cache.len_multiple, out_lengths=len_v)
        ck, cv = cache.key_cache_sp[self.layer_idx], cache.value_cache_sp[self.layer_idx]
        a = _lib.AppendArgs()
        a.dtype = _lib.dtype_code(new_k.dtype)
        a.batch, a.arenas_per_batch, a.max_dim = new_k.shape[0], new_k.shape[1], new_k.shape[2]
        a.new_k, a.new_v, a.len_k, a.len_v = new_k.data_ptr(), new_v.data_ptr(), len_k.data_ptr(), len_v.data_ptr()
        if self.project_new_rows:
            self.prepare(new_k.shape[0], new_k.device)
            a.k_basis, a.v_basis, a.tickets = self.k_up.data_ptr(), self.v_up.data_ptr(), self._tickets.data_ptr()
        a.k, a.v = cache._side(ck), cache._side(cv)
        a.seq_pos, a.seq_lens, a.seq_capacity = 0, row_counter.data_ptr(), seq_capacity
        a.len_multiple = cache.len_multiple
        a.status, a.stream = status_word(new_k.device).data_ptr(), _lib.stream_ptr(new_k.device)
        _lib.check(_lib.load().dkv_append_decode(C.byref(a)), "dkv_append_decode")

    def attend(self, cache: CustomDynamicCache, q: torch.Tensor, out: torch.Tensor, row_counter: torch.Tensor,
               seq_columns: int, route: str, route_min_tokens: int = 0, route_max_tokens: int = 0,
               prepare_only: bool = False) -> None:
        """Attention of all batch rows through one kernel (``route``); with routing bounds the kernel skips the rows
        whose current length (read from ``row_counter`` on the device) belongs to the other kernel."""
        ck, cv = cache.key_cache_sp[self.layer_idx], cache.value_cache_sp[self.layer_idx]
        args, keep = build_attn_args(
            q, ck[0], self.k_up, cv[0], self.v_up, ck[1][:, :seq_columns], ck[2][:, :seq_columns],
            cv[1][:, :seq_columns], cv[2][:, :seq_columns], self.theta, out=out, seq_lens=row_counter,
            k_norm_weight=self.k_norm_weight, k_norm_eps=self.k_norm_eps,
            len_multiple=cache.len_multiple, need_workspace=(route == "long_two_stage"),
            route_min_tokens=route_min_tokens, route_max_tokens=route_max_tokens)
        lib = _lib.load()
        if prepare_only:     # only size and allocate what the call needs (workspace, status word)
            return
        if route == "short_fused":
            _lib.check(lib.dkv_fused_decode(C.byref(args)), "dkv_fused_decode")
        else:
            _lib.check(lib.dkv_two_stage_decode(C.byref(args)), "dkv_two_stage_decode")
        del keep


class DecodeGraph:
    """CUDA-graph replay of append + routed attention over a stack of layers.

    The caches must have been filled (prefill) with ``token_counts`` so that every layer owns a device
    row counter; the graph reads the current cache lengths from those counters and the kernels route every
    row on its own length (``KernelPolicy.switch_tokens``) on the device, so one capture serves every later
    step -- also when a row crosses the switch point -- as long as no row outgrows ``seq_capacity``.
    ``horizon`` = number of steps the capture must stay valid for (default: until the cache is full); it only
    decides whether the long-cache kernels have to be in the graph at all.
    """

    def __init__(self, layers: Sequence[CompressedDecodeLayer], cache: CustomDynamicCache, batch: int,
                 n_q_heads: int, dtype: torch.dtype, device, seq_lens_host: Sequence[int],
                 horizon: Optional[int] = None):
        self.layers, self.cache = list(layers), cache
        self.batch, self.device = batch, torch.device(device)
        L, Hkv = len(self.layers), cache.arenas_per_batch
        self.q = torch.zeros((L, batch, n_q_heads, 128), dtype=dtype, device=device)
        self.new_k = torch.zeros((L, batch, Hkv, 128), dtype=dtype, device=device)
        self.new_v = torch.zeros_like(self.new_k)
        self.len_k = torch.full((L, batch, Hkv), 8, dtype=torch.int32, device=device)
        self.len_v = torch.full_like(self.len_k, 8)
        self.out = torch.zeros((L, batch, n_q_heads, 128), dtype=dtype, device=device)
        switch = self.layers[0].policy.switch_tokens
        cap = cache.key_cache_sp[self.layers[0].layer_idx][1].shape[1]
        reach = cap if horizon is None else min(cap, max(seq_lens_host) + 1 + int(horizon))
        # rows only grow: a row is short now or never, and long at some step of the horizon or never
        self._has_short = any(int(n) + 1 < switch for n in seq_lens_host)
        self._has_long = reach >= switch
        self._switch = switch
        self.kernel_launches_per_step = L * (1 + (1 if self._has_short else 0) + (2 if self._has_long else 0)) + \
            sum(1 for l in self.layers if l.gate is not None)     # the gate of both sides is one launch
        for l in self.layers:       # size the gate's scratch and the append's tickets before any capture
            l.prepare(batch, self.device)
            if l.gate is not None:
                _scratch(self.device, 8 * batch * Hkv * 128)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        status_word(self.device)
        self._run_layers(prepare_only=True)   # allocate the split workspace before any capture

    def _run_layers(self, prepare_only: bool = False) -> None:
        for li, layer in enumerate(self.layers):
            ck = self.cache.key_cache_sp[layer.layer_idx]
            counter = self.cache.seq_lens(layer.layer_idx)
            if counter is None:
                raise RuntimeError("DecodeGraph needs per-row counters: fill the cache with token_counts or adopt()")
            cap = ck[1].shape[1]
            if not prepare_only:
                layer.append(self.cache, self.new_k[li], self.new_v[li], self.len_k[li], self.len_v[li], counter, cap)
            both = self._has_short and self._has_long
            if self._has_short:
                layer.attend(self.cache, self.q[li], self.out[li], counter, cap, "short_fused",
                             route_max_tokens=self._switch if both else 0, prepare_only=prepare_only)
            if self._has_long:
                layer.attend(self.cache, self.q[li], self.out[li], counter, cap, "long_two_stage",
                             route_min_tokens=self._switch if both else 0, prepare_only=prepare_only)

    def capture(self) -> None:
        """Capture one decode step.  Nothing is executed: the cache is left as it is."""
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._run_layers()
        self.graph = g

    def step(self) -> torch.Tensor:
        """Run one decode step on the static device buffers (q, new_k, new_v, len_k, len_v -> out)."""
        if self.graph is None:
            self._run_layers()
        else:
            self.graph.replay()
        return self.out

    def step_from_host(self, q, new_k, new_v, len_k, len_v, out_host: torch.Tensor) -> torch.Tensor:
        """Host-resident step: pinned host tensors in, pinned host tensor out, copies on the current stream."""
        self.q.copy_(q, non_blocking=True)
        self.new_k.copy_(new_k, non_blocking=True)
        self.new_v.copy_(new_v, non_blocking=True)
        self.len_k.copy_(len_k, non_blocking=True)
        self.len_v.copy_(len_v, non_blocking=True)
        self.step()
        out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def h2d_bytes_per_step(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.q, self.new_k, self.new_v, self.len_k, self.len_v))

    def d2h_bytes_per_step(self) -> int:
        return self.out.numel() * self.out.element_size()
