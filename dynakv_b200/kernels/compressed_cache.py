"""Physical variable-length KV cache (replaces src/dynakv/kernels/compressed_cache.py).

Per layer and per side (K, V) the state is the reference's 6-element list
``[flat_buf, lens_buf, offs_buf, flat_ptr_gpu, seq_ptr, max_flat_ptr_cpu]``:

* ``flat_buf [rows, capacity]``  kept coefficients of every token, back to back, model dtype
* ``lens_buf / offs_buf [rows, seq_capacity]`` int32: ``lens[r, s]`` = coefficients kept for
  token s, ``offs[r, s]`` = exclusive prefix sum of ``lens[r, :s]``
* ``flat_ptr_gpu [rows]`` int32 write pointer = sum of lens; ``seq_ptr`` tokens stored (python int)
* ``max_flat_ptr_cpu`` conservative host-side bound on the write pointers, so that decode steps need
  no device synchronisation except when a buffer must grow.

``rows`` is the batch size in the reference's joint layout (``arenas_per_batch=1``: one latent row
per token shared by all heads) or ``batch * Hkv`` with one arena per KV head
(``arenas_per_batch=Hkv``), which is the layout the tensor-core decode kernels read.

Extensions over the reference: per-head arenas; ``len_multiple`` (declared granularity of the
lengths, 8 enables the 16-byte aligned kernels); ragged batches through per-row token counts
(``token_counts`` at prefill, ``seq_lens`` afterwards); ``reserve`` to pre-size the buffers.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _lib
from ._common import status_word

EXPAND_SEQ_STEP = 1024


def _round8(n: int) -> int:
    return (int(n) + 7) // 8 * 8


def _round4(n: int) -> int:
    # metadata rows that start on 16-byte boundaries can be staged with 16-byte async copies
    return (int(n) + 3) // 4 * 4


def simple_decompress(flat_values: torch.Tensor, lengths: torch.Tensor, max_dim: int,
                      offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ragged -> dense zero-padded [rows, S, max_dim].

    Without ``offsets`` the rows are taken to be packed gap-free from element 0, as the reference
    assumes (compressed_cache.py:36-56); the offsets are then the exclusive prefix sums of the lengths.
    """
    _lib.require_cuda(flat_values, lengths)
    lengths = lengths.to(torch.int32)
    if offsets is None:
        offsets = (torch.cumsum(lengths, dim=1, dtype=torch.int32) - lengths).to(torch.int32)
    rows, s = lengths.shape
    dense = torch.empty((rows, s, max_dim), dtype=flat_values.dtype, device=flat_values.device)
    side = _lib.make_side(flat_values, lengths, offsets)
    rc = _lib.load().dkv_decompress(_lib.dtype_code(flat_values.dtype), rows, s, max_dim, C.byref(side),
                                    dense.data_ptr(), _lib.stream_ptr(dense.device))
    _lib.check(rc, "dkv_decompress")
    return dense


class CustomDynamicCache:
    """Drop-in for the reference's ``CustomDynamicCache`` on the physical path."""

    def __init__(self, config=None, max_batch_size=None, max_cache_len=None, dtype=None, device=None,
                 layer_device_map=None, arenas_per_batch: int = 1, len_multiple: int = 1, **kwargs):
        self.max_batch_size = max_batch_size
        self.max_cache_len = max_cache_len
        self.dtype = dtype
        self.device = device
        self.layer_device_map = layer_device_map
        self.arenas_per_batch = int(arenas_per_batch)
        self.len_multiple = int(len_multiple)
        self.key_cache_sp: List[Optional[list]] = []
        self.value_cache_sp: List[Optional[list]] = []
        # ragged batches: tokens stored per batch row, one int32 device counter [B] per layer
        # (plus a host mirror), created by the first update that passes ``token_counts``
        self._seq_lens: List[Optional[torch.Tensor]] = []
        self._seq_lens_host: List[Optional[List[int]]] = []

    # ------------------------------------------------------------------ reference surface
    def reset(self):
        self.key_cache_sp = []
        self.value_cache_sp = []
        self._seq_lens = []
        self._seq_lens_host = []

    def seq_lens(self, layer_idx: int = 0) -> Optional[torch.Tensor]:
        """Device int32 [B] token count per batch row of a ragged batch (None for rectangular use)."""
        return self._seq_lens[layer_idx] if layer_idx < len(self._seq_lens) else None

    def seq_lens_host(self, layer_idx: int = 0) -> Optional[List[int]]:
        return self._seq_lens_host[layer_idx] if layer_idx < len(self._seq_lens_host) else None

    def get_seq_length_sp(self, layer_idx: Optional[int] = 0) -> int:
        if len(self.key_cache_sp) <= layer_idx:
            return 0
        if self.key_cache_sp[layer_idx] is None:
            return 0
        return self.key_cache_sp[layer_idx][4]

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.get_seq_length_sp(layer_idx)

    def get_origin_states(self, max_dim, layer_idx):
        c_k, c_v = self.key_cache_sp[layer_idx], self.value_cache_sp[layer_idx]
        seq = c_k[4]
        k = simple_decompress(c_k[0], c_k[1][:, :seq], max_dim, c_k[2][:, :seq])
        v = simple_decompress(c_v[0], c_v[1][:, :seq], max_dim, c_v[2][:, :seq])
        return k, v

    # ------------------------------------------------------------------ sizing
    def reserve(self, layer_idx: int, batch: int, flat_capacity: int, seq_capacity: int, dtype: torch.dtype,
                device) -> None:
        """Allocate (or enlarge) both sides of a layer up front so later updates never reallocate."""
        rows = batch * self.arenas_per_batch
        for cache_list in (self.key_cache_sp, self.value_cache_sp):
            while len(cache_list) <= layer_idx:
                cache_list.append(None)
            if cache_list[layer_idx] is None:
                cache_list[layer_idx] = self._new_state(rows, _round8(flat_capacity), seq_capacity, dtype, device)
            else:
                self._ensure_capacity(cache_list[layer_idx], _round8(flat_capacity), seq_capacity)

    def adopt(self, layer_idx: int, k_state: Sequence, v_state: Sequence, seq_lens_host: Sequence[int]) -> None:
        """Install already packed buffers as a layer's cache: ``(flat, lens, offs, ptr)`` per side, built
        elsewhere under the same layout contract, with ``seq_lens_host[b]`` tokens stored for batch row b.
        The layer gets per-row device counters, so later appends and attention follow each row's own length."""
        for cache_list, st in ((self.key_cache_sp, k_state), (self.value_cache_sp, v_state)):
            while len(cache_list) <= layer_idx:
                cache_list.append(None)
            flat, lens, offs, ptr = st
            if flat.shape[1] % 8:
                raise ValueError("flat capacity must be a multiple of 8 elements")
            cache_list[layer_idx] = [flat, lens, offs, ptr.to(torch.int32), max(seq_lens_host) if len(seq_lens_host) else 0,
                                     ptr.cpu().tolist()]
        while len(self._seq_lens) <= layer_idx:
            self._seq_lens.append(None)
            self._seq_lens_host.append(None)
        self._seq_lens[layer_idx] = torch.tensor(list(seq_lens_host), dtype=torch.int32, device=k_state[0].device)
        self._seq_lens_host[layer_idx] = [int(n) for n in seq_lens_host]

    @staticmethod
    def _new_state(rows, flat_cap, seq_cap, dtype, device):
        return [
            torch.zeros((rows, max(flat_cap, 8)), dtype=dtype, device=device),
            torch.zeros((rows, _round4(max(seq_cap, 1))), dtype=torch.int32, device=device),
            torch.zeros((rows, _round4(max(seq_cap, 1))), dtype=torch.int32, device=device),
            torch.zeros(rows, dtype=torch.int32, device=device),
            0,
            [0] * rows,
        ]

    @staticmethod
    def _ensure_capacity(cache, flat_cap, seq_cap):
        flat_buf, lens_buf, offs_buf = cache[0], cache[1], cache[2]
        if seq_cap > lens_buf.shape[1]:
            for i in (1, 2):
                new = cache[i].new_zeros(cache[i].shape[0], _round4(seq_cap))
                new[:, : cache[i].shape[1]].copy_(cache[i])
                cache[i] = new
        if flat_cap > flat_buf.shape[1]:
            new = flat_buf.new_zeros(flat_buf.shape[0], flat_cap)
            new[:, : flat_buf.shape[1]].copy_(flat_buf)
            cache[0] = new

    # ------------------------------------------------------------------ update
    def _prepare(self, cache_list, layer_idx, new_states, new_len, max_dim, is_decode, n_new):
        """Host-side capacity policy of the reference (_update_layer_cache, compressed_cache.py:96-168)."""
        while len(cache_list) <= layer_idx:
            cache_list.append(None)
        rows = new_len.shape[0]
        if cache_list[layer_idx] is None:
            # first use: exact fit (one synchronising reduction, as in the reference)
            init_flat = int(new_len.sum(dim=1).max().item())
            cache_list[layer_idx] = self._new_state(rows, _round8(init_flat), n_new, new_states.dtype,
                                                    new_states.device)
        cache = cache_list[layer_idx]
        seq_ptr = cache[4]
        if seq_ptr + n_new > cache[1].shape[1]:
            self._ensure_capacity(cache, cache[0].shape[1], max(cache[1].shape[1] + EXPAND_SEQ_STEP, seq_ptr + n_new))
        max_added = n_new * max_dim if is_decode else int(new_len.sum(dim=1).max().item())
        if max(cache[5]) + max_added > cache[0].shape[1]:
            real = cache[3].cpu().tolist()          # resynchronise the conservative bound
            cache[5] = real
            if max(real) + max_added > cache[0].shape[1]:
                step = EXPAND_SEQ_STEP * (max_dim // 2)
                self._ensure_capacity(cache, _round8(max(cache[0].shape[1] + step, max(real) + max_added)),
                                      cache[1].shape[1])
        return cache, max_added

    def _side(self, cache) -> _lib.Side:
        return _lib.make_side(cache[0], cache[1], cache[2], cache[3])

    def update_sp(self, key_states, key_len, value_states, value_len, max_dim, layer_idx, tensor_d,
                  k_scalar=None, v_scalar=None, token_counts: Optional[Sequence[int]] = None):
        """Append a block of tokens to layer ``layer_idx`` and return the cache views.

        key_states / value_states: [B, S_new, arenas_per_batch * max_dim] coefficient rows (zero beyond
        each row's length is not required; only the first ``len`` entries are read).
        key_len / value_len: int32 [B, S_new] (joint layout) or [B, arenas_per_batch, S_new].
        ``tensor_d`` is the per-row width bound used for the conservative growth estimate (int or tensor).
        ``token_counts`` (prefill of a ragged batch): only the first ``token_counts[b]`` tokens of row b
        are stored.  Returns ``(flat_k, flat_v, lens_k, lens_v, offs_k, offs_v)`` with the metadata
        sliced to the tokens stored, exactly as the reference's ``update_sp``.
        """
        lib = _lib.load()
        _lib.require_cuda(key_states, value_states, key_len, value_len)
        A = self.arenas_per_batch
        B, n_new = key_states.shape[0], key_states.shape[1]
        is_decode = n_new == 1
        row_dim = key_states.shape[2] // A
        width = int(tensor_d.max().item()) if isinstance(tensor_d, torch.Tensor) else int(tensor_d)
        width = min(width, row_dim)
        dev = key_states.device

        def lens2d(t):
            t = t.to(torch.int32)
            t = t.reshape(B * A, n_new) if t.dim() == 3 else t.reshape(B, n_new)
            if t.shape[0] != B * A:
                raise ValueError(f"lengths describe {t.shape[0]} rows, cache has {B * A}")
            return t.contiguous()

        kl, vl = lens2d(key_len), lens2d(value_len)
        ck, _ = self._prepare(self.key_cache_sp, layer_idx, key_states, kl, width, is_decode, n_new)
        cv, max_added = self._prepare(self.value_cache_sp, layer_idx, value_states, vl, width, is_decode, n_new)
        seq_ptr = ck[4]
        while len(self._seq_lens) <= layer_idx:
            self._seq_lens.append(None)
            self._seq_lens_host.append(None)
        ragged = token_counts is not None or self._seq_lens[layer_idx] is not None
        if ragged and self._seq_lens[layer_idx] is None:
            if seq_ptr != 0:
                raise ValueError("token_counts must be given from the first update of a layer on")
            self._seq_lens[layer_idx] = torch.zeros(B, dtype=torch.int32, device=dev)
            self._seq_lens_host[layer_idx] = [0] * B
        row_counter = self._seq_lens[layer_idx]
        st = status_word(dev)
        stream = _lib.stream_ptr(dev)
        dt = _lib.dtype_code(key_states.dtype)

        if is_decode and token_counts is None:
            ks = key_states.contiguous()
            vs = value_states.contiguous()
            a = _lib.AppendArgs()
            a.dtype, a.batch, a.arenas_per_batch, a.max_dim = dt, B, A, row_dim
            a.new_k, a.new_v, a.len_k, a.len_v = ks.data_ptr(), vs.data_ptr(), kl.data_ptr(), vl.data_ptr()
            a.k, a.v = self._side(ck), self._side(cv)
            a.seq_pos, a.seq_capacity = seq_ptr, ck[1].shape[1]
            a.seq_lens = _lib.ptr(row_counter)   # ragged: write at the row's own count, kernel advances it
            a.len_multiple, a.status, a.stream = self.len_multiple, st.data_ptr(), stream
            _lib.check(lib.dkv_append_decode(C.byref(a)), "dkv_append_decode")
            if ragged:
                self._seq_lens_host[layer_idx] = [n + 1 for n in self._seq_lens_host[layer_idx]]
        else:
            counts_dev = None
            if token_counts is not None:
                counts_dev = torch.tensor(list(token_counts), dtype=torch.int32, device=dev)
            for states, lens, cache in ((key_states, kl, ck), (value_states, vl, cv)):
                if states.stride(2) != 1:
                    states = states.contiguous()
                p = _lib.PackArgs()
                p.dtype, p.batch, p.arenas_per_batch, p.n_new, p.max_dim = dt, B, A, n_new, row_dim
                p.states, p.stride_b, p.stride_j, p.stride_s = states.data_ptr(), states.stride(0), row_dim, states.stride(1)
                p.new_lens = lens.data_ptr()
                p.row_counts = _lib.ptr(counts_dev)
                p.seq_lens = _lib.ptr(row_counter)
                p.side = self._side(cache)
                p.seq_pos, p.seq_capacity, p.len_multiple = seq_ptr, cache[1].shape[1], self.len_multiple
                p.status, p.stream = st.data_ptr(), stream
                _lib.check(lib.dkv_pack_bulk(C.byref(p)), "dkv_pack_bulk")
            if ragged:
                counts = list(token_counts) if token_counts is not None else [n_new] * B
                row_counter.add_(counts_dev if counts_dev is not None else n_new)
                self._seq_lens_host[layer_idx] = [a_ + int(c) for a_, c in zip(self._seq_lens_host[layer_idx], counts)]

        for cache in (ck, cv):
            cache[4] = seq_ptr + n_new
            if is_decode:
                cache[5] = [p_ + max_added for p_ in cache[5]]
            else:
                cache[5] = cache[3].cpu().tolist()
        s = ck[4]
        return ck[0], cv[0], ck[1][:, :s], cv[1][:, :s], ck[2][:, :s], cv[2][:, :s]
