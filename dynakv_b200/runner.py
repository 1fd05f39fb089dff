"""Minimal Llama-shaped decode loop on the compressed KV cache.

Stands in for the reference's model wrappers (src/dynakv/custom_llama.py:36-85 swaps the decoder layers of a
Hugging Face Llama for ``CustomAttention``; scripts/benchmark_throughput.py:37-81 times ``generate``), which need
a checkpoint, a tokenizer and transformers 4.53.  Here the model is random-init at the given shape; embeddings,
RMSNorm, the QKV / output / MLP GEMMs, RoPE of the query and greedy sampling are plain torch (library GEMMs), and
everything that touches the cache is this package: bulk projection + pack for the prompt, the projecting append
and the routed attention kernels for every generated token.

Partitioning (no collective inside attention): data parallel = each rank runs its own sequences with its own
caches; tensor parallel by KV head = rank r owns KV heads [r*Hkv/N, (r+1)*Hkv/N) with their query heads, their
arenas and the matching column / row shards of the projections and the MLP, and the partial sums after the
row-parallel ``o_proj`` and ``down_proj`` are all-reduced (NCCL on GPUs), once each per layer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import synthetic
from .kernels.compressed_attention import CompressedDecodeLayer, project_bulk
from .kernels.compressed_cache import CustomDynamicCache
from .kernels.router import KernelPolicy
from .sharding import block_range


@dataclass(frozen=True)
class ModelShape:
    layers: int = 32
    hidden: int = 4096
    mlp: int = 14336
    vocab: int = 128256
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    theta: float = 500000.0
    rms_eps: float = 1e-5


LLAMA3_8B = ModelShape()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE in fp32.  x [..., n_heads, D]; pos broadcastable to x.shape[:-2] (token positions)."""
    D = x.shape[-1]
    j = torch.arange(D // 2, device=x.device, dtype=torch.float32)
    freq = torch.exp(-(2.0 * j / D) * math.log(theta))
    ang = pos.to(torch.float32)[..., None, None] * freq
    cos, sin = torch.cos(ang), torch.sin(ang)
    lo, hi = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1).to(x.dtype)


class _LayerWeights:
    __slots__ = ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "norm1", "norm2", "k_up", "v_up", "w_cut")


class MiniLlama:
    """Random-init decoder at ``shape``; rank ``tp_rank`` of ``tp_size`` holds the KV-head shard described above.

    Every rank draws the full tensors from the same seeded generator and keeps its slice, so the model is the same
    function whatever ``tp_size`` is.
    """

    def __init__(self, shape: ModelShape, device, dtype=torch.bfloat16, seed: int = 0, tp_rank: int = 0,
                 tp_size: int = 1, group: Optional[dist.ProcessGroup] = None, cutoff_bias: float = -1.25,
                 policy: Optional[KernelPolicy] = None, trace: bool = False):
        if shape.head_dim != 128:
            raise ValueError("the per-head cache layout is built for head_dim 128")
        if shape.n_kv_heads % tp_size or shape.mlp % tp_size:
            raise ValueError("tp_size must divide the KV heads and the MLP width")
        self.shape, self.device, self.dtype = shape, torch.device(device), dtype
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        self.cutoff_bias = float(cutoff_bias)
        self.policy = policy or KernelPolicy()
        self.trace: Optional[list] = [] if trace else None
        s = shape
        G = s.n_q_heads // s.n_kv_heads
        kv_lo, kv_hi = block_range(s.n_kv_heads, tp_size, tp_rank)
        m_lo, m_hi = block_range(s.mlp, tp_size, tp_rank)
        self.kv_local, self.q_local = kv_hi - kv_lo, (kv_hi - kv_lo) * G
        D = s.head_dim
        gen = torch.Generator(device=self.device).manual_seed(seed)

        def normal(*size, std=0.02):
            return (torch.randn(*size, generator=gen, device=self.device, dtype=torch.float32) * std).to(dtype)

        self.embed = normal(s.vocab, s.hidden)
        self.lm_head = normal(s.hidden, s.vocab)
        self.final_norm = torch.ones(s.hidden, dtype=dtype, device=self.device)
        self.layers: List[_LayerWeights] = []
        for li in range(s.layers):
            w = _LayerWeights()
            w.wq = normal(s.hidden, s.n_q_heads * D)[:, kv_lo * G * D: kv_hi * G * D].contiguous()
            w.wk = normal(s.hidden, s.n_kv_heads * D)[:, kv_lo * D: kv_hi * D].contiguous()
            w.wv = normal(s.hidden, s.n_kv_heads * D)[:, kv_lo * D: kv_hi * D].contiguous()
            w.wo = normal(s.n_q_heads * D, s.hidden)[kv_lo * G * D: kv_hi * G * D].contiguous()
            w.wg = normal(s.hidden, s.mlp)[:, m_lo:m_hi].contiguous()
            w.wu = normal(s.hidden, s.mlp)[:, m_lo:m_hi].contiguous()
            w.wd = normal(s.mlp, s.hidden)[m_lo:m_hi].contiguous()
            w.norm1 = torch.ones(s.hidden, dtype=dtype, device=self.device)
            w.norm2 = torch.ones(s.hidden, dtype=dtype, device=self.device)
            w.k_up = synthetic.qr_bases(s.n_kv_heads, 7919 * li + 11, dtype, self.device)[kv_lo:kv_hi].contiguous()
            w.v_up = synthetic.qr_bases(s.n_kv_heads, 7919 * li + 13, dtype, self.device)[kv_lo:kv_hi].contiguous()
            # cutoff head: rows [K heads | V heads], drawn for all heads, this rank's rows kept
            cut = normal(2 * s.n_kv_heads, s.hidden, std=1.0 / math.sqrt(s.hidden)).float()
            w.w_cut = torch.cat((cut[kv_lo:kv_hi], cut[s.n_kv_heads + kv_lo: s.n_kv_heads + kv_hi])).contiguous()
            self.layers.append(w)
        self.cache = CustomDynamicCache(arenas_per_batch=self.kv_local, len_multiple=8)
        self.attn = [CompressedDecodeLayer(li, w.k_up, w.v_up, s.theta, policy=self.policy, project_new_rows=True)
                     for li, w in enumerate(self.layers)]
        self.batch = 0
        self.seq_lens_host: List[int] = []
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._segments: list = []
        self._ids: Optional[torch.Tensor] = None
        self._next: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ pieces
    def _all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y

    def _mlp(self, w: _LayerWeights, x: torch.Tensor) -> torch.Tensor:
        return self._all_reduce((F.silu(x @ w.wg) * (x @ w.wu)) @ w.wd)

    def _cutoffs(self, w: _LayerWeights, x: torch.Tensor):
        """Kept lengths of the new K and V rows from the layer input: [..., Hkv_local] int32 each."""
        r = synthetic.cutoff_head_lengths(x.reshape(-1, x.shape[-1]), w.w_cut, self.cutoff_bias)
        r = r.reshape(*x.shape[:-1], 2 * self.kv_local)
        return r[..., : self.kv_local].contiguous(), r[..., self.kv_local:].contiguous()

    # ------------------------------------------------------------------ prompt
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, new_tokens: int, token_chunk: int = 32768, seq_chunk: int = 4) -> torch.Tensor:
        """Run the prompt ``ids`` [B, P] (all rows the same length), fill the caches with room for ``new_tokens``
        more tokens per row, and return the first generated token per row [B].

        Attention over the prompt is dense causal attention (torch SDPA) on the keys and values the cache will hold:
        the truncated coefficient rows expanded through the bases, as the reference's prefill branch does after
        ``get_origin_states`` (kernels/compressed_attention.py:165-176, 369-382)."""
        s, D = self.shape, self.shape.head_dim
        B, P = ids.shape
        self.batch = B
        pos = torch.arange(P, device=self.device)
        h = self.embed[ids]                                    # [B, P, H]
        flat_h = h.view(B * P, s.hidden)
        for li, w in enumerate(self.layers):
            q = torch.empty(B * P, self.q_local * D, dtype=self.dtype, device=self.device)
            k = torch.empty(B * P, self.kv_local * D, dtype=self.dtype, device=self.device)
            v = torch.empty_like(k)
            len_k = torch.empty(B * P, self.kv_local, dtype=torch.int32, device=self.device)
            len_v = torch.empty_like(len_k)
            for t0 in range(0, B * P, token_chunk):
                x = rms_norm(flat_h[t0:t0 + token_chunk], w.norm1, s.rms_eps)
                q[t0:t0 + token_chunk] = x @ w.wq
                k[t0:t0 + token_chunk] = x @ w.wk
                v[t0:t0 + token_chunk] = x @ w.wv
                len_k[t0:t0 + token_chunk], len_v[t0:t0 + token_chunk] = self._cutoffs(w, x)
            ck = project_bulk(k.view(B, P, -1), w.k_up)         # spectral coefficients of the pre-RoPE rows
            cv = project_bulk(v.view(B, P, -1), w.v_up)
            lk = len_k.view(B, P, self.kv_local).permute(0, 2, 1).contiguous()      # [B, Hkv, P]
            lv = len_v.view(B, P, self.kv_local).permute(0, 2, 1).contiguous()
            need = int(torch.maximum(lk.sum(dim=2).max(), lv.sum(dim=2).max()).item()) + new_tokens * D
            self.cache.reserve(li, B, need, P + new_tokens, self.dtype, self.device)
            self.cache.update_sp(ck, lk, cv, lv, D, li, D, token_counts=[P] * B)
            # the keys and values the cache holds, dense: rows cut at their lengths, expanded through the bases
            r_idx = torch.arange(D, device=self.device)
            attn = torch.empty(B, P, self.q_local * D, dtype=self.dtype, device=self.device)
            for b0 in range(0, B, seq_chunk):
                sl = slice(b0, b0 + seq_chunk)
                nb = ck[sl].shape[0]
                xk = ck[sl].view(nb, P, self.kv_local, D) * (r_idx < lk[sl].permute(0, 2, 1)[..., None])
                xv = cv[sl].view(nb, P, self.kv_local, D) * (r_idx < lv[sl].permute(0, 2, 1)[..., None])
                k_hat = torch.einsum("bphr,hrd->bphd", xk, w.k_up)
                v_hat = torch.einsum("bphr,hrd->bphd", xv, w.v_up)
                k_hat = rope(k_hat, pos[None, :], s.theta)
                qq = rope(q.view(B, P, self.q_local, D)[sl], pos[None, :], s.theta)
                o = F.scaled_dot_product_attention(qq.transpose(1, 2), k_hat.transpose(1, 2), v_hat.transpose(1, 2),
                                                   is_causal=True, enable_gqa=True)
                attn[sl] = o.transpose(1, 2).reshape(nb, P, -1)
            for t0 in range(0, B * P, token_chunk):
                a = attn.view(B * P, -1)[t0:t0 + token_chunk]
                hh = flat_h[t0:t0 + token_chunk] + self._all_reduce(a @ w.wo)
                flat_h[t0:t0 + token_chunk] = hh + self._mlp(w, rms_norm(hh, w.norm2, s.rms_eps))
            del q, k, v, ck, cv, attn
        self.seq_lens_host = [P] * B
        last = rms_norm(h[:, -1], self.final_norm, s.rms_eps)
        return (last @ self.lm_head).argmax(dim=-1)

    # ------------------------------------------------------------------ one generated token
    def _attention_part(self, li: int, h: torch.Tensor) -> torch.Tensor:
        """Layer ``li`` from the residual stream to this rank's partial sum of the output projection [B, H]."""
        s, D, B = self.shape, self.shape.head_dim, h.shape[0]
        w = self.layers[li]
        has_short = any(n + 1 < self.policy.switch_tokens for n in self.seq_lens_host)
        counter = self.cache.seq_lens(li)                  # tokens stored per row = position of the new token
        cap = self.cache.key_cache_sp[li][1].shape[1]
        x = rms_norm(h, w.norm1, s.rms_eps)
        q = rope((x @ w.wq).view(B, self.q_local, D), counter, s.theta)
        new_k = (x @ w.wk).view(B, self.kv_local, D)       # pre-RoPE: the append projects them onto the bases
        new_v = (x @ w.wv).view(B, self.kv_local, D)
        len_k, len_v = self._cutoffs(w, x)
        out = torch.empty(B, self.q_local, D, dtype=self.dtype, device=self.device)
        layer = self.attn[li]
        layer.append(self.cache, new_k, new_v, len_k, len_v, counter, cap)
        if has_short:     # rows only grow: the long kernels are always there, the short one while a row needs it
            layer.attend(self.cache, q, out, counter, cap, "short_fused", route_max_tokens=self.policy.switch_tokens)
        layer.attend(self.cache, q, out, counter, cap, "long_two_stage",
                     route_min_tokens=self.policy.switch_tokens if has_short else 0)
        if self.trace is not None:
            self.trace.append((li, q.clone(), out.clone()))
        return out.view(B, -1) @ w.wo

    def _mlp_part(self, li: int, h: torch.Tensor) -> torch.Tensor:
        w = self.layers[li]
        return (F.silu((x := rms_norm(h, w.norm2, self.shape.rms_eps)) @ w.wg) * (x @ w.wu)) @ w.wd

    def _decode_layers(self, ids: torch.Tensor) -> torch.Tensor:
        h = self.embed[ids]                                    # [B, H]
        for li in range(len(self.layers)):
            h = h + self._all_reduce(self._attention_part(li, h))
            h = h + self._all_reduce(self._mlp_part(li, h))
        return rms_norm(h, self.final_norm, self.shape.rms_eps) @ self.lm_head

    # Tensor-parallel replay: the step is cut at its all-reduces.  Each piece between two all-reduces (a layer's
    # attention part, a layer's MLP part, the head) is its own CUDA graph on static buffers; the all-reduces run
    # eagerly between the replays, so no collective is ever captured.
    def _capture_segments(self, ids: torch.Tensor) -> None:
        B, H = ids.shape[0], self.shape.hidden
        self._ids = ids.clone()
        self._h = torch.zeros(B, H, dtype=self.dtype, device=self.device)
        self._y = torch.zeros(B, H, dtype=self.dtype, device=self.device)
        pool = torch.cuda.graph_pool_handle()
        self._segments = []

        def capture(fn):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                fn()
            self._segments.append(g)

        def first():
            self._h.copy_(self.embed[self._ids])
            self._y.copy_(self._attention_part(0, self._h))
        capture(first)
        for li in range(len(self.layers)):
            def mlp(li=li):
                self._h.add_(self._y)
                self._y.copy_(self._mlp_part(li, self._h))
            capture(mlp)
            if li + 1 < len(self.layers):
                def attn(li=li + 1):
                    self._h.add_(self._y)
                    self._y.copy_(self._attention_part(li, self._h))
                capture(attn)

        def head():
            self._h.add_(self._y)
            self.logits = rms_norm(self._h, self.final_norm, self.shape.rms_eps) @ self.lm_head
            self._next = self.logits.argmax(dim=-1)
        capture(head)

    def _replay_segments(self) -> None:
        last = len(self._segments) - 1
        for i, g in enumerate(self._segments):
            g.replay()
            if i < last:
                self._all_reduce(self._y)

    def _dry_pass(self, ids: torch.Tensor) -> None:
        """One eager step that sizes every workspace, with its effect on the caches' counters undone."""
        for layer in self.attn:
            layer.prepare(ids.shape[0], self.device)
        snap = [(self.cache.seq_lens(li).clone(), self.cache.key_cache_sp[li][3].clone(),
                 self.cache.value_cache_sp[li][3].clone()) for li in range(len(self.layers))]
        self._decode_layers(ids)
        torch.cuda.synchronize(self.device)
        for li, (c, pk, pv) in enumerate(snap):
            self.cache.seq_lens(li).copy_(c)
            self.cache.key_cache_sp[li][3].copy_(pk)
            self.cache.value_cache_sp[li][3].copy_(pv)

    @torch.no_grad()
    def decode_step(self, ids: torch.Tensor, use_graph: bool = False) -> torch.Tensor:
        """Append the token ``ids`` [B] to every row and return the next greedy token [B] (and keep the logits in
        ``self.logits``).  With ``use_graph`` the step is captured once and replayed: as one CUDA graph on a single
        rank, as one graph per piece between all-reduces on a tensor-parallel rank (the collectives stay eager; a
        captured step with ``torch.distributed`` all-reduces inside did not finish on two GPUs and is not offered).
        Rows only grow and the kernels route each row on the device, so one capture serves all later steps."""
        if use_graph and self.trace is None:
            if self._graph is None and not self._segments:
                self._dry_pass(ids)
                if self.tp_size == 1:
                    self._ids = ids.clone()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self.logits = self._decode_layers(self._ids)
                        self._next = self.logits.argmax(dim=-1)
                    self._graph = g
                else:
                    self._capture_segments(ids)
            self._ids.copy_(ids)
            if self._graph is not None:
                self._graph.replay()
            else:
                self._replay_segments()
            nxt = self._next
        else:
            self.logits = self._decode_layers(ids)
            nxt = self.logits.argmax(dim=-1)
        self.seq_lens_host = [n + 1 for n in self.seq_lens_host]
        return nxt

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, new_tokens: int, use_graph: bool = False) -> torch.Tensor:
        """Greedy generation: [B, P] prompt -> [B, new_tokens] generated ids."""
        nxt = self.prefill(prompt_ids, new_tokens)
        out = [nxt]
        for _ in range(new_tokens - 1):
            nxt = self.decode_step(nxt.clone(), use_graph=use_graph)
            out.append(nxt.clone())
        return torch.stack(out, dim=1)


def decode_throughput(model: MiniLlama, prompt_ids: torch.Tensor, new_tokens: int, use_graph: bool) -> dict:
    """Tokens per second of the generated tokens after the first (CUDA events around the decode steps), and the
    prompt time beside it."""
    dev = model.device
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize(dev)
    e[0].record()
    nxt = model.prefill(prompt_ids, new_tokens)
    e[1].record()
    warm = min(3, new_tokens - 2)
    for _ in range(warm):                     # graph capture and warm-up outside the timed steps
        nxt = model.decode_step(nxt.clone(), use_graph=use_graph)
    torch.cuda.synchronize(dev)
    e[1].synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t0.record()
    steps = new_tokens - 1 - warm
    for _ in range(steps):
        nxt = model.decode_step(nxt.clone(), use_graph=use_graph)
    e[2].record()
    torch.cuda.synchronize(dev)
    ms = t0.elapsed_time(e[2])
    return {"decode_steps_timed": steps, "ms_per_step": ms / max(steps, 1),
            "tokens_per_s": prompt_ids.shape[0] * steps / (ms * 1e-3) if steps else 0.0,
            "prefill_ms": e[0].elapsed_time(e[1]), "last_tokens": nxt[:4].tolist()}


def main(argv: Optional[Sequence[str]] = None) -> None:
    """``python -m dynakv_b200.runner`` (one process per GPU under ``torch.distributed.run`` for N > 1): random-init
    model of the given shape, uniform random prompt, greedy decode; rank 0 prints one JSON object with the
    whole-job tokens/s (device time of the decode steps, maximum over ranks)."""
    import argparse
    import json
    import os

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--mlp", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--batch", type=int, default=32, help="sequences per GPU (dp) or in total (tp)")
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--new-tokens", type=int, default=100)
    ap.add_argument("--mode", default="dp", choices=["dp", "tp"])
    ap.add_argument("--graph", action="store_true", help="replay the decode step from CUDA graphs (tp: one per piece between all-reduces)")
    ap.add_argument("--cutoff-bias", type=float, default=-1.25)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # stdout carries the one JSON line: NCCL's debug output goes to stderr, and the version banner, which NCCL
        # prints on stdout at debug level VERSION whatever the debug file is, is switched off
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    shape = ModelShape(layers=args.layers, hidden=args.hidden, mlp=args.mlp, vocab=args.vocab)
    tp = args.mode == "tp"
    model = MiniLlama(shape, dev, seed=0, tp_rank=rank if tp else 0, tp_size=world if tp else 1,
                      cutoff_bias=args.cutoff_bias)
    gen = torch.Generator(device=dev).manual_seed(1234 + (0 if tp else rank))
    ids = torch.randint(0, shape.vocab, (args.batch, args.prompt), generator=gen, device=dev)
    if world > 1:
        dist.barrier()
    res = decode_throughput(model, ids, args.new_tokens, use_graph=args.graph)
    ms = res["ms_per_step"]
    kept = sum(float(c[1][:, : args.prompt].float().mean().item()) for c in model.cache.key_cache_sp) / shape.layers / 128
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    seqs = args.batch * (1 if tp else world)
    if rank == 0:
        print(json.dumps({"metric": "generated_tokens_per_s", "value": seqs / (ms * 1e-3), "unit": "tokens/s",
                          "n_gpus": world, "mode": args.mode, "ms_per_step": ms, "sequences": seqs,
                          "config": {"workload": "random-init Llama-shaped decode", "layers": shape.layers,
                                     "hidden": shape.hidden, "mlp": shape.mlp, "vocab": shape.vocab,
                                     "prompt": args.prompt, "new_tokens": args.new_tokens,
                                     "decode_steps_timed": res["decode_steps_timed"], "cuda_graph": bool(args.graph)},
                          "prefill_ms": res["prefill_ms"], "key_retention_of_prompt": kept, "dtype": "bf16",
                          "data": "synthetic"}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
