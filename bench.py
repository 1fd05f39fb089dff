"""Benchmark of the compressed-cache decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default ``long_b8_s32768``): the long-cache configuration -- per GPU a batch of 8 sequences
with 32768 cached tokens each, Llama-3-8B attention shape (32 query heads, 8 KV heads, head_dim 128),
bf16, per-token cutoffs ~ Beta(2,8) quantised to multiples of 8 (~20 % retention), 32 layers.  One
"step" = one decode step of the attention path over all 32 layers: per layer, append one new token per
sequence (pre-RoPE K/V rows projected onto the basis in-kernel, cut at r_t from the synthetic linear
cutoff head) and run the split two-stage decode attention.  The whole step is replayed from one CUDA
graph.  ``value`` is tokens/s over all GPUs with the step inputs already in HBM; ``e2e`` is the same
step driven from pinned host buffers (H2D of q / new K,V rows / cutoffs, D2H of the attention outputs
inside the timed region).  Each GPU reads ~8 GB of distinct cache bytes per step, far more than L2,
so no L2 flush is needed between steps.  After the timed region one (layer, sequence) of the last
step's output is checked against the CPU oracle (``parity``).

Multi-GPU: the batch is sharded by sequence (one process per GPU, 8 sequences each, no collective in
the data path) -> weak scaling.  Timing: CUDA events on the launching stream, barrier + synchronize on
both sides, max over ranks.  Two more legs run at every N and are reported as extra objects:
``ragged_strong`` -- the ragged-batch configuration (64 sequences, lengths log-uniform in [128, 32768],
Qwen3 K-RMSNorm, ~48 % retention, per-row routing across the switch point) with the FIXED set of 64
sequences split over the ranks by a token-balanced partition (strong scaling, no collective); and, for
N > 1, ``kv_head_sharded`` -- one 32768-token sequence with its 8 KV heads split over the ranks, the
attention output feeding a row-parallel o_proj summed by one NCCL all-reduce, checked against the
unsharded result.

At N = 1 the line also carries ``cpu_baseline`` (the oracle's restatement of the reference's fp32
research math on the host cores) and ``gpu_reference`` (the reference's own Triton kernels, JIT-compiled
for this GPU from the copy installed under baseline/_ref, timed on the same cache tensors).

``--impl reference`` times the reference's own CPU implementation of the same math on the host cores,
rank 0 only; a step there is a bounded sample of the workload: one sequence x one layer.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (batch per GPU, cache length, length distribution, theta, layers, ragged lower bound or None)
    "long_b8_s32768": dict(batch=8, seq=32768, dist="beta:2,8", theta=500000.0, layers=32),
    "short_b4_ragged": dict(batch=4, seq=499, dist="beta:2,5", theta=500000.0, layers=32, ragged_lo=64),
    "smoke": dict(batch=2, seq=1500, dist="beta:2,8", theta=500000.0, layers=2),
    # small enough for a full ncu capture, still larger than L2 (2 layers x ~54 MB x 2 sequences... per layer)
    "profile_b2_s32768": dict(batch=2, seq=32768, dist="beta:2,8", theta=500000.0, layers=3),
}
N_Q_HEADS, N_KV_HEADS, HEAD_DIM = 32, 8, 128
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) of one split-kernel launch divided by its algorithmic bytes, as counted by ncu on the
# profile_b2_s32768 workload (the excess is the int32 lens/offs metadata)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.18
RAGGED = dict(n_seq=64, lo=128, hi=32768, dist="beta:2.4,2.6", theta=1000000.0, layers=4, seed=3017)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload_config(name, w, world, retention=None, bytes_step=None):
    cfg = {"workload": name, "batch_per_gpu": w["batch"], "cache_len": w["seq"], "layers": w["layers"],
           "q_heads": N_Q_HEADS, "kv_heads": N_KV_HEADS, "head_dim": HEAD_DIM, "length_dist": w["dist"],
           "parallelism": "sequence-sharded x%d" % world}
    if retention is not None:
        cfg["retention"] = retention
    if bytes_step is not None:
        if bytes_step > 2 * 126e6:
            cfg["l2"] = "inputs larger than L2 (%.1f GB of distinct cache bytes per step per GPU), no flush" % (bytes_step / 1e9)
        else:   # a latency-bound side workload: its bytes stay in the 126 MB L2 from step to step
            cfg["l2"] = "inputs smaller than L2 (%.0f MB per step per GPU) and not flushed: an L2-resident, latency-bound number" % (bytes_step / 1e6)
    return cfg


# ------------------------------------------------------------------------------------------ our arm
def build_workload(w, device, dtype=torch.bfloat16, extra_tokens=64):
    from dynakv_b200 import synthetic
    from dynakv_b200.kernels.compressed_attention import CompressedDecodeLayer, DecodeGraph
    from dynakv_b200.kernels.compressed_cache import CustomDynamicCache

    B, S, L = w["batch"], w["seq"], w["layers"]
    if "ragged_lo" in w:
        gen = torch.Generator().manual_seed(1017)
        seq_lens = torch.randint(w["ragged_lo"], S + 1, (B,), generator=gen).tolist()
    else:
        seq_lens = [S] * B
    cache = CustomDynamicCache(arenas_per_batch=N_KV_HEADS, len_multiple=8)
    layers, comp_bytes, tokens = [], [], sum(seq_lens)
    for li in range(L):
        case = synthetic.make_layer_case(2017 + 31 * li, seq_lens, w["dist"], w["theta"], dtype, device,
                                         N_Q_HEADS, N_KV_HEADS, extra_tokens=extra_tokens)
        cache.adopt(li, (case.k.flat, case.k.lens, case.k.offs, case.k.ptr),
                    (case.v.flat, case.v.lens, case.v.offs, case.v.ptr), seq_lens)
        comp_bytes.append(case.compressed_bytes())
        layers.append(CompressedDecodeLayer(li, case.k_up, case.v_up, w["theta"], project_new_rows=True))
    graph = DecodeGraph(layers, cache, B, N_Q_HEADS, dtype, device, seq_lens)
    return graph, cache, seq_lens, comp_bytes, tokens


def fill_step_inputs(graph, w, seed, device=None):
    """Step inputs as the configuration prescribes: q ~ N(0,1) (taken as already rotated), new pre-RoPE
    K/V rows ~ N(0,1), cutoffs from the synthetic 4096 -> 1 per-head linear head on h ~ N(0,1)."""
    from dynakv_b200 import synthetic
    gen = torch.Generator().manual_seed(seed)
    L, B = graph.q.shape[0], graph.q.shape[1]
    q = torch.randn(L, B, N_Q_HEADS, HEAD_DIM, generator=gen).to(graph.q.dtype)
    nk = torch.randn(L, B, N_KV_HEADS, HEAD_DIM, generator=gen).to(graph.q.dtype)
    nv = torch.randn(L, B, N_KV_HEADS, HEAD_DIM, generator=gen).to(graph.q.dtype)
    hidden = torch.randn(B, 4096, generator=gen)
    wgt = torch.randn(L, 2 * N_KV_HEADS, 4096, generator=gen) / 64.0
    lens = torch.stack([synthetic.cutoff_head_lengths(hidden, wgt[l], -1.75) for l in range(L)])  # [L,B,16]
    lk, lv = lens[..., :N_KV_HEADS].contiguous(), lens[..., N_KV_HEADS:].contiguous()
    host = [t.pin_memory() if torch.cuda.is_available() else t for t in (q, nk, nv, lk, lv)]
    return host



def oracle_row(cache, layer_idx, q_row, k_up, v_up, theta, row, n_tokens, k_norm_weight=None):
    """fp32 compact attention of one batch row from the cache as it is on the GPU (checker, CPU)."""
    from oracle import dynakv_oracle as O
    ck, cv = cache.key_cache_sp[layer_idx], cache.value_cache_sp[layer_idx]
    sl = slice(row * N_KV_HEADS, (row + 1) * N_KV_HEADS)
    S = int(n_tokens)
    lk, ok = ck[1][sl, :S].cpu().numpy(), ck[2][sl, :S].cpu().numpy()
    lv, ov = cv[1][sl, :S].cpu().numpy(), cv[2][sl, :S].cpu().numpy()
    fk = ck[0][sl, : int((ok + lk).max())].float().cpu().numpy()
    fv = cv[0][sl, : int((ov + lv).max())].float().cpu().numpy()
    xk = torch.from_numpy(O.decompress_gather(fk, lk, ok, 128)).view(1, N_KV_HEADS, S, 128)
    xv = torch.from_numpy(O.decompress_gather(fv, lv, ov, 128)).view(1, N_KV_HEADS, S, 128)
    valid = torch.from_numpy(lk > 0).view(1, N_KV_HEADS, S)
    return O.compact_attention_dense(q_row.float().cpu().view(1, N_Q_HEADS, HEAD_DIM), xk, xv, k_up.float().cpu(),
                                     v_up.float().cpu(), theta, valid, k_norm_weight=k_norm_weight)[0]


def parity_of_last_step(graph, cache, w):
    """Layer 0, sequence 0 of the step that ran last, against the oracle on the cache contents it left."""
    n = int(cache.seq_lens(0)[0].item())
    layer = graph.layers[0]
    ref = oracle_row(cache, 0, graph.q[0][0], layer.k_up, layer.v_up, w["theta"], 0, n)
    got = graph.out[0][0].float().cpu()
    return {"max_abs": float((got - ref).abs().max()), "mean_rel": float((got - ref).abs().mean() / ref.abs().mean()),
            "checked": "layer 0, sequence 0 of the last step (%d tokens) against the CPU oracle" % n,
            "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-2}}


def ragged_strong_leg(dev, world, rank, steps, warmup, timed, dist):
    """The ragged-batch configuration with a fixed set of sequences split over the ranks (strong scaling)."""
    from dynakv_b200 import sharding, synthetic
    from dynakv_b200.kernels.compressed_attention import CompressedDecodeLayer, DecodeGraph
    from dynakv_b200.kernels.compressed_cache import CustomDynamicCache
    r = RAGGED
    lengths = synthetic.log_uniform_lengths(r["n_seq"], r["lo"], r["hi"], seed=r["seed"])
    parts = sharding.balanced_sequence_partition(lengths, world)
    mine = parts[rank]
    tokens_rank = [sum(lengths[i] for i in p) for p in parts]
    cache = CustomDynamicCache(arenas_per_batch=N_KV_HEADS, len_multiple=8)
    layers, comp = [], 0
    knw = 1.0 + 0.02 * torch.randn(128, generator=torch.Generator().manual_seed(3))
    my_lens = [lengths[i] for i in mine]
    if mine:
        for li in range(r["layers"]):
            case = synthetic.make_layer_case(r["seed"] + 31 * li + 7919 * rank, my_lens, r["dist"], r["theta"], torch.bfloat16,
                                             dev, N_Q_HEADS, N_KV_HEADS, extra_tokens=2 * (steps + warmup) + 8)
            cache.adopt(li, (case.k.flat, case.k.lens, case.k.offs, case.k.ptr),
                        (case.v.flat, case.v.lens, case.v.offs, case.v.ptr), my_lens)
            comp += case.compressed_bytes()
            layers.append(CompressedDecodeLayer(li, case.k_up, case.v_up, r["theta"], k_norm_weight=knw))
        graph = DecodeGraph(layers, cache, len(mine), N_Q_HEADS, torch.bfloat16, dev, my_lens)
        gen = torch.Generator().manual_seed(17 + rank)
        graph.q.copy_(torch.randn(graph.q.shape, generator=gen).to(torch.bfloat16))
        graph.new_k.copy_((torch.randn(graph.new_k.shape, generator=gen) * 0.5).to(torch.bfloat16))
        graph.new_v.copy_((torch.randn(graph.new_v.shape, generator=gen) * 0.5).to(torch.bfloat16))
        graph.len_k.copy_((torch.randint(1, 17, graph.len_k.shape, generator=gen) * 8).to(torch.int32))
        graph.len_v.copy_((torch.randint(1, 17, graph.len_v.shape, generator=gen) * 8).to(torch.int32))
        graph.capture()
        fn = graph.step
    else:
        fn = lambda: None
    for _ in range(max(warmup, 3)):
        fn()
    ms = timed(fn, steps)
    comp_t = torch.tensor([float(comp)], device=dev)
    if world > 1:
        dist.all_reduce(comp_t)
    ms_step = ms / steps
    out = {"workload": "ragged_b64_loguniform_knorm", "scaling": "strong", "sequences": r["n_seq"], "layers": r["layers"],
           "length_dist": "log-uniform [%d, %d]" % (r["lo"], r["hi"]), "retention_dist": r["dist"],
           "tokens_cached_per_rank": tokens_rank, "sequences_per_rank": [len(p) for p in parts],
           "value": r["n_seq"] / (ms_step * 1e-3), "unit": "tokens/s", "ms_per_step": ms_step,
           "us_per_layer": ms_step * 1e3 / r["layers"],
           "hbm_gbs_all_ranks": float(comp_t.item()) / (ms_step * 1e-3) / 1e9,
           "routing": "per row on the device, KernelPolicy(switch_tokens=500); %d of %d sequences below the switch point"
                      % (sum(1 for n in lengths if n < 500), r["n_seq"])}
    del cache, layers
    torch.cuda.empty_cache()
    return out


def kv_head_sharded_leg(dev, world, rank, steps, timed, dist):
    """One long sequence with its KV heads split over the ranks; row-parallel o_proj + one NCCL all-reduce."""
    from dynakv_b200 import sharding, synthetic
    from dynakv_b200.kernels.two_stage import two_stage_attention
    if N_KV_HEADS % world:
        return {"skipped": "KV heads do not divide over %d ranks" % world}
    S, hidden = 32768, 4096
    case = synthetic.make_layer_case(5151, [S], "beta:2,8", 500000.0, torch.bfloat16, dev, N_Q_HEADS, N_KV_HEADS)
    (k_lo, k_hi), (q_lo, q_hi) = sharding.shard_kv_heads(N_KV_HEADS, N_Q_HEADS, world, rank)
    fk, fv, lk, lv, ok, ov = case.views()
    w_o = (torch.randn(hidden, N_Q_HEADS * HEAD_DIM, generator=torch.Generator().manual_seed(9)) / 64.0).to(torch.bfloat16).to(dev)
    sl = slice(k_lo, k_hi)
    q_loc = case.q[:, q_lo:q_hi].contiguous()

    def local_step():
        o = two_stage_attention(q_loc, fk[sl], case.k_up[sl].contiguous(), fv[sl], case.v_up[sl].contiguous(), lk[sl], ok[sl],
                                lv[sl], ov[sl], case.theta, len_multiple=8)
        return sharding.row_parallel_linear(o.reshape(1, -1), w_o[:, q_lo * HEAD_DIM:q_hi * HEAD_DIM])

    y = local_step()
    full = two_stage_attention(case.q, fk, case.k_up, fv, case.v_up, lk, ok, lv, ov, case.theta, len_multiple=8)
    y_ref = full.reshape(1, -1) @ w_o.T
    err = float((y.float() - y_ref.float()).abs().max())
    scale = float(y_ref.float().abs().mean())
    for _ in range(3):
        local_step()
    ms = timed(local_step, steps)
    return {"workload": "one sequence of %d tokens, %d KV heads per rank, o_proj %dx%d row-parallel + all-reduce" %
                        (S, k_hi - k_lo, hidden, N_Q_HEADS * HEAD_DIM),
            "us_per_layer_step": ms / steps * 1e3, "max_abs_vs_unsharded": err, "mean_abs_of_reference": scale,
            "collective": "NCCL all-reduce of [1, %d] bf16" % hidden}


def prefill_compress_leg(dev, reps=200):
    """Bulk compression of a prompt block (8 sequences x 8192 tokens x 8 KV heads, bf16): tensor-core projection onto
    the per-head bases, then the ragged pack; CUDA events, inputs larger than L2."""
    import ctypes as C
    from dynakv_b200 import _lib, synthetic
    from dynakv_b200.kernels.compressed_attention import project_bulk
    from dynakv_b200.kernels.compressed_cache import CustomDynamicCache
    B, S = 8, 8192
    gen = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(B, S, N_KV_HEADS * 128, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    basis = synthetic.qr_bases(N_KV_HEADS, 71, torch.bfloat16, dev)
    out = torch.empty_like(x)
    lens = synthetic.draw_lengths((B, N_KV_HEADS, S), "beta:2,5", gen, dev)

    def ev_time(fn, reps):
        for _ in range(reps // 2):      # long enough for the clocks to settle before the timed launches
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ms_proj = ev_time(lambda: project_bulk(x, basis, out=out), reps)
    flops = 2.0 * B * S * N_KV_HEADS * 128 * 128
    io = 2.0 * x.numel() * 2 + basis.numel() * 2
    cache = CustomDynamicCache(arenas_per_batch=N_KV_HEADS, len_multiple=8)
    cache.reserve(0, B, int(lens.sum(dim=2).max().item()) + 64, S + 8, torch.bfloat16, dev)
    ck = cache.key_cache_sp[0]
    lens2 = lens.reshape(B * N_KV_HEADS, S).contiguous()
    p = _lib.PackArgs()
    p.dtype, p.batch, p.arenas_per_batch, p.n_new, p.max_dim = _lib.DKV_BF16, B, N_KV_HEADS, S, 128
    p.states, p.stride_b, p.stride_j, p.stride_s = out.data_ptr(), out.stride(0), 128, out.stride(1)
    p.new_lens, p.side = lens2.data_ptr(), cache._side(ck)
    p.seq_pos, p.seq_capacity, p.len_multiple = 0, ck[1].shape[1], 8
    p.stream = _lib.stream_ptr(dev)
    lib = _lib.load()

    def pack():
        ck[3].zero_()
        _lib.check(lib.dkv_pack_bulk(C.byref(p)), "dkv_pack_bulk")

    ms_pack = ev_time(pack, reps)
    payload = float(lens.sum().item()) * 2
    peak_tf = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf = float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        pass
    hbm, _ = measured_peak()
    return {"workload": "8 sequences x 8192 prompt tokens x 8 KV heads, bf16",
            "project_bulk": {"ms": ms_proj, "tflops": flops / (ms_proj * 1e-3) / 1e12, "of_bf16_sustained": None if not peak_tf else flops / (ms_proj * 1e-3) / 1e12 / peak_tf,
                             "gbs": io / (ms_proj * 1e-3) / 1e9, "of_hbm_peak": io / (ms_proj * 1e-3) / 1e9 / hbm,
                             "bound": "hbm (44 flop per byte moved)"},
            "pack_bulk": {"ms": ms_pack, "payload_gbs_read_plus_write": 2 * payload / (ms_pack * 1e-3) / 1e9,
                          "of_hbm_peak": 2 * payload / (ms_pack * 1e-3) / 1e9 / hbm, "retention": payload / (x.numel() * 2)}}


def joint_layout_leg(dev):
    """The reference's literal layout next to the headline: one joint latent row per batch row (R = 1024 over all
    heads), bases [Hq, 1024, 128], any integer length (len_multiple 1).  It runs on the generic CUDA-core kernels
    (the tensor-core kernels need per-KV-head arenas and lengths in multiples of 8); with the reference's own
    Triton kernels on the same tensors beside it when the installed copy is there."""
    from dynakv_b200.kernels.fused import fused_attention_dispatch
    from dynakv_b200.kernels.two_stage import two_stage_attention
    B, S, R = 2, 2048, 1024
    gen = torch.Generator(device=dev).manual_seed(4017)
    dt = torch.bfloat16

    def side():
        lens = torch.randint(1, 411, (B, S), generator=gen, device=dev, dtype=torch.int32)
        offs = (torch.cumsum(lens.long(), 1) - lens.long()).to(torch.int32)
        cap = (int(lens.long().sum(1).max().item()) + 7) // 8 * 8
        sigma = torch.exp(-torch.arange(R, device=dev, dtype=torch.float32) / 256.0)
        flat = torch.randn(B, cap, generator=gen, device=dev) * sigma[torch.arange(cap, device=dev) % R]
        return flat.to(dt), lens, offs

    fk, lk, ok = side()
    fv, lv, ov = side()
    k_up = (torch.randn(N_Q_HEADS, R, HEAD_DIM, generator=gen, device=dev) / math.sqrt(R)).to(dt)
    v_up = (torch.randn(N_Q_HEADS, R, HEAD_DIM, generator=gen, device=dev) / math.sqrt(R)).to(dt)
    q = torch.randn(B, N_Q_HEADS, HEAD_DIM, generator=gen, device=dev).to(dt)
    theta = 500000.0
    nbytes = float((lk.long().sum() + lv.long().sum()).item()) * 2

    def timed(fn, reps=5):
        out = fn(); fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return out, e0.elapsed_time(e1) / reps * 1e3

    out2, us2 = timed(lambda: two_stage_attention(q, fk, k_up, fv, v_up, lk, ok, lv, ov, theta))
    out1, us1 = timed(lambda: fused_attention_dispatch(q, fk, k_up, fv, v_up, lk, ok, lv, ov, theta))
    res = {"workload": "joint latent rows, B=2, S=2048, R=1024, bases [32, 1024, 128], integer lengths 1..410, bf16",
           "kernels": "generic kernels (len_multiple 1, one arena per batch row): mma.sync K reconstruction, "
                      "two-stage entry split over the token axis",
           "two_stage_us": us2, "fused_us": us1, "compressed_bytes": nbytes,
           "two_stage_gbs": nbytes / (us2 * 1e-6) / 1e9,
           "max_abs_two_stage_vs_fused": float((out2.float() - out1.float()).abs().max())}
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_root, "dynakv")):
        try:
            sys.path.insert(0, ref_root)
            from dynakv.kernels.two_stage import abx_sparse, avx
            ref_out, ref_us = timed(lambda: avx(abx_sparse(q, k_up, fk, lk, offsets=ok, theta=theta), fv, v_up, lv, ov), reps=3)
            res["reference_triton_us"] = ref_us
            res["max_abs_vs_reference_triton"] = float((ref_out.float() - out2.float()).abs().max())
        except Exception as exc:
            res["reference_triton_unavailable"] = "%s: %s" % (type(exc).__name__, str(exc)[:160])
        finally:
            if sys.path and sys.path[0] == ref_root:
                sys.path.pop(0)
    return res


def tensor_pipe_probe(dev, tiles=100):
    """Cycles per 128-token tile that one SM's tensor pipe is held by the decode kernel's three tcgen05.mma chains
    (issued back to back by one thread, nothing else on the SM): the floor under the split kernel's time per tile."""
    from dynakv_b200 import _lib
    from dynakv_b200.kernels._common import status_word, read_status
    lib = _lib.load()
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    cyc = torch.zeros(2 * n_sm, dtype=torch.int64, device=dev)
    out = {}
    for name, mask in (("k_reconstruction", 1), ("scores", 2), ("latent_accumulation", 4), ("all_three", 7),
                       ("all_three_commit_per_chain", 23), ("all_three_nonzero_operands", 39),
                       ("two_issuers_nonzero_thread_1_2", 43), ("two_issuers_thread_1_2", 11)):
        for _ in range(2):
            _lib.check(lib.dkv_probe_tensor_pipe(mask, tiles, n_sm, cyc.data_ptr(), status_word(dev).data_ptr(),
                                                 _lib.stream_ptr(dev)), "dkv_probe_tensor_pipe")
        torch.cuda.synchronize()
        out[name] = float(cyc[:n_sm].double().median().item()) / tiles
        if mask == 11:
            out["two_issuers_thread_3"] = float(cyc[n_sm:].double().median().item()) / tiles
        if mask == 43:
            out["two_issuers_nonzero_thread_3"] = float(cyc[n_sm:].double().median().item()) / tiles
    out["status"] = read_status(dev)
    return {"cycles_per_tile": out, "tiles": tiles, "ctas": n_sm}


def gpu_reference_leg(graph, cache, w, dev):
    """The reference's own Triton kernels (abx_sparse -> avx, and the fused kernel) on layer 0 of the workload, one call
    pair per KV head (the reference API with a single basis group is the per-head layout), CUDA-event timed."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "dynakv")):
        return {"unavailable": "baseline/_ref holds no installed copy of the reference"}
    try:
        sys.path.insert(0, ref_root)
        from dynakv.kernels.two_stage import abx_sparse, avx
        layer = graph.layers[0]
        ck, cv = cache.key_cache_sp[0], cache.value_cache_sp[0]
        B = graph.batch
        S = int(cache.seq_lens(0).max().item())
        cap_k, cap_v = ck[0].shape[1], cv[0].shape[1]
        fk = ck[0].view(B, N_KV_HEADS, cap_k); fv = cv[0].view(B, N_KV_HEADS, cap_v)
        lk = ck[1].view(B, N_KV_HEADS, -1)[:, :, :S]; ok = ck[2].view(B, N_KV_HEADS, -1)[:, :, :S]
        lv = cv[1].view(B, N_KV_HEADS, -1)[:, :, :S]; ov = cv[2].view(B, N_KV_HEADS, -1)[:, :, :S]
        G = N_Q_HEADS // N_KV_HEADS
        q = graph.q[0]

        def one_layer():
            outs = []
            for h in range(N_KV_HEADS):
                qh = q[:, h * G:(h + 1) * G].contiguous()
                sc = abx_sparse(qh, layer.k_up[h:h + 1], fk[:, h], lk[:, h], offsets=ok[:, h], theta=w["theta"])
                outs.append(avx(sc, fv[:, h], layer.v_up[h:h + 1], lv[:, h], ov[:, h]))
            return torch.cat(outs, dim=1)

        ref_out = one_layer()            # first call compiles and autotunes
        one_layer()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            one_layer()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps * 1e3
        diff = float((ref_out.float() - graph.out[0].float()).abs().max())
        return {"kernels": "reference abx_sparse + avx (Triton %s, JIT for this GPU), %d per-KV-head call pairs per layer" %
                           (__import__("triton").__version__, N_KV_HEADS),
                "us_per_layer": us, "max_abs_vs_ours": diff,
                "note": "same cache tensors and queries as layer 0 of the last step; scores round-trip HBM in the query dtype"}
    except Exception as exc:   # the baseline is reported, never required
        return {"unavailable": "%s: %s" % (type(exc).__name__, str(exc)[:200])}
    finally:
        if sys.path and sys.path[0] == ref_root:
            sys.path.pop(0)


def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # stdout carries the one JSON line: NCCL's debug output goes to stderr, and the version banner, which NCCL
        # prints on stdout at debug level VERSION whatever the debug file is, is switched off
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    from dynakv_b200 import _lib
    from dynakv_b200.kernels import _common
    import ctypes as C

    _lib.load()
    w = WORKLOADS[args.workload]
    graph, cache, seq_lens, comp_bytes, tokens = build_workload(w, dev, extra_tokens=args.warmup * 2 + args.steps * 2 + 16)
    host_in = fill_step_inputs(graph, w, 99 + rank)
    for dst, src in zip((graph.q, graph.new_k, graph.new_v, graph.len_k, graph.len_v), host_in):
        dst.copy_(src)
    out_host = torch.empty(graph.out.shape, dtype=graph.out.dtype).pin_memory()
    graph.capture()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        from dynakv_b200.sharding import max_over_ranks
        return max_over_ranks(e0.elapsed_time(e1), dev)

    for _ in range(max(args.warmup, 3)):
        graph.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(graph.step, args.steps)
    # end-to-end: host buffers in, host buffer out, every step
    for _ in range(2):
        graph.step_from_host(*host_in, out_host)
    ms_e2e = timed(lambda: graph.step_from_host(*host_in, out_host), args.steps)
    clocks = sampler.stop() if rank == 0 else None

    h2d_bytes, d2h_bytes = graph.h2d_bytes_per_step(), graph.d2h_bytes_per_step()
    # dominant kernel: the split decode kernel, timed alone per launch on its stream
    L = len(graph.layers)
    kernel_ms = None
    if graph._has_long:
        from dynakv_b200.kernels._common import build_attn_args
        lib = _lib.load()
        calls = []
        for li, layer in enumerate(graph.layers):
            ck, cv = cache.key_cache_sp[li], cache.value_cache_sp[li]
            cap = ck[1].shape[1]
            a, keep = build_attn_args(graph.q[li], ck[0], layer.k_up, cv[0], layer.v_up, ck[1][:, :cap], ck[2][:, :cap],
                                      cv[1][:, :cap], cv[2][:, :cap], layer.theta, out=graph.out[li],
                                      seq_lens=cache.seq_lens(li), len_multiple=8, need_workspace=True)
            calls.append((a, keep))
        # all layers' split launches are captured into one graph, so the events bracket back-to-back
        # launches of this kernel only (no host gaps); duration per launch = replay time / launches
        for a, _ in calls:   # eager warm-up (also sets the function attributes outside capture)
            _lib.check(lib.dkv_split_decode(C.byref(a)), "dkv_split_decode")
        torch.cuda.synchronize()
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph):
            for a, _ in calls:
                a.stream = _lib.stream_ptr(dev)
                _lib.check(lib.dkv_split_decode(C.byref(a)), "dkv_split_decode")
        kgraph.replay()
        torch.cuda.synchronize()
        reps = max(1, min(args.steps, 5))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            kgraph.replay()
        e1.record()
        torch.cuda.synchronize()
        kernel_ms = e0.elapsed_time(e1) / (reps * len(calls))
    status = _common.read_status(dev)
    parity = parity_of_last_step(graph, cache, w) if rank == 0 else None
    gpu_ref = gpu_reference_leg(graph, cache, w, dev) if (rank == 0 and world == 1 and not args.no_gpu_reference) else None
    L = len(graph.layers)
    bytes_layer = sum(comp_bytes) / len(comp_bytes)
    n_launch = graph.kernel_launches_per_step
    # free the main workload before the extra legs build theirs
    del graph, cache
    torch.cuda.empty_cache()
    prefill = prefill_compress_leg(dev) if (rank == 0 and world == 1 and not args.no_extra_legs) else None
    ragged = None if args.no_extra_legs else ragged_strong_leg(dev, world, rank, max(2, min(args.steps, 10)), args.warmup, timed, dist)
    kvsh = None
    if world > 1 and not args.no_extra_legs:
        kvsh = kv_head_sharded_leg(dev, world, rank, max(2, min(args.steps, 10)), timed, dist)
    status |= _common.read_status(dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    ms_step = ms_total / args.steps
    total_tokens = w["batch"] * world
    line = {
        "metric": "decode_attn_tokens_per_s", "value": total_tokens / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, w, world, 0.5 * bytes_layer / (sum(seq_lens) * N_KV_HEADS * 128 * 2),
                                  sum(comp_bytes)),
        "us_per_layer": ms_step * 1e3 / L,
        "hbm_gbs_step": sum(comp_bytes) / (ms_step * 1e-3) / 1e9,
        "e2e": {"value": total_tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": n_launch * args.steps,
        "clocks": clocks, "device_status": status, "parity": parity,
    }
    if kernel_ms is not None:
        achieved = bytes_layer / (kernel_ms * 1e-3) / 1e9
        line["roofline"] = {
            "kernel": "mma_decode_kernel<bf16, split>", "bound": "hbm", "achieved": achieved, "peak": peak,
            "peak_source": "of " + peak_kind, "unit": "GB/s", "frac": achieved / peak, "us_per_launch": kernel_ms * 1e3,
            "algorithmic_bytes_per_launch": bytes_layer,
            "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer,
            "frac_of_nominal_8TBs": achieved / 8000.0,
            "us_per_layer_outside_the_kernel": ms_step * 1e3 / L - kernel_ms * 1e3}
    if ragged is not None:
        line["ragged_strong"] = ragged
    if kvsh is not None:
        line["kv_head_sharded"] = kvsh
    if gpu_ref is not None:
        line["gpu_reference"] = gpu_ref
    if prefill is not None:
        line["prefill_compress"] = prefill
        line["joint_layout"] = joint_layout_leg(dev)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(w, steps=20, warmup=2)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------- reference arm
def cpu_reference(w, steps, warmup, max_seconds=25.0):
    """The reference's CPU math (oracle restatement of the fp32 research attention) on one sequence x one layer of
    the workload per pass, all host cores; plus the CPU-runnable configuration (fp32, one sequence of 256 tokens)
    at one thread and at all threads."""
    from dynakv_b200 import synthetic
    from oracle import dynakv_oracle as O

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S, L = w["seq"], w["layers"]

    def dense_case(seed, seq, dist, theta, dtype):
        case = synthetic.make_layer_case(seed, [seq], dist, theta, dtype, "cpu", N_Q_HEADS, N_KV_HEADS)
        fk, fv, lk, lv, ok, ov = case.views()
        xk = torch.from_numpy(O.decompress_gather(fk.float().numpy(), lk.numpy(), ok.numpy(), 128)).view(1, N_KV_HEADS, seq, 128)
        xv = torch.from_numpy(O.decompress_gather(fv.float().numpy(), lv.numpy(), ov.numpy(), 128)).view(1, N_KV_HEADS, seq, 128)
        return case.q.float(), xk, xv, case.k_up.float(), case.v_up.float(), (lk > 0).view(1, N_KV_HEADS, seq)

    def time_passes(inputs, theta, n, n_warm, limit_s):
        times, t_start = [], time.perf_counter()
        for i in range(n_warm + n):
            t0 = time.perf_counter()
            O.compact_attention_dense(*inputs[:5], theta, inputs[5])
            dt = time.perf_counter() - t0
            if i >= n_warm:
                times.append(dt)
            if time.perf_counter() - t_start > limit_s and len(times) >= 3:
                break
        return times

    main = dense_case(2017, S, w["dist"], w["theta"], torch.bfloat16)
    times = time_passes(main, w["theta"], steps, warmup, max_seconds)
    t_layer_seq = statistics.median(times)
    small = dense_case(17, 256, "uniform", 500000.0, torch.float32)
    t_small_all = statistics.median(time_passes(small, 500000.0, 20, 3, 5.0))
    torch.set_num_threads(1)
    t_small_one = statistics.median(time_passes(small, 500000.0, 20, 3, 5.0))
    torch.set_num_threads(threads)
    # a decode step of one sequence is L such layer passes; sequences are independent
    tok_s = 1.0 / (t_layer_seq * L)
    return {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "1 sequence x 1 layer of the workload (cache length %d) per pass, %d timed passes, "
                      "median %.1f ms; value = 1 / (pass time x %d layers)" % (S, len(times), t_layer_seq * 1e3, L),
            "seconds_per_pass": t_layer_seq, "passes": len(times),
            "fp32_b1_s256_ms_per_layer": {"threads_1": t_small_one * 1e3, "threads_%d" % threads: t_small_all * 1e3}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    base = cpu_reference(w, steps=max(args.steps, 3), warmup=args.warmup, max_seconds=150.0)
    # a step of this arm is the bounded sample that actually ran: one sequence x one layer (the reported
    # ms_per_step times steps is the time spent); value is the whole-workload rate it implies
    line = {
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": base["value"], "unit": "tokens/s",
        "n_gpus": world, "steps": base["passes"], "warmup": args.warmup, "ms_per_step": base["seconds_per_pass"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w, world),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="long_b8_s32768", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true", help="skip the reference's Triton kernels at N=1")
    ap.add_argument("--no-extra-legs", action="store_true", help="skip the ragged strong-scaling and KV-head-sharded legs")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="REPS",
                    help="only time the bulk (prefill) projection and pack with REPS launches each, print that object")
    ap.add_argument("--pipe-probe", action="store_true",
                    help="only run the tensor-pipe occupancy probe of the decode kernel's products, print that object")
    args = ap.parse_args()
    if args.prefill_only > 0:
        torch.cuda.set_device(0)
        print(json.dumps(prefill_compress_leg(torch.device("cuda:0"), args.prefill_only)))
        return
    if args.pipe_probe:
        torch.cuda.set_device(0)
        print(json.dumps(tensor_pipe_probe(torch.device("cuda:0"))))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
