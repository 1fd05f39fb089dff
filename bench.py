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
so no L2 flush is needed between steps.

Multi-GPU: the batch is sharded by sequence (one process per GPU, 8 sequences each, no collective in
the data path) -> weak scaling.  Timing: CUDA events on the launching stream, barrier + synchronize on
both sides, max over ranks.

``--impl reference`` times the reference's own CPU implementation of the same math (fp32 compact
masked-dimension attention on dense zero-masked latents, as restated in oracle/) on the host cores,
rank 0 only, on a bounded sample: one sequence of the workload, one layer per step.
"""
from __future__ import annotations

import argparse
import json
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
# dram__bytes_read.sum + dram__bytes_write.sum of one split-kernel launch divided by its algorithmic bytes,
# from the ncu capture summarised under profiles/; None until such a capture exists.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.18   # dram read+write / algorithmic bytes, profile_b2_s32768 capture


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
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

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

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    ms_step = ms_total / args.steps
    bytes_layer = sum(comp_bytes) / len(comp_bytes)
    total_tokens = w["batch"] * world
    line = {
        "metric": "decode_attn_tokens_per_s", "value": total_tokens / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "batch_per_gpu": w["batch"], "cache_len": w["seq"], "layers": L,
                   "q_heads": N_Q_HEADS, "kv_heads": N_KV_HEADS, "head_dim": HEAD_DIM, "length_dist": w["dist"],
                   "retention": 0.5 * bytes_layer / (sum(seq_lens) * N_KV_HEADS * 128 * 2),
                   "l2": "inputs larger than L2 (%.1f GB of distinct cache bytes per step per GPU), no flush" %
                         (sum(comp_bytes) / 1e9),
                   "parallelism": "sequence-sharded x%d" % world},
        "us_per_layer": ms_step * 1e3 / L,
        "hbm_gbs_step": sum(comp_bytes) / (ms_step * 1e-3) / 1e9,
        "e2e": {"value": total_tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": graph.h2d_bytes_per_step(), "d2h_bytes_per_step": graph.d2h_bytes_per_step(),
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": graph.kernel_launches_per_step * args.steps,
        "clocks": clocks, "device_status": status,
    }
    if kernel_ms is not None:
        achieved = bytes_layer / (kernel_ms * 1e-3) / 1e9
        line["roofline"] = {
            "kernel": "mma_decode_kernel<bf16, split>", "bound": "hbm", "achieved": achieved, "peak": peak,
            "peak_source": "of " + peak_kind, "unit": "GB/s", "frac": achieved / peak, "us_per_launch": kernel_ms * 1e3,
            "algorithmic_bytes_per_launch": bytes_layer,
            "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer) if NCU_TRAFFIC_PER_ALGORITHMIC_BYTE else None,
            "frac_of_nominal_8TBs": achieved / 8000.0}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(w, steps=3, warmup=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------- reference arm
def cpu_reference(w, steps, warmup, max_seconds=25.0):
    """The reference's CPU math (oracle restatement) on one sequence x one layer of the workload."""
    from dynakv_b200 import synthetic
    from oracle import dynakv_oracle as O

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S, L = w["seq"], w["layers"]
    case = synthetic.make_layer_case(2017, [S], w["dist"], w["theta"], torch.bfloat16, "cpu", N_Q_HEADS, N_KV_HEADS)
    fk, fv, lk, lv, ok, ov = case.views()
    xk = torch.from_numpy(O.decompress(fk.float().numpy(), lk.numpy(), 128, ok.numpy())).view(1, N_KV_HEADS, S, 128)
    xv = torch.from_numpy(O.decompress(fv.float().numpy(), lv.numpy(), 128, ov.numpy())).view(1, N_KV_HEADS, S, 128)
    q, ku, vu = case.q.float(), case.k_up.float(), case.v_up.float()
    valid = (lk > 0).view(1, N_KV_HEADS, S)
    times = []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.compact_attention_dense(q, xk, xv, ku, vu, w["theta"], valid)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_start > max_seconds and len(times) >= 1:
            break
    t_layer_seq = statistics.median(times)
    # a decode step of one sequence is L such layer passes; sequences are independent
    tok_s = 1.0 / (t_layer_seq * L)
    return {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "1 sequence x 1 layer of the workload (cache length %d) per pass, %d timed passes, "
                      "median %.1f ms; value = 1 / (pass time x %d layers)" % (S, len(times), t_layer_seq * 1e3, L),
            "seconds_per_pass": t_layer_seq}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    base = cpu_reference(w, steps=args.steps, warmup=args.warmup, max_seconds=120.0)
    L = w["layers"]
    line = {
        "impl": "reference", "metric": "decode_attn_tokens_per_s", "value": base["value"], "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["seconds_per_pass"] * L * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch_per_gpu": w["batch"], "cache_len": w["seq"], "layers": L,
                   "q_heads": N_Q_HEADS, "kv_heads": N_KV_HEADS, "head_dim": HEAD_DIM, "length_dist": w["dist"]},
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
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
