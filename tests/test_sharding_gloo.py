"""Multi-process (gloo, CPU) tests of the N>1 host logic: sequence sharding, KV-head sharding with the
row-parallel o_proj all-reduce, and the max-over-ranks timing convention.  The attention math inside the
ranks is the CPU oracle here (the checker); on GPUs the same partition feeds the CUDA kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dynakv_b200 import sharding, synthetic
from oracle import dynakv_oracle as O

WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    return synthetic.make_layer_case(99, [40, 70, 33, 64], "uniform", 10000.0, torch.float32, "cpu", n_q_heads=8, n_kv_heads=4)


def _attn(case, rows=None, kv=None):
    fk, fv, lk, lv, ok, ov = case.views()
    H, G = case.n_kv_heads, case.n_q_heads // case.n_kv_heads
    B = len(case.seq_lens)
    b_lo, b_hi = rows if rows else (0, B)
    h_lo, h_hi = kv if kv else (0, H)
    idx = torch.tensor([b * H + h for b in range(b_lo, b_hi) for h in range(h_lo, h_hi)])
    q = case.q[b_lo:b_hi, h_lo * G:h_hi * G]
    return O.compact_attention(q, fk[idx], case.k_up[h_lo:h_hi], fv[idx], case.v_up[h_lo:h_hi], lk[idx], ok[idx],
                               lv[idx], ov[idx], case.theta, seq_lens=case.seq_lens[b_lo:b_hi])


def _worker(rank, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        case = _case()
        full = _attn(case)
        # by sequence: no communication, outputs are disjoint row blocks
        lo, hi = sharding.shard_sequences(len(case.seq_lens), WORLD, rank)
        seq_ok = torch.allclose(_attn(case, rows=(lo, hi)), full[lo:hi], atol=1e-6)
        # by KV head + row-parallel o_proj: one all-reduce reproduces the unsharded projection
        (k_lo, k_hi), (q_lo, q_hi) = sharding.shard_kv_heads(case.n_kv_heads, case.n_q_heads, WORLD, rank)
        local = _attn(case, kv=(k_lo, k_hi)).reshape(len(case.seq_lens), -1)
        w_o = torch.randn(64, case.n_q_heads * 128, generator=torch.Generator().manual_seed(5))
        y = sharding.row_parallel_linear(local, w_o[:, q_lo * 128:q_hi * 128])
        head_ok = torch.allclose(y, full.reshape(len(case.seq_lens), -1) @ w_o.T, atol=1e-4)
        slowest = sharding.max_over_ranks(float(rank + 1), "cpu")
        results[rank] = (seq_ok, head_ok, slowest)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(port, results), nprocs=WORLD, join=True)
        assert len(results) == WORLD
        for r in range(WORLD):
            seq_ok, head_ok, slowest = results[r]
            assert seq_ok and head_ok and slowest == float(WORLD)


def test_block_ranges_cover_everything_once():
    for n in (0, 1, 7, 8, 256):
        for w in (1, 2, 4, 8):
            spans = [sharding.block_range(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= 1
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(8, 32, 3, 0)
    assert sharding.shard_kv_heads(8, 32, 4, 1) == ((2, 4), (8, 16))


def _runner_worker(rank, port, results):
    """The decode runner's tensor-parallel shards on CPU: the column shards of the projections put side by side are
    the one-rank matrices, and the row-parallel output / MLP paths with their all-reduce give the one-rank result.
    (The attention itself needs the CUDA kernels and is covered by the two-GPU test.)"""
    from dynakv_b200.runner import MiniLlama, ModelShape, rms_norm
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        shape = ModelShape(layers=1, hidden=256, mlp=512, vocab=64, n_q_heads=8, n_kv_heads=4)
        one = MiniLlama(shape, "cpu", dtype=torch.float32, seed=9)
        mine = MiniLlama(shape, "cpu", dtype=torch.float32, seed=9, tp_rank=rank, tp_size=WORLD)
        w1, wr = one.layers[0], mine.layers[0]
        (k_lo, k_hi), (q_lo, q_hi) = sharding.shard_kv_heads(shape.n_kv_heads, shape.n_q_heads, WORLD, rank)
        cols_ok = (torch.equal(wr.wq, w1.wq[:, q_lo * 128:q_hi * 128]) and torch.equal(wr.wk, w1.wk[:, k_lo * 128:k_hi * 128])
                   and torch.equal(wr.k_up, w1.k_up[k_lo:k_hi]) and torch.equal(wr.v_up, w1.v_up[k_lo:k_hi])
                   and torch.equal(wr.w_cut, torch.cat((w1.w_cut[k_lo:k_hi], w1.w_cut[4 + k_lo:4 + k_hi]))))
        x = torch.randn(5, shape.hidden, generator=torch.Generator().manual_seed(1))
        mlp_ok = torch.allclose(mine._mlp(wr, x), one._mlp(w1, x), atol=1e-5)
        attn_out = torch.randn(5, shape.n_q_heads * 128, generator=torch.Generator().manual_seed(2))
        o_ok = torch.allclose(mine._all_reduce(attn_out[:, q_lo * 128:q_hi * 128] @ wr.wo), attn_out @ w1.wo, atol=1e-5)
        lk1, lv1 = one._cutoffs(w1, rms_norm(x, w1.norm1, shape.rms_eps))
        lkr, lvr = mine._cutoffs(wr, rms_norm(x, wr.norm1, shape.rms_eps))
        cut_ok = torch.equal(lkr, lk1[:, k_lo:k_hi]) and torch.equal(lvr, lv1[:, k_lo:k_hi])
        results[rank] = (cols_ok, mlp_ok, o_ok, cut_ok)
    finally:
        dist.destroy_process_group()


def test_runner_shards_by_kv_head_reproduce_the_one_rank_model():
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_runner_worker, args=(port, results), nprocs=WORLD, join=True)
        for rank in range(WORLD):
            assert results[rank] == (True, True, True, True), (rank, results[rank])
