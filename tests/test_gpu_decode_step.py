"""GPU parity of whole decode steps at the benchmarked sizes: the layer object and the CUDA graph the benchmark
replays (projected append with cutoff-head lengths, then routed attention), against the CPU oracle.

Outputs: max-abs <= 2e-2 and mean-relative <= 1e-2 against the oracle's fp32 compact attention evaluated on the
cache contents read back from the GPU (the same 16-bit rounded inputs); cache metadata (lens, offs, ptr, row
counters) bit-exact against the layout rule; the projected coefficient rows within 2^-7 relative of the fp32
projection (they are rounded to bf16 once).
"""
import math

import numpy as np
import pytest
import torch

from dynakv_b200 import synthetic
from dynakv_b200.kernels import _common
from dynakv_b200.kernels.compressed_attention import CompressedDecodeLayer, DecodeGraph
from dynakv_b200.kernels.compressed_cache import CustomDynamicCache
from dynakv_b200.kernels.router import KernelPolicy
from oracle import dynakv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
HQ, HKV, D = 32, 8, 128
MAX_ABS_16, MEAN_REL_16 = 2e-2, 1e-2


def _oracle_rows(cache, layer_idx, q, k_up, v_up, theta, rows, seq_lens, k_norm_weight=None):
    """fp32 compact attention (research math on dense zero-masked latents) of the given batch rows, from the cache
    as it is on the GPU now.  Returns {row: [Hq, D]}."""
    ck, cv = cache.key_cache_sp[layer_idx], cache.value_cache_sp[layer_idx]
    out = {}
    ku, vu = k_up.float().cpu(), v_up.float().cpu()
    for b in rows:
        S = int(seq_lens[b])
        sl = slice(b * HKV, (b + 1) * HKV)
        lk, ok = ck[1][sl, :S].cpu().numpy(), ck[2][sl, :S].cpu().numpy()
        lv, ov = cv[1][sl, :S].cpu().numpy(), cv[2][sl, :S].cpu().numpy()
        fk = ck[0][sl, : int((ok + lk).max()) if S else 0].float().cpu().numpy()
        fv = cv[0][sl, : int((ov + lv).max()) if S else 0].float().cpu().numpy()
        xk = torch.from_numpy(O.decompress_gather(fk, lk, ok, 128)).view(1, HKV, S, 128)
        xv = torch.from_numpy(O.decompress_gather(fv, lv, ov, 128)).view(1, HKV, S, 128)
        valid = torch.from_numpy(lk > 0).view(1, HKV, S)
        out[b] = O.compact_attention_dense(q[b:b + 1].float().cpu(), xk, xv, ku, vu, theta, valid,
                                           k_norm_weight=k_norm_weight)[0]
    return out


def _check_rows(out, ref_rows):
    got = torch.stack([out[b].float().cpu() for b in ref_rows])
    ref = torch.stack([ref_rows[b] for b in ref_rows])
    max_abs = (got - ref).abs().max().item()
    mean_rel = ((got - ref).abs().mean() / ref.abs().mean().clamp_min(1e-12)).item()
    assert max_abs <= MAX_ABS_16, f"max-abs {max_abs}"
    assert mean_rel <= MEAN_REL_16, f"mean-rel {mean_rel}"


def _step_inputs(gen, n_layers, batch, dtype):
    q = torch.randn(n_layers, batch, HQ, D, generator=gen).to(dtype)
    nk = torch.randn(n_layers, batch, HKV, D, generator=gen).to(dtype)
    nv = torch.randn(n_layers, batch, HKV, D, generator=gen).to(dtype)
    hidden = torch.randn(batch, 4096, generator=gen)
    wgt = torch.randn(n_layers, 2 * HKV, 4096, generator=gen) / 64.0
    lens = torch.stack([synthetic.cutoff_head_lengths(hidden, wgt[l], -1.75) for l in range(n_layers)])
    return q, nk, nv, lens[..., :HKV].contiguous(), lens[..., HKV:].contiguous()


def _load(graph, q, nk, nv, lk, lv):
    for dst, src in zip((graph.q, graph.new_k, graph.new_v, graph.len_k, graph.len_v), (q, nk, nv, lk, lv)):
        dst.copy_(src)


def _build(seed, seq_lens, dist, theta, n_layers, project, extra, k_norm=False):
    cache = CustomDynamicCache(arenas_per_batch=HKV, len_multiple=8)
    layers, cases = [], []
    w = (1.0 + 0.02 * torch.randn(128, generator=torch.Generator().manual_seed(3))) if k_norm else None
    for li in range(n_layers):
        case = synthetic.make_layer_case(seed + 31 * li, seq_lens, dist, theta, torch.bfloat16, DEV, HQ, HKV,
                                         extra_tokens=extra)
        cache.adopt(li, (case.k.flat, case.k.lens, case.k.offs, case.k.ptr),
                    (case.v.flat, case.v.lens, case.v.offs, case.v.ptr), seq_lens)
        layers.append(CompressedDecodeLayer(li, case.k_up, case.v_up, theta, project_new_rows=project,
                                            k_norm_weight=w))
        cases.append(case)
    return cache, layers, cases, w


def _check_appended_token(cache, li, case, pos_of_row, nk, nv, lk, lv, ptr_before):
    """Layout of the token this step appended: lens = cutoff, offs = pointer before, pointer advanced, payload =
    projection of the new row onto the basis (rounded once to bf16)."""
    for side_idx, (st, new, lens, basis) in enumerate(((cache.key_cache_sp[li], nk, lk, case.k_up),
                                                       (cache.value_cache_sp[li], nv, lv, case.v_up))):
        want = O.project_rows(new.float().cpu(), basis.float().cpu())      # [B, Hkv, R]
        lens_c, offs_c, ptr_c, flat_c = st[1].cpu(), st[2].cpu(), st[3].cpu(), st[0]
        for b, pos in enumerate(pos_of_row):
            for h in range(HKV):
                a = b * HKV + h
                n = int(lens[b, h])
                assert int(lens_c[a, pos]) == n
                assert int(offs_c[a, pos]) == int(ptr_before[side_idx][a])
                assert int(ptr_c[a]) == int(ptr_before[side_idx][a]) + n
                got = flat_c[a, int(offs_c[a, pos]): int(offs_c[a, pos]) + n].float().cpu()
                ref = want[b, h, :n]
                assert (got - ref).abs().max() <= 2.0 ** -7 * ref.abs().max().clamp_min(1e-3)


# ------------------------------------------------------------------ the long-cache configuration at its real length
def test_long_cache_decode_step_at_full_length_against_oracle():
    """One sequence of the long-cache configuration at its real size (32768 cached tokens, 8 KV heads, bf16,
    Beta(2,8) cutoffs): a decode step = append of one projected token with cutoff-head lengths, then the split
    two-stage attention over 32769 tokens, against the oracle's dense compact attention."""
    seq = [32768]
    cache, layers, cases, _ = _build(2017, seq, "beta:2,8", 500000.0, 1, project=True, extra=8)
    graph = DecodeGraph(layers, cache, 1, HQ, torch.bfloat16, DEV, seq)
    q, nk, nv, lk, lv = _step_inputs(torch.Generator().manual_seed(99), 1, 1, torch.bfloat16)
    _load(graph, q, nk, nv, lk, lv)
    ptr_before = [cache.key_cache_sp[0][3].cpu().clone(), cache.value_cache_sp[0][3].cpu().clone()]
    out = graph.step()[0]
    torch.cuda.synchronize()
    assert _common.read_status(torch.device(DEV)) == 0
    assert cache.seq_lens(0).cpu().tolist() == [32769]
    _check_appended_token(cache, 0, cases[0], [32768], nk[0], nv[0], lk[0], lv[0], ptr_before)
    ref = _oracle_rows(cache, 0, q[0], cases[0].k_up, cases[0].v_up, 500000.0, [0], [32769])
    _check_rows(out, ref)


# ------------------------------------------------------------------ the captured graph the benchmark replays
def test_decode_graph_with_projected_append_three_steps():
    seq = [700, 1200, 600]
    cache, layers, cases, _ = _build(4117, seq, "beta:2,8", 500000.0, 2, project=True, extra=16)
    graph = DecodeGraph(layers, cache, 3, HQ, torch.bfloat16, DEV, seq)
    gen = torch.Generator().manual_seed(5)
    graph.capture()
    cur = list(seq)
    for step in range(3):
        q, nk, nv, lk, lv = _step_inputs(gen, 2, 3, torch.bfloat16)
        _load(graph, q, nk, nv, lk, lv)
        before = [[cache.key_cache_sp[li][3].cpu().clone(), cache.value_cache_sp[li][3].cpu().clone()] for li in range(2)]
        out = graph.step()
        torch.cuda.synchronize()
        assert _common.read_status(torch.device(DEV)) == 0
        for li in range(2):
            _check_appended_token(cache, li, cases[li], cur, nk[li], nv[li], lk[li], lv[li], before[li])
            assert cache.seq_lens(li).cpu().tolist() == [n + 1 for n in cur]
            ref = _oracle_rows(cache, li, q[li], cases[li].k_up, cases[li].v_up, 500000.0, [0, 1, 2], [n + 1 for n in cur])
            _check_rows(out[li], ref)
        cur = [n + 1 for n in cur]


# ------------------------------------------------------------------ ragged batch, rows crossing the switch point
def test_ragged_batch_of_64_routes_on_the_device_across_the_switch_point():
    """Qwen3-shaped ragged batch (K-RMSNorm, theta 1e6, ~48 % retention): 64 sequences with log-uniform lengths in
    [128, 32768], three of them placed at 497..499 tokens so that they cross KernelPolicy(500) during three
    consecutive replays of ONE captured graph.  Every row is checked at the last step, the crossing rows at every
    step."""
    seq = synthetic.log_uniform_lengths(64, 128, 32768, seed=3017)
    seq[5], seq[17], seq[40] = 497, 498, 499
    watch = [5, 17, 40, 0, 1]
    policy = KernelPolicy(500)
    cache, layers, cases, w = _build(3017, seq, "beta:2.4,2.6", 1000000.0, 1, project=False, extra=8, k_norm=True)
    graph = DecodeGraph(layers, cache, 64, HQ, torch.bfloat16, DEV, seq)
    assert graph._has_short and graph._has_long
    graph.capture()
    gen = torch.Generator().manual_seed(8)
    cur = list(seq)
    for step in range(3):
        q = torch.randn(1, 64, HQ, D, generator=gen).to(torch.bfloat16)
        nk = (torch.randn(1, 64, HKV, D, generator=gen) * 0.5).to(torch.bfloat16)
        nv = (torch.randn(1, 64, HKV, D, generator=gen) * 0.5).to(torch.bfloat16)
        lk = (torch.randint(1, 17, (1, 64, HKV), generator=gen) * 8).to(torch.int32)
        lv = (torch.randint(1, 17, (1, 64, HKV), generator=gen) * 8).to(torch.int32)
        _load(graph, q, nk, nv, lk, lv)
        out = graph.step()[0]
        torch.cuda.synchronize()
        cur = [n + 1 for n in cur]
        assert _common.read_status(torch.device(DEV)) == 0
        assert cache.seq_lens(0).cpu().tolist() == cur
        rows = list(range(64)) if step == 2 else watch
        ref = _oracle_rows(cache, 0, q[0], cases[0].k_up, cases[0].v_up, 1000000.0, rows, cur, k_norm_weight=w)
        _check_rows(out, ref)
    # the watched rows ended on both sides of the switch point and were served by different kernels on the way
    assert [policy.select(cur[b]) for b in (5, 17, 40)] == ["long_two_stage"] * 3
    assert policy.select(seq[5] + 1) == "short_fused"


# ------------------------------------------------------------------ the cutoff gate replayed with the step
def test_decode_graph_computes_the_cutoffs_with_the_gate():
    """Coefficient rows in, the graph runs the gate (per (sequence, KV head) row, [128 x 128] weights, lengths rounded
    up to multiples of 8), appends and attends; lengths against the oracle's gate in the same dtype, outputs against
    the oracle's attention."""
    seq = [620, 900]
    cache, layers, cases, _ = _build(5217, seq, "beta:2,5", 500000.0, 1, project=False, extra=8)
    gen = torch.Generator().manual_seed(77)
    dt = torch.bfloat16
    Wk = (torch.randn(128, 128, generator=gen) * 0.4).to(dt).to(DEV)
    Wv = (torch.randn(128, 128, generator=gen) * 0.4).to(dt).to(DEV)
    bk = (torch.randn(128, generator=gen) + torch.linspace(3.0, -3.0, 128)).to(dt).to(DEV)
    bv = (torch.randn(128, generator=gen) + torch.linspace(3.0, -3.0, 128)).to(dt).to(DEV)
    layers[0].gate = (Wk, bk, Wv, bv)
    graph = DecodeGraph(layers, cache, 2, HQ, dt, DEV, seq)
    graph.capture()
    sigma = torch.exp(-torch.arange(128, dtype=torch.float32) / 24.0)
    cur = list(seq)
    for step in range(2):
        q = torch.randn(1, 2, HQ, D, generator=gen).to(dt)
        nk = (torch.randn(1, 2, HKV, D, generator=gen) * sigma).to(dt)
        nv = (torch.randn(1, 2, HKV, D, generator=gen) * sigma).to(dt)
        graph.q.copy_(q); graph.new_k.copy_(nk); graph.new_v.copy_(nv)
        out = graph.step()[0]
        torch.cuda.synchronize()
        assert _common.read_status(torch.device(DEV)) == 0
        for new, W, b, got in ((nk, Wk, bk, graph.len_k), (nv, Wv, bv, graph.len_v)):
            want = O.gate_lengths(new.view(-1, 128), W.cpu(), b.cpu(), 128)         # the reference's ops in bf16
            want8 = torch.clamp((want + 7) // 8 * 8, max=128)
            diff = (got.view(-1).cpu().to(torch.int64) - want8.to(torch.int64)).abs()
            assert int(diff.max()) <= 8 and int((diff != 0).sum()) <= 1      # at most one row moved by one position
        cur = [n + 1 for n in cur]
        st = cache.key_cache_sp[0]
        assert torch.equal(st[1][:, cur[0] - 1].view(2, HKV)[0].cpu(), graph.len_k[0, 0].cpu())
        ref = _oracle_rows(cache, 0, q[0], cases[0].k_up, cases[0].v_up, 500000.0, [0, 1], cur)
        _check_rows(out, ref)


# ------------------------------------------------------------------ bulk (prefill) compression at prompt length
def test_bulk_projection_and_pack_at_prompt_length():
    """An 8192-token prompt of 2 sequences: tensor-core projection onto the per-head bases against the oracle's fp32
    projection (one rounding to bf16), then the bulk pack of the projected rows with Beta-distributed cutoffs,
    bit-exact against the layout oracle."""
    from dynakv_b200.kernels.compressed_attention import project_bulk
    B, S = 2, 8192
    gen = torch.Generator().manual_seed(61)
    dt = torch.bfloat16
    x = torch.randn(B, S, HKV * 128, generator=gen).to(dt)
    basis = synthetic.qr_bases(HKV, 71, dt, "cpu")
    coef = project_bulk(x.to(DEV), basis.to(DEV))
    torch.cuda.synchronize()
    assert _common.read_status(torch.device(DEV)) == 0
    want = O.project_rows(x.view(B * S, HKV, 128).float(), basis.float()).reshape(B, S, HKV * 128)
    err = (coef.float().cpu() - want).abs()
    assert float(err.max()) <= 2.0 ** -8 * float(want.abs().max()) * 1.01
    assert float(err.mean()) <= 2.0 ** -9 * float(want.abs().mean())
    # a block that is not a whole tile, through a strided view
    part = project_bulk(x[:1, :333].to(DEV), basis.to(DEV))
    assert torch.equal(part.cpu(), coef[:1, :333].cpu())
    # pack the projected rows
    lens = synthetic.draw_lengths((B, HKV, S), "beta:2,5", gen)
    cache = CustomDynamicCache(arenas_per_batch=HKV, len_multiple=8)
    fk, fv, lk, lv, ok, ov = cache.update_sp(coef, lens.to(DEV), coef, lens.to(DEV), HKV * 128, 0, 128)
    lay = O.LayoutOracle(B * HKV, np.float32)
    rows = coef.float().cpu().view(B, S, HKV, 128).permute(0, 2, 1, 3).reshape(B * HKV, S, 128).numpy()
    lay.update(rows, lens.view(B * HKV, S).numpy())
    assert np.array_equal(lk.cpu().numpy(), lay.lens) and np.array_equal(ok.cpu().numpy(), lay.offs)
    assert np.array_equal(cache.key_cache_sp[0][3].cpu().numpy(), lay.ptr)
    f = fk.float().cpu().numpy()
    for n in range(lay.n):
        assert np.array_equal(f[n, : lay.ptr[n]], lay.flat[n])
    assert torch.equal(fv[:, : int(lay.ptr.max())].cpu(), fk[:, : int(lay.ptr.max())].cpu())
    assert _common.read_status(torch.device(DEV)) == 0
