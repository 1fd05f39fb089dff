"""Pins the CPU oracle against fixtures produced by the reference itself.

Fixtures: tests/golden/*.npz, made by tests/golden/make_golden.py from the
reference's research attention math, its Triton kernels under the Triton
interpreter, its cache-update code and its cutoff gate.
"""
import numpy as np
import pytest
import torch

from oracle import dynakv_oracle as O
from tests.conftest import load_golden

ATTN = ["attn_perhead_s45", "attn_perhead_s130_pad", "attn_joint_s37"]


def _t(g, *names):
    return [torch.from_numpy(g[n]) for n in names]


def _attn_args(g):
    q, ku, vu, fk, fv, lk, lv, ok, ov = _t(g, "q", "k_up", "v_up", "flat_k", "flat_v", "lens_k", "lens_v", "offs_k", "offs_v")
    return q, fk, ku, fv, vu, lk, ok, lv, ov, float(g["theta"])


@pytest.mark.parametrize("name", ATTN)
def test_compact_attention_matches_reference(name):
    g = load_golden(name)
    out = O.compact_attention(*_attn_args(g))
    # research fp32 math and the interpreter-run Triton fused kernel
    assert np.abs(out.numpy() - g["research_out"]).max() < 2e-6
    assert np.abs(out.numpy() - g["triton_fused"]).max() < 2e-6


@pytest.mark.parametrize("name", ATTN)
def test_two_stage_semantics_match_reference(name):
    g = load_golden(name)
    q, fk, ku, fv, vu, lk, ok, lv, ov, theta = _attn_args(g)
    sc = O.scores_reference(q, ku, fk, lk, ok, theta)
    assert np.abs(sc.numpy() - g["triton_scores"]).max() < 2e-5 * max(1.0, np.abs(g["triton_scores"]).max() / 100)
    av = O.softmax_v_reference(torch.from_numpy(g["triton_scores"]), fv, vu, lv, ov)
    assert np.abs(av.numpy() - g["triton_avx"]).max() < 2e-6
    # the two-stage result is the same attention (len-0 tokens get ~0 weight instead of exactly 0)
    assert np.abs(g["triton_avx"] - g["research_out"]).max() < 1e-5


def test_qwen_knorm_matches_research_math():
    g = load_golden("attn_qwen_knorm_s50")
    out = O.compact_attention(*_attn_args(g), k_norm_weight=torch.from_numpy(g["k_norm_weight"]), k_norm_eps=1e-6)
    assert np.abs(out.numpy() - g["research_out"]).max() < 2e-6


@pytest.mark.parametrize("name", ["cache_prefill_decode", "cache_anylen"])
def test_layout_oracle_bit_exact(name):
    g = load_golden(name)
    R = int(g["R"])
    lay = O.LayoutOracle(g["prefill"].shape[0], np.float32)
    lay.update(g["prefill"], g["prefill_len"])
    for s in range(g["steps"].shape[1]):
        lay.update(g["steps"][:, s:s + 1], g["step_lens"][:, s:s + 1])
    assert lay.seq == int(g["seq"])
    assert np.array_equal(lay.lens, g["lens"])
    assert np.array_equal(lay.offs, g["offs"])
    assert np.array_equal(lay.ptr, g["ptr"])
    for n in range(lay.n):
        assert np.array_equal(lay.flat[n], g["flat"][n, : lay.ptr[n]])
    dense = O.decompress(g["flat"], g["lens"], R)
    assert np.array_equal(dense, g["dense"])
    assert np.array_equal(O.decompress(g["flat"], g["lens"], R, g["offs"]), g["dense"])


def test_gate_lengths_bit_exact():
    g = load_golden("gate_d64")
    k, v = torch.from_numpy(g["k"]), torch.from_numpy(g["v"])
    d = k.shape[-1]
    lk = O.gate_lengths(k.view(-1, d), torch.from_numpy(g["Wk"]), torch.from_numpy(g["bk"]), d)
    lv = O.gate_lengths(v.view(-1, d), torch.from_numpy(g["Wv"]), torch.from_numpy(g["bv"]), d)
    assert np.array_equal(lk.numpy(), g["len_k"].reshape(-1))
    assert np.array_equal(lv.numpy(), g["len_v"].reshape(-1))


def test_router_boundary():
    # same behaviours as the reference's tests/test_kernel_router.py
    assert O.select_path(0) == "short_fused"
    assert O.select_path(499) == "short_fused"
    assert O.select_path(500) == "long_two_stage"
    assert O.select_path(127, 128) == "short_fused"
    assert O.select_path(128, 128) == "long_two_stage"
    with pytest.raises(ValueError):
        O.select_path(-1)


def test_decompress_gather_equals_the_per_token_loop():
    rng = np.random.default_rng(3)
    lens = (rng.integers(0, 17, size=(5, 37)) * 8).astype(np.int32)
    offs = (np.cumsum(lens, axis=1) - lens).astype(np.int32)
    flat = rng.standard_normal((5, int(lens.sum(axis=1).max()) + 3)).astype(np.float32)
    assert np.array_equal(O.decompress_gather(flat, lens, offs, 128), O.decompress(flat, lens, 128, offs))
    assert np.array_equal(O.decompress_gather(flat, lens, offs, 64), O.decompress(flat, lens, 64, offs))
