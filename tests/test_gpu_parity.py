"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and against the
fixtures generated from the reference.

Tolerances: fp32 paths 2e-5 absolute; 16-bit paths max-abs <= 2e-2 and mean-relative <= 1e-2 against
the oracle evaluated in fp32 on the same (16-bit rounded) inputs; cache layout bit-exact.
"""
import numpy as np
import pytest
import torch

from dynakv_b200 import synthetic
from dynakv_b200.kernels import _common
from dynakv_b200.kernels.compressed_cache import CustomDynamicCache, simple_decompress
from dynakv_b200.kernels.fused import fused_attention_dispatch
from dynakv_b200.kernels.router import KernelPolicy, compressed_decode_attention
from dynakv_b200.kernels.two_stage import abx_sparse, avx, two_stage_attention
from oracle import dynakv_oracle as O
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"

MAX_ABS_16, MEAN_REL_16 = 2e-2, 1e-2


def _check16(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    mean_rel = ((out - ref).abs().mean() / ref.abs().mean().clamp_min(1e-12)).item()
    assert max_abs <= MAX_ABS_16, f"max-abs {max_abs}"
    assert mean_rel <= MEAN_REL_16, f"mean-rel {mean_rel}"
    assert _common.read_status(torch.device(DEV)) == 0


def _golden_attn(name, dtype):
    g = load_golden(name)
    t = {k: torch.from_numpy(g[k]) for k in ("q", "k_up", "v_up", "flat_k", "flat_v", "lens_k", "lens_v", "offs_k", "offs_v")}
    for k in ("q", "k_up", "v_up", "flat_k", "flat_v"):
        t[k] = t[k].to(dtype)
    return g, t


def _pad8(flat):
    pad = (-flat.shape[1]) % 8
    return torch.nn.functional.pad(flat, (0, pad)) if pad else flat


def _run(fn, t, theta, **kw):
    d = {k: v.to(DEV) for k, v in t.items()}
    return fn(d["q"], _pad8(d["flat_k"]), d["k_up"], _pad8(d["flat_v"]), d["v_up"], d["lens_k"], d["offs_k"],
              d["lens_v"], d["offs_v"], theta, **kw)


def _oracle(t, theta, **kw):
    return O.compact_attention(t["q"], t["flat_k"], t["k_up"], t["flat_v"], t["v_up"], t["lens_k"], t["offs_k"],
                               t["lens_v"], t["offs_v"], theta, **kw)


# ------------------------------------------------------------------ golden fixtures, fp32
@pytest.mark.parametrize("name", ["attn_perhead_s45", "attn_perhead_s130_pad", "attn_joint_s37"])
@pytest.mark.parametrize("fn", [fused_attention_dispatch, two_stage_attention])
def test_fp32_matches_reference_fixtures(name, fn):
    g, t = _golden_attn(name, torch.float32)
    out = _run(fn, t, float(g["theta"])).cpu().numpy()
    assert np.abs(out - g["research_out"]).max() < 2e-5
    assert np.abs(out - g["triton_fused"]).max() < 2e-5


@pytest.mark.parametrize("name", ["attn_perhead_s45", "attn_perhead_s130_pad", "attn_joint_s37"])
def test_stage_operators_match_reference_fixtures(name):
    g, t = _golden_attn(name, torch.float32)
    d = {k: v.to(DEV) for k, v in t.items()}
    sc = abx_sparse(d["q"], d["k_up"], d["flat_k"], d["lens_k"], offsets=d["offs_k"], theta=float(g["theta"]))
    ref_sc = g["triton_scores"]
    assert np.abs(sc.cpu().numpy() - ref_sc).max() < 2e-5 * max(1.0, np.abs(ref_sc).max() / 100)
    out = avx(torch.from_numpy(ref_sc).to(DEV), d["flat_v"], d["v_up"], d["lens_v"], d["offs_v"])
    assert np.abs(out.cpu().numpy() - g["triton_avx"]).max() < 2e-5
    out4 = avx(sc.unsqueeze(2), d["flat_v"], d["v_up"], d["lens_v"], d["offs_v"])
    assert np.abs(out4.cpu().numpy() - g["triton_avx"]).max() < 5e-5


def test_qwen_knorm_fp32_matches_research_fixture():
    g, t = _golden_attn("attn_qwen_knorm_s50", torch.float32)
    w = torch.from_numpy(g["k_norm_weight"])
    out = _run(fused_attention_dispatch, t, float(g["theta"]), k_norm_weight=w.to(DEV), k_norm_eps=1e-6)
    assert np.abs(out.cpu().numpy() - g["research_out"]).max() < 2e-5


# ------------------------------------------------------------------ golden fixtures, 16-bit tensor-core path
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["attn_perhead_s45", "attn_perhead_s130_pad"])
@pytest.mark.parametrize("fn", [fused_attention_dispatch, two_stage_attention])
def test_16bit_tensor_core_path_on_fixtures(name, fn, dtype):
    g, t = _golden_attn(name, dtype)
    ref = _oracle(t, float(g["theta"]))
    out = _run(fn, t, float(g["theta"]), len_multiple=8)
    _check16(out, ref)
    # the generic kernel on the same 16-bit inputs agrees as well
    _check16(_run(fn, t, float(g["theta"]), len_multiple=1), ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fn", [fused_attention_dispatch, two_stage_attention])
def test_16bit_joint_layout_of_the_reference(fn, dtype):
    # the reference's own layout in 16 bit: one latent row shared by all heads, bases [Hq, R, D], any integer length
    g, t = _golden_attn("attn_joint_s37", dtype)
    ref = _oracle(t, float(g["theta"]))
    _check16(_run(fn, t, float(g["theta"])), ref)


def _joint_case(seed, B, S, R, Hq, dtype, ragged=False):
    """The reference's literal layout: one joint latent row per batch row, bases [Hq, R, 128], any integer length."""
    gen = torch.Generator().manual_seed(seed)

    def side():
        lens = torch.randint(0, R // 2, (B, S), generator=gen, dtype=torch.int32)
        lens[:, 0] = torch.maximum(lens[:, 0], torch.ones_like(lens[:, 0]))
        offs = (torch.cumsum(lens.long(), 1) - lens.long()).to(torch.int32)
        cap = int(lens.long().sum(1).max()) + 5
        sigma = torch.exp(-torch.arange(R, dtype=torch.float32) / (R / 4))
        flat = (torch.randn(B, cap, generator=gen) * sigma[torch.arange(cap) % R]).to(dtype)
        return flat, lens, offs

    fk, lk, ok = side()
    fv, lv, ov = side()
    t = {"q": torch.randn(B, Hq, 128, generator=gen).to(dtype), "flat_k": fk, "flat_v": fv, "lens_k": lk, "lens_v": lv,
         "offs_k": ok, "offs_v": ov,
         "k_up": (torch.randn(Hq, R, 128, generator=gen) / R ** 0.5).to(dtype),
         "v_up": (torch.randn(Hq, R, 128, generator=gen) / R ** 0.5).to(dtype)}
    return t


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
def test_joint_layout_long_cache_slices_and_merges(dtype):
    # 700 tokens: the two-stage entry cuts the token axis into slices and merges their partial records; the 16-bit
    # types reconstruct K with mma.sync.  Ragged rows (300 and 700 tokens) leave one row's last slices empty.
    t = _joint_case(21, 2, 700, 256, 8, dtype)
    seq = [300, 700]
    ref = _oracle(t, 10000.0, seq_lens=seq)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    for fn in (two_stage_attention, fused_attention_dispatch):
        out = _run(fn, t, 10000.0, seq_lens=sl)
        if dtype == torch.float32:
            assert float((out.cpu() - ref).abs().max()) < 5e-5
            assert _common.read_status(torch.device(DEV)) == 0
        else:
            _check16(out, ref)


@pytest.mark.parametrize("fn", [fused_attention_dispatch, two_stage_attention])
def test_qwen_knorm_bf16(fn):
    g, t = _golden_attn("attn_qwen_knorm_s50", torch.bfloat16)
    w = torch.from_numpy(g["k_norm_weight"])
    ref = _oracle(t, float(g["theta"]), k_norm_weight=w, k_norm_eps=1e-6)
    out = _run(fn, t, float(g["theta"]), k_norm_weight=w.to(DEV), k_norm_eps=1e-6, len_multiple=8)
    _check16(out, ref)


# ------------------------------------------------------------------ cache layout, bit exact
@pytest.mark.parametrize("name,step", [("cache_prefill_decode", 8), ("cache_anylen", 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_layout_bit_exact(name, step, dtype):
    g = load_golden(name)
    R = int(g["R"])
    cache = CustomDynamicCache(len_multiple=step)
    pre = torch.from_numpy(g["prefill"]).to(dtype).to(DEV)
    pre_len = torch.from_numpy(g["prefill_len"]).to(DEV)
    ret = cache.update_sp(pre, pre_len, pre, pre_len, R, 0, R)
    steps = torch.from_numpy(g["steps"]).to(dtype).to(DEV)
    step_lens = torch.from_numpy(g["step_lens"]).to(DEV)
    for s in range(steps.shape[1]):
        ret = cache.update_sp(steps[:, s:s + 1].contiguous(), step_lens[:, s:s + 1].contiguous(),
                              steps[:, s:s + 1].contiguous(), step_lens[:, s:s + 1].contiguous(), R, 0, R)
    flat_k, flat_v, lens_k, lens_v, offs_k, offs_v = ret
    seq = int(g["seq"])
    assert cache.get_seq_length_sp(0) == seq and cache.get_seq_length(0) == seq
    assert lens_k.shape[1] == seq
    assert np.array_equal(lens_k.cpu().numpy(), g["lens"]) and np.array_equal(lens_v.cpu().numpy(), g["lens"])
    assert np.array_equal(offs_k.cpu().numpy(), g["offs"]) and np.array_equal(offs_v.cpu().numpy(), g["offs"])
    assert np.array_equal(cache.key_cache_sp[0][3].cpu().numpy(), g["ptr"])
    want = torch.from_numpy(g["flat"]).to(dtype)
    for n in range(want.shape[0]):
        p = int(g["ptr"][n])
        assert torch.equal(flat_k[n, :p].cpu(), want[n, :p])
        assert torch.equal(flat_v[n, :p].cpu(), want[n, :p])
    dense_k, dense_v = cache.get_origin_states(R, 0)
    want_dense = torch.from_numpy(g["dense"]).to(dtype)
    assert torch.equal(dense_k.cpu(), want_dense) and torch.equal(dense_v.cpu(), want_dense)
    assert torch.equal(simple_decompress(flat_k, lens_k, R).cpu(), want_dense)
    assert _common.read_status(torch.device(DEV)) == 0


def test_cache_per_head_append_and_growth_match_layout_oracle():
    torch.manual_seed(5)
    B, H, R = 3, 8, 128
    cache = CustomDynamicCache(arenas_per_batch=H, len_multiple=8)
    lay_k, lay_v = O.LayoutOracle(B * H, np.float32), O.LayoutOracle(B * H, np.float32)
    gen = torch.Generator().manual_seed(9)
    for n_new in (5, 1, 1, 1300, 1, 1):   # prefill, decode, a block that forces both buffers to grow
        ks = torch.randn(B, n_new, H * R, generator=gen)
        vs = torch.randn(B, n_new, H * R, generator=gen)
        kl = (torch.randint(1, 17, (B, H, n_new), generator=gen) * 8).to(torch.int32)
        vl = (torch.randint(1, 17, (B, H, n_new), generator=gen) * 8).to(torch.int32)
        ret = cache.update_sp(ks.to(DEV), kl.to(DEV), vs.to(DEV), vl.to(DEV), H * R, 0, R)
        to_rows = lambda x: x.view(B, n_new, H, R).permute(0, 2, 1, 3).reshape(B * H, n_new, R).numpy()
        lay_k.update(to_rows(ks), kl.view(B * H, n_new).numpy())
        lay_v.update(to_rows(vs), vl.view(B * H, n_new).numpy())
    for lay, flat, lens, offs, st in ((lay_k, ret[0], ret[2], ret[4], cache.key_cache_sp[0]),
                                      (lay_v, ret[1], ret[3], ret[5], cache.value_cache_sp[0])):
        assert np.array_equal(lens.cpu().numpy(), lay.lens) and np.array_equal(offs.cpu().numpy(), lay.offs)
        assert np.array_equal(st[3].cpu().numpy(), lay.ptr)
        f = flat.cpu().numpy()
        for n in range(lay.n):
            assert np.array_equal(f[n, : lay.ptr[n]], lay.flat[n])
    assert _common.read_status(torch.device(DEV)) == 0


def test_append_with_projection_and_status_flags():
    import ctypes as C
    from dynakv_b200 import _lib
    B, H, R = 2, 4, 128
    dt = torch.bfloat16
    basis_k = synthetic.qr_bases(H, 3, dt, DEV)
    basis_v = synthetic.qr_bases(H, 4, dt, DEV)
    cache = CustomDynamicCache(arenas_per_batch=H, len_multiple=8)
    cache.reserve(0, B, 1024, 16, dt, DEV)
    ck, cv = cache.key_cache_sp[0], cache.value_cache_sp[0]
    x_k = torch.randn(B, H, R).to(dt).to(DEV)
    x_v = torch.randn(B, H, R).to(dt).to(DEV)
    lk = (torch.randint(1, 17, (B, H)) * 8).to(torch.int32).to(DEV)
    lv = (torch.randint(1, 17, (B, H)) * 8).to(torch.int32).to(DEV)
    st = _common.status_word(torch.device(DEV))
    a = _lib.AppendArgs()
    a.dtype, a.batch, a.arenas_per_batch, a.max_dim = _lib.DKV_BF16, B, H, R
    a.new_k, a.new_v, a.len_k, a.len_v = x_k.data_ptr(), x_v.data_ptr(), lk.data_ptr(), lv.data_ptr()
    a.k_basis, a.v_basis = basis_k.data_ptr(), basis_v.data_ptr()
    a.k, a.v = cache._side(ck), cache._side(cv)
    a.seq_pos, a.seq_capacity, a.len_multiple = 0, 16, 8
    a.status, a.stream = st.data_ptr(), _lib.stream_ptr(torch.device(DEV))
    _lib.check(_lib.load().dkv_append_decode(C.byref(a)), "append")
    want_k = O.project_rows(x_k.cpu(), basis_k.cpu())
    for b in range(B):
        for h in range(H):
            n = int(lk[b, h])
            row = b * H + h
            assert int(ck[1][row, 0]) == n and int(ck[2][row, 0]) == 0 and int(ck[3][row]) == n
            got = ck[0][row, :n].float().cpu()
            assert (got - want_k[b, h, :n]).abs().max() <= 2.0 ** -7 * want_k[b, h, :n].abs().max().clamp_min(1e-3)
    assert _common.read_status(torch.device(DEV)) == 0
    # a length that is not a multiple of 8 and one that overflows the sequence capacity are flagged, not fatal
    lk_bad = lk.clone()
    lk_bad[0, 0] = 13
    a.len_k, a.seq_pos = lk_bad.data_ptr(), 1
    _lib.check(_lib.load().dkv_append_decode(C.byref(a)), "append")
    assert _common.read_status(torch.device(DEV)) & _lib.ST_BAD_LENGTH
    a.len_k, a.seq_pos = lk.data_ptr(), 16
    _lib.check(_lib.load().dkv_append_decode(C.byref(a)), "append")
    assert _common.read_status(torch.device(DEV)) & _lib.ST_OVERFLOW


def test_bulk_pack_that_does_not_fit_records_empty_tokens_and_keeps_the_pointer():
    """Row 0 of a 2-row cache has room for its block, row 1 does not: row 1 is flagged, keeps its write pointer and
    its tokens are recorded as empty; a block past the sequence capacity is flagged and leaves the row untouched."""
    import ctypes as C

    from dynakv_b200 import _lib
    dev = torch.device(DEV)
    S, R = 40, 128
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(1, S, 2 * R, generator=gen).to(torch.bfloat16).to(dev)
    lens = torch.full((1, 2, S), 8, dtype=torch.int32)
    lens[0, 1] = 64
    cache = CustomDynamicCache(arenas_per_batch=2, len_multiple=8)
    cache.reserve(0, 1, 40 * 8 + 64, S + 8, torch.bfloat16, dev)      # 384 elements per arena row: 40*64 does not fit
    ck = cache.key_cache_sp[0]
    ck[1].fill_(-7)
    p = _lib.PackArgs()
    p.dtype, p.batch, p.arenas_per_batch, p.n_new, p.max_dim = _lib.DKV_BF16, 1, 2, S, R
    p.states, p.stride_b, p.stride_j, p.stride_s = x.data_ptr(), x.stride(0), R, x.stride(1)
    lens_d = lens.view(2, S).contiguous().to(dev)
    p.new_lens, p.side = lens_d.data_ptr(), cache._side(ck)
    p.seq_pos, p.seq_capacity, p.len_multiple = 0, ck[1].shape[1], 8
    p.status, p.stream = _common.status_word(dev).data_ptr(), _lib.stream_ptr(dev)
    _common.status_word(dev).zero_()
    _lib.check(_lib.load().dkv_pack_bulk(C.byref(p)), "dkv_pack_bulk")
    assert _common.read_status(dev) == _lib.ST_OVERFLOW
    assert ck[3].tolist() == [S * 8, 0]
    assert ck[1][0, :S].tolist() == [8] * S and ck[2][0, :S].tolist() == [8 * i for i in range(S)]
    assert ck[1][1, :S].tolist() == [0] * S and ck[2][1, :S].tolist() == [0] * S
    assert torch.equal(ck[0][0, : S * 8].view(S, 8), x[0, :, :8])
    # positions past the metadata row: nothing is written
    ck[1].fill_(-7)
    p.seq_pos = ck[1].shape[1] - S + 1
    _lib.check(_lib.load().dkv_pack_bulk(C.byref(p)), "dkv_pack_bulk")
    assert _common.read_status(dev) & _lib.ST_OVERFLOW
    assert bool((ck[1] == -7).all()) and ck[3].tolist() == [S * 8, 0]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("d", [128, 96])
def test_gate_of_both_sides_in_one_launch_gives_the_lengths_of_the_two_kernel_path(dtype, d):
    from dynakv_b200.kernels.compressed_attention import gate_lengths, gate_lengths_pair
    gen = torch.Generator().manual_seed(77)
    n = 37
    xk = (torch.randn(n, d, generator=gen) * 2).to(dtype).to(DEV)
    xv = (torch.randn(n, d, generator=gen) * 2).to(dtype).to(DEV)
    Wk = (torch.randn(d, d, generator=gen) * 0.3).to(dtype).to(DEV)
    Wv = (torch.randn(d, d, generator=gen) * 0.3).to(dtype).to(DEV)
    bk = torch.randn(d, generator=gen).to(dtype).to(DEV)
    bv = torch.randn(d, generator=gen).to(dtype).to(DEV)
    for mult in (1, 8):
        lk = torch.empty(n, dtype=torch.int32, device=DEV)
        lv = torch.empty(n, dtype=torch.int32, device=DEV)
        gate_lengths_pair(xk, Wk, bk, xv, Wv, bv, d, lk, lv, len_multiple=mult)
        _, want_k = gate_lengths(xk, Wk, bk, d, return_masked=False, len_multiple=mult)
        _, want_v = gate_lengths(xv, Wv, bv, d, return_masked=False, len_multiple=mult)
        assert torch.equal(lk, want_k) and torch.equal(lv, want_v)
        assert int(lk.min()) >= 1 and len(set(lk.tolist())) > 3     # a spread of cutoffs, not one value


# ------------------------------------------------------------------ benchmark-shaped configurations
def _case_args(case):
    fk, fv, lk, lv, ok, ov = case.views()
    return case.q, fk, case.k_up, fv, case.v_up, lk, ok, lv, ov, case.theta


def _case_oracle(case, **kw):
    c = case
    fk, fv, lk, lv, ok, ov = c.views()
    return O.compact_attention(c.q.cpu(), fk.cpu(), c.k_up.cpu(), fv.cpu(), c.v_up.cpu(), lk.cpu(), ok.cpu(),
                               lv.cpu(), ov.cpu(), c.theta, seq_lens=c.seq_lens, **kw)


def test_config0_fp32_single_layer_decode():
    case = synthetic.make_layer_case(17, [256], "uniform", 500000.0, torch.float32, DEV)
    ref = _case_oracle(case)
    for fn in (fused_attention_dispatch, two_stage_attention):
        out = fn(*_case_args(case), len_multiple=8)
        assert (out.cpu() - ref).abs().max() < 2e-5


def test_config1_short_ragged_batch_bf16():
    gen = torch.Generator().manual_seed(1017)
    seq_lens = torch.randint(64, 500, (4,), generator=gen).tolist()
    case = synthetic.make_layer_case(1017, seq_lens, "beta:2,5", 500000.0, torch.bfloat16, DEV)
    ref = _case_oracle(case)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    out = fused_attention_dispatch(*_case_args(case), seq_lens=sl, len_multiple=8)
    _check16(out, ref)
    # right-padding with zero-length tokens alone (the reference's way to express a ragged batch) agrees
    _check16(fused_attention_dispatch(*_case_args(case), len_multiple=8), ref)
    # routed through the policy: every row is below the switch point
    q4 = case.q.unsqueeze(2)
    fk, fv, lk, lv, ok, ov = case.views()
    out_r = compressed_decode_attention(q=q4, k_flat=fk, k_up=case.k_up, v_flat=fv, v_up=case.v_up, key_lengths=lk,
                                        key_offsets=ok, value_lengths=lv, value_offsets=ov, theta=case.theta,
                                        cache_length=case.S, len_multiple=8)
    _check16(out_r, ref)


def test_config2_long_cache_split_path_scaled_down():
    case = synthetic.make_layer_case(2017, [3000, 3000], "beta:2,8", 500000.0, torch.bfloat16, DEV)
    ref = _case_oracle(case)
    out = two_stage_attention(*_case_args(case), len_multiple=8)
    _check16(out, ref)
    _check16(fused_attention_dispatch(*_case_args(case), len_multiple=8), ref)


def test_config3_qwen_ragged_routing_across_switch_point():
    seq_lens = [128, 498, 499, 500, 777, 1500]
    case = synthetic.make_layer_case(3017, seq_lens, "beta:2.4,2.6", 1000000.0, torch.bfloat16, DEV)
    w = (1.0 + 0.02 * torch.randn(128, generator=torch.Generator().manual_seed(3)))
    ref = _case_oracle(case, k_norm_weight=w, k_norm_eps=1e-6)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    fk, fv, lk, lv, ok, ov = case.views()
    policy = KernelPolicy(500)
    assert policy.partition(seq_lens) == ([0, 1, 2], [3, 4, 5])
    out = compressed_decode_attention(q=case.q, k_flat=fk, k_up=case.k_up, v_flat=fv, v_up=case.v_up, key_lengths=lk,
                                      key_offsets=ok, value_lengths=lv, value_offsets=ov, theta=case.theta,
                                      cache_length=max(seq_lens), policy=policy, seq_lens=sl, seq_lens_host=seq_lens,
                                      k_norm_weight=w.to(DEV), k_norm_eps=1e-6, len_multiple=8)
    _check16(out, ref)


# ------------------------------------------------------------------ edge cases and properties
@pytest.mark.parametrize("seq_lens", [[1], [15, 16, 17], [63, 64, 65], [0, 40], [129, 1, 300]])
def test_edge_lengths_both_paths(seq_lens):
    case = synthetic.make_layer_case(77, seq_lens, "uniform", 10000.0, torch.bfloat16, DEV, n_q_heads=8, n_kv_heads=2)
    ref = _case_oracle(case)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    for fn in (fused_attention_dispatch, two_stage_attention):
        out = fn(*_case_args(case), seq_lens=sl, len_multiple=8)
        ref_f = torch.nan_to_num(ref, nan=0.0)
        out_c, ref_c = out.float().cpu(), ref_f
        assert (out_c - ref_c).abs().max() <= MAX_ABS_16
    st = _common.read_status(torch.device(DEV))
    assert st == (4 if 0 in seq_lens else 0)   # an empty row is reported, its output is zeros


def test_full_rank_and_minimum_rank_rows():
    for dist_seed, fill in ((1, 128), (2, 8)):
        case = synthetic.make_layer_case(dist_seed, [200], "uniform", 500000.0, torch.bfloat16, DEV, n_q_heads=8, n_kv_heads=2)
        # rebuild with constant lengths
        lens = torch.full((2, 200), fill, dtype=torch.int32, device=DEV)
        gen = torch.Generator(device=DEV).manual_seed(dist_seed)
        case.k = synthetic.ragged_side(lens, gen, torch.bfloat16)
        case.v = synthetic.ragged_side(lens, gen, torch.bfloat16)
        ref = _case_oracle(case)
        for fn in (fused_attention_dispatch, two_stage_attention):
            _check16(fn(*_case_args(case), len_multiple=8), ref)


def test_split_and_fused_agree_at_full_config2_size_per_sequence():
    # one sequence of the long-cache configuration at its real length: the two execution strategies compute the same
    # attention, whichever split a token lands in (the comparison with the oracle at this size is in
    # tests/test_gpu_decode_step.py)
    case = synthetic.make_layer_case(2117, [32768], "beta:2,8", 500000.0, torch.bfloat16, DEV)
    a = two_stage_attention(*_case_args(case), len_multiple=8).float()
    b = fused_attention_dispatch(*_case_args(case), len_multiple=8).float()
    assert (a - b).abs().max().item() <= 4e-3
    assert torch.isfinite(a).all()
    assert _common.read_status(torch.device(DEV)) == 0


def test_linearity_in_values():
    # out is linear in the V coefficients: scaling V by 2 doubles the output (exact in binary floating point)
    case = synthetic.make_layer_case(5, [700], "beta:2,5", 500000.0, torch.bfloat16, DEV, n_q_heads=8, n_kv_heads=2)
    out1 = two_stage_attention(*_case_args(case), len_multiple=8).float()
    case.v.flat.mul_(2.0)
    out2 = two_stage_attention(*_case_args(case), len_multiple=8).float()
    assert (out2 - 2.0 * out1).abs().max().item() <= 2.0 * 2.0 ** -8 * out1.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_reference_maximum_is_raised_late_in_a_row(dtype):
    # The scores of the last third of the row are far larger than anything before (K coefficients x 24):
    # the softmax reference has to be raised, and the accumulated O rescaled, well after the first tile --
    # in the fused kernel (one CTA walks the row) and in the split kernel (the jump falls inside a CTA's range).
    seq = 1536
    case = synthetic.make_layer_case(91, [seq, 900], "beta:2,5", 500000.0, dtype, DEV, n_q_heads=8, n_kv_heads=2)
    fk, fv, lk, lv, ok, ov = case.views()
    rows = fk.shape[0]
    for r in range(rows):
        start = int(ok[r, 1000].item())          # first coefficient of token 1000 of this arena row
        fk[r, start:] *= 24.0
    ref = _case_oracle(case)
    sl = torch.tensor(case.seq_lens, dtype=torch.int32, device=DEV)
    for fn in (fused_attention_dispatch, two_stage_attention):
        out = fn(*_case_args(case), seq_lens=sl, len_multiple=8)
        _check16(out, ref)
    assert _common.read_status(torch.device(DEV)) == 0


def test_many_short_rows_share_a_split_cta():
    # 40 rows of 1..3 tiles: in the split kernel most CTAs cover several batch rows (row flushes in the middle of
    # a CTA's tile sequence, first-tile flags, partial records of rows that end and begin inside one CTA)
    gen = torch.Generator().manual_seed(77)
    seq_lens = torch.randint(1, 384, (40,), generator=gen).tolist()
    case = synthetic.make_layer_case(78, seq_lens, "beta:2,5", 10000.0, torch.bfloat16, DEV, n_q_heads=8, n_kv_heads=2)
    ref = _case_oracle(case)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=DEV)
    out = two_stage_attention(*_case_args(case), seq_lens=sl, len_multiple=8)
    _check16(out, ref)
    assert _common.read_status(torch.device(DEV)) == 0


# ------------------------------------------------------------------ cutoff gate
def test_gate_matches_reference_fixture():
    # fp32, d = 64, six rows, straight from the reference: every length and every masked row equal
    from dynakv_b200.kernels.compressed_attention import kv_process_fused
    g = load_golden("gate_d64")
    k, v = torch.from_numpy(g["k"]).to(DEV), torch.from_numpy(g["v"]).to(DEV)
    d = k.shape[-1]
    Wk, bk, Wv, bv = (torch.from_numpy(g[n]).to(DEV) for n in ("Wk", "bk", "Wv", "bv"))
    k_out, v_out, len_k, len_v, _, _ = kv_process_fused(k, v, Wk, bk, Wv, bv, d)
    assert torch.equal(len_k.cpu(), torch.from_numpy(g["len_k"]).to(torch.int32))
    assert torch.equal(len_v.cpu(), torch.from_numpy(g["len_v"]).to(torch.int32))
    assert torch.equal(k_out.cpu(), torch.from_numpy(g["k_out"]))
    assert torch.equal(v_out.cpu(), torch.from_numpy(g["v_out"]))


@pytest.mark.parametrize("name,dtype,max_mismatch", [("gate_d1024_f32", torch.float32, 2), ("gate_d1024_bf16", torch.bfloat16, 8),
                                                     ("gate_d1024_f16", torch.float16, 8)])
def test_gate_lengths_at_model_width_against_the_reference_in_the_same_dtype(name, dtype, max_mismatch):
    """256 K rows and 256 V rows of width 1024 through the reference's kv_process_fused in fp32 / bf16 / fp16 (CPU)
    and through the kernel: no row is exempted.  The cut-off is a hard threshold on a running sum, so a different
    summation order inside the d x d product can move a sum across a rounding boundary; such rows differ by one
    position.  The count of differing rows is bounded (and printed)."""
    from tests.golden.make_golden import gate_inputs
    from dynakv_b200.kernels.compressed_attention import gate_lengths
    g = load_golden(name)
    n_rows, d = int(g["n_rows"]), int(g["d"])
    k, v, Wk, bk, Wv, bv = gate_inputs(int(g["seed"]), n_rows, d, dtype)
    chk = np.array([float(t.double().sum()) for t in (k, v, Wk, bk, Wv, bv)])
    assert np.allclose(chk, g["checksum"], rtol=0, atol=1e-6 * np.abs(g["checksum"]).max()), "seeded inputs drifted"
    bad = 0
    for x, W, b, want in ((k, Wk, bk, g["len_k"]), (v, Wv, bv, g["len_v"])):
        _, lens = gate_lengths(x.to(DEV), W.to(DEV), b.to(DEV), d, return_masked=False)
        diff = (lens.reshape(-1).cpu().numpy().astype(np.int64) - want.astype(np.int64))
        bad += int((diff != 0).sum())
        assert np.abs(diff).max() <= 1, "a row differs by more than one position"
    print(f"{name}: {bad} of {2 * n_rows} rows differ from the reference by one position")
    assert bad <= max_mismatch


@pytest.mark.parametrize("dtype,d,low_rank,rows", [(torch.float32, 1024, 1024, 37), (torch.bfloat16, 1024, 640, 37),
                                                   (torch.float16, 128, 128, 37), (torch.float32, 200, 96, 37),
                                                   (torch.bfloat16, 1024, 1024, 3), (torch.float32, 512, 300, 2)])
def test_gate_against_oracle(dtype, d, low_rank, rows):
    # rows * 3 <= 64 takes the decode-shaped path (reduction cut in chunks, weight tiles staged in shared memory).
    # The oracle is evaluated in fp32 on the stored values, so the kernel's rounding of intermediates is off here.
    from dynakv_b200.kernels.compressed_attention import gate_lengths
    gen = torch.Generator().manual_seed(11 + d)
    x = (torch.randn(3, rows, d, generator=gen) * 2).to(dtype)
    W = (torch.randn(d, d, generator=gen) / d ** 0.5).to(dtype)
    b = (torch.randn(d, generator=gen) * 0.5).to(dtype)
    ref = O.gate_lengths(x.reshape(-1, d).float(), W.float(), b.float(), low_rank).reshape(3, rows)
    masked, lens = gate_lengths(x.to(DEV), W.to(DEV), b.to(DEV), low_rank, native_rounding=False)
    diff = (lens.cpu().to(torch.int64) - ref.to(torch.int64))
    assert int(diff.abs().max()) <= 1 and int((diff != 0).sum()) <= 1    # summation order only
    keep = torch.arange(d)[None, None, :] < lens.cpu()[..., None]
    assert torch.equal(masked.cpu(), torch.where(keep, x, torch.zeros_like(x)))
    # lengths rounded up to multiples of 8: a superset of the gate's choice, capped at the row width
    _, lens8 = gate_lengths(x.to(DEV), W.to(DEV), b.to(DEV), low_rank, native_rounding=False, len_multiple=8, return_masked=False)
    want8 = torch.clamp((lens + 7) // 8 * 8, max=d - d % 8)
    assert torch.equal(lens8, want8)


def test_gate_append_attend_with_lengths_rounded_to_multiples_of_8():
    """The reference's own pipeline through the tensor-core kernels: gate (any integer length) -> rounded up to
    multiples of 8 -> append -> attention, against the oracle's attention over the rows the cache holds."""
    from dynakv_b200.kernels.compressed_attention import gate_lengths
    B, H, R, S = 2, 2, 128, 40
    gen = torch.Generator().manual_seed(123)
    dt = torch.bfloat16
    sigma = torch.exp(-torch.arange(R, dtype=torch.float32) / 16.0)
    W = (torch.randn(R, R, generator=gen) * 0.5).to(dt)
    bias = (torch.randn(R, generator=gen) + torch.linspace(3.0, -3.0, R)).to(dt)
    cache = CustomDynamicCache(arenas_per_batch=H, len_multiple=8)
    for s in range(S):
        k = (torch.randn(B, 1, H * R, generator=gen) * sigma.repeat(H)).to(dt).to(DEV)
        v = (torch.randn(B, 1, H * R, generator=gen) * sigma.repeat(H)).to(dt).to(DEV)
        _, lk = gate_lengths(k.view(B, H, R), W.to(DEV), bias.to(DEV), R, len_multiple=8, return_masked=False)
        _, lv = gate_lengths(v.view(B, H, R), W.to(DEV), bias.to(DEV), R, len_multiple=8, return_masked=False)
        assert int((lk % 8).abs().sum()) == 0 and int(lk.min()) >= 8
        fk, fv, l_k, l_v, o_k, o_v = cache.update_sp(k, lk.view(B, H, 1), v, lv.view(B, H, 1), H * R, 0, R)
    assert _common.read_status(torch.device(DEV)) == 0      # no length was flagged or truncated
    q = torch.randn(B, 8, 128, generator=gen).to(dt).to(DEV)
    k_up, v_up = synthetic.qr_bases(H, 5, dt, DEV), synthetic.qr_bases(H, 6, dt, DEV)
    ref = O.compact_attention(q.cpu(), fk.cpu(), k_up.cpu(), fv.cpu(), v_up.cpu(), l_k.cpu(), o_k.cpu(), l_v.cpu(), o_v.cpu(), 10000.0)
    out = fused_attention_dispatch(q, fk, k_up, fv, v_up, l_k, o_k, l_v, o_v, 10000.0, len_multiple=8)
    _check16(out, ref)
