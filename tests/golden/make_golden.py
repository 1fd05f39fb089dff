"""Generate the golden fixtures under tests/golden/ by running the reference.

Run once, in a container that has the reference checkout, from the repo root:

    TRITON_INTERPRET=1 PYTHONPATH=<reference>/src python tests/golden/make_golden.py <reference>

It imports the reference's own code and records inputs + outputs of
  G1  the research ("compact") attention math      src/dynakv/custom_attn.py
  G2  the Triton decode kernels run by the Triton CPU interpreter
                                                     src/dynakv/kernels/fused.py, two_stage.py
  G3  the physical cache update (prefill + decode)  src/dynakv/kernels/compressed_cache.py
  G4  the cutoff gate                                src/dynakv/kernels/compressed_attention.py:84-119
on small seeded synthetic cases.  The fixtures are compressed .npz files (tens to a few hundred KB each);
the test-suite and the GPU tests read only those files, never the reference.
"""
from __future__ import annotations

import math
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def qr_basis(gen, n_heads, rank, dim):
    """Orthonormal rows: basis[h] = first `rank` rows of Q^T from a seeded QR."""
    out = []
    for _ in range(n_heads):
        m = torch.randn(dim, dim, generator=gen, dtype=torch.float64)
        qm, _ = torch.linalg.qr(m)
        out.append(qm.T[:rank].to(torch.float32))
    return torch.stack(out)


def make_case(seed, B, Hq, Hkv, D, R, S, joint, theta, len_step, zero_tail=0):
    """Synthetic cache in the reference's own API layout.

    joint=True  -> the reference-literal layout: one latent row of R
                   coefficients per token per batch row, shared by all heads.
    joint=False -> per-KV-head arenas, expressed through the same API by
                   folding the head axis into the batch axis (num_kv_heads=1).
    """
    gen = torch.Generator().manual_seed(seed)
    n_arena = B if joint else B * Hkv
    sigma = torch.exp(-torch.arange(R, dtype=torch.float32) / 32.0)
    lat_k = torch.randn(n_arena, S, R, generator=gen) * sigma
    lat_v = torch.randn(n_arena, S, R, generator=gen) * sigma
    hi = R // len_step
    len_k = (torch.randint(1, hi + 1, (n_arena, S), generator=gen) * len_step).to(torch.int32)
    len_v = (torch.randint(1, hi + 1, (n_arena, S), generator=gen) * len_step).to(torch.int32)
    if zero_tail:
        len_k[:, S - zero_tail:] = 0
        len_v[:, S - zero_tail:] = 0
    if joint:
        # one orthonormal R x R matrix U over the concatenated heads;
        # basis[h, r, dd] = U[h*D + dd, r]  (compressed_attention.py:282)
        def joint_basis():
            m = torch.randn(R, R, generator=gen, dtype=torch.float64)
            u = torch.linalg.qr(m)[0].to(torch.float32)[: Hkv * D]
            return u.view(Hkv, D, R).transpose(1, 2).contiguous()
        k_up, v_up = joint_basis(), joint_basis()
    else:
        k_up = qr_basis(gen, Hkv, R, D)
        v_up = qr_basis(gen, Hkv, R, D)
    q = torch.randn(B, Hq, D, generator=gen)
    return dict(q=q, lat_k=lat_k, lat_v=lat_v, len_k=len_k, len_v=len_v, k_up=k_up, v_up=v_up,
                theta=theta, joint=joint, B=B, Hq=Hq, Hkv=Hkv, D=D, R=R, S=S)


def reference_cache(lat, lens, rank):
    """G3: run the reference cache update (prefill) and return its state."""
    from dynakv.kernels.compressed_cache import CustomDynamicCache

    cache = CustomDynamicCache.__new__(CustomDynamicCache)  # __init__ needs transformers 4.53
    cache.key_cache_sp, cache.value_cache_sp = [], []
    cache._update_layer_cache(cache.key_cache_sp, 0, lat, lens, rank, is_decode=False)
    flat, lens_buf, offs_buf, ptr, seq, _ = cache.key_cache_sp[0]
    return cache, flat, lens_buf[:, :seq], offs_buf[:, :seq], ptr


def research_attention(case, k_norm_weight=None, eps=1e-6):
    """G1: the research model's math, built from the reference's own functions.

    Zero-masked dense latents -> einsum up-projection + head view
    (custom_attn.py:161-168) -> optional k_norm (custom_attn.py:296) ->
    apply_rotary_pos_emb_ over positions 0..S-1 (custom_attn.py:21-25,237-240)
    -> transformers eager_attention_forward.
    """
    from dynakv.custom_attn import apply_rotary_pos_emb_
    from transformers.models.llama.modeling_llama import eager_attention_forward

    B, Hq, Hkv, D, R, S = (case[k] for k in ("B", "Hq", "Hkv", "D", "R", "S"))
    ar = torch.arange(R)
    mk = (ar[None, None, :] < case["len_k"][:, :, None]).to(torch.float32)
    mv = (ar[None, None, :] < case["len_v"][:, :, None]).to(torch.float32)
    lk, lv = case["lat_k"] * mk, case["lat_v"] * mv
    if case["joint"]:
        # joint basis [Hkv*D, R]: k_up_full[kvh*D+dd, r] = k_up[kvh, r, dd]
        ku = case["k_up"].permute(0, 2, 1).reshape(Hkv * D, R)
        vu = case["v_up"].permute(0, 2, 1).reshape(Hkv * D, R)
        key_all = torch.einsum("bsd,nd->bsn", lk, ku)
        value_all = torch.einsum("bsd,nd->bsn", lv, vu)
        key = key_all.view(B, S, Hkv, D).transpose(1, 2)
        value = value_all.view(B, S, Hkv, D).transpose(1, 2)
    else:
        lk4, lv4 = lk.view(B, Hkv, S, R), lv.view(B, Hkv, S, R)
        key = torch.einsum("bhsr,hrd->bhsd", lk4, case["k_up"])
        value = torch.einsum("bhsr,hrd->bhsd", lv4, case["v_up"])
    if k_norm_weight is not None:
        from transformers.models.qwen3.modeling_qwen3 import Qwen3RMSNorm

        norm = Qwen3RMSNorm(D, eps=eps)
        with torch.no_grad():
            norm.weight.copy_(k_norm_weight)
            key = norm(key)
    inv = torch.exp(-(torch.arange(0, D // 2, dtype=torch.float32) * 2.0 / D) * math.log(case["theta"]))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)[None]
    key = apply_rotary_pos_emb_(key, emb.cos(), emb.sin())
    mod = types.SimpleNamespace(num_key_value_groups=Hq // Hkv, training=False)
    q4 = case["q"].view(B, Hq, 1, D)
    mask = None
    if (case["len_k"] == 0).any():
        # zero-length (padding) tokens are excluded, as the kernels do (fused.py:105-106)
        dead = (case["len_k"] == 0)
        dead = dead.view(B, 1, S) if case["joint"] else dead.view(B, Hkv, S).repeat_interleave(Hq // Hkv, 1)
        mask = torch.zeros(B, Hq, 1, S).masked_fill(dead[:, :, None, :].expand(B, Hq, 1, S), float("-inf"))
    out, _ = eager_attention_forward(mod, q4, key, value, mask, scaling=D ** -0.5)
    return out.reshape(B, Hq, D)


def triton_kernels(case, flat_k, flat_v, lens_k, lens_v, offs_k, offs_v):
    """G2: the reference Triton kernels under the interpreter."""
    from dynakv.kernels import fused, two_stage

    B, Hq, Hkv, D, R, S = (case[k] for k in ("B", "Hq", "Hkv", "D", "R", "S"))
    q = case["q"]
    if case["joint"]:
        calls = [(q, case["k_up"], case["v_up"], slice(0, B))]
    else:
        G = Hq // Hkv
        calls = []
        for h in range(Hkv):
            rows = torch.arange(B) * Hkv + h
            calls.append((q[:, h * G:(h + 1) * G].contiguous(), case["k_up"][h:h + 1], case["v_up"][h:h + 1], rows))
    outs_f, outs_s, outs_a = [], [], []
    for qh, ku, vu, rows in calls:
        fk, fv = flat_k[rows].contiguous(), flat_v[rows].contiguous()
        lk, lv, ok, ov = lens_k[rows], lens_v[rows], offs_k[rows], offs_v[rows]
        nh = qh.shape[1]
        ku_h = ku.repeat_interleave(nh // ku.shape[0], 0).contiguous()
        vu_h = vu.repeat_interleave(nh // vu.shape[0], 0).contiguous()
        outs_f.append(fused.fused_attention_dispatch(qh.unsqueeze(2), fk, ku_h, fv, vu_h, lk, ok, lv, ov, case["theta"]))
        # the autotuner wants a GPU driver: call the jit functions beneath it
        sc = torch.empty(qh.shape[0], nh, S)
        grid = (qh.shape[0], nh, (S + 15) // 16)
        two_stage._abx_sparse_fwd.fn[grid](
            qh, ku, fk, sc, qh.stride(0), qh.stride(1), qh.stride(2), ku.stride(0), ku.stride(1), ku.stride(2),
            sc.stride(0), sc.stride(1), sc.stride(2), fk.stride(0), lk, lk.stride(0), lk.stride(1),
            ok, ok.stride(0), ok.stride(1), R, D, S, D, R, BLOCK_SIZE_D=64, BLOCK_SIZE_R=64, BLOCK_SIZE_L=16,
            HEADS_PER_GROUP=nh // ku.shape[0], THETA=case["theta"])
        outs_s.append(sc)
        av = torch.empty(qh.shape[0], nh, D)
        two_stage._avx_proj_fwd.fn[(qh.shape[0], nh)](
            sc, fv, av, vu, None, sc.stride(0), sc.stride(1), sc.stride(2), av.stride(0), av.stride(1),
            fv.stride(0), vu.stride(0), vu.stride(1), vu.stride(2), 0, 0, lv, lv.stride(0), lv.stride(1),
            ov, ov.stride(0), ov.stride(1), S, RANK_TOTAL=R, HEAD_DIM=D, HIDDEN_SIZE=0,
            GROUP_SIZE=nh // vu.shape[0], BLOCK_SIZE_R=1 << (R - 1).bit_length(), BLOCK_SIZE_S=16)
        outs_a.append(av)
    cat = (lambda xs: xs[0]) if case["joint"] else (lambda xs: torch.cat(xs, dim=1))
    return cat(outs_f), cat(outs_s), cat(outs_a)


def attention_fixture(name, **kw):
    knorm = kw.pop("knorm", False)
    case = make_case(**kw)
    R = case["R"]
    _, flat_k, lens_k, offs_k, ptr_k = reference_cache(case["lat_k"], case["len_k"], R)
    _, flat_v, lens_v, offs_v, ptr_v = reference_cache(case["lat_v"], case["len_v"], R)
    out = dict(
        q=case["q"], k_up=case["k_up"], v_up=case["v_up"],
        flat_k=flat_k, flat_v=flat_v, lens_k=lens_k, lens_v=lens_v, offs_k=offs_k, offs_v=offs_v,
        ptr_k=ptr_k, ptr_v=ptr_v, theta=np.float64(case["theta"]), joint=np.int32(case["joint"]),
        dims=np.array([case[k] for k in ("B", "Hq", "Hkv", "D", "R", "S")], dtype=np.int32),
    )
    if knorm:
        gen = torch.Generator().manual_seed(kw["seed"] + 1)
        w = 1.0 + 0.02 * torch.randn(case["D"], generator=gen)
        out["k_norm_weight"] = w
        out["research_out"] = research_attention(case, k_norm_weight=w)
    else:
        out["research_out"] = research_attention(case)
        f, s, a = triton_kernels(case, flat_k, flat_v, lens_k, lens_v, offs_k, offs_v)
        out.update(triton_fused=f, triton_scores=s, triton_avx=a)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k: (v.detach().numpy() if isinstance(v, torch.Tensor) else v) for k, v in out.items()})
    msg = ""
    if not knorm:
        msg = " fused-vs-research max|d|=%.2e" % float((out["triton_fused"] - out["research_out"]).abs().max())
    print("wrote", name, msg)


def cache_fixture(name, seed, n_rows, R, s_prefill, n_decode, len_step):
    """G3: prefill then n_decode single-token appends through the reference cache."""
    from dynakv.kernels.compressed_cache import CustomDynamicCache

    gen = torch.Generator().manual_seed(seed)
    cache = CustomDynamicCache.__new__(CustomDynamicCache)
    cache.key_cache_sp, cache.value_cache_sp = [], []
    hi = R // len_step
    pre = torch.randn(n_rows, s_prefill, R, generator=gen)
    pre_len = (torch.randint(1, hi + 1, (n_rows, s_prefill), generator=gen) * len_step).to(torch.int32)
    cache._update_layer_cache(cache.key_cache_sp, 0, pre, pre_len, R, is_decode=False)
    steps, step_lens = [], []
    for _ in range(n_decode):
        st = torch.randn(n_rows, 1, R, generator=gen)
        ln = (torch.randint(1, hi + 1, (n_rows, 1), generator=gen) * len_step).to(torch.int32)
        cache._update_layer_cache(cache.key_cache_sp, 0, st.contiguous(), ln.contiguous(), R, is_decode=True)
        steps.append(st)
        step_lens.append(ln)
    flat, lens_buf, offs_buf, ptr, seq, _ = cache.key_cache_sp[0]
    from dynakv.kernels.compressed_cache import simple_decompress
    dense = simple_decompress(flat, lens_buf[:, :seq], R)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        prefill=pre.numpy(), prefill_len=pre_len.numpy(),
        steps=torch.cat(steps, 1).numpy() if steps else np.zeros((n_rows, 0, R), np.float32),
        step_lens=torch.cat(step_lens, 1).numpy() if steps else np.zeros((n_rows, 0), np.int32),
        flat=flat.numpy(), lens=lens_buf[:, :seq].numpy(), offs=offs_buf[:, :seq].numpy(),
        ptr=ptr.numpy(), seq=np.int32(seq), dense=dense.numpy(), R=np.int32(R))
    print("wrote", name, "seq", seq, "ptr", ptr.tolist())


def gate_fixture(name, seed, n_rows, d):
    """G4: kv_process_fused called unbound with a stand-in self."""
    from dynakv.kernels.compressed_attention import KVProcessor

    gen = torch.Generator().manual_seed(seed)
    me = types.SimpleNamespace(
        Wk=torch.randn(d, d, generator=gen) * 0.3, bk=torch.randn(1, d, generator=gen),
        Wv=torch.randn(d, d, generator=gen) * 0.3, bv=torch.randn(1, d, generator=gen), low_rank=d)
    k = torch.randn(n_rows, 1, d, generator=gen)
    v = torch.randn(n_rows, 1, d, generator=gen)
    k_out, v_out, len_k, len_v, _, _ = KVProcessor.kv_process_fused(me, k, v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), Wk=me.Wk.numpy(), bk=me.bk.numpy(), Wv=me.Wv.numpy(),
                        bv=me.bv.numpy(), k=k.numpy(), v=v.numpy(), k_out=k_out.numpy(), v_out=v_out.numpy(),
                        len_k=len_k.numpy(), len_v=len_v.numpy())
    print("wrote", name, "len_k", len_k.flatten().tolist()[:8])


def gate_inputs(seed, n_rows, d, dtype):
    """Seeded inputs of the large gate fixtures (the weights are too big to store): K/V coefficient rows with the
    decaying spectrum of the synthetic caches, gate weights and biases.  Returns (k, v, Wk, bk, Wv, bv) in ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    sigma = torch.exp(-torch.arange(d, dtype=torch.float32) / (d / 4.0))
    k = torch.randn(n_rows, 1, d, generator=gen) * sigma * 2.0
    v = torch.randn(n_rows, 1, d, generator=gen) * sigma * 2.0
    Wk = torch.randn(d, d, generator=gen) * (2.0 / d ** 0.5)
    Wv = torch.randn(d, d, generator=gen) * (2.0 / d ** 0.5)
    bk = torch.randn(1, d, generator=gen) + torch.linspace(2.0, -2.0, d)
    bv = torch.randn(1, d, generator=gen) + torch.linspace(2.0, -2.0, d)
    return tuple(t.to(dtype) for t in (k, v, Wk, bk, Wv, bv))


def gate_seeded_fixture(name, seed, n_rows, d, dtype):
    """G4 at model width: the reference's kv_process_fused in ``dtype`` on the seeded inputs; only the lengths and
    a checksum of the inputs are stored."""
    from dynakv.kernels.compressed_attention import KVProcessor
    k, v, Wk, bk, Wv, bv = gate_inputs(seed, n_rows, d, dtype)
    me = types.SimpleNamespace(Wk=Wk, bk=bk, Wv=Wv, bv=bv, low_rank=d)
    _, _, len_k, len_v, _, _ = KVProcessor.kv_process_fused(me, k, v)
    chk = np.array([float(t.double().sum()) for t in (k, v, Wk, bk, Wv, bv)])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), len_k=len_k.numpy().reshape(-1), len_v=len_v.numpy().reshape(-1),
                        checksum=chk, seed=np.int64(seed), n_rows=np.int64(n_rows), d=np.int64(d),
                        dtype=np.array(str(dtype).replace("torch.", "")))
    print("wrote", name, "mean len_k %.1f" % float(len_k.float().mean()), "min", int(len_k.min()), "max", int(len_k.max()))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "src"))
    torch.manual_seed(0)
    # per-KV-head layout, lengths multiples of 8 (the measured configurations' form)
    attention_fixture("attn_perhead_s45", seed=11, B=2, Hq=8, Hkv=2, D=128, R=128, S=45,
                      joint=False, theta=500000.0, len_step=8)
    attention_fixture("attn_perhead_s130_pad", seed=12, B=1, Hq=8, Hkv=2, D=128, R=128, S=130,
                      joint=False, theta=500000.0, len_step=8, zero_tail=7)
    # reference-literal joint layout: one 256-wide latent row shared by 2 KV heads, any integer length
    attention_fixture("attn_joint_s37", seed=13, B=2, Hq=4, Hkv=2, D=128, R=256, S=37,
                      joint=True, theta=10000.0, len_step=1)
    # Qwen3 form: RMSNorm on reconstructed K before RoPE (research math only; no physical Qwen3 path exists)
    attention_fixture("attn_qwen_knorm_s50", seed=14, B=2, Hq=8, Hkv=2, D=128, R=128, S=50,
                      joint=False, theta=1000000.0, len_step=8, knorm=True)
    cache_fixture("cache_prefill_decode", seed=21, n_rows=3, R=128, s_prefill=9, n_decode=6, len_step=8)
    cache_fixture("cache_anylen", seed=22, n_rows=2, R=96, s_prefill=5, n_decode=4, len_step=1)
    gate_fixture("gate_d64", seed=31, n_rows=6, d=64)
    for dt, nm in ((torch.float32, "f32"), (torch.bfloat16, "bf16"), (torch.float16, "f16")):
        gate_seeded_fixture("gate_d1024_" + nm, seed=41, n_rows=256, d=1024, dtype=dt)


if __name__ == "__main__":
    main()
