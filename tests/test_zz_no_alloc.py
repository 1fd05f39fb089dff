"""The allocation-free long-cache entry point, called through the C ABI.

Some users of the library cannot allocate device memory when they call it: a serving process that has
pre-assigned all of HBM to its own pool, or a host that forbids cudaMalloc once start-up is over.  For them
``dkv_two_stage_decode_noalloc`` keeps the split path's scratch in an array built into the library.  This
test checks that it returns exactly what the ordinary entry point returns, on two calls in a row that share
the built-in array (the second with other inputs, so nothing left behind by the first can leak into it),
and that a call too large for the array is refused with a clear error instead of being run.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

from dynakv_b200 import synthetic
from dynakv_b200.kernels import _common
from dynakv_b200.kernels.two_stage import two_stage_attention, two_stage_attention_noalloc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(case):
    fk, fv, lk, lv, ok, ov = case.views()
    return case.q, fk, case.k_up, fv, case.v_up, lk, ok, lv, ov, case.theta


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    cases = [synthetic.make_layer_case(901, [1500, 700, 2100], "beta:2,8", 500000.0, torch.bfloat16, DEV),
             synthetic.make_layer_case(902, [640, 3000], "beta:2,5", 500000.0, torch.bfloat16, DEV)]
    for case in cases:                      # two calls in a row on the shared built-in scratch
        sl = torch.tensor(case.seq_lens, dtype=torch.int32, device=DEV)
        want = two_stage_attention(*_args(case), seq_lens=sl, len_multiple=8)
        out = torch.empty_like(want)
        got = two_stage_attention_noalloc(*_args(case), out=out, seq_lens=sl, len_multiple=8)
        torch.cuda.synchronize()
        assert got.data_ptr() == out.data_ptr()
        # same kernels, same order of operations: identical bits, which is within every tolerance used here
        assert torch.equal(got, want)
        assert torch.isfinite(got.float()).all()
    assert _common.read_status(torch.device(DEV)) == 0


def test_noalloc_entry_point_refuses_oversized_and_unqualified_calls():
    # 300 one-token rows need more partial records than the 2 MiB array holds
    big = synthetic.make_layer_case(903, [1] * 300, "uniform", 10000.0, torch.bfloat16, DEV)
    out = torch.empty((300, 32, 128), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="built-in array holds"):
        two_stage_attention_noalloc(*_args(big), out=out, len_multiple=8)
    # a cache whose lengths are not declared multiples of 8 never uses scratch: refused, not silently rerouted
    small = synthetic.make_layer_case(904, [600], "uniform", 10000.0, torch.bfloat16, DEV)
    out = torch.empty((1, 32, 128), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="only the split tensor-core path"):
        two_stage_attention_noalloc(*_args(small), out=out, len_multiple=1)
