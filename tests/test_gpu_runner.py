"""The minimal Llama-shaped decode loop on the compressed cache: the attention of every generated token against the
CPU oracle on the cache's own contents, the cache layout, and the CUDA-graph replay against the eager step."""
import numpy as np
import pytest
import torch

from dynakv_b200.kernels import _common
from dynakv_b200.runner import MiniLlama, ModelShape
from oracle import dynakv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TINY = ModelShape(layers=2, hidden=512, mlp=1024, vocab=1000, n_q_heads=8, n_kv_heads=2, theta=10000.0)


def _oracle_attention(model, li, q, n_tokens):
    """Oracle attention of layer ``li`` over the first ``n_tokens`` cached tokens of every row."""
    ck, cv = model.cache.key_cache_sp[li], model.cache.value_cache_sp[li]
    w = model.layers[li]
    B = q.shape[0]
    lk, ok = ck[1][:, :n_tokens].cpu(), ck[2][:, :n_tokens].cpu()
    lv, ov = cv[1][:, :n_tokens].cpu(), cv[2][:, :n_tokens].cpu()
    return O.compact_attention(q.cpu(), ck[0].cpu(), w.k_up.cpu(), cv[0].cpu(), w.v_up.cpu(), lk, ok, lv, ov,
                               model.shape.theta, seq_lens=[n_tokens] * B)


def test_generated_tokens_attend_like_the_oracle_and_the_graph_replays_the_eager_step():
    P, NEW = 520, 4            # past the switch point: the long-cache kernels run
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, TINY.vocab, (3, P), generator=gen).to(DEV)
    model = MiniLlama(TINY, DEV, seed=5, trace=True)
    nxt = model.prefill(ids, NEW + 4)
    # layout after the prompt: lengths from the cutoff head, offsets their running sums, write pointer their total
    for li in range(TINY.layers):
        ck = model.cache.key_cache_sp[li]
        lens = ck[1][:, :P].cpu().numpy().astype(np.int64)
        assert lens.min() >= 8 and lens.max() <= 128 and (lens % 8 == 0).all()
        assert np.array_equal(ck[2][:, :P].cpu().numpy(), np.cumsum(lens, axis=1) - lens)
        assert np.array_equal(ck[3].cpu().numpy(), lens.sum(axis=1))
    logits = []
    for step in range(NEW):
        model.trace.clear()
        nxt = model.decode_step(nxt.clone())
        logits.append(model.logits.float().cpu())
        for li, q, out in model.trace:
            want = _oracle_attention(model, li, q, P + step + 1)
            err = (out.float().cpu() - want).abs()
            assert float(err.max()) <= 2e-2 and float(err.mean() / want.abs().mean()) <= 1e-2, (step, li)
    assert _common.read_status(torch.device(DEV)) == 0
    assert model.cache.seq_lens(0).tolist() == [P + NEW] * 3

    # the same prompt through the graph path: the same logits as the eager steps
    replay = MiniLlama(TINY, DEV, seed=5)
    nxt = replay.prefill(ids, NEW + 4)
    for step in range(NEW):
        nxt = replay.decode_step(nxt.clone(), use_graph=True)
        assert torch.allclose(replay.logits.float().cpu(), logits[step], atol=2e-3, rtol=0), step
    assert replay.cache.seq_lens(1).tolist() == [P + NEW] * 3
    assert _common.read_status(torch.device(DEV)) == 0


def _tp_worker(rank, world, port, ids, new_tokens, out_path, use_graph):
    import os

    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    model = MiniLlama(TINY, dev, seed=5, tp_rank=rank, tp_size=world)
    nxt = model.prefill(ids.to(dev), new_tokens + 4)
    logits = []
    for _ in range(new_tokens):
        nxt = model.decode_step(nxt.clone(), use_graph=use_graph)
        logits.append(model.logits.float().cpu())
    if rank == 0:
        torch.save(torch.stack(logits), out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("use_graph", [False, True], ids=["eager", "graph-per-piece"])
def test_two_ranks_sharded_by_kv_head_give_the_logits_of_one_rank(tmp_path, use_graph):
    """Tensor parallel by KV head on 2 GPUs (this package's kernels on each rank's heads, NCCL all-reduce after the
    row-parallel output and down projections) against the same model on one GPU; eagerly, and replayed from one
    CUDA graph per piece between all-reduces."""
    import torch.multiprocessing as mp
    P, NEW = 520, 3
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, TINY.vocab, (2, P), generator=gen)
    out_path = str(tmp_path / "tp_logits.pt")
    mp.spawn(_tp_worker, args=(2, 29533 + int(use_graph), ids, NEW, out_path, use_graph), nprocs=2, join=True)
    got = torch.load(out_path)
    model = MiniLlama(TINY, DEV, seed=5)
    nxt = model.prefill(ids.to(DEV), NEW + 4)
    for step in range(NEW):
        nxt = model.decode_step(nxt.clone())
        want = model.logits.float().cpu()
        # bf16 partial sums are added in a different order: a few units of bf16 rounding on logits of size ~0.3
        assert float((got[step] - want).abs().max()) <= 2e-2 * float(want.abs().max()) + 1e-3, step
