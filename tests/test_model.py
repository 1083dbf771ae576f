"""Llama-shaped decoder: tensor-parallel equivalence on CPU (gloo, dense cache) and, on the GPU,
generation across the compression boundary."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

TINY = dict(hidden=256, layers=2, heads=8, kv_heads=2, ffn=512, vocab=320)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from reskv_b200.models import LlamaShape, ResKVLlama

        torch.manual_seed(0)
        ids = torch.randint(0, 320, (2, 12))
        model = ResKVLlama(LlamaShape(**TINY), cache="dense", device="cpu", seed=3, group=dist.group.WORLD)
        logits = [model.prefill(ids, reserve=3)]
        for _ in range(3):
            logits.append(model.decode(logits[-1].argmax(-1)))
        if rank == 0:
            results.put(torch.stack(logits))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_matches_single_rank_on_cpu():
    from reskv_b200.models import LlamaShape, ResKVLlama

    torch.manual_seed(0)
    ids = torch.randint(0, 320, (2, 12))
    single = ResKVLlama(LlamaShape(**TINY), cache="dense", device="cpu", seed=3)
    want = [single.prefill(ids, reserve=3)]
    for _ in range(3):
        want.append(single.decode(want[-1].argmax(-1)))
    want = torch.stack(want)
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = results.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # same weights, FP16 partial sums reduced in a different order
    torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_rejects_bad_arguments():
    from reskv_b200 import ResKVConfig
    from reskv_b200.models import LlamaShape, ResKVLlama

    with pytest.raises(TypeError, match="expected ResKVKernelConfig"):
        ResKVLlama(LlamaShape(**TINY), ResKVConfig(), device="cpu")
    with pytest.raises(ValueError, match="cache must be"):
        ResKVLlama(LlamaShape(**TINY), cache="paged", device="cpu")


@pytest.mark.gpu
def test_generation_across_the_compression_boundary():
    from reskv_b200 import ResKVKernelConfig
    from reskv_b200.models import LlamaShape, ResKVLlama

    cfg = ResKVKernelConfig(sparsity=0.5, layout="unstructured", num_clusters=4, max_clusters=8, group_size=16,
                            recent_size=8, kmeans_iterations=3)
    shape = LlamaShape(**TINY)
    ids = torch.randint(0, 320, (2, 70), generator=torch.Generator().manual_seed(1)).cuda()
    model = ResKVLlama(shape, cfg, cache="reskv", seed=5)
    dense = ResKVLlama(shape, cfg, cache="dense", seed=5)
    # prefill attends to dense K/V in both variants: identical logits
    a, b = model.prefill(ids, reserve=40), dense.prefill(ids, reserve=40)
    assert torch.equal(a, b)
    tok = a.argmax(-1)
    for step in range(40):
        la, lb = model.decode(tok), dense.decode(tok)
        assert torch.isfinite(la).all()
        # lossy cache: logits stay close to the dense model's
        rel = (la - lb).norm() / lb.norm()
        assert rel < 0.5, rel
        tok = lb.argmax(-1)
    layer = model.caches[0]
    assert layer.length == 110 and layer.compressed.seq_len + layer.live == 110
    assert layer.compressed.seq_len == 48 + 48 and layer.compressed.key.centroids.shape[2] == 7
    out = ResKVLlama(shape, cfg, cache="reskv", seed=5).generate(ids, 20)
    assert out.shape == (2, 20)
    assert model.cache_bytes() > 0


@pytest.mark.gpu
def test_graph_decode_matches_eager_decode():
    """Replaying the captured step (device-side position, window length and compressed-token
    count) gives the eager step's logits, across group compressions, with a single capture."""
    from reskv_b200 import ResKVKernelConfig
    from reskv_b200.models import LlamaShape, ResKVLlama

    cfg = ResKVKernelConfig(sparsity=0.75, layout="unstructured", num_clusters=4, max_clusters=8, group_size=16,
                            recent_size=8, kmeans_iterations=3)
    shape = LlamaShape(**TINY)
    ids = torch.randint(0, 320, (2, 70), generator=torch.Generator().manual_seed(1)).cuda()
    eager = ResKVLlama(shape, cfg, seed=5)
    graph = ResKVLlama(shape, cfg, seed=5)
    tok = eager.prefill(ids, reserve=64).argmax(-1)
    assert torch.equal(tok, graph.prefill(ids, reserve=64).argmax(-1))
    graph.begin_graph_decode(2)
    for step in range(40):
        le = eager.decode(tok)
        lg = graph.decode_graph(tok).clone()
        torch.testing.assert_close(lg, le, atol=2e-2, rtol=2e-2)
        tok = le.argmax(-1)
        if step == 0:
            captured = graph._graph
    assert graph._graph is captured, "the step was captured again"
    assert graph.caches[0].compressed.seq_len == eager.caches[0].compressed.seq_len
    assert graph.caches[0].live == eager.caches[0].live and graph.length == eager.length
