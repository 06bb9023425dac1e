"""World-size-2 checks of the multi-process host logic, on CPU with the gloo backend."""
import os
import socket
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bench._barrier_fn(world)()
        # the slowest rank defines the step time
        slowest = bench._max_over_ranks(0.010 * (rank + 1), world)
        results[rank] = slowest
    finally:
        dist.destroy_process_group()


def test_step_time_is_the_maximum_over_ranks():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert results[0] == pytest.approx(0.020) and results[1] == pytest.approx(0.020)


def test_single_rank_helpers_need_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    bench._barrier_fn(1)()
    assert bench._max_over_ranks(1.5, 1) == 1.5


# ---- tensor-parallel host logic ----

def _small_config():
    import dataclasses
    from nerva_b200 import synth
    return dataclasses.replace(synth.TINY_QWEN3, layers=1, vocab=512, name="tiny-1-layer")


def test_shards_partition_the_model_and_partial_sums_add_up(oracle_mod):
    import numpy as np
    from nerva_b200 import synth
    cfg = _small_config()
    full = synth.dense_checkpoint(cfg)
    world = 2
    shards = [synth.shard_checkpoint(full, r, world) for r in range(world)]
    h, ah, inter = cfg.hidden, cfg.attention_hidden, cfg.intermediate
    layer = full.layers[0]
    # row-split tensors concatenate back; column-split tensors interleave back
    for name in ("w_q", "w_k", "w_v", "w_gate", "w_up"):
        assert np.array_equal(np.concatenate([s.layers[0][name] for s in shards]), layer[name])
    assert np.array_equal(np.concatenate([s.lm_head for s in shards]), full.lm_head)
    for name, cols in (("w_o", ah), ("w_down", inter)):
        parts = [s.layers[0][name].reshape(h, cols // world) for s in shards]
        assert np.array_equal(np.concatenate(parts, axis=1).reshape(-1), layer[name])
    assert [s.shard.vocab_offset for s in shards] == [0, cfg.vocab // 2]
    assert all(s.embeddings is full.embeddings for s in shards)  # the embedding table stays whole
    # a row-parallel projection is the sum of the ranks' partial projections
    x = synth.normal_f32(0, 99, inter, 1.0)
    whole = oracle_mod.matvec(layer["w_down"], x, h, inter)
    part = sum(oracle_mod.matvec(shards[r].layers[0]["w_down"], x[r * inter // 2:(r + 1) * inter // 2], h, inter // 2)
               for r in range(world))
    assert np.abs(whole - part).max() < 1e-5
    with pytest.raises(ValueError):
        synth.shard_config(cfg, 3)  # 8 heads / 2 KV heads do not split three ways


def test_directly_generated_shard_equals_the_cut_of_the_full_model():
    import numpy as np
    from nerva_b200 import synth
    cfg = _small_config()
    full = synth.dense_checkpoint(cfg)
    for rank in range(2):
        cut = synth.shard_checkpoint(full, rank, 2)
        direct = synth.dense_checkpoint_shard(cfg, rank, 2)
        assert np.array_equal(cut.lm_head, direct.lm_head)
        for name, value in cut.layers[0].items():
            assert np.array_equal(value, direct.layers[0][name]), name
        assert direct.config.heads == 4 and direct.config.kv_heads == 1 and direct.config.intermediate == 768


class _FakeSession:
    def __init__(self, rank):
        self.rank, self.attached = rank, None

    def comm_handle(self):
        return bytes([self.rank]) * 64

    def attach_peers(self, handles):
        self.attached = handles


def _connect_main(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from nerva_b200 import tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fake = _FakeSession(rank)
        tp.connect(fake)
        results[rank] = fake.attached
    finally:
        dist.destroy_process_group()


def test_handles_reach_every_rank_in_rank_order():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_connect_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    expected = [bytes([0]) * 64, bytes([1]) * 64]
    assert results[0] == expected and results[1] == expected
