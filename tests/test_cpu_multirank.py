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


# ---- expert-parallel host logic ----

def _sparse_config():
    import dataclasses
    from nerva_b200 import synth
    return dataclasses.replace(synth.DEEPSEEK_V2_LITE, name="v2-lite-small", layers=3, vocab=512, prompt_tokens=8,
                               decode_tokens=4, hidden=256, heads=4, kv_heads=4, head_dim=32, intermediate=512,
                               num_experts=8, top_k=3, moe_intermediate=64, shared_intermediate=128,
                               kv_lora_rank=128, qk_nope_head_dim=32, qk_rope_head_dim=16)


def _f32(bits):
    import numpy as np
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _expert_mlp(x, gate, up, down):
    """down . (silu(gate . x) * (up . x)) in float64 from bf16 matrices."""
    import numpy as np
    g = _f32(gate).astype(np.float64) @ x
    u = _f32(up).astype(np.float64) @ x
    return _f32(down).astype(np.float64) @ (g / (1.0 + np.exp(-g)) * u)


def _partial_sparse_mlp(entry, cfg, x, ids, weights, expert_base, expert_local, shared_intermediate):
    """What one rank adds to the MLP output: the chosen experts it holds (the kernel's rule: id -
    expert_base below expert_local, matrices indexed by that difference) and its slice of the shared expert."""
    import numpy as np
    h, mi = cfg.hidden, cfg.moe_intermediate
    gate_up = entry["w_expert_gate_up"].reshape(-1, 2, mi, h)
    down = entry["w_expert_down"].reshape(-1, h, mi)
    out = np.zeros(h)
    for e, w in zip(ids, weights):
        local = int(e) - expert_base
        if 0 <= local < expert_local:
            out += float(w) * _expert_mlp(x, gate_up[local, 0], gate_up[local, 1], down[local])
    si = shared_intermediate
    out += _expert_mlp(x, entry["w_shared_expert_gate"].reshape(si, h), entry["w_shared_expert_up"].reshape(si, h),
                       entry["w_shared_expert_down"].reshape(h, si))
    return out


def _expert_rank_main(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, ROOT)
    import numpy as np
    import torch
    import torch.distributed as dist
    from nerva_b200 import synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = _sparse_config()
        shard = synth.expert_checkpoint_shard(cfg, rank, world)  # generated directly: no full model on this rank
        local_e = cfg.num_experts // world
        x = synth.normal_f32(0, 77, cfg.hidden, 1.0).astype(np.float64)
        ids, weights = [6, 1, 3], [0.5, 0.3, 0.2]
        part = _partial_sparse_mlp(shard.layers[1], cfg, x, ids, weights, rank * local_e, local_e,
                                   shard.config.shared_intermediate)
        total = torch.from_numpy(part.copy())
        dist.all_reduce(total)  # the sum the gather prologue forms from the ranks' partial outputs
        results[rank] = total.numpy()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_partial_outputs_add_up_to_the_whole_mlp():
    import numpy as np
    import torch.multiprocessing as mp
    from nerva_b200 import synth
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_expert_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    cfg = _sparse_config()
    full = synth.dense_checkpoint(cfg)
    x = synth.normal_f32(0, 77, cfg.hidden, 1.0).astype(np.float64)
    whole = _partial_sparse_mlp(full.layers[1], cfg, x, [6, 1, 3], [0.5, 0.3, 0.2], 0, cfg.num_experts,
                                cfg.shared_intermediate)
    assert np.abs(results[0] - whole).max() < 1e-9 * max(1.0, np.abs(whole).max()) + 1e-12
    assert np.array_equal(results[0], results[1])


def test_expert_shards_partition_the_experts_and_keep_everything_else_whole():
    import numpy as np
    from nerva_b200 import synth
    cfg = _sparse_config()
    full = synth.dense_checkpoint(cfg)
    for world in (2, 4):
        shards = [synth.expert_shard_checkpoint(full, r, world) for r in range(world)]
        for r, s in enumerate(shards):
            direct = synth.expert_checkpoint_shard(cfg, r, world)
            assert s.shard.mode == 1 and s.shard.vocab_offset == 0 and s.config.num_experts == cfg.num_experts
            assert s.config.shared_intermediate == cfg.shared_intermediate // world
            assert s.lm_head is full.lm_head and s.layers[0] is full.layers[0]  # dense parts are shared, not copied
            for a, b in zip(s.layers, direct.layers):
                assert set(a) == set(b)
                assert all(np.array_equal(a[k], b[k]) for k in a)
        sparse = full.layers[1]
        for name in ("w_expert_gate_up", "w_expert_down", "w_shared_expert_gate", "w_shared_expert_up"):
            assert np.array_equal(np.concatenate([s.layers[1][name] for s in shards]), sparse[name])
        si, h = cfg.shared_intermediate, cfg.hidden
        parts = [s.layers[1]["w_shared_expert_down"].reshape(h, si // world) for s in shards]
        assert np.array_equal(np.concatenate(parts, axis=1).reshape(-1), sparse["w_shared_expert_down"])
    with pytest.raises(ValueError):
        synth.expert_shard_config(cfg, 3)
    import dataclasses
    with pytest.raises(ValueError):  # an odd number of sparse layers: the exchange buffers would not alternate
        synth.expert_shard_config(dataclasses.replace(cfg, layers=4), 2)


def test_extra_clock_steps_are_a_function_of_the_agreed_time_only():
    """The untimed steps that keep the load up for the clock sampler are computed from the slowest
    rank's time, which every rank holds after the max over ranks: equal inputs, equal step counts
    (ranks that stepped a different number of times would leave each other waiting in an exchange)."""
    sys.path.insert(0, ROOT)
    import bench
    assert bench.extra_clock_steps(0.5, 128) == 0            # the timed and the end-to-end region cover 0.35 s
    assert bench.extra_clock_steps(0.104, 64) == int((0.35 - 0.208) / (0.104 / 64)) + 1
    assert bench.extra_clock_steps(1e-4, 4) == bench.MAX_EXTRA_CLOCK_STEPS
    assert bench.extra_clock_steps(0.0, 8) == 0 and bench.extra_clock_steps(0.1, 0) == 0
