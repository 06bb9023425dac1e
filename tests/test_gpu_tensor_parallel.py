"""Tensor parallel over 2 GPUs: one process per GPU, the tiny Qwen3-architecture model cut in two,
tokens and logits against the CPU oracle of the whole model.  Skipped on a single-GPU machine."""
import ctypes
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
LOGIT_ATOL = 2e-2  # the stated end-to-end bound, met on this configuration


def _gpu_count() -> int:
    try:
        cudart = ctypes.CDLL("libcudart.so")
    except OSError:
        try:
            cudart = ctypes.CDLL("/usr/local/cuda/lib64/libcudart.so")
        except OSError:
            return 0
    count = ctypes.c_int(0)
    return count.value if cudart.cudaGetDeviceCount(ctypes.byref(count)) == 0 else 0


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _wide_config():
    """Qwen3-8B layer shapes (32 query / 8 KV heads of 128, hidden 4096, intermediate 12288) cut to two
    layers and a small vocabulary, so that it splits 2, 4 and 8 ways and the oracle stays quick."""
    import dataclasses
    from nerva_b200 import synth
    return dataclasses.replace(synth.QWEN3_8B, name="qwen3-8b-shape-2-layers", layers=2, vocab=8192,
                               prompt_tokens=24, decode_tokens=8)


def _config(kind: str):
    from nerva_b200 import synth
    return synth.TINY_QWEN3 if kind == "tiny" else _wide_config()


def _rank_main(rank: int, world: int, port: int, steps: int, kind: str, results) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from nerva_b200 import ops, synth, tp
    from nerva_b200.session import CudaHfDecodeSequenceLoop, SmokeStatus
    tp.select_device(rank)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=180))
    try:
        cfg = _config(kind)
        full = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
        session = tp.create_session(cfg, cfg.prompt_tokens + steps + 1, rank, world, full_checkpoint=full)
        # the directly generated shard has the same bits as the slice of the full model
        direct = synth.dense_checkpoint_shard(cfg, rank, world, block_fill=ops.synth_normal_bf16_block,
                                              fill=ops.synth_normal_bf16)
        cut = synth.shard_checkpoint(full, rank, world)
        same = np.array_equal(direct.lm_head, cut.lm_head) and all(
            np.array_equal(a[k], b[k]) for a, b in zip(direct.layers, cut.layers) for k in a)
        start, loop = CudaHfDecodeSequenceLoop.start(session, synth.prompt_ids(cfg))
        assert start.status == SmokeStatus.OK, start.error
        tokens, logits = [], []
        for _ in range(steps):
            out = loop.advance(1)
            assert out.status == SmokeStatus.OK, out.error
            tokens += out.tokens
            logits.append(session.read_logits())  # this rank's rows of the vocabulary
        dist.barrier()
        session.destroy()
        results[rank] = {"tokens": tokens, "logits": np.stack(logits), "offset": session.shard.vocab_offset,
                         "shards_equal": bool(same)}
    finally:
        dist.destroy_process_group()


def _run_ranks(world: int, steps: int, kind: str):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, steps, kind, results)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(600)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
    return [results[r] for r in range(world)]


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_rank_tensor_parallel_matches_oracle(built_lib, oracle_mod, tiny_golden):
    from nerva_b200 import synth
    world, steps = 2, 32
    r0, r1 = _run_ranks(world, steps, "tiny")
    assert r0["shards_equal"] and r1["shards_equal"]
    # every rank writes the same token stream, and it is the oracle's
    assert r0["tokens"] == r1["tokens"]
    assert r0["tokens"] == tiny_golden["cuda"]["tokens"]
    # the vocabulary shards, put side by side, are the oracle's logits within the stated bound
    cfg = synth.TINY_QWEN3
    ck = synth.dense_checkpoint(cfg)
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + steps + 1, mode=oracle_mod.MODE_CUDA)
    _, ref = dec.decode_greedy(synth.prompt_ids(cfg), steps, want_logits=True)
    got = np.concatenate([r0["logits"], r1["logits"]], axis=1)
    assert r0["offset"] == 0 and r1["offset"] == cfg.vocab // 2
    assert got.shape == ref.shape
    assert float(np.abs(got - ref).max()) <= LOGIT_ATOL


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_on_qwen3_8b_layer_shapes(built_lib, oracle_mod, world):
    """Every rank count the head counts allow: same tokens on every rank, the oracle's tokens, and
    logits within max(2e-2, twice the oracle's own distance to itself under another fp32
    summation order) on the 4096-wide, two-layer model."""
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from nerva_b200 import synth
    from tests.conftest import contract_self_distance
    cfg = _wide_config()
    steps = cfg.decode_tokens
    ranks = _run_ranks(world, steps, "wide")
    assert all(r["shards_equal"] for r in ranks)
    assert all(r["tokens"] == ranks[0]["tokens"] for r in ranks)
    ck = synth.dense_checkpoint(cfg, fill=__import__("nerva_b200.ops", fromlist=["ops"]).synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + steps + 1, mode=oracle_mod.MODE_CUDA)
    ref_tokens, ref = dec.decode_greedy(prompt, steps, want_logits=True)
    got = np.concatenate([r["logits"] for r in ranks], axis=1)
    assert [r["offset"] for r in ranks] == [q * (cfg.vocab // world) for q in range(world)]
    floor = contract_self_distance(oracle_mod, ck, cfg.prompt_tokens + steps + 1, prompt, steps, ref)
    bound = max(LOGIT_ATOL, 2.0 * floor)
    worst = float(np.abs(got - ref).max())
    assert worst <= bound, (worst, bound)
    if worst <= LOGIT_ATOL / 4:  # far from any tie: the token streams must agree as well
        assert ranks[0]["tokens"] == ref_tokens.tolist()


def test_a_rank_whose_peers_never_answer_fails_the_step_within_its_wait_limit(built_lib):
    """One rank of a two-rank model with the other rank absent: the first exchange gives up after
    its bounded wait (about a second), every later exchange of the queued steps sees the error word
    and does not wait again, the call returns status -1, and the device stays usable."""
    import time
    from nerva_b200 import ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    cfg = synth.TINY_QWEN3
    full = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    shard = synth.shard_checkpoint(full, 0, 2)
    s = CudaHfDecodeSequenceSession(shard, 64)
    assert s.status == SmokeStatus.OK, s.error
    s.attach_loopback()
    t0 = time.perf_counter()
    start, loop = CudaHfDecodeSequenceLoop.start(s, synth.prompt_ids(cfg, count=24))
    elapsed = time.perf_counter() - t0
    assert start.status == SmokeStatus.FAILED
    assert "error code 6" in start.error  # kErrPeerWaitTimeout
    assert elapsed < 10.0, elapsed  # one wait limit, not one per exchange (24 tokens x 4 layers x 2 exchanges)
    s.destroy()
    # the context is intact: an ordinary session decodes afterwards
    t = CudaHfDecodeSequenceSession(full, 64)
    assert t.status == SmokeStatus.OK, t.error
    out = t.run(synth.prompt_ids(cfg, count=8), 4)
    assert out.status == SmokeStatus.OK and len(out.tokens) == 4
    t.destroy()
