"""Expert parallel over 2, 4 and 8 GPUs: one process per GPU, every rank holds the whole
DeepSeek-V2-Lite-architecture model except its share of the routed experts and of the shared expert;
the ranks' partial MLP outputs are exchanged over peer memory.  Tokens and logits against the CPU
oracle of the whole model, and against the same model on one GPU.  Skipped on a single-GPU machine."""
import dataclasses
import os
import sys

import numpy as np
import pytest

from tests.test_gpu_tensor_parallel import ROOT, _free_port, _gpu_count

pytestmark = pytest.mark.gpu

LOGIT_ATOL = 2e-2


def _config(kind: str):
    from nerva_b200 import synth
    if kind == "small":
        return dataclasses.replace(synth.DEEPSEEK_V2_LITE, name="v2-lite-small", layers=3, vocab=4096, prompt_tokens=21,
                                   decode_tokens=12, hidden=512, heads=4, kv_heads=4, head_dim=64, intermediate=1024,
                                   num_experts=8, top_k=3, moe_intermediate=128, shared_intermediate=256,
                                   kv_lora_rank=128, qk_nope_head_dim=64, qk_rope_head_dim=32)
    # full-width layers (hidden 2048, 16 heads, rank 512, 64 experts top-6, shared 2816), three of them
    return dataclasses.replace(synth.DEEPSEEK_V2_LITE, name="v2-lite cut to 3", layers=3, vocab=32768,
                               prompt_tokens=40, decode_tokens=8)


def _rank_main(rank: int, world: int, port: int, steps: int, kind: str, results) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import datetime
    import torch.distributed as dist
    from nerva_b200 import ops, synth, tp
    from nerva_b200.session import CudaHfDecodeSequenceLoop, SmokeStatus
    tp.select_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=180))
    try:
        cfg = _config(kind)
        full = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
        session = tp.create_session(cfg, cfg.prompt_tokens + steps + 1, rank, world, full_checkpoint=full)
        start, loop = CudaHfDecodeSequenceLoop.start(session, synth.prompt_ids(cfg))
        assert start.status == SmokeStatus.OK, start.error
        tokens, logits = [], []
        for _ in range(steps):
            out = loop.advance(1)
            assert out.status == SmokeStatus.OK, out.error
            tokens += out.tokens
            logits.append(session.read_logits())  # the whole vocabulary: the head is not cut
        dist.barrier()
        resident = int(session.create_result.resident_weight_bytes)
        session.destroy()
        results[rank] = {"tokens": tokens, "logits": np.stack(logits), "resident_weight_bytes": resident}
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


@pytest.mark.parametrize("world,kind", [(2, "small"), (2, "wide"), (4, "wide"), (8, "wide")])
def test_expert_parallel_matches_the_oracle_and_one_gpu(built_lib, oracle_mod, world, kind):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from nerva_b200 import ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    cfg = _config(kind)
    steps = cfg.decode_tokens
    ranks = _run_ranks(world, steps, kind)
    # every rank samples from its own full logits: same tokens, and logits equal bit for bit (the
    # partial outputs are added in rank order on every rank)
    assert all(r["tokens"] == ranks[0]["tokens"] for r in ranks)
    assert all(np.array_equal(r["logits"], ranks[0]["logits"]) for r in ranks)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + steps + 1, mode=oracle_mod.MODE_CUDA)
    want_tokens, want = dec.decode_greedy(prompt, steps, want_logits=True)
    top2 = np.sort(want, axis=1)[:, -2:]
    margins = top2[:, 1] - top2[:, 0]
    got = ranks[0]["logits"]
    at = next((i for i in range(steps) if ranks[0]["tokens"][i] != int(want_tokens[i])), None)
    compared = steps if at is None else at + 1
    assert float(np.abs(got[:compared] - want[:compared]).max()) <= LOGIT_ATOL
    assert at is None or margins[at] <= LOGIT_ATOL, (at, ranks[0]["tokens"], want_tokens.tolist())
    # one GPU, whole model: the same sums in another order (experts by routing rank instead of by owner)
    single = CudaHfDecodeSequenceSession(ck, cfg.prompt_tokens + steps + 1)
    assert single.status == SmokeStatus.OK, single.error
    _, loop = CudaHfDecodeSequenceLoop.start(single, prompt)
    loop.advance(1)
    assert float(np.abs(single.read_logits() - got[0]).max()) <= LOGIT_ATOL
    # a rank holds less than the whole model: the routed experts are divided
    assert all(r["resident_weight_bytes"] < int(single.create_result.resident_weight_bytes) for r in ranks)
    single.destroy()
