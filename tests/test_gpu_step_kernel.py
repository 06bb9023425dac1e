"""GPU parity of the whole-step kernel (engine 1) against the oracle and against engine 0."""
import numpy as np
import pytest

from nerva_b200 import ops, synth
from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
from tests.conftest import contract_self_distance

pytestmark = pytest.mark.gpu

LOGIT_ATOL = 2e-2


def test_tiny_qwen3_whole_step_kernel_matches_golden(built_lib, oracle_mod, tiny_checkpoint, tiny_golden):
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, cfg.prompt_tokens + cfg.decode_tokens, engine=1)
    assert s.status == SmokeStatus.OK, s.error
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    assert start.status == SmokeStatus.OK, start.error
    idx = tiny_golden["sample_indices"]
    logits0 = s.read_logits()
    for contract in ("cpu", "cuda"):
        want = np.array(tiny_golden[contract]["logit_samples"][0], dtype=np.float32)
        assert np.abs(logits0[idx] - want).max() <= LOGIT_ATOL
    out = loop.advance(cfg.decode_tokens)
    assert out.status == SmokeStatus.OK, out.error
    assert out.tokens == tiny_golden["cpu"]["tokens"]
    assert out.observed_token_hash == tiny_golden["cuda"]["token_hash"]
    assert out.hot_path_allocations == 0 and out.sync_calls == 1
    dec = oracle_mod.Decoder(tiny_checkpoint, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    _, ref_logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    assert np.abs(s.read_logits() - ref_logits[-1]).max() <= LOGIT_ATOL
    s.destroy()


def test_engines_agree_on_kv_pages_and_tokens(built_lib, tiny_checkpoint, tiny_golden):
    """Both engines write bit-identical K/V rows for the first layer (same projection
    arithmetic) and produce the same tokens; with a permuted page table too."""
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    perm = synth.permutation(4, synth.T_PAGE_TABLE, 128 // 16)
    rows, tokens = [], []
    for engine in (0, 1):
        s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128, engine=engine)
        s.set_kv_block_table(perm)
        _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
        tokens.append(loop.advance(10).tokens)
        rows.append([s.read_kv_row(0, tok, which) for tok in (0, 17, 63, 66) for which in (0, 1)])
        s.destroy()
    assert tokens[0] == tokens[1] == tiny_golden["cuda"]["tokens"][:10]
    for a, b in zip(rows[0], rows[1]):
        assert np.array_equal(a, b)


def test_whole_step_kernel_run_fork_and_long_context(built_lib, oracle_mod):
    """run(), fork and a context that spans several attention items per head (> 256 tokens)."""
    cfg = synth.DecoderConfig("mid", layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64,
                              intermediate=1536, vocab=4096)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg, count=700)
    s = CudaHfDecodeSequenceSession(ck, 800, engine=1)
    assert s.status == SmokeStatus.OK, s.error
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    head = loop.advance(3).tokens
    f = s.fork_shared_weights()
    a = loop.advance(5).tokens
    b = CudaHfDecodeSequenceLoop(f).advance(5).tokens
    assert a == b
    got = s.read_logits()
    f.destroy()
    s.destroy()
    dec = oracle_mod.Decoder(ck, 800, mode=oracle_mod.MODE_CUDA)
    ref_tokens, ref_logits = dec.decode_greedy(prompt, 8, want_logits=True)
    assert head + a == ref_tokens.tolist()
    assert np.abs(got - ref_logits[-1]).max() <= LOGIT_ATOL
    e0 = CudaHfDecodeSequenceSession(ck, 800, engine=0)
    assert e0.run(prompt[:40], 6).tokens == CudaHfDecodeSequenceSession(ck, 800, engine=1).run(prompt[:40], 6).tokens
    e0.destroy()


def test_whole_step_kernel_qwen3_8b_layer_shapes(built_lib, oracle_mod):
    cfg = synth.DecoderConfig("qwen3-8b-1l", layers=1, hidden=4096, heads=32, kv_heads=8, head_dim=128,
                              intermediate=12288, vocab=151936)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg, count=40)
    s = CudaHfDecodeSequenceSession(ck, 64, engine=1)
    assert s.status == SmokeStatus.OK, s.error
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    out = loop.advance(4)
    got = s.read_logits()
    s.destroy()
    dec = oracle_mod.Decoder(ck, 64, mode=oracle_mod.MODE_CUDA)
    ref_tokens, ref_logits = dec.decode_greedy(prompt, 4, want_logits=True)
    assert out.tokens == ref_tokens.tolist()
    # at these widths the contract's own summation-order sensitivity can exceed 2e-2
    bound = max(LOGIT_ATOL, 2.0 * contract_self_distance(oracle_mod, ck, 64, prompt, 4, ref_logits))
    assert np.abs(got - ref_logits[-1]).max() <= bound


def test_engine_refused_for_unsupported_head_dim(built_lib):
    cfg = synth.DecoderConfig("odd", layers=1, hidden=96, heads=3, kv_heads=3, head_dim=32, intermediate=64, vocab=64)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    with pytest.raises(RuntimeError):
        CudaHfDecodeSequenceSession(ck, 16, engine=1)
    s = CudaHfDecodeSequenceSession(ck, 16, engine=0)
    assert s.run([1, 2, 3], 4).status == SmokeStatus.OK
    s.destroy()
