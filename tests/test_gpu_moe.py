"""Sparse MoE layers of the resident session against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _moe_config(shared: int):
    from nerva_b200 import synth
    return synth.DecoderConfig("tiny-moe", layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, intermediate=1024,
                               vocab=4096, prompt_tokens=12, decode_tokens=12, num_experts=16, top_k=4,
                               moe_intermediate=256, shared_intermediate=shared, norm_topk_prob=True)


@pytest.mark.parametrize("shared", [0, 128])
def test_sparse_moe_session_matches_oracle(built_lib, oracle_mod, shared):
    """Router top-k, expert SwiGLU MLPs and the gated shared expert: tokens identical to the oracle
    and logits within the stated 2e-2 on a two-layer model."""
    from nerva_b200 import ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    cfg = _moe_config(shared)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    s = CudaHfDecodeSequenceSession(ck, cfg.prompt_tokens + cfg.decode_tokens + 1)
    assert s.status == SmokeStatus.OK, s.error
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    assert start.status == SmokeStatus.OK, start.error
    tokens, logits = [], []
    for _ in range(cfg.decode_tokens):
        out = loop.advance(1)
        assert out.status == SmokeStatus.OK, out.error
        tokens += out.tokens
        logits.append(s.read_logits())
    s.destroy()
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens + 1, mode=oracle_mod.MODE_CUDA)
    ref_tokens, ref_logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    assert float(np.abs(np.stack(logits) - ref_logits).max()) <= 2e-2
    assert tokens == ref_tokens.tolist()


def test_fork_of_a_sparse_moe_session_continues_like_its_parent(built_lib, oracle_mod):
    """A fork taken in the middle of a sequence shares the weights and clones the state; its tail,
    the parent's tail and the oracle's must be the same tokens (a fork that lost the layer kinds
    would run the dense residual wiring over MoE layers)."""
    from nerva_b200 import ops, synth
    from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
    cfg = _moe_config(128)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    s = CudaHfDecodeSequenceSession(ck, cfg.prompt_tokens + cfg.decode_tokens + 1)
    assert s.status == SmokeStatus.OK, s.error
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    assert start.status == SmokeStatus.OK, start.error
    head = loop.advance(5).tokens
    fork = s.fork_shared_weights()
    assert fork.status == SmokeStatus.OK, fork.error
    fork_tail = CudaHfDecodeSequenceLoop(fork).advance(cfg.decode_tokens - 5).tokens
    parent_tail = loop.advance(cfg.decode_tokens - 5).tokens
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens + 1, mode=oracle_mod.MODE_CUDA)
    want = dec.decode_greedy(prompt, cfg.decode_tokens).tolist()
    assert head + parent_tail == want
    assert head + fork_tail == want
    # sparse layers stay out of the packed block step: the block entry point reports no ready session
    out = CudaHfDecodeSequenceSession.batch_advance_one([s, fork], 2, 1)
    assert out.block_tokens == 0
    fork.destroy()
    s.destroy()
