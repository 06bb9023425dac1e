"""The full-size workload of the bench (Qwen3-8B architecture, 36 layers, random-init bf16) through
properties that do not need the CPU oracle to run 36 layers: bit-stable tokens, run == start +
advance, independence of the KV page placement, forks and blocks of forks continuing identically,
and the sampler drawing from the session's own full-vocabulary logits what the oracle draws."""
import numpy as np
import pytest

from nerva_b200 import ops, synth
from nerva_b200.session import (CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus, sampler_config)

pytestmark = pytest.mark.gpu

MAX_CONTEXT = 96
PROMPT_TOKENS = 40  # crosses two 16-token pages and leaves attention with more than one stage tile
STEPS = 12


@pytest.fixture(scope="module")
def full_checkpoint(built_lib):
    return synth.dense_checkpoint(synth.QWEN3_8B, fill=ops.synth_normal_bf16)


@pytest.fixture(scope="module")
def full_session(full_checkpoint):
    s = CudaHfDecodeSequenceSession(full_checkpoint, MAX_CONTEXT, use_descriptors=True)
    assert s.status == SmokeStatus.OK, s.error
    yield s
    s.destroy()


def _prompt():
    return synth.prompt_ids(synth.QWEN3_8B, count=PROMPT_TOKENS)


def test_tokens_are_bit_stable_and_run_equals_start_advance(full_session):
    s = full_session
    first = s.run(_prompt(), STEPS)
    assert first.status == SmokeStatus.OK, first.error
    assert len(first.tokens) == STEPS and first.hot_path_allocations == 0
    assert all(0 <= t < synth.QWEN3_8B.vocab for t in first.tokens)
    again = s.run(_prompt(), STEPS)
    assert again.tokens == first.tokens and again.observed_token_hash == first.observed_token_hash
    start, loop = CudaHfDecodeSequenceLoop.start(s, _prompt())
    assert start.status == SmokeStatus.OK, start.error
    stepped = loop.advance(5).tokens + loop.advance(1).tokens + loop.advance(STEPS - 6).tokens
    assert stepped == first.tokens


def test_tokens_do_not_depend_on_the_kv_page_placement(full_checkpoint, full_session):
    base = full_session.run(_prompt(), STEPS).tokens
    t = CudaHfDecodeSequenceSession(full_checkpoint, MAX_CONTEXT)
    assert t.status == SmokeStatus.OK, t.error
    pages = MAX_CONTEXT // 16
    perm = synth.permutation(5, synth.T_PAGE_TABLE, pages)
    t.set_kv_block_table(perm)
    _, loop = CudaHfDecodeSequenceLoop.start(t, _prompt())
    assert loop.advance(STEPS).tokens == base
    # the cached rows sit where the table says and hold the same bits
    full_session.run(_prompt(), STEPS)
    for layer, token, which in ((0, 0, 0), (17, 16, 1), (35, PROMPT_TOKENS + 3, 0)):
        assert np.array_equal(t.read_kv_row(layer, token, which), full_session.read_kv_row(layer, token, which))
    t.destroy()


def test_forks_and_blocks_of_forks_continue_identically(full_session):
    s = full_session
    expected = s.run(_prompt(), STEPS).tokens
    _, loop = CudaHfDecodeSequenceLoop.start(s, _prompt())
    head = loop.advance(4).tokens
    fork_a, fork_b = s.fork_shared_weights(), s.fork_shared_weights()
    assert fork_a.status == SmokeStatus.OK and fork_b.status == SmokeStatus.OK
    assert head + CudaHfDecodeSequenceLoop(fork_a).advance(STEPS - 4).tokens == expected
    block = []
    for _ in range(3):
        out = CudaHfDecodeSequenceSession.batch_advance_one([s, fork_b], 4, 2)
        assert out.status == SmokeStatus.OK and out.block_tokens == 2, out.error
        assert out.tokens[0] == out.tokens[1]
        block.append(out.tokens[0])
    assert head + block == expected[:7]
    fork_a.destroy()
    fork_b.destroy()


@pytest.mark.parametrize("config", [(0.8, 0.95, 0), (1.0, 1.0, 0), (0.7, 1.0, 40)])
def test_sampler_draws_from_the_sessions_logits(full_session, oracle_mod, config):
    temperature, top_p, top_k = config
    s = full_session
    sampler = sampler_config(temperature, top_p, top_k, seed=2718)
    start, loop = CudaHfDecodeSequenceLoop.start(s, _prompt(), sampler=sampler)
    assert start.status == SmokeStatus.OK, start.error
    tokens = []
    for i in range(6):
        out = loop.advance(1)
        assert out.status == SmokeStatus.OK, out.error
        want, margin = oracle_mod.sample_token(s.read_logits(), PROMPT_TOKENS - 1 + i, temperature, top_p, top_k, 2718)
        if margin > 1e-4:  # closer decisions may fall either way between glibc's and the device's logf / expf
            assert out.tokens[0] == want, (i, margin)
        if oracle_mod.ref_sampler_lib() is not None:  # the reference's own kernel on the same logits
            assert out.tokens[0] == oracle_mod.ref_sample_token(s.read_logits(), PROMPT_TOKENS - 1 + i, temperature,
                                                                top_p, top_k, 2718)
        tokens.append(out.tokens[0])
    assert s.run(_prompt(), 6, sampler=sampler).tokens == tokens
