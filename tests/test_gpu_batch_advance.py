"""nerva_cuda_hf_decode_sequence_batch_advance_one on the GPU: the tokens are the ones
session_advance(1) gives, only ready sessions that share weights take part, and the session
state moves exactly as if each had advanced alone."""
import numpy as np
import pytest

from nerva_b200 import synth
from nerva_b200.session import (CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus, sampler_config)

pytestmark = pytest.mark.gpu

NOT_TAKEN = 0xFFFFFFFF


def _started(checkpoint, prompt, max_context=96, sampler=None, use_descriptors=True):
    s = CudaHfDecodeSequenceSession(checkpoint, max_context, use_descriptors=use_descriptors)
    assert s.status == SmokeStatus.OK, s.error
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt, sampler=sampler)
    assert start.status == SmokeStatus.OK, start.error
    return s, loop


def test_block_of_forks_matches_individual_advances(built_lib, tiny_checkpoint):
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:11]
    parent, loop = _started(tiny_checkpoint, prompt)
    first = loop.advance(3).tokens
    forks = [parent.fork_shared_weights() for _ in range(3)]
    twins = [parent.fork_shared_weights() for _ in range(4)]  # advanced one by one as the expectation
    block = [parent] + forks
    expected = [[] for _ in twins]
    got = [[] for _ in block]
    for _ in range(6):
        out = CudaHfDecodeSequenceSession.batch_advance_one(block, target_block_tokens=8, min_block_tokens=2)
        assert out.status == SmokeStatus.OK, out.error
        assert out.reason == 0 and out.exact == 1 and out.block_tokens == 4 and out.eligible_session_count == 4
        assert out.observed_tokens == 4 and out.sampling_kernel_launches == 4 and out.hot_path_allocations == 0
        assert out.layer_count == cfg.layers and out.last_token == out.tokens[-1]
        for i, token in enumerate(out.tokens):
            got[i].append(token)
        for i, twin in enumerate(twins):
            expected[i] += CudaHfDecodeSequenceLoop(twin).advance(1).tokens
        if got != expected:
            # The packed step runs the projections on the tensor pipe, the lone advance on the streaming
            # mat-vec: two fp32 summation orders.  The streams may part only where the session's own two
            # best logits are closer than the stated logit bound; nothing can be compared after that.
            top2 = np.sort(twins[0].read_logits())[-2:]
            assert top2[1] - top2[0] <= 2e-2, (got, expected)
            for s in forks + twins:
                s.destroy()
            parent.destroy()
            return
    assert got == expected and len(first) == 3
    # the sessions go on alone from where the block left them
    tail_block = CudaHfDecodeSequenceLoop(forks[0]).advance(5).tokens
    tail_twin = CudaHfDecodeSequenceLoop(twins[1]).advance(5).tokens
    assert tail_block == tail_twin
    for s in forks + twins:
        s.destroy()
    parent.destroy()


def test_sampled_sessions_keep_their_own_sampler(built_lib, tiny_checkpoint):
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:7]
    parent, loop = _started(tiny_checkpoint, prompt, sampler=sampler_config(1.0, 0.95, 0, seed=31))
    loop.advance(2)
    fork, twin_parent, twin_fork = (parent.fork_shared_weights() for _ in range(3))
    got, expected = [], []
    for _ in range(8):
        out = CudaHfDecodeSequenceSession.batch_advance_one([parent, fork], 4, 2)
        assert out.status == SmokeStatus.OK and out.block_tokens == 2, out.error
        got.append(out.tokens)
        expected.append(CudaHfDecodeSequenceLoop(twin_parent).advance(1).tokens +
                        CudaHfDecodeSequenceLoop(twin_fork).advance(1).tokens)
    assert got == expected
    for s in (fork, twin_parent, twin_fork, parent):
        s.destroy()


def test_selection_rules(built_lib, tiny_checkpoint):
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:6]
    parent, loop = _started(tiny_checkpoint, prompt)
    loop.advance(1)
    fork = parent.fork_shared_weights()
    idle = CudaHfDecodeSequenceSession(tiny_checkpoint, 96, use_descriptors=True)  # never started
    other, other_loop = _started(tiny_checkpoint, prompt)  # same model, its own weight copy
    other_loop.advance(1)

    # nothing ready
    out = CudaHfDecodeSequenceSession.batch_advance_one([idle], 4, 1)
    assert out.status == SmokeStatus.OK and out.reason == 3 and out.tokens == [NOT_TAKEN]
    # too few compatible sessions for the requested minimum: nobody moves
    out = CudaHfDecodeSequenceSession.batch_advance_one([parent, fork, idle], 4, 3)
    assert out.status == SmokeStatus.OK and out.reason == 5 and out.eligible_session_count == 2
    assert out.tokens == [NOT_TAKEN] * 3
    # the larger compatible group wins; the stranger and the idle session are left alone
    out = CudaHfDecodeSequenceSession.batch_advance_one([other, idle, parent, fork], 4, 2)
    assert out.status == SmokeStatus.OK and out.reason == 0 and out.block_tokens == 2
    assert out.tokens[0] == NOT_TAKEN and out.tokens[1] == NOT_TAKEN
    assert out.tokens[2] != NOT_TAKEN and out.tokens[2] == out.tokens[3]  # identical histories
    # target_block_tokens caps the block, in request order
    out = CudaHfDecodeSequenceSession.batch_advance_one([parent, fork], 1, 1)
    assert out.status == SmokeStatus.OK and out.block_tokens == 1 and out.tokens[1] == NOT_TAKEN
    # a handle listed twice is refused
    out = CudaHfDecodeSequenceSession.batch_advance_one([fork, fork], 4, 1)
    assert out.status == SmokeStatus.FAILED
    for s in (fork, idle, other, parent):
        s.destroy()


def test_sessions_without_a_descriptor_hash_are_unproven(built_lib, tiny_checkpoint):
    cfg = synth.TINY_QWEN3
    parent, loop = _started(tiny_checkpoint, synth.prompt_ids(cfg)[:4], use_descriptors=False)
    loop.advance(1)
    fork = parent.fork_shared_weights()
    out = CudaHfDecodeSequenceSession.batch_advance_one([parent, fork], 4, 1)
    assert out.status == SmokeStatus.OK and out.reason == 4 and out.tokens == [NOT_TAKEN] * 2
    fork.destroy()
    parent.destroy()


def test_stop_token_and_context_end_finish_a_session(built_lib, tiny_checkpoint):
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:5]
    probe, probe_loop = _started(tiny_checkpoint, prompt, max_context=8)
    tokens = probe_loop.advance(3).tokens
    probe.destroy()
    if tokens[0] == tokens[1]:
        pytest.skip("the first two tokens coincide: no distinct stop token to test with")
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 8, use_descriptors=True)
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt, eos_token=tokens[1])
    assert start.status == SmokeStatus.OK
    # straight after start the first token is still pending: not ready for a block
    out = CudaHfDecodeSequenceSession.batch_advance_one([s], 1, 1)
    assert out.status == SmokeStatus.OK and out.reason == 3
    assert loop.advance(1).tokens == [tokens[0]]
    out = CudaHfDecodeSequenceSession.batch_advance_one([s], 1, 1)
    assert out.status == SmokeStatus.OK and out.tokens == [tokens[1]]  # the stop token: finished now
    out = CudaHfDecodeSequenceSession.batch_advance_one([s], 1, 1)
    assert out.status == SmokeStatus.OK and out.reason == 3 and out.tokens == [NOT_TAKEN]
    s.destroy()
