"""The reference's own CUDA decode library (its session and projection-bench translation units
compiled where they lie into oracle/_ref/libnerva_ref_decode.so, cuBLAS/cuBLASLt underneath) as a
second oracle on the GPU: both libraries export the same C ABI, so the same session mirror drives
both, and their greedy token streams are compared on the same seeded inputs.  This pins RoPE,
q/k-norm, attention, SwiGLU and the residual/norm plumbing to output the reference itself produced.
Skipped when that library has not been built (it needs the reference checkout at build time)."""
import os

import numpy as np
import pytest

from nerva_b200 import ffi, ops, synth
from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus
from tests.conftest import ROOT, assert_stream_matches_or_ties

pytestmark = pytest.mark.gpu

REF_LIBRARY = os.path.join(ROOT, "oracle", "_ref", "libnerva_ref_decode.so")
# A position where the oracle's two best logits are closer than this may legitimately fall either
# way between two fp32 summation orders (the reference sums in cuBLAS order).
TINY_TIE_BOUND = 2e-2


@pytest.fixture(scope="module")
def reference_library():
    if not os.path.exists(REF_LIBRARY):
        pytest.skip("oracle/_ref/libnerva_ref_decode.so has not been built")
    return ffi.load_abi_library(REF_LIBRARY)


def _decode(checkpoint, prompt, steps, library=None, stepwise=True):
    s = CudaHfDecodeSequenceSession(checkpoint, len(prompt) + steps, library=library)
    assert s.status == SmokeStatus.OK, (s.error, s.create_result.cuda_error, s.create_result.failure_stage)
    if stepwise:
        start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
        assert start.status == SmokeStatus.OK, (start.error, start.cuda_error)
        out = loop.advance(steps)
    else:
        out = s.run(prompt, steps)
    assert out.status == SmokeStatus.OK, (out.error, out.cuda_error)
    s.destroy()
    return out


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_tiny_model_tokens_equal_the_reference_cuda_path(built_lib, reference_library, oracle_mod, tiny_checkpoint,
                                                         seed):
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg, seed=seed)
    ours = _decode(tiny_checkpoint, prompt, cfg.decode_tokens)
    theirs = _decode(tiny_checkpoint, prompt, cfg.decode_tokens, library=reference_library)
    dec = oracle_mod.Decoder(tiny_checkpoint, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    tokens, logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    top2 = np.sort(logits, axis=1)[:, -2:]
    margins = (top2[:, 1] - top2[:, 0]).tolist()
    # the reference's CUDA path against the CPU restatement of its numeric contract: pins the oracle
    assert_stream_matches_or_ties(theirs.tokens, tokens.tolist(), margins, TINY_TIE_BOUND, "reference vs oracle")
    # this library against the reference's CUDA path: the parity claim itself
    assert_stream_matches_or_ties(ours.tokens, theirs.tokens, margins, TINY_TIE_BOUND, "this library vs reference")
    assert theirs.hot_path_allocations == 0 and ours.hot_path_allocations == 0


def test_one_shot_run_equals_the_reference_cuda_path(built_lib, reference_library, tiny_checkpoint, tiny_golden):
    """session_run pushes the prompt through the decode step in both libraries (the reference with
    its monolithic attention path)."""
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    ours = _decode(tiny_checkpoint, prompt, cfg.decode_tokens, stepwise=False)
    theirs = _decode(tiny_checkpoint, prompt, cfg.decode_tokens, library=reference_library, stepwise=False)
    margins = tiny_golden["cuda"]["top1_minus_top2"]
    assert_stream_matches_or_ties(theirs.tokens, tiny_golden["cuda"]["tokens"], margins, TINY_TIE_BOUND,
                                  "reference vs golden")
    assert_stream_matches_or_ties(ours.tokens, theirs.tokens, margins, TINY_TIE_BOUND, "this library vs reference")


@pytest.mark.parametrize("layers", [1, 2])
def test_qwen3_8b_layer_shapes_equal_the_reference_cuda_path(built_lib, reference_library, oracle_mod, layers):
    """Full-width Qwen3-8B layers (hidden 4096, 32/8 heads of 128, intermediate 12288, vocabulary
    151936), cut to one and two layers: this library, the reference's CUDA path and the oracle."""
    import dataclasses
    cfg = dataclasses.replace(synth.QWEN3_8B, layers=layers, prompt_tokens=24, decode_tokens=12)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    ours = _decode(ck, prompt, cfg.decode_tokens)
    theirs = _decode(ck, prompt, cfg.decode_tokens, library=reference_library)
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    tokens, logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    top2 = np.sort(logits, axis=1)[:, -2:]
    margins = (top2[:, 1] - top2[:, 0]).tolist()
    bound = 4e-2  # twice the oracle's own distance to itself at two layers of this width
    assert_stream_matches_or_ties(theirs.tokens, tokens.tolist(), margins, bound, "reference vs oracle")
    assert_stream_matches_or_ties(ours.tokens, theirs.tokens, margins, bound, "this library vs reference")


@pytest.mark.parametrize("shared", [0, 128])
def test_sparse_moe_tokens_equal_the_reference_cuda_path(built_lib, reference_library, oracle_mod, shared):
    """Softmax top-k MoE layers (16 experts, top 4, renormalised weights, with and without a gated
    shared expert): this library, the reference's CUDA path (its whole MoE MLP in one thread block,
    hf_decode_sequence/device_ops.cuh:183-315) and the oracle.  Pins the routing order, the expert
    matrix layout and the unrounded activations of the sparse path to output the reference produced."""
    cfg = synth.DecoderConfig("tiny-moe", layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, intermediate=1024,
                              vocab=4096, prompt_tokens=12, decode_tokens=12, num_experts=16, top_k=4,
                              moe_intermediate=256, shared_intermediate=shared, norm_topk_prob=True)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    ours = _decode(ck, prompt, cfg.decode_tokens)
    theirs = _decode(ck, prompt, cfg.decode_tokens, library=reference_library)
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    tokens, logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    top2 = np.sort(logits, axis=1)[:, -2:]
    margins = (top2[:, 1] - top2[:, 0]).tolist()
    assert_stream_matches_or_ties(theirs.tokens, tokens.tolist(), margins, TINY_TIE_BOUND, "reference vs oracle")
    assert_stream_matches_or_ties(ours.tokens, theirs.tokens, margins, TINY_TIE_BOUND, "this library vs reference")


def test_block_of_forks_equals_the_reference_cuda_path(built_lib, reference_library, oracle_mod, tiny_checkpoint):
    """batch_advance_one over a parent and three forks in both libraries: the same selection result
    (reason, exactness, block size, eligible and observed counts) every step, the same token for every
    session of the block, and the same stream as the reference's packed path produced (its
    cublasLt block projections, session_api_batch_fork_destroy.inc.cu)."""
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:11]
    steps = 6

    def run(library):
        # descriptors: the packed step only takes sessions whose shared weights are proven by a plan hash
        parent = CudaHfDecodeSequenceSession(tiny_checkpoint, 96, use_descriptors=True, library=library)
        assert parent.status == SmokeStatus.OK, parent.error
        start, loop = CudaHfDecodeSequenceLoop.start(parent, prompt)
        assert start.status == SmokeStatus.OK, start.error
        stream = list(loop.advance(3).tokens)
        forks = [parent.fork_shared_weights() for _ in range(3)]
        assert all(f.status == SmokeStatus.OK for f in forks)
        block = [parent] + forks
        fields = []
        for _ in range(steps):
            out = CudaHfDecodeSequenceSession.batch_advance_one(block, target_block_tokens=8, min_block_tokens=2)
            assert out.status == SmokeStatus.OK, out.error
            assert out.reason == 0 and out.exact == 1 and out.block_tokens == 4, (out.reason, out.exact, out.block_tokens)
            assert len(set(out.tokens)) == 1, out.tokens  # forks of one sequence decode the same token
            stream.append(out.tokens[0])
            fields.append((out.reason, out.exact, out.block_tokens, out.eligible_session_count, out.observed_tokens))
        for s in forks:
            s.destroy()
        parent.destroy()
        return stream, fields

    ours, our_fields = run(None)
    theirs, their_fields = run(reference_library)
    assert our_fields == their_fields, (our_fields, their_fields)
    dec = oracle_mod.Decoder(tiny_checkpoint, 96, mode=oracle_mod.MODE_CUDA)
    tokens, logits = dec.decode_greedy(prompt, 3 + steps, want_logits=True)
    top2 = np.sort(logits, axis=1)[:, -2:]
    margins = (top2[:, 1] - top2[:, 0]).tolist()
    assert_stream_matches_or_ties(theirs, tokens.tolist(), margins, TINY_TIE_BOUND, "reference block step vs oracle")
    assert_stream_matches_or_ties(ours, theirs, margins, TINY_TIE_BOUND, "this library's block step vs the reference's")


def test_file_backed_upload_equals_the_reference_cuda_path(built_lib, reference_library, tiny_checkpoint, tiny_golden,
                                                           tmp_path):
    """The same weight file and the same (file, offset, length) descriptors through both libraries'
    pinned-staging upload (hf_decode_sequence/weights.cu:797-850): the same model in both."""
    from nerva_b200.session import write_weight_file
    path = str(tmp_path / "weights.bin")
    write_weight_file(tiny_checkpoint, path, header_bytes=4096)
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    streams = []
    for library in (None, reference_library):
        s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128, weight_file=path, weight_file_header=4096,
                                        library=library)
        assert s.status == SmokeStatus.OK, (s.error, s.create_result.cuda_error, s.create_result.failure_stage)
        out = s.run(prompt, 8)
        assert out.status == SmokeStatus.OK, (out.error, out.cuda_error)
        streams.append(out.tokens)
        s.destroy()
    margins = tiny_golden["cuda"]["top1_minus_top2"]
    assert_stream_matches_or_ties(streams[1], tiny_golden["cuda"]["tokens"][:8], margins, TINY_TIE_BOUND,
                                  "reference from the file vs golden")
    assert_stream_matches_or_ties(streams[0], streams[1], margins, TINY_TIE_BOUND, "this library vs reference")


def test_fork_continues_like_its_parent_in_both_libraries(built_lib, reference_library, oracle_mod, tiny_checkpoint):
    """session_fork_shared_weights in the middle of a sequence: the fork's tail and the parent's tail are
    the same tokens, in the reference's library and in this one, and they are the oracle's."""
    cfg = synth.TINY_QWEN3
    prompt = synth.prompt_ids(cfg)[:17]
    streams = []
    for library in (None, reference_library):
        parent = CudaHfDecodeSequenceSession(tiny_checkpoint, 96, use_descriptors=True, library=library)
        assert parent.status == SmokeStatus.OK, parent.error
        start, loop = CudaHfDecodeSequenceLoop.start(parent, prompt)
        assert start.status == SmokeStatus.OK, start.error
        head = list(loop.advance(4).tokens)
        fork = parent.fork_shared_weights()
        assert fork.status == SmokeStatus.OK, fork.error
        fork_tail = list(CudaHfDecodeSequenceLoop(fork).advance(6).tokens)
        parent_tail = list(loop.advance(6).tokens)
        assert fork_tail == parent_tail, (fork_tail, parent_tail)
        streams.append(head + parent_tail)
        fork.destroy()
        parent.destroy()
    dec = oracle_mod.Decoder(tiny_checkpoint, 96, mode=oracle_mod.MODE_CUDA)
    tokens, logits = dec.decode_greedy(prompt, 10, want_logits=True)
    top2 = np.sort(logits, axis=1)[:, -2:]
    margins = (top2[:, 1] - top2[:, 0]).tolist()
    assert_stream_matches_or_ties(streams[1], tokens.tolist(), margins, TINY_TIE_BOUND, "reference vs oracle")
    assert_stream_matches_or_ties(streams[0], streams[1], margins, TINY_TIE_BOUND, "this library vs reference")
