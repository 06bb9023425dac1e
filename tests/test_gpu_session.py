"""GPU parity of the resident decode session, through the C ABI."""
import numpy as np
import pytest

from nerva_b200 import ops, synth
from nerva_b200.session import (CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus)
from tests.conftest import contract_self_distance

pytestmark = pytest.mark.gpu

LOGIT_ATOL = 2e-2  # the stated tolerance: logits within 2e-2 max-abs at fp32 accumulation


class _Checkpoint:
    pass


def _kat_checkpoint(qk_norm: bool):
    """The reference's known-answer model (crates/nerva-cuda/src/tests/decode_sequence.rs:123-200,
    decode_sequence_qk_norm.rs:12-91) with its f16 constants written as the same numbers in bf16:
    hidden 2, vocab 4, zero projections; the embedding/lm_head pair makes token t predict t+1."""
    one, zero, neg = 0x3F80, 0x0000, 0xBF80
    cfg = synth.DecoderConfig("kat", layers=1, hidden=2, heads=1, kv_heads=1, head_dim=2, intermediate=2,
                              vocab=4, rms_eps=1e-5, rope_theta=0.0, qk_norm=qk_norm)
    ck = _Checkpoint()
    ck.config = cfg
    ck.embeddings = np.array([one, zero, zero, one, neg, zero, zero, neg], dtype=np.uint16)
    ck.final_norm = np.array([one, one], dtype=np.uint16)
    ck.lm_head = np.array([zero, neg, one, zero, zero, one, neg, zero], dtype=np.uint16)
    rms = np.array([one, one], dtype=np.uint16)
    m = np.zeros(4, dtype=np.uint16)
    layer = dict(rms_attn=rms.copy(), rms_mlp=rms.copy(), w_q=m.copy(), w_k=m.copy(), w_v=m.copy(), w_o=m.copy(),
                 w_gate=m.copy(), w_up=m.copy(), w_down=m.copy())
    if qk_norm:
        layer["q_norm"] = rms.copy()
        layer["k_norm"] = rms.copy()
    ck.layers = [layer]
    return ck


@pytest.mark.parametrize("qk_norm", [False, True])
def test_reference_token_cycle_kat(built_lib, qk_norm):
    ck = _kat_checkpoint(qk_norm)
    s = CudaHfDecodeSequenceSession(ck, 8, use_descriptors=qk_norm)
    assert s.status == SmokeStatus.OK, s.error
    out = s.run([0], 4)
    assert out.status == SmokeStatus.OK, out.error
    assert out.tokens == [1, 2, 3, 0]
    assert out.graph_replays == 4 and out.sync_calls == 1 and out.hot_path_allocations == 0
    # stop token: tokens [1, 2], every replay still launched
    # (decode_sequence.rs:190-200: tokens == [1, 2], graph_replays == 4, kv_tokens == 2)
    out = s.run([0], 4, eos_token=2)
    assert out.tokens == [1, 2] and out.graph_replays == 4 and out.kv_tokens == 2
    if qk_norm:
        assert s.create_result.planned_weight_blocks == 14 and s.create_result.planned_weight_bytes == 108
    s.destroy()


def test_tiny_qwen3_tokens_and_logits(built_lib, oracle_mod, tiny_checkpoint, tiny_golden):
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    assert np.array_equal(prompt, synth.prompt_ids(cfg))
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, cfg.prompt_tokens + cfg.decode_tokens)
    assert s.status == SmokeStatus.OK, s.error
    start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    assert start.status == SmokeStatus.OK, start.error
    # logits of the first generated token against the golden samples of both contracts
    idx = tiny_golden["sample_indices"]
    logits0 = s.read_logits()
    for contract in ("cpu", "cuda"):
        want = np.array(tiny_golden[contract]["logit_samples"][0], dtype=np.float32)
        assert np.abs(logits0[idx] - want).max() <= LOGIT_ATOL
    out = loop.advance(cfg.decode_tokens)
    assert out.status == SmokeStatus.OK, out.error
    # greedy token stream identical to the reference CPU path for all 32 tokens
    assert out.tokens == tiny_golden["cpu"]["tokens"]
    assert out.tokens == tiny_golden["cuda"]["tokens"]
    assert out.observed_token_hash == tiny_golden["cpu"]["token_hash"]
    assert out.graph_replays == cfg.decode_tokens - 1 and out.host_causality_edges == 0
    assert out.hot_path_allocations == 0 and out.sync_calls == 1
    # final-step logits against a live oracle run of the CUDA contract (full vocabulary)
    dec = oracle_mod.Decoder(tiny_checkpoint, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    _, ref_logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    assert np.abs(s.read_logits() - ref_logits[-1]).max() <= LOGIT_ATOL
    s.destroy()


def test_run_equals_start_advance_and_descriptor_upload(built_lib, tiny_checkpoint, tiny_golden):
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128, use_descriptors=True)
    assert s.status == SmokeStatus.OK, s.error
    r = s.create_result
    assert r.planned_weight_bytes == r.resident_weight_bytes
    assert r.descriptor_gpu_resident_h2d_bytes + r.descriptor_gpu_staged_h2d_bytes == r.planned_weight_bytes
    out = s.run(prompt, 8)
    assert out.status == SmokeStatus.OK and out.tokens == tiny_golden["cuda"]["tokens"][:8]
    # chunked advance gives the same stream
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    got = loop.advance(3).tokens + loop.advance(1).tokens + loop.advance(4).tokens
    assert got == tiny_golden["cuda"]["tokens"][:8]
    s.destroy()


def test_kv_pages_bit_exact_and_page_table_permutation(built_lib, oracle_mod, tiny_checkpoint, tiny_golden):
    """K/V rows in the paged cache are bit-identical whatever the page placement, the
    page table reads back exactly, and the token stream does not depend on it."""
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128)
    pages = 128 // 16
    assert np.array_equal(s.kv_block_table(), np.arange(pages))
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    base_tokens = loop.advance(8).tokens
    base_rows = [s.read_kv_row(layer, tok, which) for layer in (0, 3) for tok in (0, 15, 16, 63, 70) for which in (0, 1)]
    s.destroy()
    t = CudaHfDecodeSequenceSession(tiny_checkpoint, 128)
    perm = synth.permutation(9, synth.T_PAGE_TABLE, pages)
    t.set_kv_block_table(perm)
    assert np.array_equal(t.kv_block_table(), perm)
    _, loop = CudaHfDecodeSequenceLoop.start(t, prompt)
    assert loop.advance(8).tokens == base_tokens
    rows = [t.read_kv_row(layer, tok, which) for layer in (0, 3) for tok in (0, 15, 16, 63, 70) for which in (0, 1)]
    for a, b in zip(base_rows, rows):
        assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        t.set_kv_block_table(perm)  # only before start
    t.destroy()


def test_fork_shared_weights_continues_identically(built_lib, tiny_checkpoint, tiny_golden):
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128)
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    head = loop.advance(4).tokens
    f = s.fork_shared_weights()
    assert f.status == SmokeStatus.OK
    tail_parent = loop.advance(6).tokens
    tail_fork = CudaHfDecodeSequenceLoop(f).advance(6).tokens
    assert tail_parent == tail_fork
    assert head + tail_parent == tiny_golden["cuda"]["tokens"][:10]
    f.destroy()
    s.destroy()


def test_invalid_requests_fail_without_device_work(built_lib, tiny_checkpoint):
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 32)
    assert s.status == SmokeStatus.OK
    bad, loop = CudaHfDecodeSequenceLoop.start(s, [40000])  # token outside the vocabulary
    assert bad.status == SmokeStatus.FAILED and loop is None
    bad, loop = CudaHfDecodeSequenceLoop.start(s, list(range(40)))  # longer than max_context
    assert bad.status == SmokeStatus.FAILED
    ok, loop = CudaHfDecodeSequenceLoop.start(s, [1, 2, 3])
    assert ok.status == SmokeStatus.OK
    assert loop.advance(0).status == SmokeStatus.FAILED
    assert loop.advance(31).status == SmokeStatus.FAILED  # would run past max_context
    assert loop.advance(30).status == SmokeStatus.OK
    s.destroy()


@pytest.mark.parametrize("layers", [1, 2])
def test_qwen3_8b_shapes_logits(built_lib, oracle_mod, layers):
    """Full Qwen3-8B layer and head shapes (hidden 4096, 32q/8kv, d 128, I 12288, V 151936)
    on 1 and 2 layers so that the oracle finishes in seconds.

    One layer: logits within the stated 2e-2.  From two layers on, rounding the
    projection inputs to bf16 makes the contract itself sensitive to the fp32
    summation order: the oracle evaluated with 8 interleaved partial sums per row
    instead of one serial sum (both exact restatements of the same contract) moves
    its own logits by about 2e-2 at two layers and 1e-1 at 36.  The bound for the
    deeper case is therefore that self-distance, measured here, not a constant."""
    cfg = synth.DecoderConfig(f"qwen3-8b-{layers}l", layers=layers, hidden=4096, heads=32, kv_heads=8,
                              head_dim=128, intermediate=12288, vocab=151936)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg, count=6)
    s = CudaHfDecodeSequenceSession(ck, 32)
    assert s.status == SmokeStatus.OK, s.error
    _, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
    out = loop.advance(4)
    got = s.read_logits()
    s.destroy()
    dec = oracle_mod.Decoder(ck, 32, mode=oracle_mod.MODE_CUDA)
    ref_tokens, ref_logits = dec.decode_greedy(prompt, 4, want_logits=True)
    bound = LOGIT_ATOL
    if layers > 1:
        bound = max(LOGIT_ATOL, 2.0 * contract_self_distance(oracle_mod, ck, 32, prompt, 4, ref_logits))
    srt = np.sort(ref_logits, axis=1)
    margins = srt[:, -1] - srt[:, -2]
    for step, (a, b) in enumerate(zip(out.tokens, ref_tokens.tolist())):
        if a != b:  # only a near-tie may differ, and nothing after it is comparable
            assert margins[step] <= bound, f"token {step} differs with top-2 margin {margins[step]}"
            break
    else:
        assert np.abs(got - ref_logits[-1]).max() <= bound



def test_weights_uploaded_from_byte_ranges_of_a_file(built_lib, tiny_checkpoint, tiny_golden, tmp_path):
    """Descriptors that name (file, offset, length) ranges — the file-backed load path
    (reference: hf_decode_sequence/weights.cu:797-850) — give the same model as host pointers."""
    from nerva_b200.session import write_weight_file
    path = str(tmp_path / "weights.bin")
    write_weight_file(tiny_checkpoint, path, header_bytes=4096)
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s = CudaHfDecodeSequenceSession(tiny_checkpoint, 128, weight_file=path, weight_file_header=4096)
    assert s.status == SmokeStatus.OK, s.error
    r = s.create_result
    assert r.planned_weight_bytes == r.resident_weight_bytes
    assert r.descriptor_gpu_resident_h2d_bytes + r.descriptor_gpu_staged_h2d_bytes == r.planned_weight_bytes
    out = s.run(prompt, 8)
    assert out.status == SmokeStatus.OK and out.tokens == tiny_golden["cuda"]["tokens"][:8]
    s.destroy()


def test_file_backed_upload_reports_what_went_wrong(built_lib, tiny_checkpoint, tmp_path):
    from nerva_b200.session import write_weight_file
    missing = CudaHfDecodeSequenceSession(tiny_checkpoint, 64, weight_file=str(tmp_path / "absent.bin"))
    assert missing.status == SmokeStatus.FAILED and "cannot open weight file" in missing.error
    path = str(tmp_path / "short.bin")
    write_weight_file(tiny_checkpoint, path)
    with open(path, "r+b") as f:
        f.truncate(1 << 20)
    short = CudaHfDecodeSequenceSession(tiny_checkpoint, 64, weight_file=path)
    assert short.status == SmokeStatus.FAILED and "short read" in short.error
