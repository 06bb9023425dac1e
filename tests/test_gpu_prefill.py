"""Chunked prefill of session_start (block projections on the tensor pipe, paged K/V published per
chunk) against the token-by-token prefill through the decode step and against the CPU oracle."""
import os

import numpy as np
import pytest

from nerva_b200 import ops, synth
from nerva_b200.session import CudaHfDecodeSequenceLoop, CudaHfDecodeSequenceSession, SmokeStatus

pytestmark = pytest.mark.gpu

LOGIT_ATOL = 2e-2


def _start(checkpoint, prompt, max_context, by_decode: bool):
    """A started session; by_decode selects the token-by-token prefill (NERVA_B200_PREFILL=decode)."""
    if by_decode:
        os.environ["NERVA_B200_PREFILL"] = "decode"
    try:
        s = CudaHfDecodeSequenceSession(checkpoint, max_context)
        assert s.status == SmokeStatus.OK, s.error
        start, loop = CudaHfDecodeSequenceLoop.start(s, prompt)
        assert start.status == SmokeStatus.OK, start.error
    finally:
        os.environ.pop("NERVA_B200_PREFILL", None)
    return s, loop, start


def _row_distance_in_steps(a: np.ndarray, b: np.ndarray) -> float:
    """Largest element difference of two cached rows (bf16 bit patterns), in units of the bf16
    step at the row's largest magnitude: 1.0 means one rounding step of the largest element."""
    fa, fb = synth.bf16_to_f32(a), synth.bf16_to_f32(b)
    top = float(max(np.abs(fa).max(), np.abs(fb).max()))
    if top == 0.0:
        return 0.0
    step = 2.0 ** (np.floor(np.log2(top)) - 7)  # bf16 keeps 8 significant bits
    return float(np.abs(fa - fb).max() / step)


@pytest.mark.parametrize("prompt_tokens", [2, 17, 64, 255, 256, 257, 300])
def test_chunked_prefill_matches_prefill_by_decode(built_lib, oracle_mod, tiny_checkpoint, prompt_tokens):
    """Prompt lengths around the 16-token page and the 256-token chunk: same first token and same
    continuation as the token-by-token prefill, first-token logits within the stated bound of the
    oracle, cached K/V rows within one bf16 rounding step (at the row's magnitude) of the rows the
    decode step writes: the two prefills differ in the fp32 summation order of the QKV projection."""
    cfg = synth.TINY_QWEN3
    prompt = synth.uniform_u32(3, synth.T_PROMPT, prompt_tokens, cfg.vocab)
    steps = 8
    chunked, loop_c, start_c = _start(tiny_checkpoint, prompt, prompt_tokens + steps, by_decode=False)
    serial, loop_s, start_s = _start(tiny_checkpoint, prompt, prompt_tokens + steps, by_decode=True)
    assert chunked.create_result.prefill_chunk_tokens > 1
    assert start_c.graph_replays == 0 and start_s.graph_replays == prompt_tokens
    logits_c, logits_s = chunked.read_logits(), serial.read_logits()
    dec = oracle_mod.Decoder(tiny_checkpoint, prompt_tokens + steps, mode=oracle_mod.MODE_CUDA)
    want_tokens, want_logits = dec.decode_greedy(prompt, steps, want_logits=True)
    assert np.abs(logits_c - want_logits[0]).max() <= LOGIT_ATOL
    assert np.abs(logits_c - logits_s).max() <= LOGIT_ATOL
    worst = 0.0
    for layer in (0, cfg.layers - 1):
        for token in sorted({0, prompt_tokens // 2, prompt_tokens - 1}):
            for which in (0, 1):
                worst = max(worst, _row_distance_in_steps(chunked.read_kv_row(layer, token, which),
                                                          serial.read_kv_row(layer, token, which)))
    assert worst <= 1.0, worst
    got_c = loop_c.advance(steps).tokens
    got_s = loop_s.advance(steps).tokens
    top2 = np.sort(want_logits, axis=1)[:, -2:]
    margins = top2[:, 1] - top2[:, 0]
    for got in (got_c, got_s):
        at = next((i for i in range(steps) if got[i] != int(want_tokens[i])), None)
        assert at is None or margins[at] <= LOGIT_ATOL, (at, got, want_tokens.tolist())
    chunked.destroy()
    serial.destroy()


def test_chunked_prefill_on_the_golden_prompt(built_lib, tiny_checkpoint, tiny_golden):
    cfg = synth.TINY_QWEN3
    prompt = np.array(tiny_golden["prompt"], dtype=np.uint32)
    s, loop, start = _start(tiny_checkpoint, prompt, cfg.prompt_tokens + cfg.decode_tokens, by_decode=False)
    idx = tiny_golden["sample_indices"]
    want = np.array(tiny_golden["cuda"]["logit_samples"][0], dtype=np.float32)
    assert np.abs(s.read_logits()[idx] - want).max() <= LOGIT_ATOL
    assert loop.advance(cfg.decode_tokens).tokens == tiny_golden["cuda"]["tokens"]
    s.destroy()


def test_chunked_prefill_on_qwen3_8b_layer_shapes(built_lib, oracle_mod):
    """Two full-width layers, a 300-token prompt (two chunks): first-token logits against the oracle."""
    import dataclasses
    from tests.conftest import contract_self_distance
    cfg = dataclasses.replace(synth.QWEN3_8B, layers=2, prompt_tokens=300, decode_tokens=4)
    ck = synth.dense_checkpoint(cfg, fill=ops.synth_normal_bf16)
    prompt = synth.prompt_ids(cfg)
    s, loop, start = _start(ck, prompt, cfg.prompt_tokens + cfg.decode_tokens, by_decode=False)
    logits = s.read_logits()
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens, mode=oracle_mod.MODE_CUDA)
    tokens, ref = dec.decode_greedy(prompt, 1, want_logits=True)
    floor = contract_self_distance(oracle_mod, ck, cfg.prompt_tokens + 1, prompt, 1, ref)
    assert np.abs(logits - ref[0]).max() <= max(LOGIT_ATOL, 2.0 * floor)
    s.destroy()
