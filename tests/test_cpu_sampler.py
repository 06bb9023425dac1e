"""The CPU oracle's temperature / top-k / top-p sampler: its randomness against a pure-Python
restatement of the published splitmix64 finaliser, its branches against their definitions, and
its draws against the distribution they must follow."""
import numpy as np
import pytest

M64 = (1 << 64) - 1


def _uniform(seed, position, token, salt):
    """(24 mixed bits + 1) / (2^24 + 1) of splitmix64(seed ^ position<<32 ^ token ^ salt<<48)
    (reference: hf_decode_sequence/sampler.cu:18-33)."""
    v = (seed ^ (position << 32) ^ token ^ (salt << 48)) & M64
    v = (v + 0x9E3779B97F4A7C15) & M64
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & M64
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & M64
    v ^= v >> 31
    return np.float32(np.float32(((v >> 40) & 0xFFFFFF)) + np.float32(1.0)) / np.float32(16777217.0)


def test_uniform_matches_python_restatement(oracle_mod):
    rng = np.random.default_rng(5)
    for _ in range(500):
        seed = int(rng.integers(0, 1 << 63)) * 2 + int(rng.integers(0, 2))
        position, token, salt = int(rng.integers(0, 1 << 32)), int(rng.integers(0, 1 << 32)), int(rng.integers(0, 2))
        got = oracle_mod.sampler_uniform(seed, position, token, salt)
        assert np.float32(got) == _uniform(seed, position, token, salt)
        assert 0.0 < got <= 1.0


def test_splitmix_known_answer(oracle_mod):
    # splitmix64's first output for state 0 is 0xE220A8397B1DCDAF (the generator's published
    # test vector); its top 24 bits are 0xE220A8.
    assert np.float32(oracle_mod.sampler_uniform(0, 0, 0, 0)) == np.float32(0xE220A8 + 1) / np.float32(16777217.0)


def test_greedy_cases(oracle_mod):
    rng = np.random.default_rng(1)
    logits = rng.standard_normal(4099).astype(np.float32)
    logits[[7, 900]] = logits.max() + 1.0  # a tie: the lower index wins
    for temperature, top_k in ((0.0, 0), (0.0, 40), (0.8, 1)):
        token, margin = oracle_mod.sample_token(logits, 3, temperature, 0.9, top_k, 11)
        assert token == 7 and margin == np.inf
    logits[7] = np.nan
    logits[900] = np.inf
    assert oracle_mod.sample_token(logits, 3, 0.0, 1.0, 0, 0)[0] == int(np.argmax(np.where(np.isfinite(logits), logits, -np.inf)))
    nothing = np.full(16, -np.inf, dtype=np.float32)
    for cfg in ((0.0, 1.0, 0), (1.0, 1.0, 0), (1.0, 0.9, 5)):
        assert oracle_mod.sample_token(nothing, 0, *cfg, 3)[0] == 0


def test_top_k_stays_in_the_top_k_and_is_deterministic(oracle_mod):
    rng = np.random.default_rng(2)
    logits = (rng.standard_normal(32000) * 2.0).astype(np.float32)
    order = np.lexsort((np.arange(logits.size), -logits))
    for top_k in (2, 5, 40, 128, 500):
        allowed = set(order[:min(top_k, 128)].tolist())
        seen = set()
        for position in range(200):
            token, _ = oracle_mod.sample_token(logits, position, 1.3, 1.0, top_k, 99)
            assert token in allowed
            assert token == oracle_mod.sample_token(logits, position, 1.3, 1.0, top_k, 99)[0]
            seen.add(token)
        assert len(seen) > 1


def test_small_top_p_keeps_only_the_best(oracle_mod):
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(1000).astype(np.float32)
    logits[123] = 20.0
    for position in range(50):
        assert oracle_mod.sample_token(logits, position, 1.0, 0.5, 0, position)[0] == 123


def test_non_finite_logits_are_never_drawn(oracle_mod):
    rng = np.random.default_rng(4)
    logits = rng.standard_normal(300).astype(np.float32)
    bad = rng.choice(300, 150, replace=False)
    logits[bad[:50]] = np.inf
    logits[bad[50:100]] = -np.inf
    logits[bad[100:]] = np.nan
    for position in range(100):
        for cfg in ((1.0, 1.0, 0), (1.0, 0.95, 0), (2.0, 1.0, 128)):
            assert np.isfinite(logits[oracle_mod.sample_token(logits, position, *cfg, 5)[0]])


@pytest.mark.parametrize("config", [(1.0, 1.0, 0), (0.7, 1.0, 8), (1.5, 0.8, 0)])
def test_draws_follow_the_softmax(oracle_mod, config):
    """Frequencies over 20000 positions against the (truncated, renormalised) softmax."""
    temperature, top_p, top_k = config
    logits = np.array([2.0, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, -2.0, -3.0, -4.0, -6.0, -8.0], dtype=np.float32)
    p = np.exp((logits - logits.max()) / temperature)
    p /= p.sum()
    keep = logits.size if top_k == 0 else min(top_k, logits.size)
    if top_p < 0.999999:
        keep = min(keep, int(np.searchsorted(np.cumsum(p), top_p) + 1))
    expected = np.zeros_like(p)
    expected[:keep] = p[:keep] / p[:keep].sum()
    draws = 20000
    counts = np.zeros(logits.size)
    for position in range(draws):
        counts[oracle_mod.sample_token(logits, position, temperature, top_p, top_k, 2024)[0]] += 1
    assert counts[keep:].sum() == 0
    sigma = np.sqrt(expected * (1 - expected) / draws)
    assert np.all(np.abs(counts / draws - expected) <= 5 * sigma + 1e-4)
