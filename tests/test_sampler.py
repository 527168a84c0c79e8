"""Host-side temperature / top-k / top-p sampler (llmb_sample_logits_host) against the oracle's
statement-by-statement restatement of the reference's sample_next_token chain
(src/inference/inference.cu:1030-1161).  Pure host code on both sides: no GPU needed."""
import ctypes as C

import numpy as np
import pytest


def lib_sample(pkg, logits, temperature, top_k, top_p, u):
    tok = C.c_int32(-1)
    rc = pkg.lib.llmb_sample_logits_host(logits.ctypes.data, len(logits), temperature, top_k, top_p, u, C.byref(tok))
    assert rc == 0, pkg.lib.llmb_last_error()
    return tok.value


def oracle_sample(oracle, logits, temperature, top_k, top_p, u):
    return int(oracle.lib().oracle_sample(logits.ctypes.data, len(logits), temperature, top_k, top_p, u))


def make_logits(oracle, seed, vocab, std):
    return oracle.synth_fp16(4000 + seed, 9, vocab, std=std)


@pytest.mark.parametrize("vocab,std", [(4096, 3.0), (128256, 2.0), (1000, 0.5), (50, 4.0), (7, 1.0)])
def test_matches_reference_restatement(pkg, oracle, vocab, std):
    logits = make_logits(oracle, vocab, vocab, std)
    us = [0.0, 0.001, 0.25, 0.5, 0.75, 0.9, 0.999, float(np.nextafter(np.float32(1.0), np.float32(0.0)))]
    for temperature, top_k, top_p in [(0.7, 50, 0.9), (1.0, 50, 0.9), (0.7, 5, 0.5), (0.3, 50, 1.0), (1.5, 1000, 0.95),
                                      (0.7, 1, 0.9), (0.7, 10 ** 6, 1.0), (0.7, 50, 2.0)]:
        for u in us:
            want = oracle_sample(oracle, logits, temperature, top_k, top_p, u)
            got = lib_sample(pkg, logits, temperature, top_k, top_p, u)
            assert got == want, (vocab, temperature, top_k, top_p, u, got, want)


def test_ties_go_to_the_lower_index(pkg, oracle):
    logits = np.full(64, np.float16(1.0).view(np.uint16), dtype=np.uint16)
    logits[10] = logits[40] = np.float16(3.0).view(np.uint16)
    # two equal heads: u below their first share picks index 10, above it index 40
    assert lib_sample(pkg, logits, 1.0, 2, 1.0, 0.1) == 10 == oracle_sample(oracle, logits, 1.0, 2, 1.0, 0.1)
    assert lib_sample(pkg, logits, 1.0, 2, 1.0, 0.9) == 40 == oracle_sample(oracle, logits, 1.0, 2, 1.0, 0.9)


def test_greedy_limits(pkg, oracle):
    logits = make_logits(oracle, 1, 4096, 3.0)
    best = int(oracle.lib().oracle_argmax_fp16(logits.ctypes.data, len(logits)))
    for u in (0.0, 0.3, 0.99):
        assert lib_sample(pkg, logits, 0.7, 1, 0.9, u) == best          # top_k = 1
        assert lib_sample(pkg, logits, 0.7, 50, 1e-6, u) == best        # top_p -> 0


def test_draw_is_monotone_in_u_and_stays_in_the_nucleus(pkg, oracle):
    logits = make_logits(oracle, 2, 4096, 3.0)
    order = np.argsort(-oracle.f16(logits), kind="stable")
    rank = {int(t): i for i, t in enumerate(order)}
    ranks = [rank[lib_sample(pkg, logits, 0.7, 50, 0.9, float(u))] for u in np.linspace(0.0, 0.999, 200)]
    assert ranks == sorted(ranks)
    assert ranks[0] == 0 and max(ranks) < 50


def test_frequencies_follow_the_renormalised_distribution(pkg, oracle):
    logits = make_logits(oracle, 3, 512, 2.0)
    temperature, top_k, top_p = 0.8, 8, 1.0
    p = np.exp(oracle.f16(logits).astype(np.float64) / temperature)
    order = np.argsort(-p, kind="stable")[:top_k]
    want = p[order] / p[order].sum()
    n = 20000
    counts = np.zeros(top_k)
    pos = {int(t): i for i, t in enumerate(order)}
    for i in range(n):
        u = pkg.lib.llmb_sampler_uniform(11, i)
        assert 0.0 <= u < 1.0
        counts[pos[lib_sample(pkg, logits, temperature, top_k, top_p, u)]] += 1
    assert np.abs(counts / n - want).max() < 0.015


def test_uniform_stream_matches_the_c_generator(pkg, oracle):
    for seed, draw in [(0, 0), (0, 1), (5, 123456789), (2 ** 40 + 3, 2 ** 33)]:
        assert pkg.lib.llmb_sampler_uniform(seed, draw) == oracle.lib().oracle_sampler_uniform(seed, draw)


def test_invalid_arguments_are_refused(pkg, oracle):
    logits = make_logits(oracle, 4, 64, 1.0)
    tok = C.c_int32(0)
    f = pkg.lib.llmb_sample_logits_host
    assert f(logits.ctypes.data, 64, 0.0, 50, 0.9, 0.5, C.byref(tok)) != 0    # temperature
    assert f(logits.ctypes.data, 64, 0.7, 0, 0.9, 0.5, C.byref(tok)) != 0     # the reference's k <= 0 branch draws a uniform-random id
    assert f(logits.ctypes.data, 64, 0.7, 50, 0.0, 0.5, C.byref(tok)) != 0    # and so does p <= 0
    assert f(logits.ctypes.data, 64, 0.7, 50, 0.9, 1.0, C.byref(tok)) != 0    # u outside [0, 1)
    assert f(None, 64, 0.7, 50, 0.9, 0.5, C.byref(tok)) != 0
    # the reference subtracts no maximum before expf: overflow is reported, not sampled from
    big = np.full(64, np.float16(30.0).view(np.uint16), dtype=np.uint16)
    assert f(big.ctypes.data, 64, 0.1, 50, 0.9, 0.5, C.byref(tok)) != 0
    assert b"overflow" in pkg.lib.llmb_last_error()
