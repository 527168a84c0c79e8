"""The device sampler (llmb_sample_logits) against the oracle's statement-by-statement restatement of the
reference's sample_next_token chain (src/inference/inference.cu:1030-1161): the same token on every case of
the host sampler's test matrix that the device kernel takes (it orders at most 1024 entries)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from gpu_util import dev  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def chain_f32(logits_bits, temperature, top_k, top_p, u, slack_ulps):
    """The reference's chain (inference.cu:1041-1160) in numpy float32, with the comparison `cumulative >= p`
    shifted by `slack_ulps` FP32 ulps of p (negative: reached sooner)."""
    f = np.float32
    x = logits_bits.view(np.float16).astype(np.float32)
    t = np.exp(x / f(temperature), dtype=np.float32)
    cumsum = np.cumsum(t, dtype=np.float32)[-1]
    prob = t / cumsum
    order = np.lexsort((np.arange(len(prob)), -prob))
    pr = prob[order].copy()
    k = min(top_k, len(pr))
    ssum = f(0)
    for i in range(k):
        ssum = f(ssum + pr[i])
    pr[:k] = pr[:k] / ssum
    p = f(min(top_p, 1.0))
    thr = f(p + f(slack_ulps) * np.spacing(p))
    cumulative, cutoff = f(0), len(pr)
    for i in range(len(pr)):
        cumulative = f(cumulative + pr[i])
        if cumulative >= thr:
            cutoff = i
            break
    cutoff = min(cutoff, len(pr) - 1)
    pr[:cutoff + 1] = pr[:cutoff + 1] / cumulative
    run = f(0)
    for i in range(cutoff + 1):
        run = f(run + pr[i])
        if f(u) < run:
            return int(order[i])
    return int(order[0])


def device_sample(pkg, d_logits, vocab, scratch, tok, temperature, top_k, top_p, seed, draw):
    rc = pkg.lib.llmb_sample_logits(d_logits.data_ptr(), vocab, temperature, top_k, top_p, seed, draw, scratch.data_ptr(),
                                    tok.data_ptr(), None, None, 0, 0, None)
    if rc != 0:
        return rc, None, None
    torch.cuda.synchronize()
    return 0, int(tok.item()), int(scratch[:4].view(torch.int32).item())


@pytest.mark.parametrize("vocab,std", [(4096, 3.0), (128256, 2.0), (1000, 0.5), (50, 4.0), (7, 1.0)])
def test_device_sampler_matches_reference_restatement(pkg, oracle, vocab, std):
    logits = oracle.synth_fp16(4000 + vocab, 9, vocab, std=std)
    d_logits = dev(logits)
    scratch = torch.zeros(pkg.lib.llmb_sample_scratch_bytes(vocab), dtype=torch.uint8, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    checked = 0
    for temperature, top_k, top_p in [(0.7, 50, 0.9), (1.0, 50, 0.9), (0.7, 5, 0.5), (0.3, 50, 1.0), (1.5, 1000, 0.95),
                                      (0.7, 1, 0.9), (0.7, 10 ** 6, 1.0), (0.7, 50, 2.0)]:
        for draw in range(8):
            seed = 17
            u = float(oracle.lib().oracle_sampler_uniform(seed, draw))
            rc, got, result = device_sample(pkg, d_logits, vocab, scratch, tok, temperature, top_k, top_p, seed, draw)
            if min(top_k, vocab) > 1024:
                assert rc == pkg.ERR_UNSUPPORTED
                continue
            assert rc == 0, pkg.lib.llmb_last_error()
            want = int(oracle.lib().oracle_sample(logits.ctypes.data, vocab, temperature, top_k, top_p, u))
            if result == 2:      # prefix longer than the kernel orders: reported, not guessed
                assert got == -1
                continue
            accept = {want}
            if top_p >= 1.0:
                # top_p = 1: whether the renormalised top-k mass reaches 1.0 exactly or stops an FP32 ulp short
                # decides if the prefix takes one more entry (inference.cu:1131-1136).  The device's sum of the
                # t_i is a tree and its expf is CUDA's, so it may land on the other side of that ulp: both
                # outcomes of the comparison are accepted there, each with the reference's arithmetic.
                accept |= {chain_f32(logits, temperature, top_k, 1.0, u, slack) for slack in (-4, 4)}
            assert result == 0 and got in accept, (vocab, temperature, top_k, top_p, draw, got, accept)
            checked += 1
    assert checked >= 40


def test_device_sampler_ties_overflow_and_history(pkg, oracle):
    logits = np.full(64, np.float16(1.0).view(np.uint16), dtype=np.uint16)
    logits[10] = logits[40] = np.float16(3.0).view(np.uint16)
    d = dev(logits)
    scratch = torch.zeros(pkg.lib.llmb_sample_scratch_bytes(64), dtype=torch.uint8, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    picks = set()
    for draw in range(40):   # two equal heads: index 10 comes first in the order, both get drawn
        u = float(oracle.lib().oracle_sampler_uniform(3, draw))
        rc, got, result = device_sample(pkg, d, 64, scratch, tok, 1.0, 2, 1.0, 3, draw)
        assert rc == 0 and result == 0
        assert got == int(oracle.lib().oracle_sample(logits.ctypes.data, 64, 1.0, 2, 1.0, u))
        picks.add(got)
    assert picks == {10, 40}
    # no maximum is subtracted (as in the reference): overflow is reported, nothing is sampled
    big = dev(np.full(64, np.float16(30.0).view(np.uint16), dtype=np.uint16))
    rc, got, result = device_sample(pkg, big, 64, scratch, tok, 0.1, 50, 0.9, 0, 0)
    assert rc == 0 and got == -1 and result == 1
    # bookkeeping: the token is written at history[*pos]
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    hist = torch.full((16,), -1, dtype=torch.int32, device="cuda")
    rc = pkg.lib.llmb_sample_logits(d.data_ptr(), 64, 1.0, 2, 1.0, 3, 0, scratch.data_ptr(), tok.data_ptr(), pos.data_ptr(),
                                    hist.data_ptr(), 16, 0, None)
    assert rc == 0
    torch.cuda.synchronize()
    h = hist.cpu().tolist()
    assert h[5] == int(tok.item()) and h.count(-1) == 15 and int(pos.item()) == 5


def test_engine_device_sampler_continues_from_the_sampled_token(pkg, oracle, tiny_weights):
    cfg = pkg.CONFIGS["tiny"]
    seq = oracle.synth_tokens(0, 12, cfg.vocab).tolist()
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=64)
    cache = pkg.Cache(model)
    for draw in range(4):
        greedy = cache.infer(seq)
        logits = cache.logits()
        tok = cache.sample_device(temperature=0.7, top_k=50, top_p=0.9, seed=3, draw=draw)
        u = float(oracle.lib().oracle_sampler_uniform(3, draw))
        assert tok == int(oracle.lib().oracle_sample(logits.ctypes.data, cfg.vocab, 0.7, 50, 0.9, u))
        assert tok == cache.sample(temperature=0.7, top_k=50, top_p=0.9, seed=3, draw=draw)   # host chain, same token
        assert cache.sample_device(temperature=0.7, top_k=1, top_p=0.9, seed=3, draw=draw) == greedy
        cache.sample_device(temperature=0.7, top_k=50, top_p=0.9, seed=3, draw=draw)          # leave the sampled one in place
        seq.append(tok)
    # the sampled token sits in the device history: a device-resident continuation starts from it
    more, _ = cache.continue_greedy(3)
    cache.reset()
    cache.set_prefill(False)                     # the same decode path, token by token: identical arithmetic
    assert cache.infer(seq) == more[0]           # the first continued token is the greedy successor of the sampled one
    cache.close()
    model.close()
