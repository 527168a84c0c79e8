"""Batched decode (several sequences, one new token each per step): the batched kernels through the C-ABI
against their single-sequence forms, and the engine's batch path against the CPU oracle, teacher-forced, one
independent oracle sequence per batch row.  Tolerances as everywhere: logits within 2e-2, argmax identical
unless the oracle's own top-2 gap is within twice the measured logit error."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from gpu_util import dev, host_u16  # noqa: E402

LOGIT_TOL = 2e-2


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


@pytest.mark.parametrize("lens,n_splits,split_len", [([1, 130, 257, 640, 512], 4, 256), ([640] * 7, 10, 64), ([3, 2, 1], 1, 640), ([577], 3, 200),
                                                     ([64, 65, 128, 129, 1, 640, 600, 77, 300], 3, 256)])
def test_attn_decode_batch_equals_single_sequence_calls(pkg, oracle, lens, n_splits, split_len):
    """Several sequences share one wave of CTAs, each taking an equal run of 64-row tiles across the (sequence, KV head)
    pairs; a pair's pieces therefore fall elsewhere than the fixed splits of the single-sequence call, and the two
    differ by the order of the FP32 sums: at most one FP16 step.  Two launches of the batch give identical bits.  A batch
    of one sequence keeps the fixed splits (here 200 rows, not a multiple of the 64-row tile) and fetches its tiles as
    boxes through the tensor maps all the same."""
    nq, nkv, hd, max_pos, n_seqs = 32, 8, 128, 640, len(lens)
    q = oracle.synth_fp16(1, 1, n_seqs * nq * hd, std=1.0)
    kc = oracle.synth_fp16(1, 2, n_seqs * max_pos * nkv * hd, std=1.0)
    vc = oracle.synth_fp16(1, 3, n_seqs * max_pos * nkv * hd, std=1.0)
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device="cuda")
    out = torch.zeros(n_seqs * nq * hd, dtype=torch.int16, device="cuda")
    scratch = torch.zeros(pkg.lib.llmb_attn_decode_batch_scratch_bytes(n_seqs, nq, nkv, hd, n_splits), dtype=torch.uint8, device="cuda")
    rc = pkg.lib.llmb_attn_decode_batch(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), pos.data_ptr(), n_seqs, max_pos, nq, nkv, hd,
                                        n_splits, split_len, out.data_ptr(), scratch.data_ptr(), 0, None)
    assert rc == 0, pkg.lib.llmb_last_error()
    got = host_u16(out).reshape(n_seqs, nq * hd)
    out.zero_()
    rc = pkg.lib.llmb_attn_decode_batch(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), pos.data_ptr(), n_seqs, max_pos, nq, nkv, hd,
                                        n_splits, split_len, out.data_ptr(), scratch.data_ptr(), 0, None)
    assert rc == 0, pkg.lib.llmb_last_error()
    assert np.array_equal(host_u16(out).reshape(n_seqs, nq * hd), got), "second launch differs (arrival counters, summation order)"
    one = torch.zeros(nq * hd, dtype=torch.int16, device="cuda")
    s1 = torch.zeros(pkg.lib.llmb_attn_decode_scratch_bytes(nq, nkv, hd, n_splits), dtype=torch.uint8, device="cuda")
    for b in range(n_seqs):
        off = b * max_pos * nkv * hd * 2
        rc = pkg.lib.llmb_attn_decode(dq.data_ptr() + b * nq * hd * 2, dk.data_ptr() + off, dv.data_ptr() + off,
                                      pos.data_ptr() + 4 * b, nq, nkv, hd, n_splits, split_len, one.data_ptr(), s1.data_ptr(), 0, None)
        assert rc == 0, pkg.lib.llmb_last_error()
        a = host_u16(one).view(np.float16).astype(np.float64)
        g = got[b].view(np.float16).astype(np.float64)
        assert np.all(np.abs(a - g) <= np.maximum(np.abs(a), 2.0 ** -14) * 2.0 ** -10), (b, np.abs(a - g).max())
        assert (a != g).mean() < 0.05, (b, (a != g).mean())


def test_argmax_rows(pkg, oracle):
    rows, n = 7, 4096
    bits = oracle.synth_fp16(5, 9, rows * n, std=1.0).reshape(rows, n).copy()
    bits[3, 100] = bits[3, 2000] = 0x7BFF   # a tie of the largest finite value: the first index wins
    d = dev(bits.reshape(-1))
    tok = torch.zeros(rows, dtype=torch.int32, device="cuda")
    pos = torch.arange(rows, dtype=torch.int32, device="cuda")
    hist = torch.full((rows, 16), -1, dtype=torch.int32, device="cuda")
    rc = pkg.lib.llmb_argmax_rows_f16(d.data_ptr(), n, rows, tok.data_ptr(), pos.data_ptr(), hist.data_ptr(), 16, 0, None)
    assert rc == 0, pkg.lib.llmb_last_error()
    torch.cuda.synchronize()
    want = [int(oracle.lib().oracle_argmax_fp16(bits[r].ctypes.data, n)) for r in range(rows)]
    assert tok.cpu().tolist() == want and want[3] == 100
    assert pos.cpu().tolist() == list(range(1, rows + 1))
    h = hist.cpu().numpy()
    for r in range(rows):
        assert h[r, r + 1] == want[r] and (np.delete(h[r], r + 1) == -1).all()


def batch_teacher_forced(pkg, oracle, cfg, weights, n_seqs, n_prompt, n_steps, max_seq=64):
    vocab_ids = cfg.embed_rows or cfg.vocab
    # one independent token stream per sequence
    seqs = np.stack([oracle.synth_tokens(100 + b, n_prompt + n_steps, vocab_ids) for b in range(n_seqs)])
    ref = [oracle.forward(weights, seqs[b], first_logit_row=n_prompt - 1)[0] for b in range(n_seqs)]
    model = pkg.Model.synthetic(cfg, seed=weights.seed, max_seq=max_seq)
    cache = pkg.Cache(model)
    cache.batch_init(n_seqs)
    cache.batch_prefill(seqs[:, :n_prompt])
    worst, ties = 0.0, 0
    for step in range(n_steps + 1):
        feed = None if step == 0 else seqs[:, n_prompt + step - 1]   # step 0 consumes the pending last prompt token
        nxt, logits = cache.batch_step(feed)
        for b in range(n_seqs):
            want = ref[b][step]
            diff = float(np.abs(oracle.f16(logits[b]) - oracle.f16(want)).max())
            worst = max(worst, diff)
            want_tok = int(oracle.lib().oracle_argmax_fp16(want.ctypes.data, len(want)))
            assert int(nxt[b]) == int(oracle.lib().oracle_argmax_fp16(logits[b].ctypes.data, len(want)))
            if int(nxt[b]) != want_tok:
                top2 = np.sort(oracle.f16(want))[-2:]
                assert top2[1] - top2[0] <= 2 * diff + 1e-3, "argmax differs without a tie (sequence %d, step %d)" % (b, step)
                ties += 1
    assert worst <= LOGIT_TOL, worst
    cache.close()
    model.close()
    return worst, ties


@pytest.mark.parametrize("n_seqs", [2, 32])
def test_tiny_batch_teacher_forced_parity(pkg, oracle, tiny_weights, n_seqs):
    worst, ties = batch_teacher_forced(pkg, oracle, pkg.CONFIGS["tiny"], tiny_weights, n_seqs, 20, 6)
    print("tiny batch %d: worst |dlogit| %.4g, ties %d" % (n_seqs, worst, ties))


@pytest.mark.parametrize("n_seqs,n_prompt,n_steps", [(2, 20, 4), (32, 9, 3)])
def test_8b_layer_shapes_batch_teacher_forced_parity(pkg, oracle, weights_8b_l2, n_seqs, n_prompt, n_steps):
    worst, ties = batch_teacher_forced(pkg, oracle, pkg.CONFIGS["llama3_8b_l2"], weights_8b_l2, n_seqs, n_prompt, n_steps)
    print("8b_l2 batch %d: worst |dlogit| %.4g, ties %d" % (n_seqs, worst, ties))


def test_batch_greedy_equals_stepping_and_sequences_do_not_mix(pkg, oracle):
    cfg = pkg.CONFIGS["tiny"]
    n_seqs, n_prompt, n_new = 6, 40, 12
    prompts = np.stack([oracle.synth_tokens(200 + b, n_prompt, cfg.vocab) for b in range(n_seqs)])
    prompts[3] = prompts[1]   # two equal sequences must produce equal tokens whatever their neighbours do
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=128)
    cache = pkg.Cache(model)
    cache.batch_init(n_seqs)
    cache.batch_prefill(prompts)
    stepped = []
    for _ in range(n_new):
        nxt, _ = cache.batch_step(None, want_logits=False)
        stepped.append(nxt.copy())
    stepped = np.stack(stepped, axis=1)
    cache.batch_prefill(prompts)                      # start over: same prompts, device-resident loop
    greedy, ms = cache.batch_greedy(n_new)
    assert ms > 0 and np.array_equal(greedy, stepped)
    assert np.array_equal(greedy[1], greedy[3])
    # the single-sequence engine on the same cache object is untouched by the batch state
    toks, _, _ = cache.greedy(prompts[0].tolist(), 4)
    assert len(toks) == 4
    cache.close()
    model.close()
