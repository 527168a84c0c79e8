"""Pins against the reference engine itself: tests/golden/ref_8b_l2.npz holds FP16 logits the
reference binary produced on a B200 (tests/golden/make_ref_golden.py).  The CPU oracle is checked
here without a GPU; the CUDA engine is checked against the same fixture on the GPU."""
import hashlib
import os

import numpy as np
import pytest

from conftest import ROOT

FIXTURE = os.path.join(ROOT, "tests", "golden", "ref_8b_l2.npz")
# the same bound the task states for engine-vs-reference logits
LOGIT_TOL = 2e-2


def load_fixture():
    if not os.path.exists(FIXTURE):
        pytest.skip("golden fixture not generated yet")
    return np.load(FIXTURE)


def compare(fx, logits_rows, oracle, what):
    stride = int(fx["stride"])
    exact = 0
    worst = 0.0
    for s, row in enumerate(logits_rows):
        sub = oracle.f16(row[::stride]) - oracle.f16(fx["strided_bits"][s])
        top = oracle.f16(row[fx["topk_idx"][s]]) - oracle.f16(fx["topk_bits"][s])
        worst = max(worst, float(np.abs(sub).max()), float(np.abs(top).max()))
        exact += hashlib.sha256(np.ascontiguousarray(row).tobytes()).hexdigest() == str(fx["sha256"][s])
        got_arg = int(oracle.lib().oracle_argmax_fp16(np.ascontiguousarray(row).ctypes.data, len(row)))
        if got_arg != int(fx["argmax"][s]):
            gap = oracle.f16(fx["topk_bits"][s][:2])
            assert gap[0] - gap[1] <= 2 * worst + 1e-3, "%s: argmax differs from the reference at step %d" % (what, s)
    assert worst <= LOGIT_TOL, "%s: logits differ from the reference by %g" % (what, worst)
    print("%s vs reference: worst |dlogit| %.4g, bit-identical rows %d/%d" % (what, worst, exact, len(logits_rows)))
    return worst, exact


def test_oracle_matches_reference_binary(pkg, oracle):
    fx = load_fixture()
    cfg = pkg.CONFIGS[str(fx["config"])]
    w = oracle.Weights(cfg, seed=int(fx["seed"]), keep_file=False)
    logits, _ = oracle.forward(w, fx["tokens"], first_logit_row=int(fx["n_prompt"]) - 1)
    compare(fx, logits[: len(fx["argmax"])], oracle, "oracle")


@pytest.mark.gpu
@pytest.mark.parametrize("step_kernel", [1, 0])
def test_engine_matches_reference_binary(pkg, oracle, step_kernel):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    fx = load_fixture()
    cfg = pkg.CONFIGS[str(fx["config"])]
    model = pkg.Model.synthetic(cfg, seed=int(fx["seed"]), max_seq=256)
    cache = pkg.Cache(model)
    cache.set_options(step_kernel=step_kernel)
    rows = []
    n_prompt = int(fx["n_prompt"])
    for s in range(len(fx["argmax"])):
        cache.infer(fx["tokens"][: n_prompt + s])
        rows.append(cache.logits())
    compare(fx, rows, oracle, "engine (step kernel)" if step_kernel else "engine (per-op kernels)")
    cache.close()
    model.close()
