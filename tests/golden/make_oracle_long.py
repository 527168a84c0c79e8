"""Generates tests/golden/oracle_8b_l2_long.npz with the CPU oracle (no GPU needed; minutes of CPU time).

    python tests/golden/make_oracle_long.py [output directory]

The long-context case of the benchmark shapes: the 8B layer shape (two layers, 1024-row embedding table),
a 4096-token prompt and 128 teacher-forced decode steps, i.e. cache rows up to 4224.  One causal pass of the
strict oracle (oracle/llama3_oracle.c) over the 4224 tokens yields the logits of every step.  Kept per step:
the argmax, the 16 largest logits with their ids, every 64th logit; and the residual stream after the
embedding and after each layer at the last prompt row (for the per-layer hidden-state bound).  The pass is
too slow to repeat inside every test run, so its result is committed; the oracle itself is pinned against
the reference binary by the ref_*.npz fixtures.
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

N_PROMPT, N_STEPS, SEED, STRIDE, TOPK = 4096, 128, 0, 64, 16


def main():
    from make_ref_golden import load_configs
    from oracle import oracle_lib as oracle
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    cfg = load_configs()["llama3_8b_l2"]
    weights = oracle.Weights(cfg, seed=SEED, keep_file=False)
    tokens = oracle.synth_tokens(SEED, N_PROMPT + N_STEPS, cfg.embed_rows)
    t0 = time.time()
    logits, hidden = oracle.forward(weights, tokens, first_logit_row=N_PROMPT - 1, want_hidden=True)
    print("oracle pass over %d tokens: %.0f s" % (len(tokens), time.time() - t0))
    vals = logits.view(np.float16).astype(np.float32)
    order = np.argsort(-vals, axis=1, kind="stable")[:, :TOPK]
    out = os.path.join(out_dir, "oracle_8b_l2_long.npz")
    np.savez_compressed(
        out, tokens=tokens.astype(np.int32), n_prompt=N_PROMPT, seed=SEED, stride=STRIDE,
        argmax=vals.argmax(axis=1).astype(np.int32), topk_idx=order.astype(np.int32),
        topk_bits=np.take_along_axis(logits, order, axis=1), strided_bits=logits[:, ::STRIDE],
        hidden_last_prompt_row=hidden[:, N_PROMPT - 1, :].copy(), config=cfg.name)
    print("wrote", out)


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    main()
