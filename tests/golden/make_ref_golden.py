"""Generates tests/golden/ref_8b_l2.npz by running the reference engine itself on a B200.

    python tests/golden/make_ref_golden.py [out.npz]

The reference (oracle/_ref/ref_harness: its own sources + the one-character compile fix at
inference.cu:673) can only run LLaMA3-8B layer shapes, but the layer count is a parameter
(llama3.cuh:58), so the pin uses the 8B shape with two layers and a 1024-row embedding table:
seeded BF16 weights written as two safetensors shards, a 16-token prompt and 8 teacher-forced
steps.  For every step the fixture keeps: the argmax, the 16 largest logits with their ids,
every 16th logit, and the SHA-256 of the full FP16 row.
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

N_PROMPT, N_STEPS, SEED, STRIDE, TOPK = 16, 8, 0, 16, 16


def main():
    import __graft_entry__ as ge
    from oracle import oracle_lib as oracle
    pkg = ge.load_package()
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "gpurun_out", "ref_8b_l2.npz")
    cfg = pkg.CONFIGS["llama3_8b_l2"]
    weights = oracle.Weights(cfg, seed=SEED, keep_fp16=False)
    tokens = oracle.synth_tokens(SEED, N_PROMPT + N_STEPS, cfg.embed_rows)
    with tempfile.TemporaryDirectory() as tmp:
        names = list(weights.file)
        shards = [weights.write_safetensors(os.path.join(tmp, "model-00001-of-00002.safetensors"), names[:10]),
                  weights.write_safetensors(os.path.join(tmp, "model-00002-of-00002.safetensors"), names[10:])]
        tok_path = os.path.join(tmp, "tokens.i32")
        tokens.astype(np.int32).tofile(tok_path)
        logit_path = os.path.join(tmp, "logits.f16")
        cmd = [oracle.REF_HARNESS, str(cfg.n_layers), tok_path, str(N_PROMPT), str(N_STEPS), logit_path] + shards
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.exit("reference harness failed (%d): %s" % (r.returncode, r.stderr[-500:]))
        info = json.loads(r.stdout[r.stdout.rindex('{"n_layers"'):])  # the reference prints ANSI colour codes before it
        logits = np.fromfile(logit_path, dtype=np.uint16).reshape(N_STEPS, cfg.vocab)
    vals = logits.view(np.float16).astype(np.float32)
    order = np.argsort(-vals, axis=1, kind="stable")[:, :TOPK]
    os.makedirs(os.path.dirname(out), exist_ok=True)
    np.savez_compressed(
        out, tokens=tokens.astype(np.int32), n_prompt=N_PROMPT, seed=SEED, stride=STRIDE,
        argmax=vals.argmax(axis=1).astype(np.int32), topk_idx=order.astype(np.int32),
        topk_bits=np.take_along_axis(logits, order, axis=1), strided_bits=logits[:, ::STRIDE],
        sha256=np.array([hashlib.sha256(row.tobytes()).hexdigest() for row in logits]),
        step_s=np.array(info["step_s"]), config=cfg.name)
    print("wrote %s; reference step seconds %s" % (out, info["step_s"]))


if __name__ == "__main__":
    main()
