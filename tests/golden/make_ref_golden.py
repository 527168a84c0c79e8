"""Generates the tests/golden/ref_*.npz fixtures by running the reference engine itself on a B200.

    python tests/golden/make_ref_golden.py [l2|l32|all] [output directory]

The reference (oracle/_ref/ref_harness: its own sources + the one-character compile fix at
inference.cu:673) can only run LLaMA3-8B layer shapes, but the layer count is a parameter
(llama3.cuh:58).  Seeded BF16 weights are written as safetensors shards, the harness drives the
reference's inference() teacher-forced and dumps the FP16 logits it leaves in Cache->h_token_probdist
(inference.cu:1021-1025).

  ref_8b_l2.npz         8B layer shape, 2 layers, 1024-row embedding table; 16-token prompt + 8 steps
  ref_8b_l32.npz        the full 8B model (32 layers); the benchmark's 128-token prompt + 64 steps
  ref_8b_l32_short.npz  the full 8B model; 16-token prompt + 4 steps (short enough for the CPU oracle
                        to be checked at full depth in seconds)

For every step a fixture keeps: the argmax, the 16 largest logits with their ids (so also the
reference's own top-2 gap), every `stride`-th logit, and the SHA-256 of the full FP16 row.
Without an output directory the fixtures are written next to this script.
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

SEED, TOPK = 0, 16
# name -> (config, shards, [(fixture, n_prompt, n_steps, stride)])
JOBS = {
    "l2": ("llama3_8b_l2", 2, [("ref_8b_l2.npz", 16, 8, 16)]),
    "l32": ("llama3_8b", 4, [("ref_8b_l32.npz", 128, 64, 64), ("ref_8b_l32_short.npz", 16, 4, 64)]),
}


def load_configs():
    import importlib.util
    spec = importlib.util.spec_from_file_location("llm_cu_b200_configs", os.path.join(ROOT, "llm.cu_b200", "configs.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod.CONFIGS


def run_job(oracle, cfg, n_shards, fixtures, out_dir):
    weights = oracle.Weights(cfg, seed=SEED, keep_fp16=False)
    vocab_ids = cfg.embed_rows or cfg.vocab
    with tempfile.TemporaryDirectory() as tmp:
        names = list(weights.file)
        per = (len(names) + n_shards - 1) // n_shards
        shards = []
        for i in range(n_shards):
            part = names[i * per:(i + 1) * per]
            if part:
                shards.append(weights.write_safetensors(
                    os.path.join(tmp, "model-%05d-of-%05d.safetensors" % (i + 1, n_shards)), part))
        del weights
        for fixture, n_prompt, n_steps, stride in fixtures:
            tokens = oracle.synth_tokens(SEED, n_prompt + n_steps, vocab_ids)
            tok_path = os.path.join(tmp, "tokens.i32")
            tokens.astype(np.int32).tofile(tok_path)
            logit_path = os.path.join(tmp, "logits.f16")
            cmd = [oracle.REF_HARNESS, str(cfg.n_layers), tok_path, str(n_prompt), str(n_steps), logit_path] + shards
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.exit("reference harness failed (%d): %s" % (r.returncode, r.stderr[-500:]))
            info = json.loads(r.stdout[r.stdout.rindex('{"n_layers"'):])  # the reference prints ANSI colour codes before it
            logits = np.fromfile(logit_path, dtype=np.uint16).reshape(n_steps, cfg.vocab)
            vals = logits.view(np.float16).astype(np.float32)
            order = np.argsort(-vals, axis=1, kind="stable")[:, :TOPK]
            out = os.path.join(out_dir, fixture)
            np.savez_compressed(
                out, tokens=tokens.astype(np.int32), n_prompt=n_prompt, seed=SEED, stride=stride,
                argmax=vals.argmax(axis=1).astype(np.int32), topk_idx=order.astype(np.int32),
                topk_bits=np.take_along_axis(logits, order, axis=1), strided_bits=logits[:, ::stride],
                sha256=np.array([hashlib.sha256(row.tobytes()).hexdigest() for row in logits]),
                step_s=np.array(info["step_s"]), config=cfg.name)
            print("wrote %s; reference seconds per step: first %.3f last %.3f, load %.1f s" % (
                out, info["step_s"][0], info["step_s"][-1], info["load_s"]), flush=True)


def main():
    from oracle import oracle_lib as oracle
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    out_dir = sys.argv[2] if len(sys.argv) > 2 else HERE
    os.makedirs(out_dir, exist_ok=True)
    configs = load_configs()
    for name in (JOBS if which == "all" else [which]):
        cfg_name, n_shards, fixtures = JOBS[name]
        run_job(oracle, configs[cfg_name], n_shards, fixtures, out_dir)


if __name__ == "__main__":
    main()
