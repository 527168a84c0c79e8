"""The drop-in boundary exercised from C: a driver in the shape of the reference's src/main.cu:61-126 is
compiled with gcc (plain C, no CUDA headers) against include/llama3.h and linked to libllm_b200.so.
Without a GPU the test checks that it compiles and links; on a GPU it runs it on tiny synthetic shards
and compares the generated ids with the ctypes path."""
import os
import shutil
import subprocess

import pytest

from conftest import ROOT

SRC = os.path.join(ROOT, "tests", "c_driver", "main_like.c")


def build_driver(pkg, out_dir):
    exe = os.path.join(str(out_dir), "main_like")
    lib_dir = os.path.dirname(pkg.LIB_PATH)
    cmd = [shutil.which("gcc") or "gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L", lib_dir, "-lllm_b200", "-Wl,-rpath," + lib_dir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_c_driver_compiles_and_links(pkg, tmp_path):
    exe = build_driver(pkg, tmp_path)
    assert os.path.exists(exe)
    # usage error path: no device is touched
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 2 and "usage" in r.stderr


@pytest.mark.gpu
def test_c_driver_generates_the_same_tokens_as_the_binding(pkg, oracle, tiny_weights, tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    cfg = pkg.CONFIGS["tiny"]
    exe = build_driver(pkg, tmp_path)
    names = list(tiny_weights.file)
    shards = [tiny_weights.write_safetensors(tmp_path / "model-00001-of-00002.safetensors", names[:9]),
              tiny_weights.write_safetensors(tmp_path / "model-00002-of-00002.safetensors", names[9:])]
    prompt = oracle.synth_tokens(0, 20, cfg.vocab).tolist()
    n_new = 6
    r = subprocess.run([exe, str(cfg.n_layers), str(cfg.head_dim), "64", str(n_new), ",".join(map(str, prompt))] +
                       [str(s) for s in shards], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr + r.stdout
    got = [int(x) for x in r.stdout.split()[-n_new:]]
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=64)
    cache = pkg.Cache(model)
    want, _, _ = cache.greedy(prompt, n_new)
    cache.close()
    model.close()
    assert got == want
