"""Tensor-parallel host logic on CPU ranks (gloo, world_size 2): the sharding plan of the loader
and the exchange the kernel performs after o_proj / down_proj, restated with numpy and a gloo
all-reduce.  No GPU, no compute call into the library."""
import ctypes as C
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, shard_path, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from conftest import load_package
    from oracle import oracle_lib as oracle
    pkg = load_package()
    cfg = pkg.CONFIGS["tiny"]
    m = pkg.lib.init_llama3(cfg.n_layers)
    pkg.lib.llama3_set_streaming(m, 0)   # the test slices the payloads held in host memory
    assert pkg.lib.llama3_set_tp(m, rank, world) == 0
    assert pkg.lib.llama3_load_safetensors(m, shard_path.encode()) == 0
    weights = oracle.Weights(cfg, seed=0)

    def window(layer, slot):
        out = (C.c_int * 5)()
        assert pkg.lib.llama3_tensor_shard(m, layer, slot, out) == 0
        return list(out)

    def host(t):
        t = t.contents
        return np.ctypeslib.as_array(C.cast(t.bf16_tensor, C.POINTER(C.c_uint16)), shape=(t.mem_len[0],)).copy()

    ok = True
    lay = m.contents.layers[1].contents
    # column-parallel (split by output rows): every rank holds a block of rows; gathered they are the tensor
    for slot, name in ((7, "self_attn_q_proj"), (5, "self_attn_k_proj"), (2, "mlp_gate_proj")):
        r0, rows, c0, cols, full = window(1, slot)
        full_t = host(getattr(lay, name)).reshape(-1, full)
        mine = torch.from_numpy(full_t[r0:r0 + rows, c0:c0 + cols].astype(np.int32))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ok &= bool(np.array_equal(torch.cat(parts, 0).numpy().astype(np.uint16), full_t))
        ok &= (c0, cols) == (0, full) and rows * world == full_t.shape[0]
    # row-parallel (split by input columns): partial products summed over ranks give the full product
    x = oracle.f16(oracle.synth_fp16(9, 1, cfg.q_rows, std=1.0)).astype(np.float64)
    r0, rows, c0, cols, full = window(1, 6)
    w = oracle.f16(host(lay.self_attn_o_proj)).astype(np.float64).reshape(-1, full)
    ok &= (r0, rows) == (0, cfg.d_model) and cols * world == full
    partial = torch.from_numpy(w[:, c0:c0 + cols] @ x[c0:c0 + cols])
    dist.all_reduce(partial)  # what the step kernel does with peer stores + flags after o_proj
    ok &= bool(np.allclose(partial.numpy(), w @ x, rtol=1e-12, atol=1e-12))
    # replicated tensors are whole on every rank
    ok &= window(-1, 1)[1] == cfg.vocab and window(1, 0)[1] == cfg.d_model
    # lm_head by vocabulary rows: the global argmax is the best of the per-rank bests, lowest index on ties
    r0, rows, _, _, full = window(-1, 2)
    logits = np.round(np.random.default_rng(5).standard_normal(cfg.vocab) * 4).astype(np.float32)  # many ties
    local = logits[r0:r0 + rows]
    best = torch.tensor([float(local.max()), float(r0 + int(local.argmax()))], dtype=torch.float64)
    every = [torch.empty_like(best) for _ in range(world)]
    dist.all_gather(every, best)
    top = max(v[0].item() for v in every)
    pick = min(int(v[1].item()) for v in every if v[0].item() == top)
    ok &= pick == int(logits.argmax())
    pkg.lib.free_llama3(m)
    res = torch.tensor([1 if ok else 0])
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write(str(int(res.item())))
    dist.destroy_process_group()


def test_sharding_plan_and_exchange_on_two_cpu_ranks(tmp_path, tiny_weights):
    shard = tiny_weights.write_safetensors(tmp_path / "tiny.safetensors")
    result = tmp_path / "ok.txt"
    mp.spawn(_rank_main, args=(2, _free_port(), str(shard), str(result)), nprocs=2, join=True)
    assert result.read_text() == "1"


def test_tp_size_must_divide_the_model(pkg, tiny_weights, tmp_path):
    shard = tiny_weights.write_safetensors(tmp_path / "tiny.safetensors")
    m = pkg.lib.init_llama3(pkg.CONFIGS["tiny"].n_layers)
    assert pkg.lib.llama3_set_tp(m, 0, 4) == 0  # 2 KV heads cannot be split four ways
    assert pkg.lib.llama3_load_safetensors(m, str(shard).encode()) == 0
    cfg = pkg.Llama3Config(0, 0, 0, 64, 0, 0, 64, 500000.0, 1e-5)
    pkg.lib.llama3_set_config(m, C.byref(cfg))
    # the check runs before any device work, so the refusal shows without a GPU
    rc = pkg.lib.llama3_to_cuda(m)
    assert rc == pkg.ERR_INVALID and b"tensor parallel size" in pkg.lib.llmb_last_error()
    pkg.lib.free_llama3(m)
