"""Tensor-parallel decode on real GPUs (needs at least two): one process per GPU, exchange blocks
shared through CUDA IPC, parity against the CPU oracle teacher-forced, and agreement with the
single-GPU engine.  Skipped on a single-GPU box; the CPU-rank tests in test_tp_cpu.py cover the
host logic there."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

LOGIT_TOL = 2e-2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, cfg_name, n_prompt, n_steps, result_path, shard_path=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from conftest import load_package
    from oracle import oracle_lib as oracle
    pkg = load_package()
    cfg = pkg.CONFIGS[cfg_name]
    vocab_ids = cfg.embed_rows or cfg.vocab
    tokens = oracle.synth_tokens(0, n_prompt + n_steps, vocab_ids)
    if shard_path:
        # the streaming loader under tensor parallelism: every rank reads only its windows of the shard file
        # (whole rows for q/k/v, gate/up, lm_head; a slice of every row for o_proj and down_proj)
        model = pkg.Model.from_safetensors(cfg, [shard_path], max_seq=256, tp_rank=rank, tp_size=world)
        st = model.upload_stats()
        assert st["bytes_read"] == st["bytes_uploaded"] and st["host_staging_bytes"] <= 2 * (32 << 20)
        full = 2 * (cfg.matmul_params() + 2 * cfg.vocab * cfg.d_model)
        assert st["bytes_read"] < 0.8 * full, st   # a rank does not read the other rank's shards
    else:
        model = pkg.Model.synthetic(cfg, seed=0, max_seq=256, tp_rank=rank, tp_size=world)
    cache = pkg.Cache(model)
    cache.tp_connect()
    ok, worst = True, 0.0
    if rank == 0:
        weights = oracle.Weights(cfg, seed=0, keep_file=False)
        ref_logits, _ = oracle.forward(weights, tokens, first_logit_row=n_prompt - 1)
    # The ranks wait for each other inside the kernel with a bounded spin (a few seconds): they must
    # enter a step together, so the seconds rank 0 just spent in the oracle are levelled out here.
    dist.barrier()
    for step in range(n_steps + 1):
        nxt = cache.infer(tokens[: n_prompt + step])
        mine = torch.from_numpy(cache.logits().astype(np.int32))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        every = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(every, torch.tensor([nxt], dtype=torch.int64))
        ok &= len({int(t.item()) for t in every}) == 1  # every rank picked the same token
        if rank == 0:
            got = torch.cat(parts).numpy().astype(np.uint16)
            want = ref_logits[step]
            diff = float(np.abs(oracle.f16(got) - oracle.f16(want)).max())
            worst = max(worst, diff)
            want_tok = int(oracle.lib().oracle_argmax_fp16(want.ctypes.data, len(want)))
            if nxt != want_tok:
                top2 = np.sort(oracle.f16(want))[-2:]
                ok &= bool(top2[1] - top2[0] <= 2 * diff + 1e-3)
            ok &= nxt == int(oracle.lib().oracle_argmax_fp16(got.ctypes.data, len(got)))
    # a long prompt fed without logits: the ranks drift apart here if anything lets them
    long_prompt = oracle.synth_tokens(7, 150, vocab_ids).tolist()
    cache.reset()
    dist.barrier()
    cache.greedy(long_prompt, 3)
    cache.reset()
    dist.barrier()
    toks, _, _ = cache.greedy(tokens[:n_prompt].tolist(), 6)
    st = __import__("ctypes").c_int(0)
    pkg.lib.llmb_device_status(__import__("ctypes").byref(st))
    ok &= st.value == 0
    flag = torch.tensor([1 if (ok and worst <= LOGIT_TOL) else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write("%d %.5g %s" % (int(flag.item()), worst, toks))
    cache.close()
    model.close()
    dist.destroy_process_group()


# n_prompt 16: every prompt token through the whole-step kernel; 45: the prompt as blocks of 32 rows through the
# weight-streaming projections with the all-reduce fused as peer stores, then the whole-step kernel
@pytest.mark.parametrize("cfg_name,world,n_prompt", [("tiny", 2, 16), ("llama3_8b_l2", 2, 16), ("llama3_8b_l2", 4, 16),
                                                     ("llama3_8b_l2", 8, 16), ("llama3_70b_l2", 2, 16), ("llama3_70b_l2", 8, 16),
                                                     ("tiny", 2, 45), ("llama3_8b_l2", 2, 45), ("llama3_8b_l2", 8, 45)])
def test_tensor_parallel_decode_matches_oracle(cfg_name, world, n_prompt, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    result = tmp_path / "r.txt"
    mp.spawn(_rank_main, args=(world, _free_port(), cfg_name, n_prompt, 6, str(result)), nprocs=world, join=True)
    status, worst, toks = result.read_text().split(" ", 2)
    print("TP=%d %s: worst |dlogit| %s, greedy %s" % (world, cfg_name, worst, toks))
    assert status == "1", "worst |dlogit| %s" % worst


def test_tensor_parallel_streaming_load_from_a_shard_file(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from conftest import load_package
    from oracle import oracle_lib as oracle
    pkg = load_package()
    shard = oracle.Weights(pkg.CONFIGS["tiny"], seed=0).write_safetensors(str(tmp_path / "model.safetensors"))
    result = tmp_path / "r.txt"
    mp.spawn(_rank_main, args=(2, _free_port(), "tiny", 16, 6, str(result), shard), nprocs=2, join=True)
    status, worst, toks = result.read_text().split(" ", 2)
    assert status == "1", "worst |dlogit| %s" % worst


def _rank_batch(rank, world, port, cfg_name, n_seqs, n_prompt, n_steps, result_path):
    """Batched decode under tensor parallelism: every rank feeds the same tokens; rank 0 puts the ranks' vocabulary
    slices together and compares every sequence with its own oracle run."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from conftest import load_package
    from oracle import oracle_lib as oracle
    pkg = load_package()
    cfg = pkg.CONFIGS[cfg_name]
    vocab_ids = cfg.embed_rows or cfg.vocab
    seqs = np.stack([oracle.synth_tokens(100 + b, n_prompt + n_steps, vocab_ids) for b in range(n_seqs)])
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=128, tp_rank=rank, tp_size=world)
    cache = pkg.Cache(model)
    cache.tp_connect()
    ref = None
    if rank == 0:
        weights = oracle.Weights(cfg, seed=0, keep_file=False)
        ref = [oracle.forward(weights, seqs[b], first_logit_row=n_prompt - 1)[0] for b in range(n_seqs)]
    dist.barrier()
    cache.batch_init(n_seqs)
    cache.batch_prefill(seqs[:, :n_prompt])
    ok, worst = True, 0.0
    for step in range(n_steps + 1):
        feed = None if step == 0 else seqs[:, n_prompt + step - 1]
        dist.barrier()   # rank 0 spends seconds checking 32 rows of logits: the ranks must enter a step together
        nxt, mine = cache.batch_step(feed)
        parts = [torch.empty(mine.shape, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine.astype(np.int32)))
        toks = [torch.empty(n_seqs, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(toks, torch.from_numpy(nxt.astype(np.int32)))
        ok &= all(torch.equal(toks[0], t) for t in toks)   # every rank picked the same tokens
        if rank == 0:
            logits = torch.cat(parts, dim=1).numpy().astype(np.uint16)
            for b in range(n_seqs):
                want = ref[b][step]
                diff = float(np.abs(oracle.f16(logits[b]) - oracle.f16(want)).max())
                worst = max(worst, diff)
                want_tok = int(oracle.lib().oracle_argmax_fp16(want.ctypes.data, len(want)))
                ok &= int(nxt[b]) == int(oracle.lib().oracle_argmax_fp16(np.ascontiguousarray(logits[b]).ctypes.data, len(want)))
                if int(nxt[b]) != want_tok:
                    top2 = np.sort(oracle.f16(want))[-2:]
                    ok &= bool(top2[1] - top2[0] <= 2 * diff + 1e-3)
    # device-resident greedy run: the sampled tokens are fed back on every rank alike
    dist.barrier()   # rank 0 arrives seconds late from its checks; the prefill exchanges data between the ranks
    cache.batch_prefill(seqs[:, :n_prompt])
    dist.barrier()
    greedy, _ = cache.batch_greedy(4)
    every = [torch.empty(greedy.shape, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(every, torch.from_numpy(greedy.astype(np.int32)))
    ok &= all(torch.equal(every[0], t) for t in every)
    st = __import__("ctypes").c_int(0)
    pkg.lib.llmb_device_status(__import__("ctypes").byref(st))
    ok &= st.value == 0
    flag = torch.tensor([1 if (ok and worst <= LOGIT_TOL) else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write("%d %.5g" % (int(flag.item()), worst))
    cache.close()
    model.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("cfg_name,world,n_seqs,n_prompt", [("tiny", 2, 5, 40), ("llama3_8b_l2", 2, 32, 9), ("llama3_8b_l2", 8, 8, 9),
                                                            ("llama3_70b_l2", 8, 8, 9)])
def test_tensor_parallel_batched_decode_matches_oracle(cfg_name, world, n_seqs, n_prompt, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    result = tmp_path / "r.txt"
    mp.spawn(_rank_batch, args=(world, _free_port(), cfg_name, n_seqs, n_prompt, 3, str(result)), nprocs=world, join=True)
    status, worst = result.read_text().split(" ")
    print("TP=%d %s batch %d: worst |dlogit| %s" % (world, cfg_name, n_seqs, worst))
    assert status == "1", "worst |dlogit| %s" % worst
