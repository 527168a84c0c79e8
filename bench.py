#!/usr/bin/env python
"""Benchmark of the per-token forward loop: LLaMA3-8B-shape greedy decode, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decoded token.  The workload is the 8B configuration: random-init BF16 weights
converted to FP16 at load (seeded), a 128-token uniform-random prompt, then greedy decode; the
default K = 256 is the configuration's decode length.  W warm-up tokens and K timed tokens follow
the prompt.  Prints one JSON line (rank 0).

  value        tokens/s with everything resident on the device: K launches of the whole-step kernel
               back to back, the sampled token fed back on the device, timed with CUDA events on
               the engine's stream
  e2e          tokens/s through the reference-style call inference(model, X, d_tokens, h_tokens,
               cache): host token array in, next token and 256 KB of FP16 logits out, per token
  roofline     algorithmic bytes of a decode step (weights + KV rows read + KV row written)
               divided by the measured step time, against the measured HBM copy bandwidth
  cpu_baseline the CPU oracle's KV-cached decoder timed on the host cores, a few tokens
  prefill      the prompt phase alone (128 and 4096 tokens), FLOPs / time against the measured tensor peak
  long_context_decode   decode steps behind the 4096-token prompt (cache rows up to 4224)
  batched_decode        32 sequences x 1024-token prompts on this GPU, one token each per step
  tp_parity    (N > 1) the tensor-parallel path checked against logits of the reference binary
  --impl reference   the reference engine itself (oracle/_ref/ref_harness: its own CUDA build with
               the one-character compile fix) on the same weights and prompt, a few tokens
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s_bs1"
UNIT = "tok/s"
PROMPT = 128
# decode_step_kernel, ncu --set full on the 4-layer / 32K-vocabulary case: (dram__bytes_read.sum +
# dram__bytes_write.sum) / algorithmic bytes = (2.01396 GB + 20.8 MB) / 2.01367 GB
NCU_TRAFFIC_RATIO = 1.0105
SEED = 0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def tensor_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))
    return 1590.0, 1400.0   # fallback: an earlier measurement on this pool (burst / sustained)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def load_package():
    import __graft_entry__ as ge
    return ge.load_package()


def load_configs():
    """The named model shapes without the product library: configs.py is pure Python, and the reference arm
    must not map libllm_b200.so into its process."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("llm_cu_b200_configs", os.path.join(ROOT, "llm.cu_b200", "configs.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod   # dataclasses resolves the module by name while the class is built
    spec.loader.exec_module(mod)
    return mod.CONFIGS


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def synth_ids(vocab, n, seed=SEED, first=0):
    """n uniform ids from the seeded generator (stream seed + 1, as the tests and the oracle use), computed
    without the oracle."""
    m64 = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & m64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m64
        return z ^ (z >> 31)

    key = mix(((seed + 1) * 0xD1342543DE82EF95 + mix(4)) & m64)
    return [mix((key + first + i) & m64) % vocab for i in range(n)]


def prompt_ids(vocab):
    return synth_ids(vocab, PROMPT)


def prefill_flops(cfg, n):
    """Algorithmic FLOPs of a causal prompt phase over n tokens: every projection for every row, causal
    attention (QK^T and PV over half the square), lm_head for the last row."""
    proj = 2.0 * cfg.matmul_params() * n
    attn = 4.0 * n * n * cfg.head_dim * cfg.n_q_heads * cfg.n_layers / 2.0
    return proj + attn + 2.0 * cfg.vocab * cfg.d_model, proj, attn


def tp_parity_leg(pkg, torch, dist, rank, world):
    """Correctness of the tensor-parallel path, outside any timed region: the 8B layer shape (2 layers) run
    teacher-forced over `world` GPUs and compared with the logits the reference binary itself produced
    (tests/golden/ref_8b_l2.npz: every 16th logit and the 16 largest per step)."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "ref_8b_l2.npz")
    if not os.path.exists(path):
        return {"unavailable": "tests/golden/ref_8b_l2.npz missing"}
    fx = np.load(path)
    cfg = pkg.CONFIGS[str(fx["config"])]
    model = pkg.Model.synthetic(cfg, seed=int(fx["seed"]), max_seq=256, tp_rank=rank, tp_size=world)
    cache = pkg.Cache(model)
    cache.tp_connect()
    n_prompt, stride = int(fx["n_prompt"]), int(fx["stride"])
    worst, mismatch, agree = 0.0, 0, True
    for s in range(len(fx["argmax"])):
        dist.barrier()
        nxt = cache.infer(fx["tokens"][: n_prompt + s])
        mine = torch.from_numpy(cache.logits().astype(np.int32)).cuda()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        toks = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
        dist.all_gather(toks, torch.tensor([nxt], dtype=torch.int64, device="cuda"))
        agree = agree and len({int(t.item()) for t in toks}) == 1
        row = torch.cat(parts).cpu().numpy().astype(np.uint16)
        f = lambda a: np.asarray(a, dtype=np.uint16).view(np.float16).astype(np.float32)
        worst = max(worst, float(np.abs(f(row[::stride]) - f(fx["strided_bits"][s])).max()),
                    float(np.abs(f(row[fx["topk_idx"][s]]) - f(fx["topk_bits"][s])).max()))
        mismatch += int(nxt != int(fx["argmax"][s]))
    cache.close()
    model.close()
    return {"max_dlogit": worst, "argmax_mismatch": mismatch, "steps": int(len(fx["argmax"])), "ranks_agree": bool(agree),
            "tolerance": 2e-2, "against": "logits of the reference's own CUDA build (tests/golden/ref_8b_l2.npz), 8B layer "
            "shape, 2 layers, 16-token prompt + 8 teacher-forced steps"}


def run_ours(args):
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = load_package()
    cfg = pkg.CONFIGS[args.config]
    K, W = args.steps, max(args.warmup, 3)
    single = world == 1 and not args.per_op_kernels
    # the cache also serves the long-prompt case (4096-token prompt, 128 decode steps, 4224 rows)
    long_prompt, long_decode = 4096, 128
    max_seq = max(2048, PROMPT + 2 * (W + K) + 8, (long_prompt + long_decode + 8) if (single and not args.quick) else 0)
    hbm_peak, peak_src = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tp_parity = None
    if world > 1:
        tp_parity = tp_parity_leg(pkg, torch, dist, rank, world)
    # N > 1: tensor parallel over the N GPUs (q/k/v, gate/up, lm_head by rows; o, down by columns; KV cache
    # by KV head), one process per GPU; the all-reduces after o_proj and down_proj are peer stores plus
    # tagged polls inside the step kernel, torch.distributed only carries the IPC handles and the timing barrier
    model = pkg.Model.synthetic(cfg, seed=SEED, max_seq=max_seq, tp_rank=rank, tp_size=world)
    cache = pkg.Cache(model)
    if world > 1:
        cache.tp_connect()
    if args.per_op_kernels:
        cache.set_options(step_kernel=0)
    prompt = prompt_ids(cfg.vocab)

    # ---- device-resident decode: prompt, W warm-up tokens, K timed tokens ------------------
    barrier()
    cache.greedy(prompt, 1)                       # prompt phase
    cache.continue_greedy(W)                      # warm-up (>= 3)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = cache.kernel_launches()
    toks, ms = cache.continue_greedy(K)
    launches = cache.kernel_launches() - launches0
    barrier()
    clocks = sampler.stop()
    first_pos = PROMPT + 1 + W                    # cache rows before the first timed step
    alg_bytes = sum(cfg.decode_bytes(first_pos + i, world) for i in range(K)) / K   # per GPU

    # ---- end to end through inference(): host tokens in, token + logits out ---------------
    cache.reset()
    seq = list(prompt)
    barrier()                                     # tensor-parallel ranks must enter a step together
    seq.append(cache.infer(seq))                  # prompt phase (untimed)
    for _ in range(W):
        seq.append(cache.infer(seq))
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        seq.append(cache.infer(seq))
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    # ---- prompt phase: the 128-token prompt of the headline and the long-prompt case ----------
    prefill, long_ctx = None, None
    if single:
        prefill = {}
        peak_burst, peak_sust = tensor_peaks()
        for plen in ([PROMPT] if args.quick else [PROMPT, long_prompt]):
            ids = synth_ids(cfg.vocab, plen)
            best = None
            for _ in range(3):
                cache.reset()
                _, pre_ms, _ = cache.greedy(ids, 1)
                best = pre_ms if best is None else min(best, pre_ms)
            total, proj, attn = prefill_flops(cfg, plen)
            tf = total / (best / 1e3) / 1e12
            prefill["prompt_%d" % plen] = {
                "ms": best, "tok_s": plen / (best / 1e3),
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_burst, "unit": "TFLOP/s", "frac": tf / peak_burst,
                             "frac_of_sustained": tf / peak_sust, "peak_sustained": peak_sust,
                             "flops": total, "projection_flops": proj, "attention_flops": attn,
                             "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst) / bf16_tflops_sustained"},
                "path": "rows 0..n-2 as blocks of up to 1024 rows (tcgen05 projections, block attention), last row "
                        "through the decode step (its 15 GB weight stream is inside this time)"}
        if not args.quick:
            # decode behind the long prompt: cache rows 4097..4224 (the state the last prefill run left)
            cache.continue_greedy(3)
            _, long_ms = cache.continue_greedy(long_decode - 4)
            n = long_decode - 4
            lb = sum(cfg.decode_bytes(long_prompt + 4 + i) for i in range(n)) / n
            long_ctx = {"prompt_len": long_prompt, "decode_steps": n, "tok_s": n / (long_ms / 1e3), "ms_per_step": long_ms / n,
                        "roofline": {"bound": "hbm", "achieved": lb / (long_ms / n / 1e3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                                     "frac": lb / (long_ms / n / 1e3) / 1e9 / hbm_peak, "algorithmic_bytes_per_step": lb}}

    # ---- batched decode on this GPU: n_seqs sequences, one token each per step ----------------
    batch = None
    if args.batch > 0 and not args.per_op_kernels:
        B, bp, bsteps = args.batch, args.batch_prompt, args.batch_steps
        cache.batch_init(B)
        prompts = np.array([synth_ids(cfg.vocab, bp, seed=SEED + 1 + b) for b in range(B)], dtype=np.int32)
        barrier()
        t0 = time.perf_counter()
        cache.batch_prefill(prompts)
        torch.cuda.synchronize()
        bpre_s = time.perf_counter() - t0
        barrier()
        cache.batch_greedy(3)
        barrier()
        btoks, bms = cache.batch_greedy(bsteps)
        if world > 1:
            bt = torch.tensor([bms, bpre_s], dtype=torch.float64, device="cuda")
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
            bms, bpre_s = bt.tolist()
        rows0 = bp + 3                             # cache rows per sequence before the first timed step
        bbytes = sum(cfg.weight_bytes_per_token(world) + B * (cfg.kv_bytes_per_position() // world) * (rows0 + i + 1)
                     for i in range(bsteps)) / bsteps   # per GPU
        bach = bbytes / (bms / bsteps / 1e3) / 1e9
        batch = {"n_seqs": B, "prompt_len": bp, "decode_steps": bsteps, "tok_s": B * bsteps / (bms / 1e3),
                 "ms_per_step": bms / bsteps, "prefill_tok_s": B * (bp - 1) / bpre_s,
                 "roofline": {"bound": "hbm", "achieved": bach, "peak": hbm_peak, "unit": "GB/s", "frac": bach / hbm_peak,
                              "algorithmic_bytes_per_step": bbytes,
                              "scope": "one batched step = weights once + every sequence's KV rows; %d launches per step "
                                       "in a CUDA graph" % (2 + 7 * cfg.n_layers + 2)},
                 "parallelism": "single GPU" if world == 1 else "tp%d: weight shards streamed once per step on every GPU, all-reduce as "
                                "peer stores from the projection's epilogue + a local gather kernel" % world,
                 "path": "tcgen05 projections at m = n_seqs rows (weights as the 128-row operand, K slices as a cluster), "
                         "decode attention as one balanced wave of CTAs over all sequences (TMA boxes, mma.sync), per-row argmax"}

    times = torch.tensor([ms / 1e3, e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, e2e_s = times.tolist()
    status = C.c_int(0)
    pkg.check(pkg.lib.llmb_device_status(C.byref(status)), "llmb_device_status")
    if status.value != 0:
        raise RuntimeError("a device-side wait ran out (status %d)" % status.value)

    achieved = alg_bytes / (dev_s / K) / 1e9
    out = {
        "metric": METRIC, "value": K / dev_s, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_s / K * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f16 weights/activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": "%s shape (%d layers, d %d, %dq/%dkv heads, ffn %d, vocab %d), batch 1, "
                               "prompt %d uniform-random ids, greedy decode; random-init BF16 weights (seed %d) "
                               "converted to FP16 at load" % (cfg.name, cfg.n_layers, cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads,
                                                              cfg.ffn, cfg.vocab, PROMPT, SEED),
                   "model_config": cfg.name, "prompt_len": PROMPT, "decode_len": K,
                   "parallelism": "single GPU" if world == 1 else "tp%d (one sequence, model sharded over %d GPUs)" % (world, world),
                   "l2": "inputs larger than L2: %.1f GB of weights are streamed per step and GPU (L2 is 126 MB)" % (
                       cfg.weight_bytes_per_token(world) / 1e9)},
        "e2e": {"value": K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": cfg.vocab // world * 2 + 4,
                "timer": "wall clock around K inference() calls, each ending in a stream synchronize"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": (alg_bytes * NCU_TRAFFIC_RATIO) if single else None,
                     "traffic_source": ("scaled from the ncu capture of the 4-layer case of the same kernel "
                                        "(dram read + write = %.4f x algorithmic bytes there; traffic is proportional "
                                        "to the weight and cache bytes streamed)" % NCU_TRAFFIC_RATIO) if single else None,
                     "peak_source": peak_src,
                     "scope": ("whole decode step: one kernel per fused op, 163 launches in a CUDA graph" if args.per_op_kernels else
                               "decode_step_kernel: one persistent launch per token") +
                              "; algorithmic bytes per launch and GPU = weight bytes %d + %d per cached row" % (
                                  cfg.weight_bytes_per_token(world), cfg.kv_bytes_per_position() // world),
                     "algorithmic_bytes_per_step": alg_bytes},
        "tokens_match_e2e": toks[:8] == seq[PROMPT + 1 + W:PROMPT + 1 + W + 8],
    }
    if prefill:
        out["prefill"] = prefill
    if long_ctx:
        out["long_context_decode"] = long_ctx
    if batch:
        out["batched_decode"] = batch
    if tp_parity is not None:
        out["tp_parity"] = tp_parity
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(pkg, cfg, prompt)
    cache.close()
    model.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out))


def cpu_baseline(pkg, cfg, prompt, budget_s=20.0, max_tokens=8):
    """The CPU oracle's KV-cached decoder on the host cores: a bounded sample of the same decode."""
    from oracle import oracle_lib as oracle
    weights = oracle.Weights(cfg, seed=SEED, keep_file=False)
    dec = oracle.Decoder(weights, max_tokens + 1)
    n, t0 = 0, time.perf_counter()
    while n < max_tokens and (n < 2 or time.perf_counter() - t0 < budget_s):
        dec.step(prompt[n])
        n += 1
    dt = time.perf_counter() - t0
    dec.close()
    return {"value": n / dt, "unit": UNIT, "cores": oracle.lib().oracle_num_threads(), "kind": "port",
            "sample": "%d decode steps at cache lengths 0..%d of the same model (weights regenerated on the host "
                      "from the same seed), all host threads via OpenMP" % (n, n - 1)}


def run_reference(args):
    """The reference's own engine (its CUDA build; it has no CPU path) through its public functions."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": world, "higher_is_better": True}
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    if not os.path.exists(harness):
        print(json.dumps(dict(base, unavailable="oracle/_ref/ref_harness was not built (reference tree absent at build time)")))
        return
    from oracle import oracle_lib as oracle
    cfg = load_configs()[args.config]
    if (cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab) != (4096, 32, 8, 128, 14336, 128256):
        print(json.dumps(dict(base, unavailable="the reference's dimensions are literals of the 8B shape (inference.cu:212-220, "
                                                ":700, :752, :799); it cannot run %s" % cfg.name)))
        return
    steps = min(args.steps, args.ref_max_steps)
    warm = min(max(args.warmup, 1), 2)
    need = cfg.weight_bytes_per_token() + (1 << 30)
    tmp_root = args.tmpdir or tempfile.gettempdir()
    st = os.statvfs(tmp_root)
    if st.f_bavail * st.f_frsize < need:
        print(json.dumps(dict(base, unavailable="not enough scratch disk under %s for the %.1f GB checkpoint the "
                                                "reference loader reads" % (tmp_root, need / 1e9))))
        return
    with tempfile.TemporaryDirectory(dir=tmp_root) as tmp:
        weights = oracle.Weights(cfg, seed=SEED, keep_fp16=False)
        names = list(weights.file)
        quarter = (len(names) + 3) // 4
        shards = []
        for i in range(4):  # four shards, as src/main.cu:73-76 loads
            part = names[i * quarter:(i + 1) * quarter]
            if part:
                shards.append(weights.write_safetensors(os.path.join(tmp, "model-%05d-of-00004.safetensors" % (i + 1)), part))
        del weights
        import numpy as np
        ids = np.array(prompt_ids(cfg.vocab) + [0] * (warm + steps), dtype=np.int32)
        tok_path = os.path.join(tmp, "tokens.i32")
        ids.tofile(tok_path)
        cmd = [harness, str(cfg.n_layers), tok_path, str(PROMPT), str(warm + steps), "-"] + [str(s) for s in shards]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(json.dumps(dict(base, unavailable="reference harness exited %d: %s" % (r.returncode, r.stderr[-200:]))))
            return
        info = json.loads(r.stdout[r.stdout.rindex('{"n_layers"'):])  # the reference prints ANSI colour codes before it
    secs = info["step_s"][warm:]
    total = sum(secs)
    val = len(secs) / total
    out = dict(base, value=val, steps=len(secs), warmup=warm, ms_per_step=total / len(secs) * 1e3, scaling="weak",
               vs_baseline=None, dtype="f16 weights/activations, f32 accumulate", data="synthetic",
               config={"workload": "same 8B model, prompt and seed as the main arm; the reference recomputes the whole "
                                   "sequence on every call (no KV cache), so each step costs prompt+generated rows",
                       "model_config": cfg.name, "prompt_len": PROMPT, "decode_len": len(secs)},
               e2e={"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
               cpu_baseline={"value": val, "unit": UNIT, "cores": 0, "kind": "reference",
                             "sample": "the reference has no CPU implementation of this path: this is its own CUDA "
                                       "build (inference.cu:673 one-character compile fix, nvcc -O3 sm_100a) on the "
                                       "GPU, %d inference() calls after the %d-token prompt, wall clock per call; "
                                       "first %.3f s, last %.3f s; load %.1f s" % (len(secs), PROMPT, secs[0], secs[-1], info["load_s"])})
    print(json.dumps(out))


def main():
    global PROMPT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama3_8b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-max-steps", type=int, default=6)
    ap.add_argument("--tmpdir", default=None)
    ap.add_argument("--per-op-kernels", action="store_true", help="one kernel per fused op in a CUDA graph instead of the whole-step kernel")
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="shorter prompts are for profiling runs only")
    ap.add_argument("--quick", action="store_true", help="skip the long-prompt case (profiling runs)")
    ap.add_argument("--batch", type=int, default=32, help="sequences of the batched-decode leg (0 = skip it)")
    ap.add_argument("--batch-prompt", type=int, default=1024)
    ap.add_argument("--batch-steps", type=int, default=64)
    args = ap.parse_args()
    PROMPT = args.prompt_len
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
