"""Prompt-phase kernels (tensor-core GEMM with fused epilogues, row RMSNorm, block attention) through
the C-ABI, and the engine's block prefill against the token-by-token path and the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from gpu_util import assert_close_fp16, dev, f16, host_u16, rmsnorm_ref, to_f16_bits  # noqa: E402

EPI_STORE, EPI_RESIDUAL, EPI_ROPE_KV, EPI_SWIGLU = 0, 1, 2, 3


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def check_status(pkg):
    st = C.c_int(-1)
    assert pkg.lib.llmb_device_status(C.byref(st)) == 0, pkg.lib.llmb_last_error()
    assert st.value == 0, "device status %d" % st.value


def gemm(pkg, **kw):
    a = pkg.GemmArgs()
    for k, v in kw.items():
        setattr(a, k, v.data_ptr() if hasattr(v, "data_ptr") else v)
    rc = pkg.lib.llmb_gemm_f16(C.byref(a), None)
    assert rc == 0, (rc, pkg.lib.llmb_last_error())
    torch.cuda.synchronize()
    check_status(pkg)


def mats(oracle, m, n, k, seed=0):
    a = oracle.synth_fp16(900 + seed, 1, m * k, std=1.0).reshape(m, k)
    b = oracle.synth_fp16(900 + seed, 2, n * k, std=0.02).reshape(n, k)
    return a, b


def matmul64(a_bits, b_bits):
    return f16(a_bits).astype(np.float64) @ f16(b_bits).astype(np.float64).T


def tc_tol(want, k):
    """Absolute tolerance of a tensor-core FP32 accumulation over k terms: the MMA aligns its addends to
    the largest exponent and truncates, so the error grows with k times 2^-24 of the running magnitude
    instead of with the FP32 rounding of a sequential sum.  Matters only for outputs that cancel to far
    below the typical magnitude, where one FP16 ulp is smaller than that."""
    return k * 2.0 ** -23 * float(np.abs(want).max())


def test_epilogue_constants_match_header(pkg):
    import re, os
    hdr = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "llm_b200.h")).read()
    for name, val in (("STORE", EPI_STORE), ("RESIDUAL", EPI_RESIDUAL), ("ROPE_KV", EPI_ROPE_KV), ("SWIGLU", EPI_SWIGLU)):
        m = re.search(r"LLMB_EPI_%s\s*=?\s*(\d+)" % name, hdr)
        assert m and int(m.group(1)) == val, name


@pytest.mark.parametrize("tile_n", [0, 32, 64, 128])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (16, 256, 256), (200, 384, 768), (300, 512, 4096), (1, 128, 128)])
def test_gemm_store(pkg, oracle, m, n, k, tile_n):
    a, b = mats(oracle, m, n, k)
    out = torch.full((m + 3, n), 0x7BFF, dtype=torch.int16, device="cuda")  # rows past m must stay untouched
    gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_STORE, tile_n=tile_n)
    got = host_u16(out)
    want = matmul64(a, b)
    print("gemm %dx%dx%d: max abs err %.3g" % (m, n, k, np.abs(f16(got[:m]) - want).max()))
    assert_close_fp16(got[:m], want, what="gemm %dx%dx%d" % (m, n, k), abs_tol=tc_tol(want, k))
    assert (got[m:] == 0x7BFF).all()


@pytest.mark.parametrize("tile_n", [32, 64, 128])
def test_gemm_residual(pkg, oracle, tile_n):
    m, n, k = 150, 256, 512
    a, b = mats(oracle, m, n, k, 1)
    res = oracle.synth_fp16(7, 3, m * n, std=1.0).reshape(m, n)
    out = dev(res.copy())
    gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_RESIDUAL, tile_n=tile_n)
    acc = matmul64(a, b)
    want = acc.astype(np.float16).astype(np.float64) + f16(res).astype(np.float64)
    # half(acc) may sit one FP16 ulp from the FP64 product's rounding; after the add cancels, that ulp of
    # the product is many ulps of a small sum
    assert_close_fp16(host_u16(out).reshape(m, n), want, what="gemm residual", max_frac=0.1,
                      abs_tol=np.abs(acc) * 2.0 ** -10 + tc_tol(acc, k))


@pytest.mark.parametrize("tile_n", [32, 64, 128])
def test_gemm_swiglu(pkg, oracle, tile_n):
    m, n, k = 130, 384, 256
    a, b = mats(oracle, m, n, k, 2)
    b2 = oracle.synth_fp16(8, 4, n * k, std=0.02).reshape(n, k)
    out = torch.zeros((m, n), dtype=torch.int16, device="cuda")
    gemm(pkg, a=dev(a), b=dev(b), b2=dev(b2), c=out, m=m, n=n, k=k, epilogue=EPI_SWIGLU, tile_n=tile_n)
    g, u = matmul64(a, b), matmul64(a, b2)
    want = g / (1.0 + np.exp(-g)) * u
    assert_close_fp16(host_u16(out).reshape(m, n), want, what="gemm swiglu", abs_tol=tc_tol(want, k))


@pytest.mark.parametrize("tile_n,k,split", [(32, 256, False), (64, 256, False), (128, 256, False), (0, 2048, True)])
def test_gemm_rope_kv(pkg, oracle, tile_n, k, split):
    hd, nqh, nkvh, m, pos0, max_pos = 64, 4, 2, 70, 5, 128
    ws = torch.zeros(4096 + 148 * 131072, dtype=torch.uint8, device="cuda") if split else None
    n_q, n_kv = nqh * hd, nkvh * hd
    n = n_q + 2 * n_kv
    a, b = mats(oracle, m, n, k, 3)
    pos = np.arange(pos0, pos0 + m, dtype=np.float32)
    i = np.arange(hd // 2, dtype=np.float32)
    freq = (1.0 / np.power(np.float32(500000.0), 2.0 * i / np.float32(hd))).astype(np.float32)
    ang = (pos[:, None] * freq[None, :]).astype(np.float32)
    cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)  # [m][hd/2][2]
    q_out = torch.zeros((m, n_q), dtype=torch.int16, device="cuda")
    kc = torch.zeros((max_pos, n_kv), dtype=torch.int16, device="cuda")
    vc = torch.zeros((max_pos, n_kv), dtype=torch.int16, device="cuda")
    gemm(pkg, a=dev(a), b=dev(b), c=q_out, m=m, n=n, k=k, epilogue=EPI_ROPE_KV, n_q=n_q, n_kv=n_kv, head_dim=hd,
         rope_cs=dev(cs), k_cache=kc, v_cache=vc, pos0=pos0, max_pos=max_pos, tile_n=tile_n,
         **(dict(workspace=ws, workspace_bytes=ws.numel()) if split else {}))
    y = matmul64(a, b).astype(np.float16).astype(np.float64)

    def rope(block, heads):
        r = block.reshape(m, heads, hd // 2, 2)
        c, s = cs[:, None, :, 0].astype(np.float64), cs[:, None, :, 1].astype(np.float64)
        out = np.empty_like(r)
        out[..., 0] = c * r[..., 0] - s * r[..., 1]
        out[..., 1] = s * r[..., 0] + c * r[..., 1]
        return out.reshape(m, heads * hd)

    def pair_tol(block):
        """One FP16 ulp of either input of a rotated pair (the projection is rounded to FP16 before RoPE)."""
        mag = np.abs(block).reshape(m, -1, 2).sum(axis=2, keepdims=True) * 2.0 ** -10
        return np.broadcast_to(mag, (m, block.shape[1] // 2, 2)).reshape(m, -1) + tc_tol(y, k)

    assert_close_fp16(host_u16(q_out).reshape(m, n_q), rope(y[:, :n_q], nqh), what="q rope", max_frac=0.1,
                      abs_tol=pair_tol(y[:, :n_q]))
    kgot, vgot = host_u16(kc).reshape(max_pos, n_kv), host_u16(vc).reshape(max_pos, n_kv)
    assert_close_fp16(kgot[pos0:pos0 + m], rope(y[:, n_q:n_q + n_kv], nkvh), what="k rope", max_frac=0.1,
                      abs_tol=pair_tol(y[:, n_q:n_q + n_kv]))
    assert_close_fp16(vgot[pos0:pos0 + m], y[:, n_q + n_kv:], what="v", abs_tol=tc_tol(y, k))
    assert not kgot[:pos0].any() and not kgot[pos0 + m:].any() and not vgot[:pos0].any() and not vgot[pos0 + m:].any()


def test_gemm_split_k_all_epilogues(pkg, oracle):
    """Few output tiles and a workspace: K is split across CTAs, partials meet in the workspace, the last
    CTA of a tile adds them in slice order.  Every epilogue, twice on the same workspace (the arrival
    counters must come back to zero)."""
    ws = torch.zeros(4096 + 148 * 131072, dtype=torch.uint8, device="cuda")
    kw = dict(workspace=ws, workspace_bytes=ws.numel())
    for rep in range(2):
        # store
        m, n, k = 300, 512, 4096
        a, b = mats(oracle, m, n, k, 10 + rep)
        out = torch.full((m + 3, n), 0x7BFF, dtype=torch.int16, device="cuda")
        gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_STORE, **kw)
        want = matmul64(a, b)
        got = host_u16(out)
        assert_close_fp16(got[:m], want, what="split-k store", abs_tol=tc_tol(want, k))
        assert (got[m:] == 0x7BFF).all()
        # residual
        m, n, k = 150, 256, 4096
        a, b = mats(oracle, m, n, k, 20 + rep)
        res = oracle.synth_fp16(7, 3, m * n, std=1.0).reshape(m, n)
        out = dev(res.copy())
        gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_RESIDUAL, **kw)
        acc = matmul64(a, b)
        want = acc.astype(np.float16).astype(np.float64) + f16(res).astype(np.float64)
        assert_close_fp16(host_u16(out).reshape(m, n), want, what="split-k residual", max_frac=0.1,
                          abs_tol=np.abs(acc) * 2.0 ** -10 + tc_tol(acc, k))
        # SwiGLU
        m, n, k = 130, 384, 2048
        a, b = mats(oracle, m, n, k, 30 + rep)
        b2 = oracle.synth_fp16(8, 4, n * k, std=0.02).reshape(n, k)
        out = torch.zeros((m, n), dtype=torch.int16, device="cuda")
        gemm(pkg, a=dev(a), b=dev(b), b2=dev(b2), c=out, m=m, n=n, k=k, epilogue=EPI_SWIGLU, **kw)
        g, u = matmul64(a, b), matmul64(a, b2)
        want = g / (1.0 + np.exp(-g)) * u
        assert_close_fp16(host_u16(out).reshape(m, n), want, what="split-k swiglu", abs_tol=tc_tol(want, k))
        assert not host_u16(ws[:4096].view(torch.int16)).any(), "arrival counters not back to zero"


def test_gemm_rejects_unaligned_shapes(pkg):
    t = torch.zeros(1 << 16, dtype=torch.int16, device="cuda")
    a = pkg.GemmArgs(a=t.data_ptr(), b=t.data_ptr(), c=t.data_ptr(), m=4, n=100, k=64, epilogue=EPI_STORE)
    assert pkg.lib.llmb_gemm_f16(C.byref(a), None) != 0
    a = pkg.GemmArgs(a=t.data_ptr(), b=t.data_ptr(), c=t.data_ptr(), m=4, n=128, k=40, epilogue=EPI_STORE)
    assert pkg.lib.llmb_gemm_f16(C.byref(a), None) != 0
    a = pkg.GemmArgs(a=t.data_ptr(), b=t.data_ptr(), c=t.data_ptr(), m=0, n=128, k=64, epilogue=EPI_STORE)
    assert pkg.lib.llmb_gemm_f16(C.byref(a), None) != 0
    a = pkg.GemmArgs(a=t.data_ptr(), b=t.data_ptr(), c=t.data_ptr(), m=4, n=128, k=64, epilogue=EPI_STORE, tile_n=48)
    assert pkg.lib.llmb_gemm_f16(C.byref(a), None) != 0


@pytest.mark.parametrize("m,d", [(5, 256), (33, 4096), (3, 1000)])
def test_rmsnorm_rows_bit_exact(pkg, oracle, m, d):
    x = oracle.synth_fp16(11, 1, m * d, std=1.0).reshape(m, d)
    g = oracle.synth_fp16(11, 2, d, std=1.0)
    y = torch.zeros((m, d), dtype=torch.int16, device="cuda")
    dx, dg = dev(x), dev(g)
    assert pkg.lib.llmb_rmsnorm_rows(dx.data_ptr(), dg.data_ptr(), y.data_ptr(), m, d, 1e-5, None) == 0
    got = host_u16(y).reshape(m, d)
    for r in range(m):
        want = rmsnorm_ref(x[r], g)
        # the device fuses the partial's multiply-adds; a value may sit one ulp across a rounding boundary
        assert_close_fp16(got[r], f16(want).astype(np.float64), what="rmsnorm row %d" % r)


@pytest.mark.parametrize("hd,nqh,nkvh,m,pos0", [(64, 4, 2, 45, 0), (128, 8, 2, 70, 37), (128, 4, 4, 1, 3), (128, 4, 1, 200, 100), (64, 2, 2, 130, 0)])
def test_attn_prefill_matches_fp64(pkg, oracle, hd, nqh, nkvh, m, pos0):
    total = pos0 + m
    n_q, n_kv = nqh * hd, nkvh * hd
    q = oracle.synth_fp16(21, 1, m * n_q, std=1.0).reshape(m, n_q)
    kc = oracle.synth_fp16(21, 2, (total + 4) * n_kv, std=1.0).reshape(total + 4, n_kv)
    vc = oracle.synth_fp16(21, 3, (total + 4) * n_kv, std=1.0).reshape(total + 4, n_kv)
    kc[total:] = 0x7E00  # rows past the causal limit hold NaN: they must never be read into the result
    vc[total:] = 0x7E00
    out = torch.zeros((m, n_q), dtype=torch.int16, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    rc = pkg.lib.llmb_attn_prefill(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m, pos0, nqh, nkvh, hd,
                                   out.data_ptr(), None)
    assert rc == 0, pkg.lib.llmb_last_error()
    got = host_u16(out).reshape(m, nqh, hd)
    qf = f16(q).astype(np.float64).reshape(m, nqh, hd)
    kf = f16(kc[:total]).astype(np.float64).reshape(total, nkvh, hd)
    vf = f16(vc[:total]).astype(np.float64).reshape(total, nkvh, hd)
    want = np.zeros((m, nqh, hd))
    for h in range(nqh):
        g = h // (nqh // nkvh)
        s = qf[:, h] @ kf[:, g].T / np.sqrt(float(hd))
        for r in range(m):
            s[r, pos0 + r + 1:] = -np.inf
        p = np.exp(s - s.max(axis=1, keepdims=True))
        want[:, h] = (p / p.sum(axis=1, keepdims=True)) @ vf[:, g]
    assert_close_fp16(got.reshape(m, -1), want.reshape(m, -1), what="attn prefill", max_frac=0.2, abs_tol=2e-3)


def run_prompt(pkg, model, prompt, n_new, block, step_kernel=1):
    cache = pkg.Cache(model)
    cache.set_options(step_kernel=step_kernel)
    cache.set_prefill(block, 4)
    nxt = cache.infer(prompt)
    logits = cache.logits()
    launches = cache.kernel_launches()
    toks, _, _ = cache.greedy(prompt, n_new)
    cache.close()
    return nxt, logits, toks, launches


@pytest.mark.parametrize("n_prompt", [6, 40, 161])
def test_tiny_block_prefill_matches_stepwise_and_oracle(pkg, oracle, tiny_weights, n_prompt):
    cfg = pkg.CONFIGS["tiny"]
    prompt = oracle.synth_tokens(3, n_prompt, cfg.vocab).tolist()
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=256)
    a = run_prompt(pkg, model, prompt, 8, True)
    b = run_prompt(pkg, model, prompt, 8, False)
    ref_logits, _ = oracle.forward(tiny_weights, np.asarray(prompt, dtype=np.int32), first_logit_row=n_prompt - 1)
    da = np.abs(oracle.f16(a[1]) - oracle.f16(ref_logits[0])).max()
    db = np.abs(oracle.f16(b[1]) - oracle.f16(ref_logits[0])).max()
    print("tiny prompt %d: block |dlogit| %.4g, stepwise %.4g" % (n_prompt, da, db))
    assert da <= 2e-2 and db <= 2e-2
    assert a[0] == b[0] and a[2] == b[2]
    L = cfg.n_layers
    assert a[3] == (2 + 7 * L) + 1 and b[3] == n_prompt  # one block + one decode step vs one step per token
    model.close()


def test_block_prefill_extends_a_cached_prefix(pkg, oracle, tiny_weights):
    """A second inference() call that appends 30 tokens to a 50-token prefix prefills only the new rows
    (pos0 = 50) and must agree with a fresh run on all 80."""
    cfg = pkg.CONFIGS["tiny"]
    ids = oracle.synth_tokens(4, 80, cfg.vocab).tolist()
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=256)
    c1 = pkg.Cache(model)
    c1.set_prefill(True, 4)
    c1.infer(ids[:50])
    n1 = c1.infer(ids)
    l1 = c1.logits()
    c2 = pkg.Cache(model)
    c2.set_prefill(True, 4)
    n2 = c2.infer(ids)
    l2 = c2.logits()
    assert n1 == n2
    assert np.abs(oracle.f16(l1) - oracle.f16(l2)).max() <= 4e-3
    c1.close(); c2.close(); model.close()


def test_8b_layer_shapes_block_prefill(pkg, oracle, weights_8b_l2):
    cfg = pkg.CONFIGS["llama3_8b_l2"]
    n_prompt = 48
    prompt = oracle.synth_tokens(0, n_prompt, cfg.embed_rows).tolist()
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=256)
    a = run_prompt(pkg, model, prompt, 4, True)
    ref_logits, _ = oracle.forward(weights_8b_l2, np.asarray(prompt, dtype=np.int32), first_logit_row=n_prompt - 1)
    d = np.abs(oracle.f16(a[1]) - oracle.f16(ref_logits[0])).max()
    print("8b_l2 block prefill: |dlogit| %.4g" % d)
    assert d <= 2e-2
    want_tok = int(oracle.lib().oracle_argmax_fp16(ref_logits[0].ctypes.data, len(ref_logits[0])))
    assert a[0] == want_tok
    model.close()


@pytest.mark.parametrize("m,use_ws,use_pdl", [(1, False, 0), (7, True, 1), (32, True, 1), (20, False, 1)])
def test_gemm_small_m_weight_stream_all_epilogues(pkg, oracle, m, use_ws, use_pdl):
    """m <= 32 rows take the weight-streaming kernel (weights as the 128-row MMA operand, K split across the CTAs
    of a cluster: 8 slices for the store case, 2 for the residual case, 4 for SwiGLU, none for the cache append).
    Every epilogue, twice in a row, with and without a workspace argument (not used at this m) and programmatic
    dependent launch; the batched-decode form of the cache append (one sequence per row)."""
    ws = torch.zeros(4096 + 148 * 131072, dtype=torch.uint8, device="cuda") if use_ws else None
    kw = dict(use_pdl=use_pdl, **(dict(workspace=ws, workspace_bytes=ws.numel()) if use_ws else {}))
    for rep in range(2):
        # store: k long enough for several K slices
        n, k = 384, 4096
        a, b = mats(oracle, m, n, k, 40 + rep)
        out = torch.full((m + 2, n), 0x7BFF, dtype=torch.int16, device="cuda")
        gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_STORE, **kw)
        want = matmul64(a, b)
        got = host_u16(out)
        assert_close_fp16(got[:m], want, what="small-m store", abs_tol=tc_tol(want, k))
        assert (got[m:] == 0x7BFF).all()
        # residual
        n, k = 256, 1024
        a, b = mats(oracle, m, n, k, 50 + rep)
        res = oracle.synth_fp16(7, 3, m * n, std=1.0).reshape(m, n)
        out = dev(res.copy())
        gemm(pkg, a=dev(a), b=dev(b), c=out, m=m, n=n, k=k, epilogue=EPI_RESIDUAL, **kw)
        acc = matmul64(a, b)
        want = acc.astype(np.float16).astype(np.float64) + f16(res).astype(np.float64)
        assert_close_fp16(host_u16(out).reshape(m, n), want, what="small-m residual", max_frac=0.1,
                          abs_tol=np.abs(acc) * 2.0 ** -10 + tc_tol(acc, k))
        # SwiGLU
        n, k = 512, 2048
        a, b = mats(oracle, m, n, k, 60 + rep)
        b2 = oracle.synth_fp16(8, 4, n * k, std=0.02).reshape(n, k)
        out = torch.zeros((m, n), dtype=torch.int16, device="cuda")
        gemm(pkg, a=dev(a), b=dev(b), b2=dev(b2), c=out, m=m, n=n, k=k, epilogue=EPI_SWIGLU, **kw)
        g, u = matmul64(a, b), matmul64(a, b2)
        want = g / (1.0 + np.exp(-g)) * u
        assert_close_fp16(host_u16(out).reshape(m, n), want, what="small-m swiglu", abs_tol=tc_tol(want, k))
        # RoPE + cache append, one sequence per row: row r goes to cache row r * seq_stride + row_pos[r]
        hd, nqh, nkvh, seq_stride, k = 64, 4, 2, 16, 512
        n_q, n_kv = nqh * hd, nkvh * hd
        n = n_q + 2 * n_kv
        a, b = mats(oracle, m, n, k, 70 + rep)
        row_pos = ((np.arange(m) * 5 + rep) % seq_stride).astype(np.int32)
        i = np.arange(hd // 2, dtype=np.float32)
        freq = (1.0 / np.power(np.float32(500000.0), 2.0 * i / np.float32(hd))).astype(np.float32)
        ang = (row_pos.astype(np.float32)[:, None] * freq[None, :]).astype(np.float32)
        cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
        q_out = torch.zeros((m, n_q), dtype=torch.int16, device="cuda")
        kc = torch.zeros((m * seq_stride, n_kv), dtype=torch.int16, device="cuda")
        vc = torch.zeros((m * seq_stride, n_kv), dtype=torch.int16, device="cuda")
        gemm(pkg, a=dev(a), b=dev(b), c=q_out, m=m, n=n, k=k, epilogue=EPI_ROPE_KV, n_q=n_q, n_kv=n_kv, head_dim=hd,
             rope_cs=dev(cs), k_cache=kc, v_cache=vc, row_pos=dev(row_pos), seq_stride=seq_stride, max_pos=seq_stride, **kw)
        y = matmul64(a, b).astype(np.float16).astype(np.float64)

        def rope(block, heads):
            r = block.reshape(m, heads, hd // 2, 2)
            c, s = cs[:, None, :, 0].astype(np.float64), cs[:, None, :, 1].astype(np.float64)
            o = np.empty_like(r)
            o[..., 0] = c * r[..., 0] - s * r[..., 1]
            o[..., 1] = s * r[..., 0] + c * r[..., 1]
            return o.reshape(m, heads * hd)

        def pair_tol(block):
            mag = np.abs(block).reshape(m, -1, 2).sum(axis=2, keepdims=True) * 2.0 ** -10
            return np.broadcast_to(mag, (m, block.shape[1] // 2, 2)).reshape(m, -1) + tc_tol(y, k)

        assert_close_fp16(host_u16(q_out).reshape(m, n_q), rope(y[:, :n_q], nqh), what="small-m q rope", max_frac=0.1,
                          abs_tol=pair_tol(y[:, :n_q]))
        rows = np.arange(m) * seq_stride + row_pos
        kgot, vgot = host_u16(kc).reshape(m * seq_stride, n_kv), host_u16(vc).reshape(m * seq_stride, n_kv)
        assert_close_fp16(kgot[rows], rope(y[:, n_q:n_q + n_kv], nkvh), what="small-m k rope", max_frac=0.1,
                          abs_tol=pair_tol(y[:, n_q:n_q + n_kv]))
        assert_close_fp16(vgot[rows], y[:, n_q + n_kv:], what="small-m v", abs_tol=tc_tol(y, k))
        untouched = np.ones(m * seq_stride, dtype=bool)
        untouched[rows] = False
        assert not kgot[untouched].any() and not vgot[untouched].any()
        if use_ws:
            assert not host_u16(ws[:4096].view(torch.int16)).any(), "arrival counters not back to zero"


@pytest.mark.parametrize("m,d,k_local", [(32, 512, 256), (7, 4096, 2048)])
def test_tensor_parallel_row_exchange_two_ranks_on_one_gpu(pkg, oracle, m, d, k_local):
    """The all-reduce of the row-batched tensor-parallel path with both ranks' kernels run on one GPU in an order
    in which nothing waits: projection of rank 0 and of rank 1 (LLMB_EPI_TP_SCATTER: each stores its tagged FP32
    partial sums into BOTH exchange blocks), then the gather kernel of each rank (sum in rank order + residual +
    RMSNorm).  Two exchanges per step (they alternate between the two receive buffers), two steps (the exchange
    counter moves on).  Both ranks must end with identical bits, equal to the one-GPU arithmetic."""
    tp = 2
    xbytes = pkg.lib.llmb_decode_step_exchange_bytes(tp, d)
    ex = [torch.zeros(xbytes, dtype=torch.uint8, device="cuda") for _ in range(tp)]
    peers = (C.c_void_p * 8)(*[e.data_ptr() for e in ex], *([None] * 6))
    ws = torch.zeros(4096 + 148 * 131072, dtype=torch.uint8, device="cuda")
    gamma = oracle.synth_fp16(77, 5, d, std=1.0)
    x_bits = oracle.synth_fp16(77, 6, m * d, std=1.0).reshape(m, d)
    xs = [dev(x_bits.copy()) for _ in range(tp)]
    xn = [torch.zeros((m, d), dtype=torch.int16, device="cuda") for _ in range(tp)]
    d_gamma = dev(gamma)
    want_x = f16(x_bits).astype(np.float64)
    for step in range(2):
        for index in range(2):
            a_full, b_full = mats(oracle, m, d, tp * k_local, 80 + 2 * step + index)
            for r in range(tp):   # both projections first: afterwards every partial sum is in place
                a_r = dev(np.ascontiguousarray(a_full[:, r * k_local:(r + 1) * k_local]))
                b_r = dev(np.ascontiguousarray(b_full[:, r * k_local:(r + 1) * k_local]))
                g = pkg.GemmArgs(a=a_r.data_ptr(), b=b_r.data_ptr(), c=None, m=m, n=d, k=k_local, epilogue=pkg.EPI_TP_SCATTER,
                                 workspace=ws.data_ptr(), workspace_bytes=ws.numel(), use_pdl=1, tp_rank=r, tp_size=tp, tp_index=index)
                for i in range(tp):
                    g.tp_peers[i] = peers[i]
                assert pkg.lib.llmb_gemm_f16(C.byref(g), None) == 0, pkg.lib.llmb_last_error()
            for r in range(tp):
                rc = pkg.lib.llmb_tp_gather_rows(ex[r].data_ptr(), tp, index, xs[r].data_ptr(), d_gamma.data_ptr(), xn[r].data_ptr(), m, d,
                                                 1e-5, 1 << 12, 1, None)
                assert rc == 0, pkg.lib.llmb_last_error()
            torch.cuda.synchronize()
            check_status(pkg)
            # expected: per-rank FP32 partials added in rank order, rounded to FP16, residual added in FP32, rounded
            parts = [matmul64(a_full[:, r * k_local:(r + 1) * k_local], b_full[:, r * k_local:(r + 1) * k_local]) for r in range(tp)]
            acc = parts[0] + parts[1]
            want_x = acc.astype(np.float16).astype(np.float64) + want_x
            got0, got1 = host_u16(xs[0]).reshape(m, d), host_u16(xs[1]).reshape(m, d)
            assert np.array_equal(got0, got1), "the ranks disagree"
            assert_close_fp16(got0, want_x, what="tp gather x", max_frac=0.1, abs_tol=np.abs(acc) * 2.0 ** -10 + tc_tol(acc, tp * k_local))
            want_x = f16(got0).astype(np.float64)   # carry the engine's own rounding forward
            assert np.array_equal(host_u16(xn[0]), host_u16(xn[1]))
            for row in (0, m - 1):
                assert np.array_equal(host_u16(xn[0]).reshape(m, d)[row], rmsnorm_ref(got0[row], gamma)), "fused RMSNorm row %d" % row
        for r in range(tp):
            assert pkg.lib.llmb_tp_advance(ex[r].data_ptr(), tp, d, 2, 1, None) == 0
    torch.cuda.synchronize()
    assert not host_u16(ws[:4096].view(torch.int16)).any(), "arrival counters not back to zero"
