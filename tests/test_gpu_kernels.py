"""Kernel-level parity through the C-ABI (include/llm_b200.h) on a B200."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from gpu_util import assert_close_fp16, dev, f16, host_u16, rmsnorm_ref, to_f16_bits  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def check_status(pkg):
    st = C.c_int(-1)
    assert pkg.lib.llmb_device_status(C.byref(st)) == 0, pkg.lib.llmb_last_error()
    assert st.value == 0, "device status %d" % st.value


def rand_w(oracle, sid, n, k, std=0.02):
    return oracle.synth_fp16(123, sid, n * k, std=std).reshape(n, k)


def test_bf16_to_fp16_every_pattern_and_ragged(pkg, oracle):
    bits = np.arange(0, 1 << 16, dtype=np.uint16)
    for n, off in ((65536, 0), (65533, 0), (7, 0), (1000, 3)):
        src = dev(np.concatenate([np.zeros(off, np.uint16), bits[:n]]))
        dst = torch.zeros(off + n, dtype=torch.int16, device="cuda")
        rc = pkg.lib.llmb_bf16_to_fp16(src.data_ptr() + 2 * off, dst.data_ptr() + 2 * off, n, None)
        assert rc == 0
        got = host_u16(dst)[off:]
        want = oracle.bf16_to_fp16(bits[:n])
        nan = np.isnan(want.view(np.float16))
        assert np.array_equal(got[~nan], want[~nan])
        assert np.isnan(got.view(np.float16)[nan]).all()


def test_synth_matches_cpu_generator(pkg, oracle):
    n = 100003
    out = torch.zeros(n, dtype=torch.int16, device="cuda")
    assert pkg.lib.llmb_synth_bf16(out.data_ptr(), 5, 77, 0.02, 11, n, None) == 0
    assert np.array_equal(host_u16(out), oracle.synth_bf16(5, 77, n, first=11))
    assert pkg.lib.llmb_synth_fp16(out.data_ptr(), 5, 78, 0.02, 0, n, None) == 0
    assert np.array_equal(host_u16(out), oracle.synth_fp16(5, 78, n))


def gemv(pkg, **kw):
    a = pkg.GemvArgs()
    for k, v in kw.items():
        setattr(a, k, v.data_ptr() if hasattr(v, "data_ptr") else v)
    rc = pkg.lib.llmb_gemv_f16(C.byref(a), None)
    assert rc == 0, (rc, pkg.lib.llmb_last_error())
    torch.cuda.synchronize()


@pytest.mark.parametrize("n,k", [(4096, 4096), (1003, 256), (6144, 4096), (4096, 14336), (3, 4096), (1024, 8192),
                                 (257, 512), (4096, 1792), (33, 2048)])
@pytest.mark.parametrize("pdl", [0, 1])
def test_gemv_store(pkg, oracle, n, k, pdl):
    w = rand_w(oracle, 1, n, k)
    x = oracle.synth_fp16(9, 2, k, std=1.0)
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    gemv(pkg, w=dev(w), x=dev(x), y=y, n=n, k=k, epilogue=pkg.EPI_STORE, use_pdl=pdl)
    want = f16(w).astype(np.float64) @ f16(x).astype(np.float64)
    assert_close_fp16(host_u16(y), want, what="store %dx%d" % (n, k))
    check_status(pkg)


def test_gemv_lm_head_shape(pkg, oracle):
    n, k = 128256, 4096
    w = torch.zeros(n * k, dtype=torch.int16, device="cuda")
    assert pkg.lib.llmb_synth_fp16(w.data_ptr(), 1, 2, 0.02, 0, n * k, None) == 0
    x = oracle.synth_fp16(9, 2, k, std=1.0)
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    gemv(pkg, w=w, x=dev(x), y=y, n=n, k=k, epilogue=pkg.EPI_STORE, use_pdl=1)
    rows = np.r_[0:64, 64000:64064, n - 64:n]
    wh = np.stack([oracle.synth_fp16(1, 2, k, first=int(r) * k) for r in rows])
    want = f16(wh).astype(np.float64) @ f16(x).astype(np.float64)
    assert_close_fp16(host_u16(y)[rows], want, what="lm_head rows")
    check_status(pkg)


@pytest.mark.parametrize("k", [256, 4096, 8192])
def test_gemv_rmsnorm_prologue_uses_reference_tree(pkg, oracle, k):
    n = 512
    w = rand_w(oracle, 3, n, k)
    x = oracle.synth_fp16(9, 4, k, std=0.7)
    g = to_f16_bits(1.0 + 0.1 * f16(oracle.synth_fp16(9, 5, k, std=1.0)))
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    gemv(pkg, w=dev(w), x=dev(x), y=y, n=n, k=k, prologue=pkg.PRO_RMSNORM, gamma=dev(g), eps=1e-5,
         epilogue=pkg.EPI_STORE)
    xn = rmsnorm_ref(x, g)
    want = f16(w).astype(np.float64) @ f16(xn).astype(np.float64)
    assert_close_fp16(host_u16(y), want, what="rmsnorm k=%d" % k)
    # identity weights expose the normalised vector itself: must be bit-exact (same tree, same division)
    eye = np.zeros((k, k), dtype=np.float16)
    np.fill_diagonal(eye, 1.0)
    y2 = torch.zeros(k, dtype=torch.int16, device="cuda")
    gemv(pkg, w=dev(eye.view(np.uint16)), x=dev(x), y=y2, n=k, k=k, prologue=pkg.PRO_RMSNORM, gamma=dev(g), eps=1e-5,
         epilogue=pkg.EPI_STORE)
    assert np.array_equal(host_u16(y2), xn)
    check_status(pkg)


def test_gemv_residual(pkg, oracle):
    n, k = 4096, 14336
    w = rand_w(oracle, 6, n, k)
    x = oracle.synth_fp16(9, 7, k, std=0.5)
    res = oracle.synth_fp16(9, 8, n, std=1.0)
    y = dev(res.copy())
    gemv(pkg, w=dev(w), x=dev(x), y=y, n=n, k=k, epilogue=pkg.EPI_RESIDUAL, use_pdl=1)
    acc = (f16(w).astype(np.float64) @ f16(x).astype(np.float64)).astype(np.float16).astype(np.float64)
    # the projection is rounded to FP16 before the add: one ulp of it may exceed an ulp of a small sum
    assert_close_fp16(host_u16(y), acc + f16(res).astype(np.float64), max_ulp=2, what="residual",
                      abs_tol=np.abs(acc) * 2.0 ** -10)
    check_status(pkg)


@pytest.mark.parametrize("n,k", [(14336, 4096), (768, 256), (1001, 4096), (1792, 8192)])
def test_gemv_swiglu(pkg, oracle, n, k):
    wg, wu = rand_w(oracle, 10, n, k), rand_w(oracle, 11, n, k)
    x = oracle.synth_fp16(9, 12, k, std=1.0)
    y = torch.zeros(n, dtype=torch.int16, device="cuda")
    gemv(pkg, w=dev(wg), w2=dev(wu), x=dev(x), y=y, n=n, k=k, epilogue=pkg.EPI_SWIGLU, use_pdl=1)
    xf = f16(x).astype(np.float64)
    gate, up = f16(wg).astype(np.float64) @ xf, f16(wu).astype(np.float64) @ xf
    want = gate / (1.0 + np.exp(-gate)) * up
    assert_close_fp16(host_u16(y), want, what="swiglu")
    check_status(pkg)


@pytest.mark.parametrize("nq,nkv,hd,k", [(32, 8, 128, 4096), (4, 2, 64, 256), (64, 8, 128, 8192)])
def test_gemv_rope_kv(pkg, oracle, nq, nkv, hd, k):
    n_q, n_kv = nq * hd, nkv * hd
    n = n_q + 2 * n_kv
    pos, max_pos = 37, 64
    w = rand_w(oracle, 13, n, k)
    x = oracle.synth_fp16(9, 14, k, std=1.0)
    half = hd // 2
    cs = torch.zeros(half * 2, dtype=torch.float32, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    dpos = torch.full((1,), pos, dtype=torch.int32, device="cuda")
    emb = torch.zeros(k, dtype=torch.int16, device="cuda")
    xo = torch.zeros(k, dtype=torch.int16, device="cuda")
    assert pkg.lib.llmb_embed_rope(emb.data_ptr(), tok.data_ptr(), dpos.data_ptr(), 1, k, 1, hd, 500000.0,
                                   xo.data_ptr(), cs.data_ptr(), 0, 0, None) == 0
    q = torch.zeros(n_q, dtype=torch.int16, device="cuda")
    kc = torch.zeros(max_pos * n_kv, dtype=torch.int16, device="cuda")
    vc = torch.zeros(max_pos * n_kv, dtype=torch.int16, device="cuda")
    gemv(pkg, w=dev(w), x=dev(x), y=q, n=n, k=k, epilogue=pkg.EPI_ROPE_KV, n_q=n_q, n_kv=n_kv, head_dim=hd,
         rope_cs=cs, k_cache=kc, v_cache=vc, pos=dpos, max_pos=max_pos, use_pdl=1)
    csh = cs.cpu().numpy().reshape(half, 2).astype(np.float64)
    # angles: FP32 formula of the reference, compared loosely against float64
    ang = pos * (1.0 / 500000.0 ** (2.0 * np.arange(half) / hd))
    assert np.abs(csh[:, 0] - np.cos(ang)).max() < 2e-5 and np.abs(csh[:, 1] - np.sin(ang)).max() < 2e-5
    raw = (f16(w).astype(np.float64) @ f16(x).astype(np.float64)).astype(np.float16).astype(np.float64)

    def rope(v):
        v = v.reshape(-1, half, 2)
        e, o = v[..., 0], v[..., 1]
        return np.stack([csh[:, 0] * e - csh[:, 1] * o, csh[:, 1] * e + csh[:, 0] * o], -1).reshape(-1)

    # two roundings (projection, rotation): allow 2 ulp
    def pair_mag(v):  # a rotated value mixes both elements of its pair, each rounded to FP16 first
        m = np.abs(v).reshape(-1, 2).max(axis=1)
        return np.repeat(m, 2) * 2.0 ** -10
    assert_close_fp16(host_u16(q), rope(raw[:n_q]), max_ulp=2, what="q", abs_tol=pair_mag(raw[:n_q]))
    kc_h, vc_h = host_u16(kc).reshape(max_pos, n_kv), host_u16(vc).reshape(max_pos, n_kv)
    assert_close_fp16(kc_h[pos], rope(raw[n_q:n_q + n_kv]), max_ulp=2, what="k", abs_tol=pair_mag(raw[n_q:n_q + n_kv]))
    assert_close_fp16(vc_h[pos], raw[n_q + n_kv:], what="v")
    others = np.delete(np.arange(max_pos), pos)
    assert not kc_h[others].any() and not vc_h[others].any()
    check_status(pkg)


@pytest.mark.parametrize("nq,nkv,hd", [(32, 8, 128), (4, 2, 64), (64, 8, 128)])
@pytest.mark.parametrize("length,n_splits,split_len", [(1, 16, 32), (31, 16, 32), (33, 16, 32), (129, 16, 32),
                                                        (512, 16, 32), (700, 16, 64), (2048, 16, 128),
                                                        (3000, 32, 128), (300, 2, 256)])
def test_attn_decode(pkg, oracle, nq, nkv, hd, length, n_splits, split_len):
    max_pos = max(length, 8)
    q = oracle.synth_fp16(21, 1, nq * hd, std=1.0)
    kc = oracle.synth_fp16(21, 2, max_pos * nkv * hd, std=1.0)
    vc = oracle.synth_fp16(21, 3, max_pos * nkv * hd, std=1.0)
    out = torch.zeros(nq * hd, dtype=torch.int16, device="cuda")
    nbytes = pkg.lib.llmb_attn_decode_scratch_bytes(nq, nkv, hd, n_splits)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    dpos = torch.full((1,), length - 1, dtype=torch.int32, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    for _ in range(2):  # second call checks that the counters were left at zero
        out.zero_()
        rc = pkg.lib.llmb_attn_decode(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dpos.data_ptr(), nq, nkv, hd,
                                      n_splits, split_len, out.data_ptr(), scratch.data_ptr(), 1, None)
        assert rc == 0, pkg.lib.llmb_last_error()
        qf = f16(q).astype(np.float64).reshape(nq, hd)
        kf = f16(kc).astype(np.float64).reshape(max_pos, nkv, hd)[:length]
        vf = f16(vc).astype(np.float64).reshape(max_pos, nkv, hd)[:length]
        grp = nq // nkv
        want = np.zeros((nq, hd))
        for h in range(nq):
            s = kf[:, h // grp] @ qf[h] / np.sqrt(hd)
            p = np.exp(s - s.max())
            want[h] = (p / p.sum()) @ vf[:, h // grp]
        assert_close_fp16(host_u16(out), want.reshape(-1), what="attn L=%d" % length)
    assert not scratch[: 4 * nkv].any()
    check_status(pkg)


def test_argmax_first_maximum_and_bookkeeping(pkg):
    n = 128256
    v = np.random.default_rng(0).standard_normal(n).astype(np.float16)
    v[[5, 70000, 128255]] = 9.0  # three-way tie: the first wins
    v[100] = np.nan
    logits = dev(v.view(np.uint16))
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    pos = torch.full((1,), 41, dtype=torch.int32, device="cuda")
    hist = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert pkg.lib.llmb_argmax_f16(logits.data_ptr(), n, tok.data_ptr(), pos.data_ptr(), hist.data_ptr(), 64, 0,
                                   None) == 0
    torch.cuda.synchronize()
    assert tok.item() == 5 and pos.item() == 42 and hist[42].item() == 5
    v[5] = 1.0
    logits = dev(v.view(np.uint16))
    assert pkg.lib.llmb_argmax_f16(logits.data_ptr(), n - 3, tok.data_ptr(), None, None, 0, 0, None) == 0
    torch.cuda.synchronize()
    assert tok.item() == 70000


def test_embed_rope_rows(pkg, oracle):
    d, vocab, hd = 256, 50, 64
    emb = oracle.synth_fp16(4, 4, vocab * d).reshape(vocab, d)
    toks = np.array([3, 49, 0, 77, -2], dtype=np.int32)  # out-of-range ids are clamped, never read past the table
    pos = np.array([0, 5, 100, 2000, 7], dtype=np.int32)
    x = torch.zeros(len(toks) * d, dtype=torch.int16, device="cuda")
    cs = torch.zeros(len(toks) * hd, dtype=torch.float32, device="cuda")
    assert pkg.lib.llmb_embed_rope(dev(emb).data_ptr(), dev(toks).data_ptr(), dev(pos).data_ptr(), len(toks), d,
                                   vocab, hd, 500000.0, x.data_ptr(), cs.data_ptr(), 0, 0, None) == 0
    got = host_u16(x).reshape(len(toks), d)
    assert np.array_equal(got, emb[np.clip(toks, 0, vocab - 1)])
    csh = cs.cpu().numpy().reshape(len(toks), hd // 2, 2)
    freq = (1.0 / np.float32(500000.0) ** (np.float32(2.0) * np.arange(hd // 2, dtype=np.float32) / np.float32(hd)))
    ang = pos[:, None].astype(np.float64) * freq[None, :].astype(np.float64)
    assert np.abs(csh[..., 0] - np.cos(ang)).max() < 3e-4 and np.abs(csh[..., 1] - np.sin(ang)).max() < 3e-4
