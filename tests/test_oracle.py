"""The CPU oracle against an independent float64 restatement (loose) and against its own
invariants (tight).  The tight pin against the reference binary lives in test_golden.py."""
import numpy as np
import pytest


def f64_forward(cfg, w, tokens, oracle):
    """Plain float64 LLaMA3 forward with the reference's conventions (interleaved RoPE, pos from 0,
    scale 1/sqrt(head_dim), eps 1e-5), no intermediate rounding."""
    g = lambda n: oracle.f16(w.fp16[n]).astype(np.float64).reshape(w.shapes[n])
    T, d, hd = len(tokens), cfg.d_model, cfg.head_dim
    x = g("model.embed_tokens.weight")[tokens]
    half = hd // 2
    freq = 1.0 / cfg.rope_theta ** (2.0 * np.arange(half) / hd)
    ang = np.arange(T)[:, None] * freq[None, :]
    cos, sin = np.cos(ang), np.sin(ang)

    def norm(v, gain):
        return v * gain / np.sqrt(cfg.eps + (v * v).mean(-1, keepdims=True))

    def rope(v, nh):
        v = v.reshape(T, nh, half, 2)
        e, o = v[..., 0], v[..., 1]
        out = np.stack([cos[:, None] * e - sin[:, None] * o, sin[:, None] * e + cos[:, None] * o], -1)
        return out.reshape(T, nh, hd)

    hidden = [x.copy()]
    for l in range(cfg.n_layers):
        p = "model.layers.%d." % l
        h = norm(x, g(p + "input_layernorm.weight"))
        q = rope(h @ g(p + "self_attn.q_proj.weight").T, cfg.n_q_heads)
        k = rope(h @ g(p + "self_attn.k_proj.weight").T, cfg.n_kv_heads)
        v = (h @ g(p + "self_attn.v_proj.weight").T).reshape(T, cfg.n_kv_heads, hd)
        grp = cfg.n_q_heads // cfg.n_kv_heads
        out = np.zeros((T, cfg.n_q_heads, hd))
        mask = np.tril(np.ones((T, T), bool))
        for hq in range(cfg.n_q_heads):
            s = q[:, hq] @ k[:, hq // grp].T / np.sqrt(hd)
            s = np.where(mask, s, -np.inf)
            pr = np.exp(s - s.max(-1, keepdims=True))
            pr /= pr.sum(-1, keepdims=True)
            out[:, hq] = pr @ v[:, hq // grp]
        x = x + out.reshape(T, -1) @ g(p + "self_attn.o_proj.weight").T
        h = norm(x, g(p + "post_attention_layernorm.weight"))
        gate, up = h @ g(p + "mlp.gate_proj.weight").T, h @ g(p + "mlp.up_proj.weight").T
        x = x + (gate / (1 + np.exp(-gate)) * up) @ g(p + "mlp.down_proj.weight").T
        hidden.append(x.copy())
    logits = norm(x, g("model.norm.weight")) @ g("lm_head.weight").T
    return logits, np.stack(hidden)


def test_forward_close_to_float64(pkg, oracle, tiny_weights):
    cfg = pkg.CONFIGS["tiny"]
    tokens = oracle.synth_tokens(0, 24, cfg.vocab)
    logits, hidden = oracle.forward(tiny_weights, tokens, want_hidden=True)
    ref_logits, ref_hidden = f64_forward(cfg, tiny_weights, tokens, oracle)
    got = oracle.f16(logits).astype(np.float64)
    # FP16 rounding points only: well inside the engine's own tolerance (2e-2 abs on logits)
    assert np.abs(got - ref_logits).max() < 5e-3
    hid = oracle.f16(hidden).astype(np.float64)
    for l in range(cfg.n_layers + 1):
        rel = np.linalg.norm(hid[l] - ref_hidden[l]) / np.linalg.norm(ref_hidden[l])
        assert rel < 2e-3, (l, rel)


def test_row_r_does_not_depend_on_later_rows(pkg, oracle, tiny_weights):
    """The property that lets one causal pass stand for the reference's per-step recomputation."""
    cfg = pkg.CONFIGS["tiny"]
    tokens = oracle.synth_tokens(0, 20, cfg.vocab)
    full, _ = oracle.forward(tiny_weights, tokens)
    for n in (1, 7, 20):
        part, _ = oracle.forward(tiny_weights, tokens[:n], first_logit_row=n - 1)
        assert np.array_equal(part[0], full[n - 1])


def test_cached_decoder_tracks_strict_forward(pkg, oracle, tiny_weights):
    cfg = pkg.CONFIGS["tiny"]
    tokens = oracle.synth_tokens(0, 16, cfg.vocab)
    full, _ = oracle.forward(tiny_weights, tokens)
    dec = oracle.Decoder(tiny_weights, 64)
    for i, t in enumerate(tokens):
        tok, lg = dec.step(t, want_logits=True)
        diff = np.abs(oracle.f16(lg) - oracle.f16(full[i])).max()
        assert diff < 4e-3, (i, diff)  # same rounding points, different FP32 summation order
    dec.close()


def test_bf16_to_fp16_matches_torch(oracle):
    torch = pytest.importorskip("torch")
    bits = np.arange(0, 1 << 16, dtype=np.uint16)  # every BF16 value
    got = oracle.bf16_to_fp16(bits)
    want = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(torch.float32).to(torch.float16)
    want = want.view(torch.int16).numpy().view(np.uint16)
    nan = np.isnan(got.view(np.float16))
    assert np.array_equal(nan, np.isnan(want.view(np.float16)))
    assert np.array_equal(got[~nan], want[~nan])


def test_argmax_first_maximum(oracle):
    v = np.array([1.0, 5.0, np.nan, 5.0, -np.inf], dtype=np.float16).view(np.uint16)
    assert oracle.lib().oracle_argmax_fp16(v.ctypes.data, len(v)) == 1
