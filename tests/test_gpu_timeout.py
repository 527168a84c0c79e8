"""A bounded device-side wait that runs out, made to do so on purpose in the allowed form: the whole-step
kernel is launched as rank 0 of a tensor-parallel pair whose rank 1 is a zeroed local block that nobody
ever writes, with a spin limit of a few thousand polls.  Nothing faults and nothing spins without a bound:
the kernel gives up, records status 205, runs to its end; the next launch sees the sticky status and takes
no wait at all; llmb_device_status() reports the code once and clears it."""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_tensor_parallel_wait_gives_up_and_recovers(pkg):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    cfg = pkg.CONFIGS["tiny"]
    model = pkg.Model.synthetic(cfg, seed=0, max_seq=64)
    L, d, hd = cfg.n_layers, cfg.d_model, cfg.head_dim
    nq, nkv, ffn, vocab = cfg.n_q_heads // 2, cfg.n_kv_heads // 2, cfg.ffn // 2, cfg.vocab // 2  # rank 0's shares
    max_pos = 64
    z16 = lambda n: torch.zeros(n, dtype=torch.int16, device="cuda")
    kc, vc = z16(L * max_pos * nkv * hd), z16(L * max_pos * nkv * hd)
    layers = (pkg.LayerArgs * L)()
    for l in range(L):
        # any readable weights of at least the shard's size do: the results of this test are never looked at
        layers[l].wqkv = model.tensor_ptr("self_attn_q_proj", l)
        layers[l].wo = model.tensor_ptr("self_attn_o_proj", l)
        layers[l].wgate = model.tensor_ptr("mlp_gate_proj", l)
        layers[l].wup = model.tensor_ptr("mlp_up_proj", l)
        layers[l].wdown = model.tensor_ptr("mlp_down_proj", l)
        layers[l].g_in = model.tensor_ptr("input_layernorm", l)
        layers[l].g_post = model.tensor_ptr("post_attention_layernorm", l)
        layers[l].k_cache = kc.data_ptr() + l * max_pos * nkv * hd * 2
        layers[l].v_cache = vc.data_ptr() + l * max_pos * nkv * hd * 2
    d_layers = torch.from_numpy(np.frombuffer(bytes(layers), dtype=np.uint8).copy()).cuda()
    hist = torch.zeros(max_pos + 1, dtype=torch.int32, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    nxt = torch.zeros(1, dtype=torch.int32, device="cuda")
    x, x_alt, q, attn, h, logits = z16(d), z16(d), z16(nq * hd), z16(nq * hd), z16(ffn), z16(vocab)
    max_splits = 2
    scratch = torch.zeros(pkg.lib.llmb_decode_step_scratch_bytes(nq, nkv, hd, max_splits), dtype=torch.uint8, device="cuda")
    xbytes = pkg.lib.llmb_decode_step_exchange_bytes(2, d)
    mine = torch.zeros(xbytes, dtype=torch.uint8, device="cuda")
    absent_peer = torch.zeros(xbytes, dtype=torch.uint8, device="cuda")  # rank 1 never launches: its tags never come
    a = pkg.DecodeStepArgs()
    a.layers, a.n_layers, a.d_model, a.n_q_heads, a.n_kv_heads, a.head_dim = d_layers.data_ptr(), L, d, nq, nkv, hd
    a.ffn, a.vocab, a.embed_rows, a.max_pos, a.rope_theta, a.eps = ffn, vocab, cfg.vocab, max_pos, cfg.rope_theta, cfg.eps
    a.embed, a.lm_head, a.g_final = model.tensor_ptr("embed_tokens"), model.tensor_ptr("lm_head"), model.tensor_ptr("norm")
    a.history, a.history_len, a.pos = hist.data_ptr(), max_pos + 1, pos.data_ptr()
    a.x, a.q, a.attn, a.h, a.logits, a.next_token = x.data_ptr(), q.data_ptr(), attn.data_ptr(), h.data_ptr(), logits.data_ptr(), nxt.data_ptr()
    a.scratch, a.max_splits, a.n_splits, a.split_len, a.with_logits = scratch.data_ptr(), max_splits, 1, 32, 1
    a.tp_rank, a.tp_size, a.vocab_offset, a.x_alt = 0, 2, 0, x_alt.data_ptr()
    a.peers[0], a.peers[1] = mine.data_ptr(), absent_peer.data_ptr()
    a.tag_poll_limit = 4096
    st = C.c_int(-1)
    pkg.check(pkg.lib.llmb_device_status(C.byref(st)), "llmb_device_status")  # start from a clean word
    stream = torch.cuda.current_stream().cuda_stream

    t0 = time.perf_counter()
    assert pkg.lib.llmb_decode_step(C.byref(a), stream) == 0, pkg.lib.llmb_last_error()
    torch.cuda.synchronize()
    first_s = time.perf_counter() - t0
    assert first_s < 5.0, "the wait did not give up within its limit (%.1f s)" % first_s
    # the status word is sticky: a second launch takes no wait at all and returns at once
    t0 = time.perf_counter()
    assert pkg.lib.llmb_decode_step(C.byref(a), stream) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    pkg.check(pkg.lib.llmb_device_status(C.byref(st)), "llmb_device_status")
    assert st.value == 205, st.value       # a tensor-parallel peer did not deliver its partial sums
    pkg.check(pkg.lib.llmb_device_status(C.byref(st)), "llmb_device_status")
    assert st.value == 0                   # reported once, then cleared
    # the context is intact: an ordinary single-GPU engine works right afterwards
    cache = pkg.Cache(model)
    toks, _, _ = cache.greedy([1, 2, 3, 4], 3)
    assert len(toks) == 3
    cache.close()
    model.close()
