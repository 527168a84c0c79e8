"""Thin Python handles over the host surface of include/llama3.h (same call order as the
reference driver src/main.cu:61-123)."""
import ctypes as C

import numpy as np

from . import Llama3Config, TensorStruct, check, lib


def _cfg_struct(cfg, max_seq):
    return Llama3Config(cfg.d_model, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, max_seq,
                        cfg.rope_theta, cfg.eps)


class Model:
    """init_llama3 -> load_safetensor_weights* -> to_cuda, or init_llama3 -> synthetic weights."""

    def __init__(self, n_layers):
        self.ptr = lib.init_llama3(n_layers)
        if not self.ptr:
            raise MemoryError("init_llama3 failed")

    @classmethod
    def from_safetensors(cls, cfg, paths, max_seq=2048, tp_rank=0, tp_size=1, streaming=True):
        m = cls(cfg.n_layers)
        if not streaming:
            check(lib.llama3_set_streaming(m.ptr, 0), "llama3_set_streaming")
        if tp_size > 1:
            check(lib.llama3_set_tp(m.ptr, tp_rank, tp_size), "llama3_set_tp")
        partial = Llama3Config(0, 0, 0, cfg.head_dim, 0, 0, max_seq, cfg.rope_theta, cfg.eps)
        check(lib.llama3_set_config(m.ptr, C.byref(partial)), "llama3_set_config")
        for p in paths:
            check(lib.llama3_load_safetensors(m.ptr, str(p).encode()), "load_safetensor_weights")
        check(lib.llama3_to_cuda(m.ptr), "to_cuda")
        return m

    @classmethod
    def synthetic(cls, cfg, seed=0, max_seq=2048, tp_rank=0, tp_size=1):
        m = cls(cfg.n_layers)
        if tp_size > 1:
            check(lib.llama3_set_tp(m.ptr, tp_rank, tp_size), "llama3_set_tp")
        c = _cfg_struct(cfg, max_seq)
        check(lib.llama3_synth_weights(m.ptr, C.byref(c), seed, 1 if cfg.bf16_weights else 0), "llama3_synth_weights")
        return m

    def upload_stats(self):
        """Figures of the last to_cuda(): seconds, bytes read from files, bytes uploaded, pinned staging bytes."""
        s, a, b, c = C.c_double(0), C.c_ulonglong(0), C.c_ulonglong(0), C.c_ulonglong(0)
        check(lib.llama3_upload_stats(self.ptr, C.byref(s), C.byref(a), C.byref(b), C.byref(c)), "llama3_upload_stats")
        return {"seconds": s.value, "bytes_read": a.value, "bytes_uploaded": b.value, "host_staging_bytes": c.value}

    @property
    def config(self):
        return self.ptr.contents.config

    def tensor_ptr(self, name, layer=None):
        """Device address of a weight tensor (FP16)."""
        if layer is None:
            t = getattr(self.ptr.contents, name)
        else:
            t = getattr(self.ptr.contents.layers[layer].contents, name)
        return t.contents.d_fp16_tensor

    def close(self):
        if self.ptr:
            lib.free_llama3(self.ptr)
            self.ptr = None


class Cache:
    """init_cache + inference(): KV cache, scratch and the captured decode step."""

    def __init__(self, model):
        self.model = model
        rc = C.c_int(0)
        self.ptr = lib.llama3_init_cache(model.ptr, C.byref(rc))
        if not self.ptr:
            check(rc.value or 1, "init_cache")
        self.tp_size = model.ptr.contents.tp_size
        self.tp_rank = model.ptr.contents.tp_rank
        self.vocab = model.config.vocab // self.tp_size  # this rank's slice of the logits
        self.max_seq = model.config.max_seq
        self._tokens = (C.c_int * (self.max_seq + 2))()
        self._x = TensorStruct()
        self._d_tokens = None

    def set_options(self, use_graph=-1, use_pdl=-1, copy_logits=-1, step_kernel=-1):
        check(lib.cache_set_options(self.ptr, int(use_graph), int(use_pdl), int(copy_logits)), "cache_set_options")
        if step_kernel >= 0:
            check(lib.cache_use_step_kernel(self.ptr, int(step_kernel)), "cache_use_step_kernel")

    def set_tp_poll_limit(self, limit):
        """Spin limit of the step kernel's waits for tensor-parallel peers (0 = default, about a second)."""
        check(lib.cache_set_tp_poll_limit(self.ptr, int(limit)), "cache_set_tp_poll_limit")

    def set_prefill(self, enable=True, min_rows=0):
        """Prompt tokens as blocks of rows through the tensor-core projections (default), or one by one
        through the decode step; `min_rows` > 0 changes the smallest run that takes the block path."""
        check(lib.cache_set_prefill(self.ptr, 1 if enable else 0, int(min_rows)), "cache_set_prefill")

    def tp_connect(self, group=None):
        """Exchanges the CUDA IPC handles of the ranks' exchange blocks over torch.distributed and maps the
        peers' blocks (one process per GPU; every rank calls this once before the first step)."""
        import torch
        import torch.distributed as dist
        mine = (C.c_ubyte * 64)()
        check(lib.cache_tp_handle(self.ptr, mine), "cache_tp_handle")
        t = torch.tensor(list(bytes(mine)), dtype=torch.uint8)
        use_cuda = dist.get_backend(group) == "nccl"
        if use_cuda:
            t = t.cuda()
        out = [torch.empty_like(t) for _ in range(self.tp_size)]
        dist.all_gather(out, t, group=group)
        blob = b"".join(bytes(o.cpu().tolist()) for o in out)
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        check(lib.cache_tp_connect(self.ptr, buf), "cache_tp_connect")
        dist.barrier(group=group)

    def reset(self):
        check(lib.cache_reset(self.ptr), "cache_reset")

    def infer(self, token_ids):
        """One reference-style inference() call on the whole id list; returns the next token."""
        n = len(token_ids)
        self._tokens[0] = n + 1
        self._tokens[1:n + 1] = [int(t) for t in token_ids]
        r = lib.inference(self.model.ptr, C.byref(self._x), self._d_tokens, self._tokens, self.ptr)
        if r < 0:
            check(-r, "inference")
        return r

    def logits(self):
        """FP16 logits of the last inference() call as a numpy uint16 bit-pattern array."""
        buf = (C.c_uint16 * self.vocab).from_address(self.ptr.contents.h_token_probdist)
        return np.frombuffer(buf, dtype=np.uint16).copy()

    def sample(self, temperature=0.7, top_k=50, top_p=0.9, seed=0, draw=0):
        """Temperature / top-k / top-p sample from the logits of the last infer() call (the reference's host
        sampler and its default constants); `draw` numbers the call."""
        r = lib.cache_sample_next_token(self.ptr, temperature, top_k, top_p, seed, draw)
        if r < 0:
            check(-r, "cache_sample_next_token")
        return r

    def sample_device(self, temperature=0.7, top_k=50, top_p=0.9, seed=0, draw=0):
        """The same sampling chain as sample(), run by one kernel on the device logits of the last step."""
        r = lib.cache_sample_next_token_device(self.ptr, temperature, top_k, top_p, seed, draw)
        if r < 0:
            check(-r, "cache_sample_next_token_device")
        return r

    def enable_hidden_dump(self, on=True):
        check(lib.cache_enable_hidden_dump(self.ptr, 1 if on else 0), "cache_enable_hidden_dump")

    def hidden(self):
        cfg = self.model.config
        out = np.empty((self.model.ptr.contents.n_layers + 1, cfg.d_model), dtype=np.uint16)
        check(lib.cache_read_hidden(self.ptr, out.ctypes.data), "cache_read_hidden")
        return out

    def greedy(self, prompt, n_new):
        """Device-resident greedy generation; returns (tokens, prefill_ms, decode_ms)."""
        p = (C.c_int * len(prompt))(*[int(t) for t in prompt])
        out = (C.c_int * n_new)()
        pre, dec = C.c_float(0), C.c_float(0)
        check(lib.inference_greedy(self.model.ptr, self.ptr, p, len(prompt), n_new, out, C.byref(pre), C.byref(dec)),
              "inference_greedy")
        return list(out), pre.value, dec.value

    def continue_greedy(self, n_steps):
        """n_steps more device-resident greedy steps from the current state; returns (tokens, ms)."""
        out = (C.c_int * n_steps)()
        ms = C.c_float(0)
        check(lib.inference_continue(self.model.ptr, self.ptr, n_steps, out, C.byref(ms)), "inference_continue")
        return list(out), ms.value

    # ---- batched decode: n_seqs sequences, one token each per step -------------------------------
    def batch_init(self, n_seqs):
        check(lib.cache_batch_init(self.ptr, int(n_seqs)), "cache_batch_init")
        self.n_seqs = int(n_seqs)

    def batch_set_split_len(self, split_len):
        """Cache rows per attention CTA of the batched step (a power of two, 32..512)."""
        check(lib.cache_batch_set_split_len(self.ptr, int(split_len)), "cache_batch_set_split_len")

    def batch_prefill(self, prompts):
        """prompts: [n_seqs][n_tokens] ids; the last token of each stays pending as the next step's input."""
        a = np.ascontiguousarray(prompts, dtype=np.int32)
        assert a.ndim == 2 and a.shape[0] == self.n_seqs
        check(lib.cache_batch_prefill(self.ptr, a.ctypes.data, a.shape[1]), "cache_batch_prefill")

    def batch_step(self, tokens=None, want_logits=True):
        """One step for every sequence; returns (next tokens [n_seqs], logits uint16 [n_seqs][vocab] or None)."""
        t = None if tokens is None else np.ascontiguousarray(tokens, dtype=np.int32)
        lg = np.empty((self.n_seqs, self.vocab), dtype=np.uint16) if want_logits else None
        nxt = np.empty(self.n_seqs, dtype=np.int32)
        check(lib.cache_batch_step(self.ptr, None if t is None else t.ctypes.data, None if lg is None else lg.ctypes.data,
                                   nxt.ctypes.data), "cache_batch_step")
        return nxt, lg

    def batch_greedy(self, n_steps):
        """n_steps device-resident greedy steps; returns (tokens [n_seqs][n_steps], ms)."""
        out = np.empty((self.n_seqs, int(n_steps)), dtype=np.int32)
        ms = C.c_float(0)
        check(lib.cache_batch_greedy(self.ptr, int(n_steps), out.ctypes.data, C.byref(ms)), "cache_batch_greedy")
        return out, ms.value

    def kernel_launches(self):
        return lib.cache_kernel_launches(self.ptr)

    def close(self):
        if self.ptr:
            lib.free_cache(self.ptr)
            self.ptr = None
