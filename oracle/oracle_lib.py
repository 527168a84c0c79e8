"""TEST INFRASTRUCTURE ONLY: ctypes binding of oracle/liboracle.so (the CPU restatement of the
reference forward loop) plus helpers that build seeded weights for it.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may import
this module; the product package never does.
"""
import ctypes as C
import json
import os
import struct
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")
REF_HARNESS = os.path.join(HERE, "_ref", "ref_harness")

# stream ids of include/llm_b200_synth.h
SID_EMBED, SID_LM_HEAD, SID_NORM, SID_TOKENS = 1, 2, 3, 4
SLOTS = ["input_layernorm", "mlp_down_proj", "mlp_gate_proj", "mlp_up_proj", "post_attention_layernorm",
         "self_attn_k_proj", "self_attn_o_proj", "self_attn_q_proj", "self_attn_v_proj"]
HF_NAMES = {
    "input_layernorm": "model.layers.%d.input_layernorm.weight",
    "mlp_down_proj": "model.layers.%d.mlp.down_proj.weight",
    "mlp_gate_proj": "model.layers.%d.mlp.gate_proj.weight",
    "mlp_up_proj": "model.layers.%d.mlp.up_proj.weight",
    "post_attention_layernorm": "model.layers.%d.post_attention_layernorm.weight",
    "self_attn_k_proj": "model.layers.%d.self_attn.k_proj.weight",
    "self_attn_o_proj": "model.layers.%d.self_attn.o_proj.weight",
    "self_attn_q_proj": "model.layers.%d.self_attn.q_proj.weight",
    "self_attn_v_proj": "model.layers.%d.self_attn.v_proj.weight",
}


def layer_sid(layer, slot):
    return 16 + 16 * layer + slot


class OracleConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("d_model", C.c_int), ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("ffn", C.c_int), ("vocab", C.c_int), ("rope_theta", C.c_float),
                ("eps", C.c_double)]


def build(force=False):
    """Compiles liboracle.so (and, when the reference tree is present, oracle/_ref/ref_harness)."""
    src = os.path.join(HERE, "llama3_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "oracle"], check=True, capture_output=True)
    return LIB_PATH


def build_reference(ref_root=None):
    """Builds oracle/_ref/ref_harness from the reference sources if they are present. `ref_root` (or the
    environment variable LLM_CU_REFERENCE) names the reference checkout. Returns the path of the harness,
    or None when there is neither a checkout nor a prebuilt binary."""
    ref_root = ref_root or os.environ.get("LLM_CU_REFERENCE", "")
    if ref_root and os.path.isdir(os.path.join(ref_root, "src")):
        subprocess.run(["make", "-C", HERE, "ref", "REF=" + ref_root], check=True, capture_output=True)
    return REF_HARNESS if os.path.exists(REF_HARNESS) else None


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(LIB_PATH)
        vp, u64 = C.c_void_p, C.c_uint64
        l.oracle_bf16_to_fp16.argtypes = [vp, vp, C.c_size_t]
        l.oracle_bf16_to_fp16.restype = None
        l.oracle_forward.argtypes = [C.POINTER(OracleConfig), vp, vp, C.c_int, C.c_int, vp, vp]
        l.oracle_argmax_fp16.argtypes = [vp, C.c_int]
        l.oracle_sample.argtypes = [vp, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float]
        l.oracle_sampler_uniform.argtypes = [C.c_uint64, C.c_uint64]
        l.oracle_sampler_uniform.restype = C.c_float
        l.oracle_decoder_new.argtypes = [C.POINTER(OracleConfig), vp, C.c_int]
        l.oracle_decoder_new.restype = vp
        l.oracle_decoder_free.argtypes = [vp]
        l.oracle_decoder_free.restype = None
        l.oracle_decoder_reset.argtypes = [vp]
        l.oracle_decoder_reset.restype = None
        l.oracle_decoder_step.argtypes = [vp, C.c_int, vp]
        l.oracle_synth_bf16.argtypes = [u64, u64, C.c_float, u64, u64, vp]
        l.oracle_synth_bf16.restype = None
        l.oracle_synth_fp16.argtypes = [u64, u64, C.c_float, u64, u64, vp]
        l.oracle_synth_fp16.restype = None
        l.oracle_synth_tokens.argtypes = [u64, u64, C.c_int, u64, u64, vp]
        l.oracle_synth_tokens.restype = None
        l.oracle_fill_u16.argtypes = [C.c_uint16, u64, vp]
        l.oracle_fill_u16.restype = None
        l.oracle_num_threads.restype = C.c_int
        _lib = l
    return _lib


def synth_bf16(seed, sid, n, std=0.02, first=0):
    out = np.empty(n, dtype=np.uint16)
    lib().oracle_synth_bf16(seed, sid, std, first, n, out.ctypes.data)
    return out


def synth_fp16(seed, sid, n, std=0.02, first=0):
    out = np.empty(n, dtype=np.uint16)
    lib().oracle_synth_fp16(seed, sid, std, first, n, out.ctypes.data)
    return out


def synth_tokens(seed, n, vocab, sid=SID_TOKENS, first=0):
    """Token ids of the benchmark prompts: uniform in [0, vocab), stream of seed + 1."""
    out = np.empty(n, dtype=np.int32)
    lib().oracle_synth_tokens(seed + 1, sid, vocab, first, n, out.ctypes.data)
    return out


def bf16_to_fp16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty_like(a)
    lib().oracle_bf16_to_fp16(a.ctypes.data, out.ctypes.data, a.size)
    return out


class Weights:
    """Seeded random-init weights of a ModelConfig in host memory.

    `file` holds what a checkpoint would (BF16 or FP16 bit patterns), `fp16` what the engine
    holds after its load-time conversion (llama3.cu:240-254)."""

    def __init__(self, cfg, seed=0, keep_file=True, keep_fp16=True):
        self.cfg, self.seed = cfg, seed
        gen = synth_bf16 if cfg.bf16_weights else synth_fp16
        one = 0x3F80 if cfg.bf16_weights else 0x3C00
        d, F = cfg.d_model, cfg.ffn
        erows = cfg.embed_rows or cfg.vocab
        self.shapes, self.file, self.fp16 = {}, {}, {}

        def put(name, sid, shape, norm=False):
            n = int(np.prod(shape))
            self.shapes[name] = tuple(shape)
            raw = np.full(n, one, dtype=np.uint16) if norm else gen(seed, sid, n)
            if keep_fp16:
                self.fp16[name] = bf16_to_fp16(raw) if cfg.bf16_weights else raw
            if keep_file:
                self.file[name] = raw

        put("model.embed_tokens.weight", SID_EMBED, (erows, d))
        put("lm_head.weight", SID_LM_HEAD, (cfg.vocab, d))
        put("model.norm.weight", SID_NORM, (d,), norm=True)
        dims = {"input_layernorm": (d,), "mlp_down_proj": (d, F), "mlp_gate_proj": (F, d), "mlp_up_proj": (F, d),
                "post_attention_layernorm": (d,), "self_attn_k_proj": (cfg.kv_rows, d),
                "self_attn_o_proj": (d, cfg.q_rows), "self_attn_q_proj": (cfg.q_rows, d),
                "self_attn_v_proj": (cfg.kv_rows, d)}
        for l in range(cfg.n_layers):
            for slot, s in enumerate(SLOTS):
                put(HF_NAMES[s] % l, layer_sid(l, slot), dims[s], norm="layernorm" in s)

    def oracle_pointers(self):
        """Flat pointer array in the order oracle_forward expects (llama3_oracle.h)."""
        names = ["model.embed_tokens.weight", "lm_head.weight", "model.norm.weight"]
        for l in range(self.cfg.n_layers):
            names += [HF_NAMES[s] % l for s in SLOTS]
        arr = (C.c_void_p * len(names))(*[self.fp16[n].ctypes.data for n in names])
        return arr

    def oracle_config(self):
        c = self.cfg
        return OracleConfig(c.n_layers, c.d_model, c.n_q_heads, c.n_kv_heads, c.head_dim, c.ffn, c.vocab,
                            c.rope_theta, c.eps)

    def write_safetensors(self, path, names=None):
        """Writes the tensors (all, or the listed ones) as one safetensors shard with HF key names."""
        names = list(self.file) if names is None else list(names)
        header, off = {}, 0
        for n in names:
            nbytes = self.file[n].size * 2
            header[n] = {"dtype": "BF16" if self.cfg.bf16_weights else "F16", "shape": list(self.shapes[n]),
                         "data_offsets": [off, off + nbytes]}
            off += nbytes
        header["__metadata__"] = {"format": "pt"}
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            for n in names:
                f.write(self.file[n].tobytes())
        return path


def forward(weights, tokens, first_logit_row=0, want_hidden=False):
    """Teacher-forced causal pass of the strict oracle. Returns (logits uint16 [rows][vocab], hidden or None)."""
    cfg = weights.cfg
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    T = len(tokens)
    logits = np.empty((T - first_logit_row, cfg.vocab), dtype=np.uint16)
    hidden = np.empty((cfg.n_layers + 1, T, cfg.d_model), dtype=np.uint16) if want_hidden else None
    oc = weights.oracle_config()
    ptrs = weights.oracle_pointers()
    rc = lib().oracle_forward(C.byref(oc), ptrs, tokens.ctypes.data, T, first_logit_row, logits.ctypes.data,
                              hidden.ctypes.data if want_hidden else None)
    if rc != 0:
        raise RuntimeError("oracle_forward failed: %d" % rc)
    return logits, hidden


class Decoder:
    """KV-cached CPU decoder (timed CPU baseline)."""

    def __init__(self, weights, max_pos):
        self.weights = weights
        self._oc = weights.oracle_config()
        self._ptrs = weights.oracle_pointers()
        self.h = lib().oracle_decoder_new(C.byref(self._oc), self._ptrs, max_pos)
        self.vocab = weights.cfg.vocab

    def step(self, token, want_logits=False):
        lg = np.empty(self.vocab, dtype=np.uint16) if want_logits else None
        t = lib().oracle_decoder_step(self.h, int(token), lg.ctypes.data if want_logits else None)
        return (t, lg) if want_logits else t

    def reset(self):
        lib().oracle_decoder_reset(self.h)

    def close(self):
        if self.h:
            lib().oracle_decoder_free(self.h)
            self.h = None


def f16(a):
    """uint16 bit patterns -> float32 values."""
    return np.asarray(a, dtype=np.uint16).view(np.float16).astype(np.float32)
