"""ctypes binding of libllm_b200.so: the sm_100a kernels (include/llm_b200.h) and the host
surface that mirrors the reference engine's entry points (include/llama3.h).

The directory name contains a dot, so load the package by path::

    spec = importlib.util.spec_from_file_location(
        "llm_cu_b200", "<repo>/llm.cu_b200/__init__.py",
        submodule_search_locations=["<repo>/llm.cu_b200"])

There is no CPU fallback: importing raises if the shared library has not been built
(`python llm.cu_b200/build.py`), and every compute call goes to the CUDA library.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libllm_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_IO, ERR_NOMEM = range(7)
PRO_NONE, PRO_RMSNORM = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_ROPE_KV, EPI_SWIGLU, EPI_TP_SCATTER = 0, 1, 2, 3, 4

# Symbols include/llm_b200.h and include/llama3.h declare; tests check each is exported.
KERNEL_SYMBOLS = [
    "llmb_last_error", "llmb_device_status", "llmb_build_info", "llmb_bf16_to_fp16", "llmb_synth_bf16",
    "llmb_synth_fp16", "llmb_synth_2d", "llmb_fill_u16", "llmb_embed_rope", "llmb_gemv_f16", "llmb_attn_decode_scratch_bytes",
    "llmb_attn_decode", "llmb_attn_decode_batch_scratch_bytes", "llmb_attn_decode_batch", "llmb_attn_decode_trace", "llmb_attn_decode_static", "llmb_argmax_rows_f16", "llmb_argmax_f16", "llmb_advance_pos", "llmb_gemm_f16",
    "llmb_rmsnorm_rows", "llmb_tp_gather_rows", "llmb_tp_argmax_rows", "llmb_tp_advance", "llmb_attn_prefill", "llmb_iota_i32", "llmb_sample_logits_host", "llmb_sampler_uniform", "llmb_sample_scratch_bytes", "llmb_sample_logits", "llmb_decode_step_scratch_bytes", "llmb_decode_step_exchange_bytes", "llmb_decode_step",
]
HOST_SYMBOLS = [
    "init_llama3", "free_llama3", "_free_tensor", "load_safetensor_weights", "to_cuda", "init_cache",
    "tokens_to_cuda", "inference", "llama3_set_config", "llama3_set_tp", "llama3_load_safetensors", "llama3_set_streaming", "llama3_upload_stats",
    "llama3_to_cuda", "llama3_tensor_shard", "llama3_synth_weights", "llama3_init_cache", "free_cache", "cache_reset",
    "cache_set_options", "cache_use_step_kernel", "cache_set_tp_poll_limit", "cache_tp_handle", "cache_tp_connect", "cache_enable_hidden_dump", "cache_read_hidden", "inference_greedy", "inference_continue", "cache_debug_read", "cache_debug_trace",
    "cache_kernel_launches", "cache_set_prefill", "cache_sample_next_token", "cache_sample_next_token_device", "cache_batch_init", "cache_batch_set_split_len", "cache_batch_prefill",
    "cache_batch_step", "cache_batch_greedy", "cache_debug_rows_trace",
]


class LlmbError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib.llmb_last_error().decode("utf-8", "replace") if lib is not None else ""
        super().__init__("%s failed with status %d%s" % (where, code, (": " + msg) if msg else ""))


class TensorStruct(C.Structure):
    _fields_ = [
        ("ndim", C.POINTER(C.c_int)), ("mem_len", C.POINTER(C.c_int)), ("shape", C.POINTER(C.c_int)),
        ("bf16_tensor", C.c_void_p), ("d_ndim", C.c_void_p), ("d_mem_len", C.c_void_p), ("d_shape", C.c_void_p),
        ("d_bf16_tensor", C.c_void_p), ("d_fp16_tensor", C.c_void_p), ("file_dtype", C.c_int),
        ("device_is_view", C.c_int), ("loaded", C.c_int),
    ]


class Llama3LayerStruct(C.Structure):
    _fields_ = [("layernum", C.c_int)] + [
        (n, C.POINTER(TensorStruct))
        for n in ("input_layernorm", "mlp_down_proj", "mlp_gate_proj", "mlp_up_proj", "post_attention_layernorm",
                  "self_attn_k_proj", "self_attn_o_proj", "self_attn_q_proj", "self_attn_v_proj")
    ]


class Llama3Config(C.Structure):
    _fields_ = [
        ("d_model", C.c_int), ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
        ("ffn", C.c_int), ("vocab", C.c_int), ("max_seq", C.c_int), ("rope_theta", C.c_float), ("eps", C.c_double),
    ]


class Llama3Struct(C.Structure):
    _fields_ = [
        ("embed_tokens", C.POINTER(TensorStruct)), ("lm_head", C.POINTER(TensorStruct)),
        ("norm", C.POINTER(TensorStruct)), ("layers", C.POINTER(C.POINTER(Llama3LayerStruct))),
        ("n_layers", C.c_int), ("config", Llama3Config), ("config_ready", C.c_int), ("tp_rank", C.c_int),
        ("tp_size", C.c_int), ("priv", C.c_void_p),
    ]


class CudaCacheStruct(C.Structure):
    _fields_ = [
        ("PN_X", C.POINTER(TensorStruct)), ("Q", C.POINTER(TensorStruct)), ("K", C.POINTER(TensorStruct)),
        ("V", C.POINTER(TensorStruct)), ("d_attention_score_cache", C.c_void_p),
        ("d_feedforward_cache_upgate", C.c_void_p), ("d_token_probdist", C.c_void_p),
        ("h_token_probdist", C.c_void_p), ("f_token_probdist", C.c_void_p), ("priv", C.c_void_p),
    ]


class GemvArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("w2", C.c_void_p), ("x", C.c_void_p), ("y", C.c_void_p), ("n", C.c_int), ("k", C.c_int),
        ("prologue", C.c_int), ("gamma", C.c_void_p), ("eps", C.c_double), ("epilogue", C.c_int), ("n_q", C.c_int),
        ("n_kv", C.c_int), ("head_dim", C.c_int), ("rope_cs", C.c_void_p), ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p), ("pos", C.c_void_p), ("max_pos", C.c_int), ("use_pdl", C.c_int),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("b2", C.c_void_p), ("c", C.c_void_p), ("m", C.c_int), ("n", C.c_int),
        ("k", C.c_int), ("epilogue", C.c_int), ("n_q", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int),
        ("rope_cs", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("pos0", C.c_int),
        ("max_pos", C.c_int), ("tile_n", C.c_int), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("row_pos", C.c_void_p), ("seq_stride", C.c_int), ("use_pdl", C.c_int),
        ("tp_peers", C.c_void_p * 8), ("tp_rank", C.c_int), ("tp_size", C.c_int), ("tp_index", C.c_int),
        ("trace", C.c_void_p),
    ]


class LayerArgs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wqkv", "wo", "wgate", "wup", "wdown", "g_in", "g_post", "k_cache", "v_cache")]


class DecodeStepArgs(C.Structure):
    _fields_ = [("layers", C.c_void_p)] + [
        (n, C.c_int) for n in ("n_layers", "d_model", "n_q_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "embed_rows",
                               "max_pos")] + [
        ("rope_theta", C.c_float), ("eps", C.c_double), ("embed", C.c_void_p), ("lm_head", C.c_void_p),
        ("g_final", C.c_void_p), ("history", C.c_void_p), ("history_len", C.c_int), ("pos", C.c_void_p),
        ("x", C.c_void_p), ("q", C.c_void_p), ("attn", C.c_void_p), ("h", C.c_void_p), ("logits", C.c_void_p),
        ("next_token", C.c_void_p), ("scratch", C.c_void_p), ("max_splits", C.c_int), ("n_splits", C.c_int),
        ("split_len", C.c_int), ("with_logits", C.c_int), ("hidden", C.c_void_p), ("tp_rank", C.c_int),
        ("tp_size", C.c_int), ("vocab_offset", C.c_int), ("x_alt", C.c_void_p), ("peers", C.c_void_p * 8),
        ("trace", C.c_void_p), ("tag_poll_limit", C.c_uint32),
    ]


def _declare(l):
    vp, i32, u64, sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
    l.llmb_last_error.restype = C.c_char_p
    l.llmb_build_info.restype = C.c_char_p
    l.llmb_device_status.argtypes = [C.POINTER(C.c_int)]
    l.llmb_bf16_to_fp16.argtypes = [vp, vp, sz, vp]
    l.llmb_synth_bf16.argtypes = [vp, u64, u64, C.c_float, u64, u64, vp]
    l.llmb_synth_fp16.argtypes = [vp, u64, u64, C.c_float, u64, u64, vp]
    l.llmb_synth_2d.argtypes = [vp, u64, u64, C.c_float, i32, u64, u64, u64, u64, vp]
    l.llmb_fill_u16.argtypes = [vp, C.c_uint16, u64, vp]
    l.llmb_embed_rope.argtypes = [vp, vp, vp, i32, i32, i32, i32, C.c_float, vp, vp, i32, i32, vp]
    l.llmb_gemv_f16.argtypes = [C.POINTER(GemvArgs), vp]
    l.llmb_attn_decode_scratch_bytes.argtypes = [i32, i32, i32, i32]
    l.llmb_attn_decode_scratch_bytes.restype = sz
    l.llmb_attn_decode.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp]
    l.llmb_attn_decode_batch_scratch_bytes.argtypes = [i32, i32, i32, i32, i32]
    l.llmb_attn_decode_batch_scratch_bytes.restype = sz
    l.llmb_attn_decode_batch.argtypes = [vp, vp, vp, vp, i32, sz, i32, i32, i32, i32, i32, vp, vp, i32, vp]
    l.llmb_attn_decode_trace.argtypes = [vp]
    l.llmb_argmax_rows_f16.argtypes = [vp, i32, i32, vp, vp, vp, i32, i32, vp]
    l.llmb_attn_decode_static.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp]
    l.llmb_argmax_f16.argtypes = [vp, i32, vp, vp, vp, i32, i32, vp]
    l.llmb_advance_pos.argtypes = [vp, i32, vp]
    l.llmb_gemm_f16.argtypes = [C.POINTER(GemmArgs), vp]
    l.llmb_rmsnorm_rows.argtypes = [vp, vp, vp, i32, i32, C.c_double, vp]
    l.llmb_tp_gather_rows.argtypes = [vp, i32, i32, vp, vp, vp, i32, i32, C.c_double, C.c_uint32, i32, vp]
    l.llmb_tp_argmax_rows.argtypes = [vp, i32, i32, i32, i32, vp, i32, i32, i32, vp, vp, vp, i32, C.c_uint32, i32, vp]
    l.llmb_tp_advance.argtypes = [vp, i32, i32, i32, i32, vp]
    l.llmb_attn_prefill.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
    l.llmb_iota_i32.argtypes = [vp, i32, i32, vp]
    l.llmb_sample_logits_host.argtypes = [vp, i32, C.c_float, i32, C.c_float, C.c_float, C.POINTER(C.c_int32)]
    l.llmb_sampler_uniform.argtypes = [u64, u64]
    l.llmb_sample_scratch_bytes.argtypes = [i32]
    l.llmb_sample_scratch_bytes.restype = sz
    l.llmb_sample_logits.argtypes = [vp, i32, C.c_float, i32, C.c_float, u64, u64, vp, vp, vp, vp, i32, i32, vp]
    l.llmb_sampler_uniform.restype = C.c_float
    M, K = C.POINTER(Llama3Struct), C.POINTER(CudaCacheStruct)
    l.init_llama3.argtypes = [i32]
    l.init_llama3.restype = M
    l.free_llama3.argtypes = [M]
    l.free_llama3.restype = None
    l._free_tensor.argtypes = [C.POINTER(TensorStruct)]
    l._free_tensor.restype = None
    l.load_safetensor_weights.argtypes = [M, C.c_char_p]
    l.load_safetensor_weights.restype = None
    l.to_cuda.argtypes = [M]
    l.to_cuda.restype = None
    l.init_cache.argtypes = [M]
    l.init_cache.restype = K
    l.tokens_to_cuda.argtypes = [C.POINTER(C.c_int), i32, C.POINTER(TensorStruct)]
    l.tokens_to_cuda.restype = vp
    l.inference.argtypes = [M, C.POINTER(TensorStruct), vp, C.POINTER(C.c_int), K]
    l.llama3_set_config.argtypes = [M, C.POINTER(Llama3Config)]
    l.llama3_set_tp.argtypes = [M, i32, i32]
    l.llama3_load_safetensors.argtypes = [M, C.c_char_p]
    l.llama3_to_cuda.argtypes = [M]
    l.llama3_set_streaming.argtypes = [M, i32]
    l.llama3_upload_stats.argtypes = [M, C.POINTER(C.c_double), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)]
    l.llama3_tensor_shard.argtypes = [M, i32, i32, C.POINTER(C.c_int)]
    l.llama3_synth_weights.argtypes = [M, C.POINTER(Llama3Config), u64, i32]
    l.llama3_init_cache.argtypes = [M, C.POINTER(C.c_int)]
    l.llama3_init_cache.restype = K
    l.free_cache.argtypes = [K]
    l.free_cache.restype = None
    l.cache_reset.argtypes = [K]
    l.cache_set_options.argtypes = [K, i32, i32, i32]
    l.cache_use_step_kernel.argtypes = [K, i32]
    l.cache_set_tp_poll_limit.argtypes = [K, C.c_uint]
    l.cache_tp_handle.argtypes = [K, vp]
    l.cache_tp_connect.argtypes = [K, vp]
    l.llmb_decode_step_exchange_bytes.argtypes = [i32, i32]
    l.llmb_decode_step_exchange_bytes.restype = sz
    l.cache_enable_hidden_dump.argtypes = [K, i32]
    l.llmb_decode_step_scratch_bytes.argtypes = [i32, i32, i32, i32]
    l.llmb_decode_step_scratch_bytes.restype = sz
    l.llmb_decode_step.argtypes = [C.POINTER(DecodeStepArgs), vp]
    l.cache_read_hidden.argtypes = [K, vp]
    l.inference_greedy.argtypes = [M, K, C.POINTER(C.c_int), i32, i32, C.POINTER(C.c_int), C.POINTER(C.c_float),
                                   C.POINTER(C.c_float)]
    l.inference_continue.argtypes = [M, K, i32, C.POINTER(C.c_int), C.POINTER(C.c_float)]
    l.cache_debug_read.argtypes = [K, i32, vp, sz]
    l.cache_debug_trace.argtypes = [K, i32]
    l.cache_kernel_launches.argtypes = [K]
    l.cache_set_prefill.argtypes = [K, i32, i32]
    l.cache_sample_next_token.argtypes = [K, C.c_float, i32, C.c_float, u64, u64]
    l.cache_sample_next_token_device.argtypes = [K, C.c_float, i32, C.c_float, u64, u64]
    l.cache_kernel_launches.restype = C.c_longlong
    l.cache_batch_init.argtypes = [K, i32]
    l.cache_batch_set_split_len.argtypes = [K, i32]
    l.cache_batch_prefill.argtypes = [K, vp, i32]
    l.cache_batch_step.argtypes = [K, vp, vp, vp]
    l.cache_batch_greedy.argtypes = [K, i32, vp, C.POINTER(C.c_float)]
    l.cache_debug_rows_trace.argtypes = [K, i32, vp]


lib = None
if not os.path.exists(LIB_PATH):
    raise ImportError(
        "llm.cu_b200: %s is missing. Build it with `python llm.cu_b200/build.py` "
        "(nvcc, sm_100a). There is no CPU or PyTorch fallback." % LIB_PATH)
lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
_declare(lib)


def check(code, where):
    if code != OK:
        raise LlmbError(code, where)


from .configs import CONFIGS, ModelConfig  # noqa: E402
from .engine import Cache, Model  # noqa: E402

__all__ = ["lib", "check", "LlmbError", "Llama3Config", "GemvArgs", "GemmArgs", "LayerArgs", "DecodeStepArgs", "Model", "Cache", "CONFIGS", "ModelConfig",
           "KERNEL_SYMBOLS", "HOST_SYMBOLS", "LIB_PATH"]
