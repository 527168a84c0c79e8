"""The C-ABI library loads without a GPU and exports every function include/*.h declares."""
import ctypes
import os
import re

from conftest import ROOT


def declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"typedef\s+struct\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"enum\s*\{.*?\}\s*;", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_]\w*)\s*\([^;{}]*\)\s*;", text)
    return [n for n in names if n not in ("defined",)]


def test_kernel_header_symbols_exported(pkg):
    names = declared_functions("llm_b200.h")
    assert set(names) == set(pkg.KERNEL_SYMBOLS), set(names) ^ set(pkg.KERNEL_SYMBOLS)
    raw = ctypes.CDLL(pkg.LIB_PATH)
    for n in names:
        assert getattr(raw, n) is not None


def test_host_header_symbols_exported(pkg):
    names = declared_functions("llama3.h")
    assert set(names) == set(pkg.HOST_SYMBOLS), set(names) ^ set(pkg.HOST_SYMBOLS)
    raw = ctypes.CDLL(pkg.LIB_PATH)
    for n in names:
        assert getattr(raw, n) is not None


def test_struct_layouts_match_reference_prefix(pkg):
    # the first fields are the reference's (llama3.cuh:10-50, inference.cuh:19-34), in its order
    t = [f[0] for f in pkg.TensorStruct._fields_][:9]
    assert t == ["ndim", "mem_len", "shape", "bf16_tensor", "d_ndim", "d_mem_len", "d_shape", "d_bf16_tensor",
                 "d_fp16_tensor"]
    m = [f[0] for f in pkg.Llama3Struct._fields_][:5]
    assert m == ["embed_tokens", "lm_head", "norm", "layers", "n_layers"]
    c = [f[0] for f in pkg.CudaCacheStruct._fields_][:9]
    assert c == ["PN_X", "Q", "K", "V", "d_attention_score_cache", "d_feedforward_cache_upgate", "d_token_probdist",
                 "h_token_probdist", "f_token_probdist"]


def test_build_info_names_the_architecture(pkg):
    assert b"sm_100a" in pkg.lib.llmb_build_info()


def test_invalid_arguments_are_rejected_without_a_gpu(pkg):
    a = pkg.GemvArgs()
    assert pkg.lib.llmb_gemv_f16(ctypes.byref(a), None) == pkg.ERR_INVALID
    assert pkg.lib.llmb_attn_decode(None, None, None, None, 32, 8, 128, 16, 32, None, None, 0, None) == pkg.ERR_INVALID
    assert pkg.lib.llmb_attn_decode_scratch_bytes(32, 8, 128, 16) > 32 * 16 * 128 * 4
    assert pkg.lib.llmb_argmax_f16(None, 10, None, None, None, 0, 0, None) == pkg.ERR_INVALID
