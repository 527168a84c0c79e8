"""Host-side loader logic (no GPU): header parsing, key -> slot mapping, error paths.
Mirrors what the reference's loader does (src/safetensor/safetensor.cu:16-162) and the failures
it does not check for."""
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest


def loaded_tensor(t):
    t = t.contents
    n = t.mem_len[0]
    arr = np.ctypeslib.as_array(C.cast(t.bf16_tensor, C.POINTER(C.c_uint16)), shape=(n,)).copy()
    return arr, [t.shape[i] for i in range(t.ndim[0])], t.file_dtype


def test_load_maps_every_key_to_its_slot(pkg, oracle, tiny_weights, tmp_path):
    cfg = pkg.CONFIGS["tiny"]
    names = list(tiny_weights.file)
    # two shards, as the reference loads four (src/main.cu:73-76)
    p1 = tiny_weights.write_safetensors(tmp_path / "a.safetensors", names[: len(names) // 2])
    p2 = tiny_weights.write_safetensors(tmp_path / "b.safetensors", names[len(names) // 2:])
    m = pkg.lib.init_llama3(cfg.n_layers)
    assert pkg.lib.llama3_set_streaming(m, 0) == 0   # keep the payloads in host memory, as the reference does
    for p in (p1, p2):
        assert pkg.lib.llama3_load_safetensors(m, str(p).encode()) == 0, pkg.lib.llmb_last_error()
    mc = m.contents
    arr, shape, dt = loaded_tensor(mc.lm_head)
    assert shape == [cfg.vocab, cfg.d_model] and dt == 1
    assert np.array_equal(arr, tiny_weights.file["lm_head.weight"])
    for l in range(cfg.n_layers):
        lay = mc.layers[l].contents
        assert lay.layernum == l
        for slot in oracle.SLOTS:
            arr, shape, _ = loaded_tensor(getattr(lay, slot))
            name = oracle.HF_NAMES[slot] % l
            assert shape == list(tiny_weights.shapes[name]), name
            assert np.array_equal(arr, tiny_weights.file[name]), name
    pkg.lib.free_llama3(m)


def write_raw(path, header, payload=b"", header_len=None):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob) if header_len is None else header_len))
        f.write(blob)
        f.write(payload)


@pytest.fixture
def model(pkg):
    m = pkg.lib.init_llama3(2)
    pkg.lib.llama3_set_streaming(m, 0)
    yield m
    pkg.lib.free_llama3(m)


def test_missing_file(pkg, model, tmp_path):
    assert pkg.lib.llama3_load_safetensors(model, str(tmp_path / "nope.safetensors").encode()) == pkg.ERR_IO
    assert b"opening" in pkg.lib.llmb_last_error()


def test_header_length_past_eof(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    write_raw(p, {}, header_len=1 << 20)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_IO


def test_truncated_payload(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"model.norm.weight": {"dtype": "BF16", "shape": [256], "data_offsets": [0, 512]}}
    write_raw(p, hdr, payload=b"\0" * 100)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_IO
    assert b"truncated" in pkg.lib.llmb_last_error()


def test_wrong_dtype(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"model.norm.weight": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}
    write_raw(p, hdr, payload=b"\0" * 8)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_UNSUPPORTED


def test_offsets_do_not_match_shape(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"model.norm.weight": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}
    write_raw(p, hdr, payload=b"\0" * 8)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_IO


def test_layer_index_outside_model(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"model.layers.7.mlp.up_proj.weight": {"dtype": "BF16", "shape": [2, 2], "data_offsets": [0, 8]}}
    write_raw(p, hdr, payload=b"\0" * 8)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_INVALID


def test_unknown_key_and_malformed_json(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"model.rotary.inv_freq": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}}
    write_raw(p, hdr, payload=b"\0" * 4)
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_INVALID
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 9) + b'{"a": [1,')
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == pkg.ERR_IO


def test_metadata_and_escapes_are_skipped(pkg, model, tmp_path):
    p = tmp_path / "x.safetensors"
    hdr = {"__metadata__": {"format": "pt", "note": "a \"quoted\" {brace}", "n": [1, [2, 3], {"k": None}]},
           "model.norm.weight": {"dtype": "F16", "shape": [4], "data_offsets": [0, 8]}}
    write_raw(p, hdr, payload=np.arange(4, dtype=np.uint16).tobytes())
    assert pkg.lib.llama3_load_safetensors(model, str(p).encode()) == 0, pkg.lib.llmb_last_error()
    arr, shape, dt = loaded_tensor(model.contents.norm)
    assert arr.tolist() == [0, 1, 2, 3] and shape == [4] and dt == 1


def test_to_cuda_rejects_incomplete_model(pkg, model):
    assert pkg.lib.llama3_to_cuda(model) == pkg.ERR_INVALID
    assert b"never loaded" in pkg.lib.llmb_last_error()


def test_tp_arguments(pkg, model):
    assert pkg.lib.llama3_set_tp(model, 0, 1) == 0
    assert pkg.lib.llama3_set_tp(model, 1, 2) == 0
    assert pkg.lib.llama3_set_tp(model, 7, 8) == 0
    assert pkg.lib.llama3_set_tp(model, 2, 2) == pkg.ERR_INVALID
    assert pkg.lib.llama3_set_tp(model, 0, 16) == pkg.ERR_UNSUPPORTED


def test_streaming_load_keeps_no_payload_on_the_host(pkg, oracle, tiny_weights, tmp_path):
    """Default mode: the loader records where each payload lies (shape, dtype, file offset) and leaves
    Tensor::bf16_tensor empty; to_cuda() later reads the windows it needs straight from the file."""
    cfg = pkg.CONFIGS["tiny"]
    path = tiny_weights.write_safetensors(tmp_path / "all.safetensors")
    m = pkg.lib.init_llama3(cfg.n_layers)
    assert pkg.lib.llama3_load_safetensors(m, str(path).encode()) == 0, pkg.lib.llmb_last_error()
    t = m.contents.lm_head.contents
    assert not t.bf16_tensor and t.loaded == 1
    assert [t.shape[0], t.shape[1]] == [cfg.vocab, cfg.d_model] and t.mem_len[0] == cfg.vocab * cfg.d_model
    lay = m.contents.layers[1].contents
    assert not lay.mlp_down_proj.contents.bf16_tensor and lay.mlp_down_proj.contents.shape[1] == cfg.ffn
    out = (C.c_int * 5)()
    assert pkg.lib.llama3_tensor_shard(m, 1, 1, out) == 0 and list(out) == [0, cfg.d_model, 0, cfg.ffn, cfg.ffn]
    pkg.lib.free_llama3(m)
