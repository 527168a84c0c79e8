"""The roofline denominators bench.py uses (algorithmic bytes per decoded token) against the figures
derived from the reference's tensor shapes (src/llama3/llama3.cu, src/inference/inference.cu:110-145)."""


def test_algorithmic_bytes_per_token(pkg):
    c = pkg.CONFIGS
    assert c["llama3_8b"].weight_bytes_per_token() == 15_009_857_536
    assert c["llama3_8b"].kv_bytes_per_position() == 131_072
    assert c["tiny"].weight_bytes_per_token() == 5_245_952
    assert c["tiny"].kv_bytes_per_position() == 1_024
    assert c["llama3_70b"].weight_bytes_per_token() == 139_006_083_072
    assert c["llama3_70b"].kv_bytes_per_position() == 327_680
    # one step over L cached rows reads L rows and writes one
    assert c["llama3_8b"].decode_bytes(128) == 15_009_857_536 + 131_072 * 129


def test_tensor_parallel_share(pkg):
    cfg = pkg.CONFIGS["llama3_8b"]
    norms = 2 * (2 * cfg.n_layers + 1) * cfg.d_model + 2 * cfg.d_model  # replicated gains + one embedding row
    for tp in (2, 4, 8):
        sharded = cfg.weight_bytes_per_token() - norms
        assert cfg.weight_bytes_per_token(tp) == sharded // tp + norms
        assert cfg.decode_bytes(100, tp) == cfg.weight_bytes_per_token(tp) + cfg.kv_bytes_per_position() // tp * 101


def test_reference_layer_bytes(pkg):
    # 436,207,616 bytes of projection weights per 8B layer, 1,050,673,152 for lm_head
    cfg = pkg.CONFIGS["llama3_8b"]
    assert 2 * cfg.matmul_params() // cfg.n_layers == 436_207_616
    assert 2 * cfg.vocab * cfg.d_model == 1_050_673_152
