"""The seeded generator (include/llm_b200_synth.h) must give the same bits in C, numpy and CUDA."""
import numpy as np

M64 = (1 << 64) - 1


def mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def stream_key(seed, sid):
    return mix64((seed * 0xD1342543DE82EF95 + mix64(sid)) & M64)


def unit(key, i):
    a, b = mix64((key + 2 * i) & M64), mix64((key + 2 * i + 1) & M64)
    s = sum((v >> sh) & 0xFFFF for v in (a, b) for sh in (0, 16, 32, 48)) - 4 * 65535
    return np.float32(s) * np.float32(1.8688567e-05)


def bf16_rne(f):
    u = int(np.float32(f).view(np.uint32))
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFFFFFF
    return u >> 16


def test_bf16_stream_matches_python_restatement(oracle):
    got = oracle.synth_bf16(7, 35, 64, std=0.02, first=1000)
    key = stream_key(7, 35)
    want = [bf16_rne(unit(key, 1000 + i) * np.float32(0.02)) for i in range(64)]
    assert got.tolist() == want


def test_fp16_stream_matches_numpy_rounding(oracle):
    got = oracle.synth_fp16(3, 2, 4096, std=0.02)
    key = stream_key(3, 2)
    want = np.array([unit(key, i) * np.float32(0.02) for i in range(4096)], dtype=np.float32).astype(np.float16)
    assert np.array_equal(got, want.view(np.uint16))


def test_fp16_rounding_edge_cases(oracle):
    # std scales the unit draw; huge and tiny scales reach overflow, subnormals and zero
    for std in (1e-9, 3e-8, 6e-6, 1e-4, 1.0, 3e4, 1e6):
        got = oracle.synth_fp16(11, 5, 2048, std=std)
        key = stream_key(11, 5)
        with np.errstate(over="ignore"):
            want = np.array([unit(key, i) * np.float32(std) for i in range(2048)], dtype=np.float32).astype(np.float16)
        assert np.array_equal(got, want.view(np.uint16)), std


def test_distribution_is_close_to_normal(oracle):
    v = oracle.f16(oracle.synth_fp16(0, 1, 1 << 18, std=0.02))
    assert abs(v.mean()) < 2e-4
    assert abs(v.std() - 0.02) < 2e-4
    assert 2.7 < ((v / v.std()) ** 4).mean() < 3.05  # Irwin-Hall(8): kurtosis 2.85


def test_slices_are_independent_of_chunking(oracle):
    whole = oracle.synth_bf16(1, 99, 1000)
    parts = np.concatenate([oracle.synth_bf16(1, 99, 400), oracle.synth_bf16(1, 99, 600, first=400)])
    assert np.array_equal(whole, parts)


def test_tokens_in_range(oracle):
    t = oracle.synth_tokens(0, 4096, 128256)
    assert t.min() >= 0 and t.max() < 128256 and len(set(t.tolist())) > 3900


def test_bench_prompt_is_the_oracle_token_stream(oracle):
    import bench
    want = oracle.synth_tokens(bench.SEED, bench.PROMPT, 128256).tolist()
    assert bench.prompt_ids(128256) == want
