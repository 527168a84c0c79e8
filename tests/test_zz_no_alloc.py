"""llmb_attn_decode_static: the decode attention for callers that may not allocate device memory
(their own pool owns the device, or they only ever hold input and output buffers).  Its partial
results live in a fixed array inside the library, so this test calls it twice in a row through the
C-ABI, with different shapes, and compares each result with llmb_attn_decode given a workspace.
The file name sorts last so that a run that stops at the first failure has already run every other
test; the test does not depend on anything the other tests leave behind."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from gpu_util import dev, host_u16  # noqa: E402


def run_pair(pkg, oracle, nq, nkv, hd, length, n_splits, split_len, seed, use_pdl=0, check_free=False):
    max_pos = max(length, 8)
    q = dev(oracle.synth_fp16(seed, 1, nq * hd, std=1.0))
    kc = dev(oracle.synth_fp16(seed, 2, max_pos * nkv * hd, std=1.0))
    vc = dev(oracle.synth_fp16(seed, 3, max_pos * nkv * hd, std=1.0))
    pos = torch.full((1,), length - 1, dtype=torch.int32, device="cuda")
    want = torch.zeros(nq * hd, dtype=torch.int16, device="cuda")
    got = torch.zeros_like(want)
    scratch = torch.zeros(pkg.lib.llmb_attn_decode_scratch_bytes(nq, nkv, hd, n_splits), dtype=torch.uint8,
                          device="cuda")
    rc = pkg.lib.llmb_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), nq, nkv, hd, n_splits,
                                  split_len, want.data_ptr(), scratch.data_ptr(), 0, None)
    assert rc == 0, pkg.lib.llmb_last_error()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = pkg.lib.llmb_attn_decode_static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), nq, nkv, hd,
                                         n_splits, split_len, got.data_ptr(), use_pdl, None)
    assert rc == 0, pkg.lib.llmb_last_error()
    torch.cuda.synchronize()
    if check_free:  # the driver's free-memory figure does not move: the call took nothing from the device
        assert torch.cuda.mem_get_info()[0] == free_before
    return host_u16(got), host_u16(want)


def test_static_workspace_matches_caller_workspace_twice_in_a_row(pkg, oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    # first call: long sequence, many splits; second call: fewer heads, shorter sequence, so anything
    # the first call left in the shared array would show
    # the third call launches with programmatic stream serialization, as the engine's captured step does
    calls = (((32, 8, 128, 1500, 16, 128, 31), 0), ((4, 2, 64, 70, 16, 32, 32), 0), ((32, 8, 128, 900, 8, 128, 33), 1))
    for i, (args, pdl) in enumerate(calls):
        # the first call on a device may make the CUDA runtime load the library's device code (the array
        # itself included); from the second call on, free device memory must not change at all
        got, want = run_pair(pkg, oracle, *args, use_pdl=pdl, check_free=i > 0)
        # same kernel, same split order: the results are identical, well inside the 1-ulp
        # tolerance the attention tests allow against a float64 softmax
        assert np.array_equal(got, want), args


def test_static_workspace_on_a_second_device(pkg, oracle):
    """The array's address and the kernels' shared-memory opt-in are per device: a process that uses two
    GPUs gets a correct result on both (64 KB of shared memory at head_dim 128 needs the opt-in)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    for d in (0, 1):
        with torch.cuda.device(d):
            got, want = run_pair(pkg, oracle, 32, 8, 128, 600, 8, 128, 40 + d)
            assert np.array_equal(got, want), d


def test_static_workspace_rejects_oversized_requests(pkg):
    rc = pkg.lib.llmb_attn_decode_static(None, None, None, None, 64, 8, 128, 128, 128, None, 0, None)
    assert rc == pkg.ERR_UNSUPPORTED
    assert b"built-in workspace" in pkg.lib.llmb_last_error()
    assert pkg.lib.llmb_attn_decode_static(None, None, None, None, 32, 8, 256, 16, 128, None, 0, None) == pkg.ERR_UNSUPPORTED
