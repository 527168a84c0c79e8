"""Helpers for the GPU tests: device buffers through torch (plumbing only) and FP16 comparisons."""
import numpy as np
import torch


def dev(a):
    """numpy array -> device tensor with the same bits (uint16 travels as int16)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    return torch.from_numpy(a).cuda()


def host_u16(t):
    torch.cuda.synchronize()
    return t.cpu().numpy().view(np.uint16)


def f16(a):
    return np.asarray(a, dtype=np.uint16).view(np.float16).astype(np.float32)


def to_f16_bits(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def ulp_diff(a_bits, b_bits):
    """Distance in FP16 units in the last place between two bit-pattern arrays (finite values)."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return np.abs(key(np.asarray(a_bits)) - key(np.asarray(b_bits)))


def assert_close_fp16(got_bits, want_f64, max_ulp=1, max_frac=0.05, what="", abs_tol=None):
    """got (FP16 bits) must equal RN(want) up to `max_ulp`, with at most `max_frac` of elements off at all:
    the kernels sum in FP32 in a different order than a sequential loop, which can move a value
    across an FP16 rounding boundary but never further.  Outputs that cancel to nearly zero have an
    FP16 ulp below the FP32 accumulation error, so an absolute error of 2^-20 of the largest output is
    accepted as well."""
    want_f64 = np.asarray(want_f64, dtype=np.float64)
    want_bits = want_f64.astype(np.float16).view(np.uint16)
    d = ulp_diff(got_bits, want_bits)
    tol = (1.0 + np.abs(want_f64).max()) * 2.0 ** -20
    if abs_tol is not None:
        tol = np.maximum(tol, abs_tol)
    abs_ok = np.abs(f16(got_bits).astype(np.float64) - want_f64) <= tol
    d = np.where(abs_ok & (d > max_ulp), max_ulp, d)
    assert d.max() <= max_ulp, "%s: max ulp distance %d" % (what, d.max())
    frac = float((d > 0).mean())
    assert frac <= max_frac, "%s: %.4f of elements differ" % (what, frac)


def rmsnorm_ref(x_bits, g_bits, eps=1e-5):
    """RMSNorm with the reference's reduction tree (inference.cu:293-363), vectorised numpy."""
    x = f16(x_bits)
    d = x.size
    sq = x * x
    part = ((sq[0::4] + sq[1::4]) + sq[2::4]) + sq[3::4]
    n = 1
    while n < part.size:
        n <<= 1
    buf = np.zeros(n, dtype=np.float32)
    buf[: part.size] = part
    while n > 1:
        n //= 2
        buf[:n] = buf[:n] + buf[n:2 * n]
    rms = np.float32(np.sqrt(np.float32(eps + np.float64(buf[0] / np.float32(d)))))
    return ((x * f16(g_bits)) / rms).astype(np.float16).view(np.uint16)
