"""The preprocessing kernels divide a whole tile by one scale with a correctly rounded reciprocal and
one fused remainder correction.  The quotient bits must be those of an IEEE division, because every
quantised byte is a rounding of such a quotient (the reference divides, quant.py:416-430).  This runs
the library's exhaustive self-test: every dividend significand, both signs, four quotient binades,
for ordinary, extreme and adversarial divisors."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_shared_divisor_division_has_the_bits_of_ieee_division(pkg, cuda):
    from attn_kernel_lab_b200 import kernel as K

    lib = K.load()
    rng = np.random.default_rng(20260829)
    scales = [
        1.0, 448.0, 127.0, 1.0 / 448.0, 1e-8 / 448.0, 1e-8 / 127.0, 3.0, 1.0 / 3.0,
        np.float32(1.0) + np.float32(2.0 ** -23),                 # 1 + ulp
        np.float32(2.0) - np.float32(2.0 ** -23),                 # significand all ones: the excluded pattern
        np.float32(2.0 ** -60) * (np.float32(2.0) - np.float32(2.0 ** -23)),
        2.0 ** -87, 2.0 ** -88, 2.0 ** 73, 2.0 ** 74, 2.0 ** -120, 2.0 ** 100,   # around and beyond the fast path's range
    ]
    # scales as the kernels form them: amax / 448 and amax / 127 for random amax over many binades
    amax = np.exp2(rng.uniform(-20, 20, size=120)).astype(np.float32)
    scales += list((amax[:60] / np.float32(448.0)).astype(np.float32)) + list((amax[60:] / np.float32(127.0)).astype(np.float32))
    # random significands, exponent 0
    scales += list((np.float32(1.0) + rng.integers(0, 2 ** 23, size=70).astype(np.float32) * np.float32(2.0 ** -23)))
    s = torch.tensor(np.asarray(scales, dtype=np.float32), device=cuda)
    bad = torch.zeros(1, dtype=torch.int64, device=cuda)
    code = lib.akl_selftest_exact_division(s.data_ptr(), s.numel(), bad.data_ptr(), torch.cuda.current_stream().cuda_stream)
    K.check(code, "akl_selftest_exact_division")
    torch.cuda.synchronize()
    assert int(bad.item()) == 0, f"{int(bad.item())} quotients differ from IEEE division over {s.numel()} divisors"
    assert lib.akl_selftest_exact_division(None, 1, bad.data_ptr(), None) == K.AKL_ERR_INVALID
