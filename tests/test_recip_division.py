"""The unpack kernels divide a code by a group's scale as  y = RN(1/s), q0 = RN(c y),
r = c - s q0 (one FMA), q = RN(q0 + r y)  when the scale is a 16-bit value in [2^-60, 2^60]
(csrc/quant_math.cuh: group_reciprocal / dequant_bits_recip).  That must be the exactly rounded
float32 quotient, the value the reference's division produces.  Checked here with numpy for every
code 1..255 against every finite positive float16 scale and every bfloat16 scale in the range;
float64 holds the products of two float32 numbers exactly, so the FMAs are emulated without error
up to the final rounding."""
import numpy as np


def _mismatches(scales: np.ndarray) -> int:
    b = scales.astype(np.float32)
    y = (np.float32(1) / b).astype(np.float32)
    b64, y64 = b.astype(np.float64), y.astype(np.float64)
    bad = 0
    for code in range(1, 256):
        a = np.float32(code)
        q0 = (a * y).astype(np.float32)
        r = np.float64(a) - b64 * q0.astype(np.float64)            # exact
        assert np.all(r.astype(np.float32).astype(np.float64) == r)   # ... and a float32 value, as the FMA returns it
        q = (q0.astype(np.float64) + r * y64).astype(np.float32)
        bad += int(np.count_nonzero(q != (a / b).astype(np.float32)))
    return bad


def test_every_float16_scale():
    halves = np.arange(1, 0x7c00, dtype=np.uint16).view(np.float16)     # subnormals included
    assert _mismatches(halves.astype(np.float32)) == 0


def test_every_bfloat16_scale_in_range():
    bf = (np.arange(0x0080, 0x7f80, dtype=np.uint32) << 16).view(np.float32)
    bf = bf[(bf >= 2.0 ** -60) & (bf <= 2.0 ** 60)]
    assert bf.size == 121 * 128 - 127
    assert _mismatches(bf) == 0
