"""CPU checks of the NVFP4 oracle: the reference's known-answer fixture, the
numpy restatement against the CUDA toolkit's host conversions, and the
independent decoder."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import nvfp4
from oracle.build import build_oracle


@pytest.fixture(scope="module")
def cref():
    lib = C.CDLL(str(build_oracle()))
    lib.oracle_nvfp4_quantize.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_float]
    lib.oracle_e4m3_to_float.restype = C.c_float
    lib.oracle_e4m3_to_float.argtypes = [C.c_uint8]
    lib.oracle_float_to_e4m3.restype = C.c_uint8
    lib.oracle_float_to_e4m3.argtypes = [C.c_float]
    lib.oracle_float_to_e2m1.restype = C.c_uint8
    lib.oracle_float_to_e2m1.argtypes = [C.c_float]
    return lib


def c_quantize(lib, w_bf16: torch.Tensor, ts: float):
    rows, k = w_bf16.shape
    bits = w_bf16.contiguous().view(torch.int16).numpy()
    packed = np.zeros((rows, k // 2), np.uint8)
    scales = np.zeros((rows, k // 16), np.uint8)
    decoded = np.zeros((rows, k), np.float32)
    rc = lib.oracle_nvfp4_quantize(bits.ctypes.data, packed.ctypes.data, scales.ctypes.data, decoded.ctypes.data,
                                   rows, k, C.c_float(ts))
    assert rc == 0
    return packed, scales, decoded


def test_reference_sixteen_level_fixture_round_trips_exactly():
    """tools/analysis/nvfp4/check.py:12-17: a 128x256 matrix that repeats the 16
    code values, tensor scale 1, must decode to itself bit for bit."""
    levels = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.])
    src = levels.repeat(128 * 16).reshape(128, 256).bfloat16()
    packed, scales, decoded = nvfp4.quantize(src.float().numpy(), np.float32(1.0))
    assert np.array_equal(decoded, src.float().numpy())
    assert np.array_equal(np.signbit(decoded), np.signbit(src.float().numpy()))
    assert (scales == 0x38).all()  # amax 6 / 6 = 1.0 = E4M3 0x38
    assert np.array_equal(packed[0, :8], np.array([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE], np.uint8))
    assert np.array_equal(nvfp4.dequantize(packed, scales, 1.0), src.float().numpy())


def test_code_table_matches_the_toolkit(cref):
    for code in range(8):
        assert cref.oracle_float_to_e2m1(float(nvfp4.E2M1_LEVELS[code])) == code
        assert cref.oracle_float_to_e2m1(-float(nvfp4.E2M1_LEVELS[code])) == (code | 8)
    for bits in range(0x7F):  # 0x7f is NaN
        assert nvfp4.e4m3_decode(np.array([bits], np.uint8))[0] == cref.oracle_e4m3_to_float(bits)


def test_roundings_match_the_toolkit_on_ties_and_random_values(cref):
    rng = np.random.default_rng(0)
    grid = nvfp4.e4m3_decode(np.arange(0, 0x7F, dtype=np.uint8)).astype(np.float64)
    xs = np.concatenate([np.exp2(rng.uniform(-12, 10, 4000)), (grid[:-1] + grid[1:]) / 2, grid, [449, 464, 465, 1e6]]).astype(np.float32)
    want = np.array([cref.oracle_float_to_e4m3(float(x)) for x in xs], np.uint8)
    assert np.array_equal(nvfp4.e4m3_encode_positive(xs), want)
    xs = np.concatenate([rng.normal(0, 3, 4000), np.linspace(-8, 8, 1601),
                         [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 7, 100, -0.0, 0.0]]).astype(np.float32)
    want = np.array([cref.oracle_float_to_e2m1(float(x)) for x in xs], np.uint8)
    assert np.array_equal(nvfp4.e2m1_encode(xs), want)


@pytest.mark.parametrize("rows,k,std", [(128, 256, 0.02), (264, 512, 1.0), (64, 2048, 0.02), (16, 8192, 0.02)])
def test_numpy_quantiser_equals_toolkit_quantiser(cref, rows, k, std):
    torch.manual_seed(2)
    w = (torch.randn(rows, k) * std).bfloat16()
    w[0, :16] = 0  # an all-zero group takes the 2^-9 scale floor
    ts = nvfp4.tensor_scale_for(w.abs().max().item())
    a = nvfp4.quantize(w.float().numpy(), ts)
    b = c_quantize(cref, w, float(ts))
    for x, y, name in zip(a, b, ("packed", "scales", "decoded")):
        assert np.array_equal(x, y), name
    assert a[1][0, 0] == 0x01  # 2^-9, the smallest subnormal
    assert np.array_equal(nvfp4.dequantize(a[0], a[1], ts), a[2])
    # quantisation error stays within half a code step of the block scale
    err = np.abs(a[2] - w.float().numpy())
    step = np.repeat(nvfp4.e4m3_decode(a[1]), 16, axis=-1) * ts
    assert (err <= step * 1.0 + 1e-12).all()
