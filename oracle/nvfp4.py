"""TEST INFRASTRUCTURE ONLY - numpy restatement of the reference's NVFP4 weight
format and weight-only GEMV.

Follows
    tools/analysis/nvfp4/primitive.cu:50-75   quantiser (the format definition)
    tools/analysis/nvfp4/bench.py:68          per-tensor scale rule
    tools/analysis/nvfp4/check.py:12,25-29    code table and the independent decoder
    tools/analysis/nvfp4/primitive.cu:79-96   weight-only GEMV (fp32 fma, bf16 out)
    tools/analysis/nvfp4/model_reference.py:39-61  model-level oracle (fp32 linear on
                                               dequantised weights, one bf16 rounding)

The reference's quantiser exists only as a CUDA kernel, so it cannot be run on a
CPU box.  Its two roundings are restated here from the published formats:
E4M3 (4 exponent bits, bias 7, 3 mantissa bits, subnormals, max 448, no
infinity) and E2M1 (values 0, .5, 1, 1.5, 2, 3, 4, 6 and their negatives), both
round-to-nearest-even and saturating.  ``oracle/nvfp4_ref.cpp`` computes the same
thing through the CUDA toolkit's host-callable conversion functions and the
tests require both to agree bit for bit; the reference's own known-answer
fixture (check.py:12-17) pins the table.
"""
from __future__ import annotations

import numpy as np

# check.py:12 - code value table; bit 3 is the sign
E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                       dtype=np.float32)


def tensor_scale_for(weight_amax: float) -> np.float32:
    """bench.py:68: amax / (6 * 448), floored at 1e-12, narrowed to fp32 at the C boundary."""
    return np.float32(max(float(weight_amax) / (6 * 448), 1e-12))


def _round_half_even(x: np.ndarray) -> np.ndarray:
    return np.rint(x)  # IEEE default rounding: ties to even


def e4m3_encode_positive(x: np.ndarray) -> np.ndarray:
    """fp32 >= 0 -> E4M3 bit pattern, round-to-nearest-even, saturating at 448."""
    x = np.asarray(x, dtype=np.float32)
    xd = x.astype(np.float64)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.maximum(xd, 2.0 ** -20)))
    e = np.clip(e, -6, 8)
    quantum = np.exp2(e - 3)
    q = _round_half_even(xd / quantum) * quantum
    q = np.minimum(q, 448.0)
    # re-derive exponent after a possible carry into the next binade
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.maximum(q, 2.0 ** -20)))
    normal = q >= 2.0 ** -6
    e2 = np.clip(e2, -6, 8)
    exp_field = np.where(normal, e2 + 7, 0).astype(np.int64)
    mant = np.where(normal, (q / np.exp2(e2) - 1.0) * 8.0, q / 2.0 ** -9)
    bits = (exp_field << 3) | np.rint(mant).astype(np.int64)
    return bits.astype(np.uint8)


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    bits = np.asarray(bits, dtype=np.uint8).astype(np.int64)
    sign = np.where(bits & 0x80, -1.0, 1.0)
    exp_field = (bits >> 3) & 0xF
    mant = bits & 0x7
    val = np.where(exp_field == 0, mant * 2.0 ** -9, (1.0 + mant / 8.0) * np.exp2(exp_field - 7.0))
    return (sign * val).astype(np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit E2M1 code, round-to-nearest-even, saturating at +-6."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    # quantum: 0.5 below 2 (subnormal + first two binades share it), 1 in [2,4), 2 in [4,6]
    quantum = np.where(a < 2.0, 0.5, np.where(a < 4.0, 1.0, 2.0))
    q = np.minimum(_round_half_even(a / quantum) * quantum, 6.0)
    code = np.searchsorted(E2M1_LEVELS[:8].astype(np.float64), q).astype(np.uint8)
    return (code | (np.signbit(x).astype(np.uint8) << 3)).astype(np.uint8)


def quantize(weight_bf16_as_f32: np.ndarray, tensor_scale: np.float32):
    """primitive.cu:58-74.  ``weight_bf16_as_f32``: fp32 array holding bf16 values,
    shape [rows, k] with k % 16 == 0.  Returns (packed [rows,k/2] u8,
    scales [rows,k/16] u8, decoded [rows,k] f32)."""
    w = np.asarray(weight_bf16_as_f32, dtype=np.float32)
    rows, k = w.shape
    ts = np.float32(tensor_scale)
    v = (w / ts).astype(np.float32).reshape(rows, k // 16, 16)
    amax = np.abs(v).max(axis=-1)
    sf_in = np.maximum((amax / np.float32(6.0)).astype(np.float32), np.float32(1.0 / 512.0))
    sf_bits = e4m3_encode_positive(sf_in)
    scale = e4m3_decode(sf_bits)
    codes = e2m1_encode((v / scale[..., None]).astype(np.float32)).reshape(rows, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    decoded = (E2M1_LEVELS[codes].reshape(rows, k // 16, 16) * scale[..., None]).astype(np.float32) * ts
    return packed, sf_bits.reshape(rows, k // 16), decoded.reshape(rows, k).astype(np.float32)


def dequantize(packed: np.ndarray, scales: np.ndarray, tensor_scale) -> np.ndarray:
    """check.py:25-29: low nibble first, lookup, times block scale, times tensor scale."""
    packed = np.asarray(packed, dtype=np.uint8)
    rows = packed.shape[0]
    codes = np.stack((packed & 15, packed >> 4), axis=-1).reshape(rows, -1)
    sf = np.repeat(e4m3_decode(scales), 16, axis=-1)
    return (E2M1_LEVELS[codes] * sf).astype(np.float32) * np.float32(tensor_scale)


def gemv_reference(dequantized: np.ndarray, x_bf16_as_f32: np.ndarray) -> np.ndarray:
    """bf16(dequantised_fp32 @ x_fp32) - the reference's accuracy target
    (check.py:36, bench.py ref_w4).  Returned as fp32 holding bf16 values."""
    import torch

    y = torch.from_numpy(np.ascontiguousarray(dequantized)).double() @ torch.from_numpy(
        np.ascontiguousarray(x_bf16_as_f32)).double().T
    return y.T.float().bfloat16().float().numpy()
