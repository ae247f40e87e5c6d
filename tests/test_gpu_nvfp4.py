"""GPU parity of the NVFP4 quantiser and the fused dequantise-GEMV, through the
C-ABI, against the numpy oracle.  Codes, scale bytes and the fp32 decode are
bit-exact; the bf16 GEMV output is held to the reference's own gate
(relative L2 <= 1e-3 against bf16(dequantised_fp32 @ x), check.py:36-43) and
to |a-ref| <= 3e-2 + 1e-2 |ref|."""
import numpy as np
import pytest
import torch

from helpers import assert_close
from oracle import nvfp4 as oracle

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def test_sixteen_level_fixture_on_device():
    from thor_megakernels_b200.nvfp4 import quantize_weight

    levels = torch.tensor([0., .5, 1., 1.5, 2., 3., 4., 6., -0., -.5, -1., -1.5, -2., -3., -4., -6.])
    src = levels.repeat(128 * 16).reshape(128, 256).bfloat16().cuda()
    q = quantize_weight(src, tensor_scale=1.0, reference=True)
    assert torch.equal(q.decoded.cpu(), src.float().cpu())


@pytest.mark.parametrize("rows,k", [(128, 256), (264, 512), (8192, 2048), (2048, 8192)])
def test_quantiser_bit_exact(rows, k):
    from thor_megakernels_b200.nvfp4 import quantize_weight

    torch.manual_seed(2)
    w = (torch.randn(rows, k) * 0.02).bfloat16()
    w[0, :32] = 0
    q = quantize_weight(w.cuda(), reference=True)
    ts = oracle.tensor_scale_for(w.abs().max().item())
    assert q.tensor_scale == float(ts)
    packed, scales, decoded = oracle.quantize(w.float().numpy(), ts)
    assert np.array_equal(q.packed.cpu().numpy(), packed)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    assert np.array_equal(q.decoded.cpu().numpy(), decoded)
    assert np.array_equal(oracle.dequantize(q.packed.cpu().numpy(), q.scales.cpu().numpy(), q.tensor_scale), decoded)


@pytest.mark.parametrize("rows,k", [(8192, 2048), (2048, 8192), (128, 256), (264, 512)])
@pytest.mark.parametrize("batch", [1, 4])
def test_weight_only_gemv(rows, k, batch):
    from thor_megakernels_b200.nvfp4 import gemv, quantize_weight

    torch.manual_seed(2)
    w = (torch.randn(rows, k) * 0.02).bfloat16()
    x = torch.randn(batch, k).bfloat16()
    q = quantize_weight(w.cuda())
    dq = oracle.dequantize(q.packed.cpu().numpy(), q.scales.cpu().numpy(), q.tensor_scale)
    want = torch.from_numpy(oracle.gemv_reference(dq, x.float().numpy()))
    got = gemv(q, x.cuda()).float().cpu()
    assert got.shape == (batch, rows)
    assert rel_l2(got, want) <= 1e-3
    assert_close("w4a16 gemv", got, want)
    # bf16 weights through the same entry point
    want_bf = (w.double() @ x.double().T).T.float().bfloat16().float()
    got_bf = gemv(w.cuda(), x.cuda()).float().cpu()
    assert rel_l2(got_bf, want_bf) <= 1e-3
    assert_close("bf16 gemv", got_bf, want_bf)


def test_weight_only_gemv_activation_range():
    """The NVFP4 GEMV feeds the tensor cores f16 activations.  Magnitudes around
    1e4 (inside f16's range) must match the oracle like any other input; values
    beyond 65504 are clamped to it rather than turning into infinities; tiny
    values lose precision but only in proportion to their (negligible) size."""
    from thor_megakernels_b200.nvfp4 import gemv, quantize_weight

    torch.manual_seed(6)
    rows, k = 512, 2048
    w = (torch.randn(rows, k) * 0.02).bfloat16()
    q = quantize_weight(w.cuda())
    dq = torch.from_numpy(oracle.dequantize(q.packed.cpu().numpy(), q.scales.cpu().numpy(), q.tensor_scale)).double()
    # large but representable
    x = (torch.randn(1, k) * 1e4).bfloat16()
    want = (dq @ x.double().T).T.float().bfloat16().float()
    got = gemv(q, x.cuda()).float().cpu()
    assert torch.isfinite(got).all()
    assert rel_l2(got, want) <= 1e-3
    # beyond f16: the result is that of the clamped activations, and finite
    x_big = x.clone()
    x_big[0, ::7] = 3.0e5
    x_big[0, 3::11] = -2.0e6
    got = gemv(q, x_big.cuda()).float().cpu()
    want = (dq @ x_big.double().clamp(-65504, 65504).T).T.float().bfloat16().float()
    assert torch.isfinite(got).all()
    assert rel_l2(got, want) <= 1e-3
    # tiny values next to ordinary ones: absolute error stays at the ordinary values' rounding level
    x_small = torch.randn(1, k).bfloat16()
    x_small[0, ::2] = 1e-6
    want = (dq @ x_small.double().T).T.float().bfloat16().float()
    got = gemv(q, x_small.cuda()).float().cpu()
    assert rel_l2(got, want) <= 1e-3


def test_gemv_rejects_bad_shapes():
    from thor_megakernels_b200.nvfp4 import gemv, quantize_weight

    w = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        gemv(w, torch.zeros(32, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError):
        gemv(w, torch.zeros(9, 64, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        quantize_weight(torch.zeros(16, 24, dtype=torch.bfloat16, device="cuda"))
