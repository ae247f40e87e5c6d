"""mk_gemv_static (split-K scratch in a fixed array of the library, no allocation)
against mk_gemv on the same inputs.  Collected last on purpose: it has to pass
both alone and after every other test has used the library."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, w, q, x, y):
    from thor_megakernels_b200 import _lib

    batch, k = x.shape
    stream = torch.cuda.current_stream().cuda_stream
    if q is not None:
        return fn(None, q.packed.data_ptr(), q.scales.data_ptr(), x.data_ptr(), y.data_ptr(), q.rows, k,
                  q.tensor_scale, 1, batch, stream)
    return fn(w.data_ptr(), None, None, x.data_ptr(), y.data_ptr(), w.shape[0], k, 1.0, 0, batch, stream)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("m,k", [(2048, 8192), (8192, 2048), (1000, 4096)])
def test_two_calls_in_a_row_equal_mk_gemv(packed, m, k):
    from thor_megakernels_b200 import _lib
    from thor_megakernels_b200.nvfp4 import quantize_weight

    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(2)
    w = (torch.randn(m, k, device="cuda", generator=gen) * 0.02).bfloat16()
    q = quantize_weight(w) if packed else None
    for batch in (1, 4):  # two calls in a row, different activations and batch
        x = torch.randn(batch, k, device="cuda", generator=gen).bfloat16()
        want = torch.full((batch, m), float("nan"), dtype=torch.bfloat16, device="cuda")
        got = torch.full((batch, m), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _call(lib.mk_gemv, w, q, x, want) == 0
        assert _call(lib.mk_gemv_static, w, q, x, got) == 0, lib.mk_last_error()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_sizes_beyond_the_fixed_scratch_are_refused():
    from thor_megakernels_b200 import _lib

    lib = _lib.load()
    dummy = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # 131072 rows need 8192 tickets; the array holds 4096.  Refused before any launch, so the buffers are never touched.
    code = lib.mk_gemv_static(dummy.data_ptr(), None, None, dummy.data_ptr(), dummy.data_ptr(), 131072, 4096, 1.0, 0, 1, stream)
    assert code == _lib.MK_ERR_UNSUPPORTED
    assert b"fixed scratch" in lib.mk_last_error()
    # k must be a multiple of 256
    code = lib.mk_gemv_static(dummy.data_ptr(), None, None, dummy.data_ptr(), dummy.data_ptr(), 16, 96, 1.0, 0, 1, stream)
    assert code == _lib.MK_ERR_BAD_ARGUMENT
    torch.cuda.synchronize()
