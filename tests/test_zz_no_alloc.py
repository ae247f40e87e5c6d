"""mk_gemv_static (split-K scratch in a fixed array of the library, no allocation)
against mk_gemv on the same inputs.  Collected last on purpose: it has to pass
both alone and after every other test has used the library."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, w, q, x, y, workspace=None):
    """mk_gemv_static when ``workspace`` is None, else mk_gemv with that workspace."""
    batch, k = x.shape
    stream = torch.cuda.current_stream().cuda_stream
    extra = () if workspace is None else (workspace.data_ptr(), workspace.numel())
    if q is not None:
        return fn(None, q.packed.data_ptr(), q.scales.data_ptr(), x.data_ptr(), y.data_ptr(), q.rows, k,
                  q.tensor_scale, 1, batch, *extra, stream)
    return fn(w.data_ptr(), None, None, x.data_ptr(), y.data_ptr(), w.shape[0], k, 1.0, 0, batch, *extra, stream)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("m,k", [(2048, 8192), (8192, 2048), (1000, 4096)])
def test_two_calls_in_a_row_equal_mk_gemv(packed, m, k):
    from thor_megakernels_b200 import _lib
    from thor_megakernels_b200.nvfp4 import quantize_weight

    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(2)
    w = (torch.randn(m, k, device="cuda", generator=gen) * 0.02).bfloat16()
    q = quantize_weight(w) if packed else None
    workspace = torch.zeros(max(256, int(lib.mk_gemv_workspace_bytes(m, k))), dtype=torch.uint8, device="cuda")
    # one call first: it resolves the fixed array's address on this device (no allocation, but a driver look-up)
    x = torch.randn(1, k, device="cuda", generator=gen).bfloat16()
    assert _call(lib.mk_gemv_static, w, q, x, torch.empty((1, m), dtype=torch.bfloat16, device="cuda")) == 0
    torch.cuda.synchronize()
    for batch in (1, 4):  # two calls in a row, different activations and batch
        x = torch.randn(batch, k, device="cuda", generator=gen).bfloat16()
        want = torch.full((batch, m), float("nan"), dtype=torch.bfloat16, device="cuda")
        got = torch.full((batch, m), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _call(lib.mk_gemv, w, q, x, want, workspace) == 0, lib.mk_last_error()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        assert _call(lib.mk_gemv_static, w, q, x, got) == 0, lib.mk_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the property the entry point exists for: the device's free memory is what it was before the call
        assert free_after == free_before, (free_before, free_after)
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_largest_supported_split_matches_mk_gemv():
    """16384 x 16384 bf16: 8 K-chunks, 1024 row blocks, exactly the 1 048 576
    partial floats the fixed array holds."""
    from thor_megakernels_b200 import _lib

    lib = _lib.load()
    m = k = 16384
    gen = torch.Generator(device="cuda").manual_seed(4)
    w = (torch.randn(m, k, device="cuda", generator=gen) * 0.02).bfloat16()
    x = torch.randn(1, k, device="cuda", generator=gen).bfloat16()
    workspace = torch.zeros(int(lib.mk_gemv_workspace_bytes(m, k)), dtype=torch.uint8, device="cuda")
    want = torch.empty((1, m), dtype=torch.bfloat16, device="cuda")
    got = torch.empty((1, m), dtype=torch.bfloat16, device="cuda")
    assert _call(lib.mk_gemv, w, None, x, want, workspace) == 0, lib.mk_last_error()
    for _ in range(2):
        got.fill_(float("nan"))
        assert _call(lib.mk_gemv_static, w, None, x, got) == 0, lib.mk_last_error()
        torch.cuda.synchronize()
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
