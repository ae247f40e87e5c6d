"""The C-ABI shared library: it builds for sm_100a, loads without a GPU, exports
every symbol the public header declares, and its struct layouts are the ones the
ctypes binding assumes.  No compute calls here."""
import ctypes as C
import re
from pathlib import Path

import pytest

from thor_megakernels_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "b200_megakernel.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_list_the_same_functions():
    assert declared_functions() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_struct_layouts_match():
    lib = _lib.load()
    for which, struct in enumerate((_lib.MkModelDesc, _lib.MkLaunchInfo, _lib.MkStatus, _lib.MkNvfp4Matrix)):
        assert lib.mk_abi_sizeof(which) == C.sizeof(struct), struct.__name__
    assert lib.mk_abi_sizeof(99) == -1


def test_bad_arguments_are_rejected_without_a_device():
    lib = _lib.load()
    handle = C.c_void_p()
    assert lib.mk_create(None, C.byref(handle)) == _lib.MK_ERR_BAD_ARGUMENT
    desc = _lib.MkModelDesc()
    desc.abi_version = 999
    assert lib.mk_create(C.byref(desc), C.byref(handle)) == _lib.MK_ERR_BAD_ARGUMENT
    assert b"ABI version" in lib.mk_last_error()
    desc.abi_version = _lib.MK_ABI_VERSION
    desc.weight_format = 7
    assert lib.mk_create(C.byref(desc), C.byref(handle)) == _lib.MK_ERR_UNSUPPORTED
    assert lib.mk_step(None, 0, 0, None, None, None) == _lib.MK_ERR_BAD_ARGUMENT
    assert lib.mk_query(None, None) == _lib.MK_ERR_BAD_ARGUMENT
    assert lib.mk_gemv(None, None, None, None, None, 16, 32, 1.0, 0, 1, None, 0, None) != 0
    # split-K scratch is the caller's: size query only, no device needed
    assert lib.mk_gemv_workspace_bytes(8192, 2048) == 0
    assert lib.mk_gemv_workspace_bytes(2048, 8192) == 512 + 4 * 8 * 2048 * 4
    assert lib.mk_tp_connect(None, None, 2) == _lib.MK_ERR_BAD_ARGUMENT
    assert lib.mk_nvfp4_quantize(None, None, None, None, 1, 16, 1.0, None) != 0
    lib.mk_destroy(None)


def test_product_package_never_imports_the_oracle():
    for path in (ROOT / "thor_megakernels_b200").rglob("*.py"):
        text = path.read_text()
        assert "import oracle" not in text and "from oracle" not in text, path


def test_cpu_tensors_are_refused():
    import torch

    from thor_megakernels_b200.runtime import Megakernel

    t = torch.zeros(4, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        Megakernel(barriers=t, qkv_w=t, attn_norm_w=t, o_w=t, mlp_norm_w=t, up_w=t, gate_w=t, down_w=t,
                   lm_head_norm_w=t, lm_head_w=t, k_cache=t, v_cache=t, rope_cos=t, rope_sin=t, hidden_states=t,
                   q_post_rope=t, attn_out=t, attn_lse_intermediates=t, attn_out_intermediates=t, silu_out=t,
                   logits=t, attn_scale=1.0, rms_norm_eps=1e-5)
