"""Loader for the native step function (reference ``megakernels/mk.py:5-17``).

``mk_dir`` is any directory holding a module ``mk_llama`` that exports a
function ``mk_llama``.  The reference builds one such module per instruction
set; this package ships ``native/`` (batch-1 latency set, ``DEFAULT_MK_DIR``)
and ``native_throughput/`` (batched set).
"""
from __future__ import annotations

import importlib
import importlib.util
import sys
from pathlib import Path

DEFAULT_MK_DIR = Path(__file__).resolve().parent / "native"
THROUGHPUT_MK_DIR = Path(__file__).resolve().parent / "native_throughput"

_loaded: dict[str, object] = {}


def get_mk_func(mk_dir: Path | str | None = None):
    mk_dir = Path(mk_dir).expanduser().absolute() if mk_dir is not None else DEFAULT_MK_DIR
    source = mk_dir / "mk_llama.py"
    if source.exists():
        # loaded by path, so that two directories' ``mk_llama`` modules can live in one process
        key = str(source)
        if key not in _loaded:
            spec = importlib.util.spec_from_file_location(f"mk_llama_{len(_loaded)}", source)
            module = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(module)
            _loaded[key] = module
        return _loaded[key].mk_llama
    if str(mk_dir) not in sys.path:
        sys.path.append(str(mk_dir))
    return importlib.import_module("mk_llama").mk_llama


class MK_Interpreter:
    default_mk_dir = DEFAULT_MK_DIR

    def __init__(self, mk_dir: Path | str | None = None):
        self.mk_func = get_mk_func(mk_dir if mk_dir is not None else self.default_mk_dir)

    def interpret(self, globs):
        raise NotImplementedError
