"""Loader for the native step function (reference ``megakernels/mk.py:5-17``).

``mk_dir`` is any directory holding a module ``mk_llama`` that exports a
function ``mk_llama``; ``DEFAULT_MK_DIR`` is the one shipped with this package.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

DEFAULT_MK_DIR = Path(__file__).resolve().parent / "native"


def get_mk_func(mk_dir: Path | str | None = None):
    mk_dir = Path(mk_dir).expanduser().absolute() if mk_dir is not None else DEFAULT_MK_DIR
    if str(mk_dir) not in sys.path:
        sys.path.append(str(mk_dir))
    return importlib.import_module("mk_llama").mk_llama


class MK_Interpreter:
    def __init__(self, mk_dir: Path | str | None = None):
        self.mk_func = get_mk_func(mk_dir)

    def interpret(self, globs):
        raise NotImplementedError
