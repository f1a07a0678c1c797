"""Loader of the compiled megakernel entry point.

Reference: megakernels/mk.py:5-17.  ``mk_dir`` is a directory holding an
importable ``mk_llama`` module that exposes the callable ``mk_llama``; by
default that is this package's ``native/`` directory, whose module is a ctypes
shim over the C-ABI library ``libmkb200.so``.
"""

from __future__ import annotations

import importlib
import sys
from pathlib import Path

DEFAULT_MK_DIR = Path(__file__).resolve().parent / "native"


def get_mk_func(mk_dir: Path | None = None):
    mk_dir = Path(mk_dir or DEFAULT_MK_DIR).expanduser().absolute()
    if str(mk_dir) not in sys.path:
        sys.path.append(str(mk_dir))
    module = importlib.import_module("mk_llama")
    module.load_library()  # fail here, loudly, when the CUDA library is absent
    return module.mk_llama


class MK_Interpreter:
    def __init__(self, mk_dir: Path | None = None):
        self.mk_func = get_mk_func(mk_dir)

    def interpret(self, globs):
        raise NotImplementedError
