"""The shared library loads without a GPU and exports every function the public header declares."""
import ctypes as C
import re

import numpy as np
import pytest

import cubit_b200
from cubit_b200 import _native

HEADER = cubit_b200.build.PKG.parent / "include" / "cubit_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(cubit_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _native.load_library()
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(names) == set(_native.SIGNATURES), set(names) ^ set(_native.SIGNATURES)


def test_compute_calls_fail_loudly_without_a_device(host_codec):
    words = np.zeros((4, 16), np.uint8)
    for call in (lambda: host_codec.decode_batch(words), lambda: host_codec.roundtrip_batch(words),
                 lambda: host_codec.encode_batch(np.zeros(4, np.uint16), np.zeros((8, 4), np.uint32), np.zeros(4, np.uint32)),
                 lambda: host_codec.synth(0, 0, 4), lambda: host_codec.decode(0, 0)):
        with pytest.raises(cubit_b200.CubitError) as e:
            call()
        assert e.value.code == -4


def test_bad_arguments_return_codes_not_crashes():
    lib = _native.load_library()
    assert lib.cubit_ctx_create(None, None, 0, None) == -1
    assert lib.cubit_table_info(None, None, None) == -1
    elf = C.c_void_p()
    assert lib.cubit_elf_parse(None, 0, C.byref(elf)) == -1
    lib.cubit_ctx_destroy(None)
    lib.cubit_elf_free(None)
    assert lib.cubit_elf_num_text(None) == 0


def test_context_creation_failure_returns_a_code_and_a_message(monkeypatch):
    """A device that cannot be opened and a table that cannot be read: an error code, a message
    under cubit_last_error(NULL), no context, and nothing thrown through the C frames."""
    lib = _native.load_library()
    ctx = C.c_void_p()
    import torch
    if not torch.cuda.is_available():
        devices = (C.c_int * 1)(0)
        assert lib.cubit_ctx_create(None, devices, 1, C.byref(ctx)) == -3 and not ctx.value
        assert b"cuda" in lib.cubit_last_error(None).lower()
    assert lib.cubit_ctx_create(b"/nonexistent/sm120.json", None, 0, C.byref(ctx)) == -2 and not ctx.value
    assert b"/nonexistent/sm120.json" in lib.cubit_last_error(None)


def test_text_layer_entry_points_say_what_is_missing():
    with pytest.raises(NotImplementedError, match="scheduling pass"):
        cubit_b200.asm("NOP")
