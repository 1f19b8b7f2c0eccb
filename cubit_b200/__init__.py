"""cubit_b200 — B200-native batch SM120 SASS codec behind cubit's Python interface.

Module-level functions carry the names and signatures of the reference's PyO3 module
(reference src/python.rs:215-225): ``decode``, ``decode_kernel``, ``table_info`` run on the
GPU through a process-wide :class:`Codec` created on first use (the reference keeps a
process-wide table and index the same way, src/python.rs:28-42).  ``encode``, ``to_sass`` and
``asm`` work on SASS *text*; the text layer is not part of this package yet and they raise
NotImplementedError — record-level encoding is :meth:`Codec.encode_batch`.
"""
from __future__ import annotations

import os
import threading

from .codec import (FORM_NONE, MEM_DEVICE, MEM_HOST, MIX_FAMILY, MIX_UNIFORM, MIX_ZIPF, RT_EXACT, RT_MISMATCH,
                    RT_REJECTED, SCHED_MASK, Codec, CubitError, FieldMeta, VariantMeta, build_cubin, unpack_ctrl)
from .sharding import shard_range, shard_sections

__all__ = ["Codec", "CubitError", "FieldMeta", "VariantMeta", "build_cubin", "unpack_ctrl", "shard_range",
           "shard_sections", "decode", "decode_kernel", "table_info", "encode", "to_sass", "asm", "FORM_NONE",
           "MEM_HOST", "MEM_DEVICE", "MIX_UNIFORM", "MIX_ZIPF", "MIX_FAMILY", "RT_EXACT", "RT_MISMATCH", "RT_REJECTED",
           "SCHED_MASK"]

_default: Codec | None = None
_lock = threading.Lock()


def default_codec() -> Codec:
    """Process-wide codec on the devices named by CUBIT_B200_DEVICES (comma-separated CUDA
    ordinals, default "0")."""
    global _default
    with _lock:
        if _default is None:
            spec = os.environ.get("CUBIT_B200_DEVICES", "0")
            _default = Codec(tuple(int(x) for x in spec.split(",") if x.strip() != ""))
        return _default


def decode(lo: int, hi: int, addr: int = 0) -> dict:
    """Decode one 128-bit word to a dict with key, mod_group, opcode, addr, fields, scheduling."""
    return default_codec().decode(lo, hi, addr)


def decode_kernel(cubin_path, kernel_name: str) -> list:
    """Decode every instruction of the first text section whose name contains `kernel_name`."""
    return default_codec().decode_kernel(cubin_path, kernel_name)


def table_info() -> tuple:
    """(number of instruction keys, number of encoding variants)."""
    return default_codec().table_info()


def encode(sass: str, addr: int = 0):
    raise NotImplementedError("text-level encode needs the SASS parser, which this package does not include; "
                              "use Codec.encode_batch on records")


def to_sass(lo: int, hi: int, addr: int = 0) -> str:
    raise NotImplementedError("the SASS printer is not part of this package")


def asm(code: str, addr: int = 0):
    raise NotImplementedError("the assembler front end is not part of this package")
