"""cubit_b200 — B200-native batch SM120 SASS codec behind cubit's Python interface.

Module-level functions carry the names and signatures of the reference's PyO3 module
(reference src/python.rs:215-225): ``decode``, ``decode_kernel``, ``table_info`` run on the
GPU through a process-wide :class:`Codec` created on first use (the reference keeps a
process-wide table and index the same way, src/python.rs:28-42).  ``encode`` parses the text
on the host, encodes the record on the GPU and applies the text-derived bits on the host;
``encode_lines`` does the same for a program with labels; ``to_sass`` decodes on the GPU and
prints on the host.  ``asm`` (which runs the reference's scheduling pass before encoding) is
not part of this package and raises NotImplementedError.
"""
from __future__ import annotations

import os
import threading

from .codec import (FORM_NONE, MEM_DEVICE, MEM_HOST, MIX_FAMILY, MIX_UNIFORM, MIX_ZIPF, RT_EXACT, RT_MISMATCH,
                    RT_REJECTED, SCHED_MASK, Codec, CubitError, FieldMeta, VariantMeta, build_cubin, patch_text, unpack_ctrl)
from .sharding import shard_range, shard_sections

__all__ = ["Codec", "CubitError", "FieldMeta", "VariantMeta", "build_cubin", "patch_text", "unpack_ctrl", "shard_range",
           "shard_sections", "decode", "decode_kernel", "table_info", "encode", "encode_lines", "to_sass", "asm", "FORM_NONE",
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


_host_only: Codec | None = None


def table_info() -> tuple:
    """(number of instruction keys, number of encoding variants).  Answered from the table alone, so it
    also works on a machine without a GPU."""
    global _host_only
    with _lock:
        if _default is not None:
            return _default.table_info()
        if _host_only is None:
            _host_only = Codec(devices=())
        return _host_only.table_info()


def encode(sass: str, addr: int = 0) -> tuple:
    """Encode one SASS instruction to (lo64, hi64); ValueError("parse error: ..." /
    "encode error: ...") as the reference raises."""
    return default_codec().encode(sass, addr)


def encode_lines(code: str, addr: int = 0) -> tuple:
    """(bytes, count) for a program: ';' / newline separated statements, labels, comments and
    optional "[B------:R-:W-:-:S01]" prefixes.  Control codes are taken as written; the
    reference's asm() reschedules them first, which this function does not do."""
    words = default_codec().encode_text(code, addr, program=True)
    return words.tobytes(), len(words)


def to_sass(lo: int, hi: int, addr: int = 0) -> str:
    """SASS text of one 128-bit word, e.g. "IADD3 R5, PT, PT, R9, R4, R5"; encode() reads it back."""
    return default_codec().to_sass(lo, hi, addr)


def asm(code: str, addr: int = 0):
    raise NotImplementedError("asm() runs the reference's scheduling pass before encoding, which is not part of "
                              "this package; encode_lines() assembles the same text with control codes as written")
