"""ctypes access to the CPU oracle (cubit_oracle.cpp).  Test infrastructure only: imported by the
tests, the smoke check and the CPU-baseline leg of the benchmark, never by the product package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
ROOT = ORACLE_DIR.parent
ORACLE_SO = ORACLE_DIR / "_build" / "liboracle.so"
TABLE = ROOT / "cubit_b200" / "tables" / "sm120.json"


def build_oracle() -> Path:
    """Compiles the oracle with its Makefile when the library is missing or stale."""
    src = ORACLE_DIR / "cubit_oracle.cpp"
    if not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    return ORACLE_SO


class Oracle:
    """The reference algorithm on host cores: decode / encode / roundtrip / stream generator."""

    def __init__(self, table_path: os.PathLike | str | None = None, text: bytes | None = None):
        self.lib = C.CDLL(str(build_oracle()))
        L = self.lib
        L.orc_load.restype = C.c_void_p
        L.orc_load.argtypes = [C.c_char_p]
        L.orc_load_text.restype = C.c_void_p
        L.orc_load_text.argtypes = [C.c_char_p, C.c_uint64]
        L.orc_last_error.restype = C.c_char_p
        L.orc_free.argtypes = [C.c_void_p]
        L.orc_table_info.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.orc_variant_name.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p)]
        L.orc_decode_full.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint32), C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32), C.c_void_p,
                                      C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.orc_variant_opcode.argtypes = [C.c_void_p, C.c_uint32, C.c_char_p, C.c_uint32]
        L.orc_kernel_meta.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                      C.c_void_p, C.c_uint32]
        L.orc_field_extraction.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_char_p, C.c_uint32]
        L.orc_decode_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_encode_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int]
        L.orc_roundtrip_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int]
        L.orc_synth_batch.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_elf_text_sections.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint32, C.c_char_p, C.c_uint64]
        if text is not None:
            self.h = L.orc_load_text(text, len(text))
        else:
            self.h = L.orc_load(str(table_path or TABLE).encode())
        if not self.h:
            raise ValueError(L.orc_last_error().decode())

    def close(self):
        if self.h:
            self.lib.orc_free(self.h)
            self.h = None

    def table_info(self):
        k, g = C.c_uint32(), C.c_uint32()
        self.lib.orc_table_info(self.h, k, g)
        return k.value, g.value

    def variant_name(self, v: int):
        k, m = C.c_char_p(), C.c_char_p()
        if self.lib.orc_variant_name(self.h, v, k, m):
            raise IndexError(v)
        return k.value.decode(), m.value.decode()

    def decode_full(self, lo: int, hi: int):
        """One word -> dict with key, mod_group, per-field values, scheduling; None-like status on reject."""
        cap = 64
        vals = np.zeros(cap, np.uint64); sh = np.zeros(cap, np.uint32); bits = np.zeros(cap, np.uint32)
        tok = np.zeros(cap, np.int32); sched = np.zeros(5, np.uint32)
        variant, synth, tie, score = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        n = self.lib.orc_decode_full(self.h, lo, hi, variant, vals.ctypes.data, sh.ctypes.data, bits.ctypes.data,
                                     tok.ctypes.data, cap, synth, sched.ctypes.data, tie, score)
        out = {"status": 0 if n >= 0 else -n,
               "scheduling": dict(stall=int(sched[0]), yield_flag=bool(sched[1]), write_bar=int(sched[2]),
                                  read_bar=int(sched[3]), wait_mask=int(sched[4]))}
        if n < 0:
            return out
        key, mg = self.variant_name(variant.value)
        buf = C.create_string_buffer(64)
        fields = []
        for i in range(n):
            self.lib.orc_field_extraction(self.h, variant.value, i, buf, 64)
            fields.append(dict(shift=int(sh[i]), bits=int(bits[i]), value=int(vals[i]), token_idx=int(tok[i]),
                               extraction=buf.value.decode()))
        self.lib.orc_variant_opcode(self.h, variant.value, buf, 64)
        out.update(variant=variant.value, key=key, mod_group=mg, opcode=buf.value.decode(), fields=fields, synth=synth.value, tie=bool(tie.value),
                   score=C.c_int32(score.value).value)
        return out

    def kernel_meta(self, code: bytes):
        """Reference metadata inference over one kernel's code: regcount, num_barriers, exit offsets."""
        buf = np.frombuffer(code, np.uint8)
        cap = max(len(buf) // 16, 1)
        exits = np.zeros(cap, np.uint32)
        mr, bm = C.c_uint32(), C.c_uint32()
        n = self.lib.orc_kernel_meta(self.h, buf.ctypes.data if len(buf) else None, len(buf), mr, bm, exits.ctypes.data, cap)
        return dict(max_reg=mr.value, barrier_mask=bm.value, regcount=max(((mr.value + 32) & ~31), 32),
                    num_barriers=bin(bm.value).count("1"), exit_offsets=exits[:n].tolist())

    def decode_batch(self, words: np.ndarray, threads: int = 1):
        words = np.ascontiguousarray(words, dtype=np.uint8).reshape(-1, 16)
        n = len(words)
        form = np.zeros(n, np.uint16); slots = np.zeros((8, n), np.uint32); ctrl = np.zeros(n, np.uint32)
        self.lib.orc_decode_batch(self.h, words.ctypes.data, n, form.ctypes.data, slots.ctypes.data, ctrl.ctypes.data, threads)
        return form, slots, ctrl

    def encode_batch(self, form, slots, ctrl, threads: int = 1):
        form = np.ascontiguousarray(form, np.uint16); slots = np.ascontiguousarray(slots, np.uint32)
        ctrl = np.ascontiguousarray(ctrl, np.uint32)
        n = len(form)
        assert slots.shape == (8, n)
        words = np.zeros((n, 16), np.uint8)
        self.lib.orc_encode_batch(self.h, form.ctypes.data, slots.ctypes.data, ctrl.ctypes.data, n, words.ctypes.data, threads)
        return words

    def roundtrip_batch(self, words: np.ndarray, threads: int = 1):
        words = np.ascontiguousarray(words, dtype=np.uint8).reshape(-1, 16)
        status = np.zeros(len(words), np.uint8)
        self.lib.orc_roundtrip_batch(self.h, words.ctypes.data, len(words), status.ctypes.data, threads)
        return status

    def synth(self, mix: int, seed: int, n: int, noise_ppm: int = 0, first: int = 0, threads: int = 1, records: bool = True):
        words = np.zeros((n, 16), np.uint8)
        if records:
            form = np.zeros(n, np.uint16); slots = np.zeros((8, n), np.uint32); ctrl = np.zeros(n, np.uint32)
            self.lib.orc_synth_batch(self.h, mix, seed, noise_ppm, first, n, words.ctypes.data, form.ctypes.data,
                                     slots.ctypes.data, ctrl.ctypes.data, threads)
            return words, form, slots, ctrl
        self.lib.orc_synth_batch(self.h, mix, seed, noise_ppm, first, n, words.ctypes.data, None, None, None, threads)
        return words

    def elf_text_sections(self, data: bytes):
        cap = 1 << 16
        offs = np.zeros(cap, np.uint64); sizes = np.zeros(cap, np.uint64)
        names = C.create_string_buffer(cap * 24)
        buf = (C.c_char * len(data)).from_buffer_copy(data)
        n = self.lib.orc_elf_text_sections(buf, len(data), offs.ctypes.data, sizes.ctypes.data, cap, names, len(names))
        if n < 0:
            raise ValueError("not a little-endian ELF64")
        parts = names.raw.split(b"\0")[:n]
        return [(parts[i].decode(), int(offs[i]), int(sizes[i])) for i in range(n)]


def words_from_ints(values) -> np.ndarray:
    """List of 128-bit Python ints -> (n, 16) uint8 little-endian words."""
    return np.frombuffer(b"".join(int(v).to_bytes(16, "little") for v in values), np.uint8).reshape(-1, 16).copy()


def ints_from_words(words: np.ndarray):
    return [int.from_bytes(bytes(w), "little") for w in np.asarray(words, np.uint8).reshape(-1, 16)]
