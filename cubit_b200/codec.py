"""Host-side mirror of cubit's codec interface over the CUDA library.

`Codec` owns one library context (ISA table compiled and resident on the chosen GPUs) and
offers batch decode / encode / roundtrip on numpy arrays or raw device pointers, plus the
single-word and per-kernel calls of the reference's Python module (reference
src/python.rs:46-177) with the same names, argument meaning, result shapes and errors.
All instruction work runs in the CUDA kernels; nothing here decodes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from . import _native
from ._native import Counts, VariantInfo

MEM_HOST, MEM_DEVICE = 0, 1
MIX_UNIFORM, MIX_ZIPF, MIX_FAMILY = 0, 1, 2
FORM_NONE = 0xFFFF
RT_EXACT, RT_MISMATCH, RT_REJECTED = 0, 1, 2
SCHED_MASK = 0x1FFFF << 105
NOT_STORED = 0xFFFFFFFF
TEXT_ONE, TEXT_PROGRAM = 0, 1
ERR_TEXT = -8
STATIC_MAX_WORDS = 65536


class CubitError(RuntimeError):
    """A library call failed; `.code` is the negative cubit_status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"cubit_b200 error {code}: {message}")
        self.code = code
        self.message = message


@dataclass(frozen=True)
class FieldMeta:
    name: str
    shift: int
    bits: int
    token_idx: int
    extraction: str
    dst_pos: int       # bit position inside the 256-bit slot area, or NOT_STORED
    stored_bits: int   # width held there: the part of the field below bit 96 of the word


@dataclass(frozen=True)
class VariantMeta:
    variant: int
    key: str
    mod_group: str
    opcode: str
    key_id: int
    layout_kind: int
    synth_mask: int
    ra_tok: int
    rb_tok: int
    fields: tuple


def unpack_ctrl(ctrl: int) -> dict:
    """Splits a record's ctrl word; the scheduling part follows reference src/scheduling.rs:70-78."""
    c = int(ctrl)
    return dict(stall=c & 0xF, yield_flag=bool((c >> 4) & 1), write_bar=(c >> 5) & 7, read_bar=(c >> 8) & 7,
                wait_mask=(c >> 11) & 0x3F, reuse=(c >> 17) & 7, guard=(c >> 20) & 0xF, synth=(c >> 24) & 0xF,
                tie=bool((c >> 28) & 1), status=(c >> 30) & 3)


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    return C.c_void_p(int(a))


class Codec:
    """One ISA table compiled and resident on `devices` (CUDA ordinals).  `devices=()` gives a
    host-only object: table metadata and ELF helpers work, codec calls raise CubitError."""

    def __init__(self, devices: Sequence[int] = (0,), table_path: str | os.PathLike | None = None):
        self._lib = _native.load_library()
        self._ctx = C.c_void_p()
        devs = (C.c_int * max(len(devices), 1))(*devices)
        path = os.fspath(table_path).encode() if table_path else None
        rc = self._lib.cubit_ctx_create(path, devs, len(devices), C.byref(self._ctx))
        if rc:
            raise CubitError(rc, self._lib.cubit_last_error(None).decode())
        self.devices = tuple(devices)
        self._meta: dict[int, VariantMeta] = {}

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.cubit_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc:
            raise CubitError(rc, self._lib.cubit_last_error(self._ctx).decode())

    # ---- table -------------------------------------------------------------------------

    def table_info(self) -> tuple[int, int]:
        k, g = C.c_uint32(), C.c_uint32()
        self._check(self._lib.cubit_table_info(self._ctx, k, g))
        return k.value, g.value

    def variant(self, variant: int) -> VariantMeta:
        m = self._meta.get(variant)
        if m is None:
            info = VariantInfo()
            self._check(self._lib.cubit_variant_lookup(self._ctx, variant, C.byref(info)))
            fields = tuple(FieldMeta(info.fields[i].name.decode(), info.fields[i].shift, info.fields[i].bits,
                                     info.fields[i].token_idx, info.fields[i].extraction.decode(), info.fields[i].dst_pos,
                                     info.fields[i].stored_bits)
                           for i in range(info.n_fields))
            m = VariantMeta(variant, info.key.decode(), info.mod_group.decode(), info.opcode.decode(), info.key_id,
                            info.layout_kind, info.synth_mask, info.ra_tok, info.rb_tok, fields)
            self._meta[variant] = m
        return m

    def find_variant(self, key: str, mod_group: str = "") -> int:
        v = C.c_uint32()
        self._check(self._lib.cubit_variant_find(self._ctx, key.encode(), mod_group.encode(), v))
        return v.value

    def key_name(self, key_id: int) -> tuple[str, int, int]:
        name, first, count = C.c_char_p(), C.c_uint32(), C.c_uint32()
        self._check(self._lib.cubit_key_name(self._ctx, key_id, name, first, count))
        return name.value.decode(), first.value, count.value

    # ---- batch calls on host arrays -------------------------------------------------------

    @staticmethod
    def _words(words) -> np.ndarray:
        w = np.ascontiguousarray(words, dtype=np.uint8)
        if w.size % 16:
            raise ValueError("word buffer length is not a multiple of 16 bytes")
        return w.reshape(-1, 16)

    def decode_batch(self, words):
        """(n,16) uint8 little-endian words -> (form u16[n], slots u32[8,n], ctrl u32[n], counts)."""
        w = self._words(words)
        n = len(w)
        form = np.empty(n, np.uint16); slots = np.empty((8, n), np.uint32); ctrl = np.empty(n, np.uint32)
        counts = Counts()
        self._check(self._lib.cubit_decode_batch(self._ctx, _ptr(w), n, _ptr(form), _ptr(slots), _ptr(ctrl),
                                                 C.byref(counts), MEM_HOST, None))
        return form, slots, ctrl, counts.as_dict()

    def decode_batch_static(self, words, device_slot: int = 0):
        """decode_batch for at most STATIC_MAX_WORDS words without any device allocation: the batch is
        staged through a fixed array built into the library.  For callers that must not call cudaMalloc
        while running (device memory reserved by someone else, or no tolerance for its implicit
        synchronisation).  All calls on one GPU share that array, from whichever Codec; the library
        serialises them with one lock per GPU, so they are safe but do not run in parallel."""
        w = self._words(words)
        n = len(w)
        form = np.empty(n, np.uint16); slots = np.empty((8, n), np.uint32); ctrl = np.empty(n, np.uint32)
        counts = Counts()
        self._check(self._lib.cubit_decode_batch_static(self._ctx, device_slot, _ptr(w), n, _ptr(form), _ptr(slots),
                                                        _ptr(ctrl), C.byref(counts)))
        return form, slots, ctrl, counts.as_dict()

    def encode_batch(self, form, slots, ctrl) -> np.ndarray:
        form = np.ascontiguousarray(form, np.uint16); slots = np.ascontiguousarray(slots, np.uint32)
        ctrl = np.ascontiguousarray(ctrl, np.uint32)
        n = len(form)
        if slots.shape != (8, n) or ctrl.shape != (n,):
            raise ValueError("slots must be (8, n) and ctrl (n,)")
        words = np.empty((n, 16), np.uint8)
        self._check(self._lib.cubit_encode_batch(self._ctx, _ptr(form), _ptr(slots), _ptr(ctrl), n, _ptr(words),
                                                 MEM_HOST, None))
        return words

    def roundtrip_batch(self, words):
        w = self._words(words)
        status = np.empty(len(w), np.uint8)
        counts = Counts()
        self._check(self._lib.cubit_roundtrip_batch(self._ctx, _ptr(w), len(w), _ptr(status), C.byref(counts),
                                                    MEM_HOST, None))
        return status, counts.as_dict()

    def synth(self, mix: int, seed: int, n: int, noise_ppm: int = 0, first: int = 0):
        """Words [first, first+n) of a seeded synthetic stream and the generator's records."""
        words = np.empty((n, 16), np.uint8); form = np.empty(n, np.uint16)
        slots = np.empty((8, n), np.uint32); ctrl = np.empty(n, np.uint32)
        self._check(self._lib.cubit_synth_batch(self._ctx, mix, seed, noise_ppm, first, n, _ptr(words), _ptr(form),
                                                _ptr(slots), _ptr(ctrl), MEM_HOST, None))
        return words, form, slots, ctrl

    # ---- batch calls on device pointers (integers), queued on `stream` ---------------------

    def decode_device(self, words_ptr, n, form_ptr, slots_ptr, ctrl_ptr, stream=None, want_counts=False):
        counts = Counts() if want_counts else None
        self._check(self._lib.cubit_decode_batch(self._ctx, _ptr(words_ptr), n, _ptr(form_ptr), _ptr(slots_ptr),
                                                 _ptr(ctrl_ptr), C.byref(counts) if counts else None, MEM_DEVICE,
                                                 _ptr(stream)))
        return counts.as_dict() if counts else None

    def encode_device(self, form_ptr, slots_ptr, ctrl_ptr, n, words_ptr, stream=None):
        self._check(self._lib.cubit_encode_batch(self._ctx, _ptr(form_ptr), _ptr(slots_ptr), _ptr(ctrl_ptr), n,
                                                 _ptr(words_ptr), MEM_DEVICE, _ptr(stream)))

    def roundtrip_device(self, words_ptr, n, status_ptr, stream=None, want_counts=False):
        counts = Counts() if want_counts else None
        self._check(self._lib.cubit_roundtrip_batch(self._ctx, _ptr(words_ptr), n, _ptr(status_ptr),
                                                    C.byref(counts) if counts else None, MEM_DEVICE, _ptr(stream)))
        return counts.as_dict() if counts else None

    def synth_device(self, mix, seed, n, words_ptr=None, form_ptr=None, slots_ptr=None, ctrl_ptr=None, noise_ppm=0,
                     first=0, stream=None):
        self._check(self._lib.cubit_synth_batch(self._ctx, mix, seed, noise_ppm, first, n, _ptr(words_ptr),
                                                _ptr(form_ptr), _ptr(slots_ptr), _ptr(ctrl_ptr), MEM_DEVICE,
                                                _ptr(stream)))

    # ---- records -> named fields ------------------------------------------------------------

    def field_values(self, form: int, slots) -> list[int]:
        """Values of the variant's table fields, in table order, from the 8 slots of one record."""
        area = 0
        for s in range(8):
            area |= int(slots[s]) << (32 * s)
        return [0 if f.dst_pos == NOT_STORED else (area >> f.dst_pos) & ((1 << f.stored_bits) - 1)
                for f in self.variant(int(form)).fields]

    def pack_fields(self, form: int, values: Sequence[int]) -> np.ndarray:
        """Inverse of field_values: table-order values -> the 8 slots of a record."""
        area = 0
        for f, v in zip(self.variant(int(form)).fields, values):
            if f.dst_pos == NOT_STORED:
                continue
            mask = ((1 << f.stored_bits) - 1) << f.dst_pos
            area = (area & ~mask) | ((int(v) << f.dst_pos) & mask)   # later fields overwrite shared bits
        return np.array([(area >> (32 * s)) & 0xFFFFFFFF for s in range(8)], np.uint32)

    def record_to_dict(self, form, slots, ctrl, addr: int = 0, brief: bool = False) -> dict:
        """The dict cubit.decode returns (reference src/python.rs:71-97); `brief` gives the
        shorter per-instruction shape of cubit.decode_kernel (src/python.rs:131-155)."""
        m = self.variant(int(form))
        c = unpack_ctrl(ctrl)
        fields = []
        for f, v in zip(m.fields, self.field_values(form, slots)):
            d = dict(name=f.name, shift=f.shift, bits=f.bits, value=v)
            if not brief:
                d.update(token_idx=f.token_idx, extraction=f.extraction)
            fields.append(d)
        # Generic abs/neg modifiers the reference appends after the table fields (src/decoder.rs:340-343).
        for k, (bit, tok, ext) in enumerate(((63, m.rb_tok, "neg"), (62, m.rb_tok, "abs"), (72, m.ra_tok, "neg"),
                                             (73, m.ra_tok, "abs"))):
            if (c["synth"] >> k) & 1:
                d = dict(name=ext, shift=bit, bits=1, value=1)
                if not brief:
                    d.update(token_idx=tok, extraction=ext)
                fields.append(d)
        if brief:
            sched = dict(stall=c["stall"], yield_flag=c["yield_flag"], wait_mask=c["wait_mask"])
            return dict(addr=addr, key=m.key, mod_group=m.mod_group, opcode=m.opcode, fields=fields, scheduling=sched)
        sched = dict(stall=c["stall"], yield_flag=c["yield_flag"], write_bar=c["write_bar"], read_bar=c["read_bar"],
                     wait_mask=c["wait_mask"])
        return dict(key=m.key, mod_group=m.mod_group, opcode=m.opcode, addr=addr, fields=fields, scheduling=sched)

    # ---- the reference's Python surface -------------------------------------------------------

    def decode(self, lo: int, hi: int, addr: int = 0) -> dict:
        """cubit.decode(lo, hi, addr=0): one word through the batch kernel."""
        word = (int(lo) & (2**64 - 1)).to_bytes(8, "little") + (int(hi) & (2**64 - 1)).to_bytes(8, "little")
        form, slots, ctrl, _ = self.decode_batch(np.frombuffer(word, np.uint8))
        self._raise_if_rejected(lo, hi, int(ctrl[0]))
        return self.record_to_dict(form[0], slots[:, 0], ctrl[0], addr)

    @staticmethod
    def _raise_if_rejected(lo: int, hi: int, ctrl: int):
        """The two decode failures of the reference, with its messages (src/decoder.rs:173, :287)."""
        status = (ctrl >> 30) & 3
        opcode_bits = int(lo) & 0xFFF
        if status == 1:
            raise ValueError(f"decode error: no instruction matches opcode 0x{opcode_bits:04x}")
        if status == 2:
            clean = (int(lo) & (2**64 - 1)) | ((int(hi) & 0xFFFFFFFF) << 64)
            raise ValueError(f"decode error: no instruction matches code 0x{clean:032x} at opcode 0x{opcode_bits:04x}")

    # ---- SASS text (host parse, GPU record encode, host patch) ----------------------------

    def parse_text(self, line: str, addr: int = 0) -> dict:
        """The parsed form of one instruction line (key, opcode, guard, typed operands, ...);
        ValueError("parse error: ...") when the line is not an instruction."""
        import json
        need = C.c_uint64()
        text = line.encode()
        rc = self._lib.cubit_text_parse(self._ctx, text, addr, None, 0, need)
        if rc == ERR_TEXT:
            raise ValueError(self._lib.cubit_last_error(self._ctx).decode())
        self._check(rc)
        buf = C.create_string_buffer(need.value)
        self._check(self._lib.cubit_text_parse(self._ctx, text, addr, buf, need.value, need))
        return json.loads(buf.value.decode())

    def lower_text(self, text: str, addr: int = 0, program: bool = True):
        """Text -> (form, slots, ctrl, clear, set): the records cubit_encode_batch takes and the
        128-bit patches ((word & ~clear) | set) that carry the text-derived bits.  clear / set
        are uint8[n, 16] little-endian.  ValueError with the reference's message on failure."""
        mode = TEXT_PROGRAM if program else TEXT_ONE
        raw = text.encode()
        n = C.c_uint64()
        rc = self._lib.cubit_text_lower(self._ctx, raw, addr, mode, 0, None, None, None, None, None, n)
        if rc == ERR_TEXT:
            raise ValueError(self._lib.cubit_last_error(self._ctx).decode())
        self._check(rc)
        cap = max(int(n.value), 1)
        form = np.zeros(cap, np.uint16); slots = np.zeros((8, cap), np.uint32); ctrl = np.zeros(cap, np.uint32)
        clear = np.zeros((cap, 16), np.uint8); set_ = np.zeros((cap, 16), np.uint8)
        self._check(self._lib.cubit_text_lower(self._ctx, raw, addr, mode, cap, _ptr(form), _ptr(slots), _ptr(ctrl),
                                               _ptr(clear), _ptr(set_), n))
        k = int(n.value)
        return form[:k], slots[:, :k], ctrl[:k], clear[:k], set_[:k]

    def encode_text(self, text: str, addr: int = 0, program: bool = True) -> np.ndarray:
        """Text -> uint8[n, 16] words.  `program=False`: one bare instruction, as the reference's
        encode(sass, addr); `program=True`: statements with labels, comments and optional
        control-code prefixes, as its assembler reads them (without its scheduling pass)."""
        mode = TEXT_PROGRAM if program else TEXT_ONE
        raw = text.encode()
        n = C.c_uint64()
        rc = self._lib.cubit_text_encode(self._ctx, raw, addr, mode, 0, None, n)
        if rc == ERR_TEXT:
            raise ValueError(self._lib.cubit_last_error(self._ctx).decode())
        self._check(rc)
        words = np.zeros((max(int(n.value), 1), 16), np.uint8)
        rc = self._lib.cubit_text_encode(self._ctx, raw, addr, mode, len(words), _ptr(words), n)
        if rc == ERR_TEXT:
            raise ValueError(self._lib.cubit_last_error(self._ctx).decode())
        self._check(rc)
        return words[:int(n.value)]

    def print_text(self, words, addr: int = 0, records=None) -> list[str]:
        """SASS text of each 16-byte word (uint8[n, 16]); word i is taken to sit at addr + 16 i.
        `records` = (form, slots, ctrl) of the words skips the decode (and then needs no GPU).
        Words that match no variant print as the disassembler's "/* ? 0x... */" comment."""
        words = np.ascontiguousarray(words, np.uint8).reshape(-1, 16)
        n = len(words)
        if n == 0:
            return []
        if records is None:
            form, slots, ctrl, _ = self.decode_batch(words)
        else:
            form, slots, ctrl = records
        form = np.ascontiguousarray(form, np.uint16); slots = np.ascontiguousarray(slots, np.uint32)
        ctrl = np.ascontiguousarray(ctrl, np.uint32)
        need = C.c_uint64()
        cap = 96 * n + 64                      # nearly always enough; the call reports the exact size otherwise
        for _ in range(2):
            buf = C.create_string_buffer(cap)
            self._check(self._lib.cubit_text_print(self._ctx, _ptr(words), n, addr, _ptr(form), _ptr(slots), _ptr(ctrl),
                                                   buf, cap, need))
            if need.value <= cap:
                break
            cap = need.value
        return buf.value.decode().split("\n")[:n]

    def to_sass(self, lo: int, hi: int, addr: int = 0) -> str:
        """cubit.to_sass(lo, hi, addr=0) (reference src/python.rs:186-197)."""
        word = (int(lo) & (2**64 - 1)).to_bytes(8, "little") + (int(hi) & (2**64 - 1)).to_bytes(8, "little")
        words = np.frombuffer(word, np.uint8).reshape(1, 16)
        form, slots, ctrl, _ = self.decode_batch(words)
        self._raise_if_rejected(lo, hi, int(ctrl[0]))
        return self.print_text(words, addr, (form, slots, ctrl))[0]

    def encode(self, sass: str, addr: int = 0) -> tuple[int, int]:
        """cubit.encode(sass, addr=0) -> (lo, hi) (reference src/python.rs:48-60)."""
        w = self.encode_text(sass, addr, program=False)[0].tobytes()
        return int.from_bytes(w[:8], "little"), int.from_bytes(w[8:], "little")

    def decode_elf(self, data: bytes, kernel_name: str | None = None, want_raw: bool = True):
        """All words of the text sections of a cubin image (or of the first section whose name
        contains `kernel_name`) in one launch per GPU.  Returns (sections, word_start, form,
        slots, ctrl, raw_words, counts) with sections = [(name, offset, size)]."""
        buf = np.frombuffer(data, np.uint8)
        elf = C.c_void_p()
        rc = self._lib.cubit_elf_parse(_ptr(buf), len(buf), C.byref(elf))
        if rc:
            raise OSError("load error: " + self._lib.cubit_last_error(None).decode())
        try:
            n_text = self._lib.cubit_elf_num_text(elf)
            sections = []
            for i in range(n_text):
                name, off, size = C.c_char_p(), C.c_uint64(), C.c_uint64()
                self._lib.cubit_elf_text(elf, i, name, off, size)
                sections.append((name.value.decode(), off.value, size.value))
            indices = None
            if kernel_name is not None:
                idx = C.c_uint32()
                if self._lib.cubit_elf_find(elf, kernel_name.encode(), idx):
                    names = ", ".join('"' + s[0] + '"' for s in sections)
                    raise ValueError(f"kernel '{kernel_name}' not found. Available: [{names}]")
                indices = np.array([idx.value], np.uint32)
                sections = [sections[idx.value]]
            k = len(sections)
            word_start = np.zeros(k + 1, np.uint64)
            self._check(self._lib.cubit_decode_elf(self._ctx, elf, _ptr(indices), k, _ptr(word_start), 0, None, None,
                                                   None, None, None))
            total = int(word_start[k])
            form = np.empty(total, np.uint16); slots = np.empty((8, total), np.uint32); ctrl = np.empty(total, np.uint32)
            raw = np.empty((total, 16), np.uint8) if want_raw else None
            counts = Counts()
            self._check(self._lib.cubit_decode_elf(self._ctx, elf, _ptr(indices), k, _ptr(word_start), total, _ptr(form),
                                                   _ptr(slots), _ptr(ctrl), _ptr(raw), C.byref(counts)))
            return sections, word_start, form, slots, ctrl, raw, counts.as_dict()
        finally:
            self._lib.cubit_elf_free(elf)

    def infer_kernel_meta(self, data: bytes, kernel_name: str | None = None) -> list[dict]:
        """Per text section of a cubin image (or only the first whose name contains `kernel_name`): the
        metadata the reference infers from code (src/main.rs:787-867) — regcount, num_barriers and the byte
        offsets of EXIT instructions — from one GPU launch over all sections."""
        buf = np.frombuffer(data, np.uint8)
        elf = C.c_void_p()
        if self._lib.cubit_elf_parse(_ptr(buf), len(buf), C.byref(elf)):
            raise OSError("load error: " + self._lib.cubit_last_error(None).decode())
        try:
            names = []
            for i in range(self._lib.cubit_elf_num_text(elf)):
                name = C.c_char_p()
                self._lib.cubit_elf_text(elf, i, name, None, None)
                names.append(name.value.decode())
            indices = None
            if kernel_name is not None:
                idx = C.c_uint32()
                if self._lib.cubit_elf_find(elf, kernel_name.encode(), idx):
                    listed = ", ".join('"' + s + '"' for s in names)
                    raise ValueError(f"kernel '{kernel_name}' not found. Available: [{listed}]")
                indices = np.array([idx.value], np.uint32)
                names = [names[idx.value]]
            k = len(names)
            meta = (_native.KernelMeta * max(k, 1))()
            total = C.c_uint64()
            self._check(self._lib.cubit_infer_kernel_meta(self._ctx, elf, _ptr(indices), k, meta, None, 0, C.byref(total)))
            exits = np.zeros(max(total.value, 1), np.uint32)
            self._check(self._lib.cubit_infer_kernel_meta(self._ctx, elf, _ptr(indices), k, meta, _ptr(exits), len(exits),
                                                          C.byref(total)))
            return [dict(name=names[i], regcount=meta[i].regcount, num_barriers=meta[i].num_barriers,
                         max_reg=meta[i].max_reg, barrier_mask=meta[i].barrier_mask,
                         exit_offsets=exits[meta[i].first_exit:meta[i].first_exit + meta[i].n_exits].tolist())
                    for i in range(k)]
        finally:
            self._lib.cubit_elf_free(elf)

    def disassemble(self, data: bytes, kernel: str | None = None, frozen: bool = False, want_raw_count: bool = False):
        """Listing of a cubin image in the reference's `disassemble` formats (src/main.rs:401-627):
        plain (address comments and "@sched" annotations) or, with `frozen`, a re-assemblable
        .entry block with labels and control-code prefixes in which every line that would not
        encode back to its word is written as __raw__0x...  Returns the text (and the number of
        raw / undecodable lines with `want_raw_count`)."""
        buf = np.frombuffer(data, np.uint8)
        elf = C.c_void_p()
        rc = self._lib.cubit_elf_parse(_ptr(buf), len(buf), C.byref(elf))
        if rc:
            raise OSError("load error: " + self._lib.cubit_last_error(None).decode())
        try:
            need, n_raw = C.c_uint64(), C.c_uint64()
            only = kernel.encode() if kernel is not None else None
            n_text = self._lib.cubit_elf_num_text(elf)
            size = C.c_uint64()
            total = 0
            for i in range(n_text):
                self._lib.cubit_elf_text(elf, i, None, None, C.byref(size))
                total += size.value // 16
            cap = 112 * total + 512 * n_text + 64   # nearly always enough; the call reports the exact size otherwise
            for _ in range(2):
                out = C.create_string_buffer(cap)
                self._check(self._lib.cubit_disassemble(self._ctx, elf, only, int(frozen), out, cap, need, n_raw))
                if need.value <= cap:
                    break
                cap = need.value
        finally:
            self._lib.cubit_elf_free(elf)
        text = out.value.decode()
        return (text, int(n_raw.value)) if want_raw_count else text

    def assemble_listing(self, listing: str, kernel: str, want_failed: bool = False):
        """Code bytes of `kernel` from a plain listing as `disassemble` writes it (the encode loop of the
        reference's listing assembler, src/main.rs:997-1075): every line is encoded at its address, the
        "@sched" value replaces the scheduling field, placeholder comments give their raw word."""
        need, failed = C.c_uint64(), C.c_uint64()
        raw = listing.encode()
        self._check(self._lib.cubit_listing_assemble(self._ctx, raw, kernel.encode(), None, 0, need, failed))
        out = np.zeros(max(int(need.value), 1), np.uint8)
        self._check(self._lib.cubit_listing_assemble(self._ctx, raw, kernel.encode(), _ptr(out), len(out), need, failed))
        code = out[:int(need.value)].tobytes()
        return (code, int(failed.value)) if want_failed else code

    def patch(self, data: bytes) -> tuple[bytes, dict]:
        """The reference's `patch` over a cubin image (src/main.rs:691-764): every instruction goes
        decode -> print -> parse -> encode and, where that works, gets its low 64 bits rewritten
        (high 64 bits are kept).  Returns (new image, counters)."""
        buf = np.frombuffer(data, np.uint8)
        elf = C.c_void_p()
        rc = self._lib.cubit_elf_parse(_ptr(buf), len(buf), C.byref(elf))
        if rc:
            raise OSError("load error: " + self._lib.cubit_last_error(None).decode())
        try:
            out = np.empty(len(buf), np.uint8)
            need = C.c_uint64()
            stats = _native.PatchStats()
            self._check(self._lib.cubit_patch_elf(self._ctx, elf, _ptr(out), len(out), need, C.byref(stats)))
        finally:
            self._lib.cubit_elf_free(elf)
        return out.tobytes(), {name: int(getattr(stats, name)) for name, _ in stats._fields_}

    def decode_kernel(self, cubin_path: str | os.PathLike, kernel_name: str) -> list[dict]:
        """cubit.decode_kernel(cubin_path, kernel_name) (reference src/python.rs:104-169)."""
        try:
            with open(cubin_path, "rb") as fh:
                data = fh.read()
        except OSError as e:
            raise OSError(f"load error: failed to read {os.fspath(cubin_path)}: {e}") from None
        _, _, form, slots, ctrl, raw, _ = self.decode_elf(data, kernel_name)
        out = []
        for i in range(len(form)):
            addr = (16 * i) & 0xFFFFFFFF
            if (int(ctrl[i]) >> 30) & 3:
                out.append(dict(addr=addr, key="UNKNOWN", raw_lo=int.from_bytes(bytes(raw[i, :8]), "little"),
                                raw_hi=int.from_bytes(bytes(raw[i, 8:]), "little")))
            else:
                out.append(self.record_to_dict(form[i], slots[:, i], ctrl[i], addr, brief=True))
        return out


def build_cubin(kernels: Sequence[tuple[str, bytes]]) -> bytes:
    """Synthetic multi-kernel cubin image: [(name, code bytes)] -> ELF bytes, laid out like the
    reference's Mercury-free builder (src/elf_builder.rs:535-847)."""
    lib = _native.load_library()
    n = len(kernels)
    names = (C.c_char_p * max(n, 1))(*[k[0].encode() for k in kernels])
    bufs = [np.frombuffer(k[1], np.uint8) for k in kernels]
    codes = (C.c_void_p * max(n, 1))(*[b.ctypes.data if len(b) else None for b in bufs])
    sizes = (C.c_uint64 * max(n, 1))(*[len(b) for b in bufs])
    need = C.c_uint64()
    rc = lib.cubit_elf_build(names, codes, sizes, n, None, 0, C.byref(need))
    if rc:
        raise CubitError(rc, lib.cubit_last_error(None).decode())
    out = np.empty(need.value, np.uint8)
    rc = lib.cubit_elf_build(names, codes, sizes, n, _ptr(out), need.value, C.byref(need))
    if rc:
        raise CubitError(rc, lib.cubit_last_error(None).decode())
    return out.tobytes()


def patch_text(data: bytes, index: int, code: bytes) -> bytes:
    """The cubin image with text section `index` replaced by `code`; a different length moves every
    offset behind it (reference CubinFile::patch_text, src/elf.rs:71-219)."""
    lib = _native.load_library()
    buf = np.frombuffer(data, np.uint8)
    elf = C.c_void_p()
    rc = lib.cubit_elf_parse(_ptr(buf), len(buf), C.byref(elf))
    if rc:
        raise OSError("load error: " + lib.cubit_last_error(None).decode())
    try:
        new = np.frombuffer(code, np.uint8)
        need = C.c_uint64()
        rc = lib.cubit_elf_patch_text(elf, index, _ptr(new) if len(new) else None, len(new), None, 0, need)
        if rc:
            raise CubitError(rc, lib.cubit_last_error(None).decode())
        out = np.empty(need.value, np.uint8)
        rc = lib.cubit_elf_patch_text(elf, index, _ptr(new) if len(new) else None, len(new), _ptr(out), len(out), need)
        if rc:
            raise CubitError(rc, lib.cubit_last_error(None).decode())
    finally:
        lib.cubit_elf_free(elf)
    return out.tobytes()
