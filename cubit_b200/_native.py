"""ctypes binding of libcubit_b200.so (the C ABI declared in include/cubit_b200.h)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

u8p, u16p, u32p, u64p = C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)


class Counts(C.Structure):
    _fields_ = [("n_decoded", C.c_uint64), ("n_rejected", C.c_uint64), ("n_tie", C.c_uint64),
                ("n_exact", C.c_uint64), ("n_mismatch", C.c_uint64)]

    def as_dict(self):
        return {name: int(getattr(self, name)) for name, _ in self._fields_}


class FieldInfo(C.Structure):
    _fields_ = [("shift", C.c_uint32), ("bits", C.c_uint32), ("token_idx", C.c_int32), ("dst_pos", C.c_uint32),
                ("stored_bits", C.c_uint32), ("name", C.c_char_p), ("extraction", C.c_char_p)]


class PatchStats(C.Structure):
    _fields_ = [("n_words", C.c_uint64), ("n_reencoded", C.c_uint64), ("n_kept", C.c_uint64), ("n_changed", C.c_uint64),
                ("n_unfaithful", C.c_uint64)]


class KernelMeta(C.Structure):
    _fields_ = [("regcount", C.c_uint32), ("num_barriers", C.c_uint32), ("max_reg", C.c_uint32),
                ("barrier_mask", C.c_uint32), ("first_exit", C.c_uint64), ("n_exits", C.c_uint64)]


class VariantInfo(C.Structure):
    _fields_ = [("key", C.c_char_p), ("mod_group", C.c_char_p), ("opcode", C.c_char_p), ("key_id", C.c_uint32),
                ("layout_kind", C.c_uint32), ("synth_mask", C.c_uint32), ("ra_tok", C.c_int32), ("rb_tok", C.c_int32),
                ("n_fields", C.c_uint32), ("fields", C.POINTER(FieldInfo))]


# Every symbol include/cubit_b200.h declares: name -> (restype, argtypes).
SIGNATURES = {
    "cubit_ctx_create": (C.c_int, [C.c_char_p, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_void_p)]),
    "cubit_ctx_destroy": (None, [C.c_void_p]),
    "cubit_last_error": (C.c_char_p, [C.c_void_p]),
    "cubit_table_info": (C.c_int, [C.c_void_p, u32p, u32p]),
    "cubit_variant_lookup": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(VariantInfo)]),
    "cubit_variant_find": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, u32p]),
    "cubit_key_name": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(C.c_char_p), u32p, u32p]),
    "cubit_host_alloc": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]),
    "cubit_host_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cubit_decode_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.POINTER(Counts), C.c_int, C.c_void_p]),
    "cubit_decode_batch_static": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.POINTER(Counts)]),
    "cubit_encode_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int,
                                     C.c_void_p]),
    "cubit_roundtrip_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.POINTER(Counts), C.c_int,
                                        C.c_void_p]),
    "cubit_synth_batch": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "cubit_elf_parse": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]),
    "cubit_elf_free": (None, [C.c_void_p]),
    "cubit_elf_num_text": (C.c_uint32, [C.c_void_p]),
    "cubit_elf_text": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(C.c_char_p), u64p, u64p]),
    "cubit_elf_find": (C.c_int, [C.c_void_p, C.c_char_p, u32p]),
    "cubit_decode_elf": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Counts)]),
    "cubit_infer_kernel_meta": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(KernelMeta), C.c_void_p,
                                          C.c_uint64, u64p]),
    "cubit_elf_build": (C.c_int, [C.POINTER(C.c_char_p), C.POINTER(C.c_void_p), u64p, C.c_uint32, C.c_void_p, C.c_uint64,
                                  u64p]),
    "cubit_text_lower": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint32, C.c_int, C.c_uint64, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, u64p]),
    "cubit_text_encode": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint32, C.c_int, C.c_uint64, C.c_void_p, u64p]),
    "cubit_text_parse": (C.c_int, [C.c_void_p, C.c_char_p, C.c_uint32, C.c_char_p, C.c_uint64, u64p]),
    "cubit_listing_assemble": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_void_p, C.c_uint64, u64p, u64p]),
    "cubit_patch_elf": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, u64p, C.POINTER(PatchStats)]),
    "cubit_elf_patch_text": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, u64p]),
    "cubit_disassemble": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_int, C.c_char_p, C.c_uint64, u64p, u64p]),
    "cubit_text_print": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_char_p, C.c_uint64, u64p]),
}

_lib = None


def library_path() -> Path:
    return _build.LIB


def load_library() -> C.CDLL:
    """Loads the CUDA library, building it first if needed.  There is no fallback: without the
    library every codec call fails."""
    global _lib
    if _lib is None:
        # CUBIT_B200_LIB names a library file to load instead of the in-tree build (for comparing builds).
        path = os.environ.get("CUBIT_B200_LIB") or _build.build()
        lib = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError here means the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
