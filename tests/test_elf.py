"""Cubin (ELF64) text-section reader, synthetic builder and the per-kernel offset table — host side only."""
import ctypes as C
import struct

import numpy as np
import pytest

import cubit_b200
from cubit_b200 import _native


def parse(data: bytes):
    lib = _native.load_library()
    buf = np.frombuffer(data, np.uint8)
    elf = C.c_void_p()
    rc = lib.cubit_elf_parse(C.c_void_p(buf.ctypes.data), len(buf), C.byref(elf))
    if rc:
        raise ValueError(lib.cubit_last_error(None).decode())
    out = []
    for i in range(lib.cubit_elf_num_text(elf)):
        name, off, size = C.c_char_p(), C.c_uint64(), C.c_uint64()
        assert lib.cubit_elf_text(elf, i, name, off, size) == 0
        out.append((name.value.decode(), off.value, size.value))
    lib.cubit_elf_free(elf)
    return out


def kernels(counts):
    rng = np.random.default_rng(0)
    return [(f"k{k:05d}", rng.integers(0, 256, size=16 * n, dtype=np.uint8).tobytes()) for k, n in enumerate(counts)]


def test_builder_layout_matches_the_reference_builder(oracle):
    """9 + 4N sections, one .text.<name> per kernel, 128-byte aligned, NOP padding ending in a self-branch
    (reference src/elf_builder.rs:535-847)."""
    ks = kernels([8, 13, 1, 40, 16])
    image = cubit_b200.build_cubin(ks)
    assert image[:4] == b"\x7fELF" and image[4] == 2 and image[5] == 1
    e_shnum, = struct.unpack_from("<H", image, 0x3C)
    e_phnum, = struct.unpack_from("<H", image, 0x38)
    e_machine, = struct.unpack_from("<H", image, 0x12)
    assert e_shnum == 9 + 4 * len(ks) and e_phnum == 3 + 2 * len(ks) and e_machine == 190
    text = parse(image)
    assert text == oracle.elf_text_sections(image)
    assert [t[0] for t in text] == [".text." + k[0] for k in ks]
    nop = bytes([0x18, 0x79] + [0] * 11 + [0xc0, 0x0f, 0])
    for (name, off, size), (_, code) in zip(text, ks):
        assert off % 128 == 0 and size == (len(code) + 127) // 128 * 128
        assert image[off:off + len(code)] == code
        pad = image[off + len(code):off + size]
        if pad:
            assert pad[-16:-14] == b"\x47\x79"                       # the last padding word is the self-branch
            assert all(pad[i:i + 16] == nop for i in range(0, len(pad) - 16, 16))
    # consecutive text sections touch, so a whole cubin is fetched with one copy
    assert all(a[1] + a[2] == b[1] for a, b in zip(text, text[1:]))


def test_word_start_table_without_a_gpu(host_codec):
    image = cubit_b200.build_cubin(kernels([8, 13, 1, 40]))
    lib = _native.load_library()
    buf = np.frombuffer(image, np.uint8)
    elf = C.c_void_p()
    assert lib.cubit_elf_parse(C.c_void_p(buf.ctypes.data), len(buf), C.byref(elf)) == 0
    start = np.zeros(5, np.uint64)
    assert lib.cubit_decode_elf(host_codec._ctx, elf, None, 4, C.c_void_p(start.ctypes.data), 0, None, None, None, None, None) == 0
    assert start.tolist() == [0, 8, 24, 32, 72]
    pick = np.array([3, 1], np.uint32)
    start2 = np.zeros(3, np.uint64)
    assert lib.cubit_decode_elf(host_codec._ctx, elf, C.c_void_p(pick.ctypes.data), 2, C.c_void_p(start2.ctypes.data), 0, None,
                                None, None, None, None) == 0
    assert start2.tolist() == [0, 40, 56]
    idx = C.c_uint32()
    assert lib.cubit_elf_find(elf, b"k0000", C.byref(idx)) == 0 and idx.value == 0     # substring, first hit
    assert lib.cubit_elf_find(elf, b"00003", C.byref(idx)) == 0 and idx.value == 3
    assert lib.cubit_elf_find(elf, b"zzz", C.byref(idx)) == -6
    assert b"Available" in lib.cubit_last_error(None)
    # decoding needs a device: loud failure, not a silent CPU path
    form = np.zeros(72, np.uint16); slots = np.zeros((8, 72), np.uint32); ctrl = np.zeros(72, np.uint32)
    rc = lib.cubit_decode_elf(host_codec._ctx, elf, None, 4, C.c_void_p(start.ctypes.data), 72, C.c_void_p(form.ctypes.data),
                              C.c_void_p(slots.ctypes.data), C.c_void_p(ctrl.ctypes.data), None, None)
    assert rc == -4
    lib.cubit_elf_free(elf)


def test_reader_filters_sections_like_the_reference():
    """Only PROGBITS sections named .text / .text.* with size > 0 (reference src/elf.rs:45-48)."""
    image = bytearray(cubit_b200.build_cubin(kernels([8, 8])))
    shoff, = struct.unpack_from("<Q", image, 0x28)
    text = parse(bytes(image))
    # find the header of the first text section and turn it into NOBITS, then into an empty section
    shnum, = struct.unpack_from("<H", image, 0x3C)
    headers = [shoff + 64 * i for i in range(shnum)]
    first = next(h for h in headers if struct.unpack_from("<Q", image, h + 0x18)[0] == text[0][1]
                 and struct.unpack_from("<I", image, h + 4)[0] == 1)
    struct.pack_into("<I", image, first + 4, 8)
    assert [t[0] for t in parse(bytes(image))] == [text[1][0]]
    struct.pack_into("<I", image, first + 4, 1)
    struct.pack_into("<Q", image, first + 0x20, 0)
    assert [t[0] for t in parse(bytes(image))] == [text[1][0]]


@pytest.mark.parametrize("damage", ["magic", "class", "endian", "short", "shoff", "shstrndx"])
def test_malformed_images_are_errors(damage):
    image = bytearray(cubit_b200.build_cubin(kernels([8])))
    if damage == "magic": image[0] = 0
    elif damage == "class": image[4] = 1
    elif damage == "endian": image[5] = 2
    elif damage == "short": image = image[:40]
    elif damage == "shoff": struct.pack_into("<Q", image, 0x28, len(image) + 4096)
    elif damage == "shstrndx": struct.pack_into("<H", image, 0x3E, 60000)
    with pytest.raises(ValueError, match="failed to parse ELF"):
        parse(bytes(image))


def test_builder_rejects_ragged_code_and_sizes_first():
    lib = _native.load_library()
    names = (C.c_char_p * 1)(b"k")
    code = np.zeros(24, np.uint8)
    codes = (C.c_void_p * 1)(code.ctypes.data)
    sizes = (C.c_uint64 * 1)(24)
    need = C.c_uint64()
    assert lib.cubit_elf_build(names, codes, sizes, 1, None, 0, C.byref(need)) == -5
    sizes[0] = 16
    assert lib.cubit_elf_build(names, codes, sizes, 1, None, 0, C.byref(need)) == 0 and need.value > 1000
    small = np.zeros(64, np.uint8)
    assert lib.cubit_elf_build(names, codes, sizes, 1, C.c_void_p(small.ctypes.data), 64, C.byref(need)) == -5
