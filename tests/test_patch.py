"""Cubin rewriting: text-section replacement (reference src/elf.rs:71-219) and the patch
command (reference src/main.rs:691-764).  No reference test covers either, so the checks are
structural: the ELF64 layout after a splice, read back by the oracle's independent reader, and
the invariants of the patch loop (high halves kept, faithful words unchanged)."""
import struct

import numpy as np
import pytest

import cubit_b200


def image():
    a = bytes(range(16)) * 5
    b = bytes([7]) * 16 * 3
    c = bytes([9]) * 16 * 11
    return cubit_b200.build_cubin([("k0", a), ("k1", b), ("k2", c)])


def section_headers(img):
    shoff, = struct.unpack_from("<Q", img, 0x28)
    shnum, = struct.unpack_from("<H", img, 0x3C)
    return [struct.unpack_from("<IIQQQQIIQQ", img, shoff + 64 * i) for i in range(shnum)]


def test_patch_text_same_size_is_in_place(oracle):
    img = image()
    secs = oracle.elf_text_sections(img)
    new_code = bytes([0xAB]) * secs[1][2]
    out = cubit_b200.patch_text(img, 1, new_code)
    assert len(out) == len(img) and oracle.elf_text_sections(out) == secs
    off = secs[1][1]
    assert out[off:off + len(new_code)] == new_code
    assert out[:off] == img[:off] and out[off + len(new_code):] == img[off + len(new_code):]


@pytest.mark.parametrize("new_words", [1, 3, 9, 40])
def test_patch_text_splice_moves_everything_behind_it(oracle, new_words):
    img = image()
    before = oracle.elf_text_sections(img)
    new_code = bytes([0x5A]) * 16 * new_words
    out = cubit_b200.patch_text(img, 1, new_code)
    delta = len(new_code) - before[1][2]
    assert len(out) == len(img) + delta
    after = oracle.elf_text_sections(out)
    assert after[0] == before[0]
    assert after[1] == (before[1][0], before[1][1], len(new_code))
    assert after[2] == (before[2][0], before[2][1] + delta, before[2][2])
    start = before[1][1]
    assert out[start:start + len(new_code)] == new_code
    # every other section keeps its contents, wherever it now lives
    old_h, new_h = section_headers(img), section_headers(out)
    assert len(old_h) == len(new_h)
    text_index = None
    for i, (o, n) in enumerate(zip(old_h, new_h)):
        o_off, o_size, n_off, n_size = o[4], o[5], n[4], n[5]
        if o_off == start and o_size == before[1][2]:
            text_index = i
            assert (n_off, n_size) == (start, len(new_code))
            continue
        assert n_size == o_size and n_off == (o_off + delta if o_off > start else o_off)
        if o[1] != 8 and o_size:                                   # not NOBITS
            assert out[n_off:n_off + n_size] == img[o_off:o_off + o_size] or o[1] == 2   # symtab sizes change
    assert text_index is not None
    # symbols defined in the section carry the new size; the others are untouched
    for o, n in zip(old_h, new_h):
        if o[1] != 2:
            continue
        for k in range(o[5] // 24):
            os_ = struct.unpack_from("<IBBHQQ", img, o[4] + 24 * k)
            ns_ = struct.unpack_from("<IBBHQQ", out, n[4] + 24 * k)
            assert os_[:5] == ns_[:5]
            if os_[3] == text_index and (os_[1] >> 4) >= 1:
                assert ns_[5] == len(new_code)
            else:
                assert ns_[5] == os_[5]
    # program headers: a segment holding the section grows, later ones move
    phoff, = struct.unpack_from("<Q", out, 0x20)
    phnum, = struct.unpack_from("<H", out, 0x38)
    o_phoff, = struct.unpack_from("<Q", img, 0x20)
    for p in range(phnum):
        o = struct.unpack_from("<IIQQQQQQ", img, o_phoff + 56 * p)
        n = struct.unpack_from("<IIQQQQQQ", out, phoff + 56 * p)
        if o[2] <= start < o[2] + o[5]:
            assert (n[2], n[5], n[6]) == (o[2], o[5] + delta, o[6] + delta)
        elif o[2] > start:
            assert (n[2], n[5]) == (o[2] + delta, o[5])
        else:
            assert n == o


def test_patch_text_errors():
    img = image()
    with pytest.raises(cubit_b200.CubitError, match="text section index out of range"):
        cubit_b200.patch_text(img, 7, b"")
    with pytest.raises(OSError, match="load error"):
        cubit_b200.patch_text(b"not an elf", 0, b"")


@pytest.mark.parametrize("what", ["e_phoff", "e_shoff_after_parse", "symtab_offset"])
def test_patch_text_rejects_header_offsets_near_2_to_64(what):
    """Offsets whose sums wrap around 2^64 must end in an error, not in reads or writes outside the image
    (reference src/elf.rs:109-190 walks the same tables with bounds-checked slices)."""
    img = bytearray(image())
    huge = 0xFFFFFFFFFFFFFFF8
    if what == "e_phoff":
        struct.pack_into("<Q", img, 0x20, huge)
        struct.pack_into("<H", img, 0x38, 2)
    elif what == "symtab_offset":
        heads = section_headers(bytes(img))
        shoff, = struct.unpack_from("<Q", img, 0x28)
        sym = next(i for i, h in enumerate(heads) if h[1] == 2)
        struct.pack_into("<Q", img, shoff + 64 * sym + 0x18, huge)
    else:
        # the section table itself is read by the parser first: a bad e_shoff never reaches the splice
        struct.pack_into("<Q", img, 0x28, huge)
    with pytest.raises((cubit_b200.CubitError, OSError), match="ELF|load error"):
        cubit_b200.patch_text(bytes(img), 1, bytes(16 * 5))


@pytest.mark.gpu
def test_patch_keeps_faithful_words_and_high_halves(codec, oracle):
    import json
    from pathlib import Path
    golden = json.loads((Path(__file__).parent / "golden" / "encoding_words.json").read_text())
    texts = [c["sass"] for c in golden["cases"] if c["kind"] in ("clean128", "lo64")]
    faithful = codec.encode_text("\n".join(texts + ["BRA 0x0", "EXIT"]), 0, program=True)
    words, *_ = oracle.synth(0, 11, 3000, noise_ppm=20000)              # random forms and some noise
    img = cubit_b200.build_cubin([("faithful", faithful.tobytes()), ("mixed", np.asarray(words, np.uint8).tobytes())])
    out, stats = codec.patch(img)
    assert len(out) == len(img)
    secs = oracle.elf_text_sections(img)
    total = sum(s[2] // 16 for s in secs)
    assert stats["n_words"] == total == stats["n_reencoded"] + stats["n_kept"]
    assert stats["n_kept"] > 0 and stats["n_changed"] <= stats["n_unfaithful"] <= stats["n_reencoded"]
    a, b = np.frombuffer(img, np.uint8), np.frombuffer(out, np.uint8)
    changed = np.flatnonzero(a != b)
    in_text = np.zeros(len(a), bool)
    for _, off, size in secs:
        in_text[off:off + size] = True
    assert in_text[changed].all()                                        # nothing outside the text sections moves
    for _, off, size in secs:
        w_old = a[off:off + size].reshape(-1, 16)
        w_new = b[off:off + size].reshape(-1, 16)
        assert (w_old[:, 8:] == w_new[:, 8:]).all()                      # high halves are the original's
    # Only the STS.U16 word of the first section is rewritten: it decodes to a sibling form
    # (tests/encoding.rs:412), every other word of that section reads back to itself.
    _, off, size = secs[0]
    diff = np.flatnonzero((a[off:off + size].reshape(-1, 16) != b[off:off + size].reshape(-1, 16)).any(axis=1))
    assert [texts[i] for i in diff] == ["STS.U16 [R20+UR13+0x4008], R129 ;"]
    # the same counters from the pieces: decode, print, CPU re-encode
    sec_words = np.concatenate([a[off:off + size].reshape(-1, 16) for _, off, size in secs])
    changed_words = int((sec_words[:, :8] != np.concatenate([b[off:off + size].reshape(-1, 16) for _, off, size in secs])[:, :8]).any(axis=1).sum())
    assert changed_words == stats["n_changed"]
    # patching the patched image again changes nothing more than the first pass already did
    again, stats2 = codec.patch(out)
    assert stats2["n_words"] == total
