"""GPU parity: every result of the CUDA path, through the C ABI, equals the CPU oracle's bit for bit."""
import ctypes as C
import json

import numpy as np
import pytest

import cubit_b200
from cubit_b200 import MIX_FAMILY, MIX_UNIFORM, MIX_ZIPF
from oracle_lib import ints_from_words, words_from_ints

pytestmark = pytest.mark.gpu
T = 8


def assert_records_equal(got, want):
    for name, g, w in zip(("form", "slots", "ctrl"), got, want):
        assert g.shape == w.shape and g.dtype == w.dtype, name
        bad = np.nonzero((g != w).any(axis=0))[0] if g.ndim == 2 else np.nonzero(g != w)[0]
        assert len(bad) == 0, f"{name} differs at {len(bad)} records, first {bad[:5]}"


@pytest.mark.parametrize("mix,seed,noise", [(MIX_UNIFORM, 0, 0), (MIX_ZIPF, 1, 0), (MIX_ZIPF, 7, 10000),
                                            (MIX_FAMILY, 3, 0), (MIX_UNIFORM, 5, 500000)])
def test_stream_decode_encode_roundtrip(codec, oracle, mix, seed, noise):
    n = 47244
    words, form, slots, ctrl = codec.synth(mix, seed, n, noise_ppm=noise)
    owords, oform, oslots, octrl = oracle.synth(mix, seed, n, noise_ppm=noise, threads=T)
    assert (words == owords).all(), "generated words differ"
    assert_records_equal((form, slots, ctrl), (oform, oslots, octrl))
    d = codec.decode_batch(words)
    od = oracle.decode_batch(words, threads=T)
    assert_records_equal(d[:3], od)
    counts = d[3]
    assert counts["n_rejected"] == int((od[0] == 0xFFFF).sum())
    assert counts["n_decoded"] == n - counts["n_rejected"]
    assert counts["n_tie"] == int(((od[2] >> 28) & 1).sum())
    # encode: generator records give back the stream; decoded records equal the oracle's encode
    assert (codec.encode_batch(form, slots, ctrl) == oracle.encode_batch(oform, oslots, octrl, threads=T)).all()
    noise_free = oform != 0xFFFF
    assert (codec.encode_batch(form, slots, ctrl)[noise_free] == words[noise_free]).all()
    assert (codec.encode_batch(*d[:3]) == oracle.encode_batch(*od, threads=T)).all()
    status, rc = codec.roundtrip_batch(words)
    ostatus = oracle.roundtrip_batch(words, threads=T)
    assert (status == ostatus).all()
    assert [rc["n_exact"], rc["n_mismatch"], rc["n_rejected"]] == np.bincount(ostatus, minlength=3).tolist()


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 255, 256, 257, 1023, 4097])
def test_ragged_sizes(codec, oracle, n):
    words = oracle.synth(MIX_ZIPF, 11, n, noise_ppm=20000, records=False)
    form, slots, ctrl, counts = codec.decode_batch(words)
    assert_records_equal((form, slots, ctrl), oracle.decode_batch(words))
    assert counts["n_decoded"] + counts["n_rejected"] == n
    assert (codec.encode_batch(form, slots, ctrl) == oracle.encode_batch(form, slots, ctrl)).all()
    status, _ = codec.roundtrip_batch(words)
    assert (status == oracle.roundtrip_batch(words)).all()


def adversarial_words(rng, per_variant):
    """Every variant's constant bits plus random variable bits, with flips, stray ones, sparse fields, Rc=RZ."""
    table = json.loads((cubit_b200.build.PKG / "tables" / "sm120.json").read_text())["instructions"]
    out = []
    for key in sorted(table, key=str.encode):
        for mods in sorted(table[key]["mod_groups"], key=str.encode):
            e = table[key]["mod_groups"][mods]
            base, fmask = int(e["and_base"], 16), 0
            for f in e["fields"]:
                fmask |= ((1 << f["bits"]) - 1) << f["shift"]
            vmask = (int(e["variable_mask"], 16) if "variable_mask" in e else fmask) | fmask
            draws = rng.integers(0, 2**64, size=(per_variant, 4), dtype=np.uint64)
            for i, r in enumerate(draws):
                x, y = int(r[0]) | (int(r[1]) << 64), int(r[2]) | (int(r[3]) << 64)
                w = base | (x & vmask)
                mode = i % 5
                if mode == 1: w ^= 1 << (y % 128)
                elif mode == 2: w |= (y >> 7) & ((1 << 96) - 1) & ~0xFFF
                elif mode == 3: w &= ~(y & vmask)
                elif mode == 4: w = (w & ~(0xFF << 64)) | (0xFF << 64)
                out.append(w)
    return words_from_ints(out)


# Batches of at least this many words run on the kernels that stage the table in shared memory
# (the ones the benchmark times); smaller ones on the kernels that read it through global memory.
STAGED_MIN_WORDS = 1 << 17


@pytest.mark.parametrize("per_variant", [48, 12])
def test_adversarial_words(codec, oracle, per_variant):
    """The real table's edge words through both kernel flavours: 48 per variant is 137,856 words (staged table),
    12 per variant 34,464 (table in global memory)."""
    words = adversarial_words(np.random.default_rng(1), per_variant)
    assert (len(words) >= STAGED_MIN_WORDS) == (per_variant == 48)
    d = codec.decode_batch(words)
    od = oracle.decode_batch(words, threads=T)
    assert_records_equal(d[:3], od)
    assert (codec.encode_batch(*d[:3]) == oracle.encode_batch(*od, threads=T)).all()
    status, _ = codec.roundtrip_batch(words)
    assert (status == oracle.roundtrip_batch(words, threads=T)).all()


def test_wide_index_kernels_agree(oracle, monkeypatch):
    """Batches of 2^31 words and more use 64-bit word indices in the decode kernel; CUBIT_WIDE_INDEX=1 selects
    those kernels at any size so that they can be compared with the oracle here."""
    monkeypatch.setenv("CUBIT_WIDE_INDEX", "1")
    wide = cubit_b200.Codec(devices=(0,))
    try:
        for n in (STAGED_MIN_WORDS + 4099, 5000):
            words = oracle.synth(MIX_UNIFORM, 31, n, noise_ppm=50000, records=False, threads=T)
            got = wide.decode_batch(words)
            assert_records_equal(got[:3], oracle.decode_batch(words, threads=T))
    finally:
        wide.close()


def test_uniform_random_words_are_rejected_like_the_oracle(codec, oracle):
    rng = np.random.default_rng(2)
    words = rng.integers(0, 256, size=(200000, 16), dtype=np.uint8)
    d = codec.decode_batch(words)
    assert_records_equal(d[:3], oracle.decode_batch(words, threads=T))
    assert d[3]["n_rejected"] > 0.99 * len(words)


def test_encode_arbitrary_records(codec, oracle):
    """Random slots and ctrl for every variant, plus out-of-range forms (zero word)."""
    rng = np.random.default_rng(3)
    nv = codec.table_info()[1]
    form = np.repeat(np.arange(nv, dtype=np.uint16), 20)
    n = len(form)
    slots = rng.integers(0, 2**32, size=(8, n), dtype=np.uint32)
    ctrl = rng.integers(0, 2**32, size=n, dtype=np.uint32)
    form[::97] = 0xFFFF
    form[5::101] = nv
    words = codec.encode_batch(form, slots, ctrl)
    assert (words == oracle.encode_batch(form, slots, ctrl, threads=T)).all()
    assert not words[::97].any()


def test_golden_words(codec, golden):
    """Known-answer words of the reference's tests: decode selects the named variant and the
    record-level re-encode reproduces the word outside the scheduling field."""
    mask = int(golden["sched_mask"], 16)
    # Branch targets/modes are written by the reference's text-level branch fixup, and the STS.U16 word is
    # shadowed by a sibling form: these re-encode differently at record level.
    not_exact = {"tests/encoding.rs:290", "tests/encoding.rs:295", "tests/encoding.rs:412"}
    cases = [c for c in golden["cases"] if c["kind"] != "lo64"]
    words = words_from_ints([int(c["word"], 16) for c in cases])
    form, slots, ctrl, _ = codec.decode_batch(words)
    enc = ints_from_words(codec.encode_batch(form, slots, ctrl))
    status, _ = codec.roundtrip_batch(words)
    for i, c in enumerate(cases):
        m = codec.variant(int(form[i]))
        if "key" in c:
            assert m.key == c["key"], c
        if "mod_group" in c:
            assert m.mod_group == c["mod_group"], c
        if "opcode" in c:
            assert m.opcode == c["opcode"], c
        exact = (enc[i] & ~mask) == (int(c["word"], 16) & ~mask)
        assert exact == (c["source"] not in not_exact), c
        assert status[i] == (0 if exact else 1)
    for p in golden["padding_words"]:
        w = int(p["word"], 16)
        assert codec.decode(w & (2**64 - 1), w >> 64)["key"] == p["key"]


def test_python_decode_matches_oracle_fields(codec, oracle):
    """cubit.decode's dict: key, opcode, every field (name, shift, bits, value, token_idx, extraction), scheduling."""
    words = oracle.synth(MIX_UNIFORM, 21, 300, records=False)
    for w in ints_from_words(words):
        lo, hi = w & (2**64 - 1), w >> 64
        want = oracle.decode_full(lo, hi)
        if want["status"]:
            with pytest.raises(ValueError, match="decode error: no instruction matches"):
                codec.decode(lo, hi)
            continue
        got = codec.decode(lo, hi, addr=16)
        assert (got["key"], got["mod_group"], got["addr"]) == (want["key"], want["mod_group"], 16)
        assert got["scheduling"] == want["scheduling"] and got["opcode"] == want["opcode"]
        table_fields = [f for f in got["fields"] if f["name"] not in ("neg", "abs") or f["bits"] != 1 or f["shift"] not in (62, 63, 72, 73)]
        synth = [f for f in got["fields"] if f not in table_fields]
        assert [(f["shift"], f["bits"], f["value"], f["token_idx"], f["extraction"]) for f in got["fields"][:len(want["fields"])]] == \
               [(f["shift"], f["bits"], f["value"], f["token_idx"], f["extraction"]) for f in want["fields"]]
        assert len(got["fields"]) - len(want["fields"]) == bin(want["synth"]).count("1")
        del synth


@pytest.mark.parametrize("n", [STAGED_MIN_WORDS + 20003, 100003])
def test_device_pointer_path(codec, oracle, n):
    """Buffers in device memory, kernel queued on a caller stream (torch is only the allocator here); once above and
    once below the batch size from which the kernels stage the table in shared memory."""
    torch = pytest.importorskip("torch")
    words = oracle.synth(MIX_ZIPF, 5, n, noise_ppm=10000, records=False, threads=T)
    dev = torch.device("cuda", 0)
    dw = torch.from_numpy(words.reshape(-1)).to(dev)
    form = torch.empty(n, dtype=torch.int16, device=dev)
    slots = torch.empty(8 * n, dtype=torch.int32, device=dev)
    ctrl = torch.empty(n, dtype=torch.int32, device=dev)
    status = torch.empty(n, dtype=torch.uint8, device=dev)
    out = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        counts = codec.decode_device(dw.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), stream=s.cuda_stream,
                                     want_counts=True)
        codec.encode_device(form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), n, out.data_ptr(), stream=s.cuda_stream)
        rcounts = codec.roundtrip_device(dw.data_ptr(), n, status.data_ptr(), stream=s.cuda_stream, want_counts=True)
    s.synchronize()
    oform, oslots, octrl = oracle.decode_batch(words, threads=T)
    assert (form.cpu().numpy().view(np.uint16) == oform).all()
    assert (slots.cpu().numpy().view(np.uint32).reshape(8, n) == oslots).all()
    assert (ctrl.cpu().numpy().view(np.uint32) == octrl).all()
    assert (out.cpu().numpy().reshape(n, 16) == oracle.encode_batch(oform, oslots, octrl, threads=T)).all()
    ostatus = oracle.roundtrip_batch(words, threads=T)
    assert (status.cpu().numpy() == ostatus).all()
    assert counts["n_decoded"] == int((oform != 0xFFFF).sum())
    assert rcounts["n_exact"] == int((ostatus == 0).sum())


def test_one_context_from_several_host_threads(codec, oracle):
    """Four host threads share the context: two decode device buffers on streams of their own
    (counted launches, so they also share the counter slots), two go through the host-buffer
    path (which shares the staging area).  ctypes releases the GIL during the calls."""
    import threading
    torch = pytest.importorskip("torch")
    dev = torch.device("cuda", 0)
    n = 300001
    batches = [oracle.synth(MIX_ZIPF, 20 + k, n, noise_ppm=5000, records=False) for k in range(4)]
    want = [oracle.decode_batch(b, threads=T) for b in batches]
    got, errors = [None] * 4, []

    def device_worker(k):
        try:
            torch.cuda.set_device(dev)
            s = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(s):
                dw = torch.from_numpy(batches[k].reshape(-1)).to(dev, non_blocking=False)
                form = torch.empty(n, dtype=torch.int16, device=dev)
                slots = torch.empty(8 * n, dtype=torch.int32, device=dev)
                ctrl = torch.empty(n, dtype=torch.int32, device=dev)
                for _ in range(5):
                    c = codec.decode_device(dw.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(),
                                            stream=s.cuda_stream, want_counts=True)
                    assert c["n_decoded"] + c["n_rejected"] == n
                s.synchronize()
                got[k] = (form.cpu().numpy().view(np.uint16), slots.cpu().numpy().view(np.uint32).reshape(8, n),
                          ctrl.cpu().numpy().view(np.uint32))
        except BaseException as e:   # noqa: BLE001 - reported by the main thread
            errors.append(e)

    def host_worker(k):
        try:
            for _ in range(3):
                got[k] = codec.decode_batch(batches[k])[:3]
        except BaseException as e:   # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=device_worker, args=(0,)), threading.Thread(target=device_worker, args=(1,)),
               threading.Thread(target=host_worker, args=(2,)), threading.Thread(target=host_worker, args=(3,))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(4):
        assert_records_equal(got[k], want[k])


def test_stream_ranges_compose(codec):
    """Any range of a stream can be generated on its own: shards of one stream agree with the whole."""
    whole = codec.synth(MIX_ZIPF, 9, 5000, noise_ppm=10000)
    for begin, end in ((0, 1), (1, 1700), (1700, 5000)):
        part = codec.synth(MIX_ZIPF, 9, end - begin, noise_ppm=10000, first=begin)
        assert (part[0] == whole[0][begin:end]).all() and (part[1] == whole[1][begin:end]).all()
        assert (part[2] == whole[2][:, begin:end]).all() and (part[3] == whole[3][begin:end]).all()


def test_full_size_properties(codec, oracle):
    """64 Mi-word batch (the benchmark's size) on device memory: properties that need no full oracle pass,
    plus an exact comparison on a strided sample."""
    torch = pytest.importorskip("torch")
    n = 64 * 1024 * 1024
    dev = torch.device("cuda", 0)
    words = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    form = torch.empty(n, dtype=torch.int16, device=dev)
    slots = torch.empty(8 * n, dtype=torch.int32, device=dev)
    ctrl = torch.empty(n, dtype=torch.int32, device=dev)
    status = torch.empty(n, dtype=torch.uint8, device=dev)
    enc = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    codec.synth_device(MIX_ZIPF, 1, n, words_ptr=words.data_ptr(), noise_ppm=10000)
    counts = codec.decode_device(words.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), want_counts=True)
    codec.encode_device(form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), n, enc.data_ptr())
    rc = codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), want_counts=True)
    torch.cuda.synchronize()
    assert counts["n_decoded"] + counts["n_rejected"] == n
    assert rc["n_exact"] + rc["n_mismatch"] + rc["n_rejected"] == n and rc["n_rejected"] == counts["n_rejected"]
    # status == exact  <=>  encode(decode(w)) == w outside bits 121:105; rejected <=> form 0xFFFF.
    w32 = words.view(torch.int32).view(n, 4)
    e32 = enc.view(torch.int32).view(n, 4)
    keep = torch.tensor([-1, -1, -1, ~(0x1FFFF << 9)], dtype=torch.int32, device=dev)
    same = ((w32 ^ e32) & keep).eq(0).all(dim=1)
    rejected = form.eq(-1)
    assert bool((status.eq(2) == rejected).all())
    assert bool((status.eq(0) == (same & ~rejected)).all())
    assert int(rejected.sum()) == counts["n_rejected"]
    # Exact comparison with the oracle on every 64th word.
    idx = torch.arange(0, n, 64, device=dev)
    sample = words.view(n, 16)[idx].cpu().numpy()
    oform, oslots, octrl = oracle.decode_batch(sample, threads=T)
    assert (form[idx].cpu().numpy().view(np.uint16) == oform).all()
    assert (slots.view(8, n)[:, idx].cpu().numpy().view(np.uint32) == oslots).all()
    assert (ctrl[idx].cpu().numpy().view(np.uint32) == octrl).all()
    assert (status[idx].cpu().numpy() == oracle.roundtrip_batch(sample, threads=T)).all()


def test_roundtrip_at_the_largest_configuration(codec, oracle):
    """256 Mi words (4 GiB) with 1 % raw random words in one fused roundtrip launch: the status
    classes partition the batch, a second launch over a sub-range reproduces the first one's
    bytes, and every 256th word has the oracle's status."""
    torch = pytest.importorskip("torch")
    n = 256 * 1024 * 1024
    dev = torch.device("cuda", 0)
    if torch.cuda.mem_get_info(dev)[0] < 6 * (1 << 30):
        pytest.skip("needs 6 GiB of free device memory")
    words = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    status = torch.empty(n, dtype=torch.uint8, device=dev)
    codec.synth_device(MIX_ZIPF, 1, n, words_ptr=words.data_ptr(), noise_ppm=10000)
    rc = codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), want_counts=True)
    torch.cuda.synchronize()
    assert rc["n_exact"] + rc["n_mismatch"] + rc["n_rejected"] == n
    hist = torch.bincount(status.to(torch.int64), minlength=3)
    assert hist.tolist() == [rc["n_exact"], rc["n_mismatch"], rc["n_rejected"]]
    assert rc["n_rejected"] >= n // 200          # the raw random words are nearly all rejected
    begin, m = 3 * n // 4 + 5, 1 << 20            # an unaligned-by-word sub-range, as another launch
    again = torch.empty(m, dtype=torch.uint8, device=dev)
    codec.roundtrip_device(words.data_ptr() + begin * 16, m, again.data_ptr())
    torch.cuda.synchronize()
    assert bool((again == status[begin:begin + m]).all())
    idx = torch.arange(0, n, 256, device=dev)
    sample = words.view(n, 16)[idx].cpu().numpy()
    assert (status[idx].cpu().numpy() == oracle.roundtrip_batch(sample, threads=T)).all()


def test_decode_kernel_and_multi_kernel_cubin(codec, oracle, tmp_path):
    """decode_kernel on a synthetic multi-kernel cubin: one launch over all kernels, per-kernel offsets,
    NOP / self-branch padding, substring name match, UNKNOWN entries."""
    rng = np.random.default_rng(4)
    kernels = []
    for k, words_in in enumerate((8, 13, 1, 40)):
        w = oracle.synth(MIX_FAMILY, 30 + k, words_in, noise_ppm=100000 if k == 3 else 0, records=False)
        kernels.append((f"k{k:05d}", w.tobytes()))
    image = cubit_b200.build_cubin(kernels)
    sections, word_start, form, slots, ctrl, raw, counts = codec.decode_elf(image)
    assert [s[0] for s in sections] == [".text." + k[0] for k in kernels]
    assert [s[2] for s in sections] == [128, 256, 128, 640]
    assert word_start.tolist() == [0, 8, 24, 32, 72]
    assert sections == oracle.elf_text_sections(image)
    of, os_, oc = oracle.decode_batch(raw)
    assert_records_equal((form, slots, ctrl), (of, os_, oc))
    assert raw[word_start[1]:word_start[1] + 13].tobytes() == kernels[1][1]
    assert codec.variant(int(form[23])).key == "BRA_II" and codec.variant(int(form[22])).key == "NOP"
    path = tmp_path / "synthetic.cubin"
    path.write_bytes(image)
    insns = codec.decode_kernel(path, "k00003")
    assert len(insns) == 40 and [i["addr"] for i in insns] == [16 * j for j in range(40)]
    for j, ins in enumerate(insns):
        want = oracle.decode_full(int.from_bytes(kernels[3][1][16 * j:16 * j + 8], "little"),
                                  int.from_bytes(kernels[3][1][16 * j + 8:16 * j + 16], "little"))
        if want["status"]:
            assert ins["key"] == "UNKNOWN" and set(ins) == {"addr", "key", "raw_lo", "raw_hi"}
        else:
            assert ins["key"] == want["key"] and set(ins["scheduling"]) == {"stall", "yield_flag", "wait_mask"}
            assert all(set(f) == {"name", "shift", "bits", "value"} for f in ins["fields"])
    assert len(codec.decode_kernel(path, "k0000")) == 8      # substring, first hit
    with pytest.raises(ValueError, match="kernel 'nope' not found. Available"):
        codec.decode_kernel(path, "nope")
    with pytest.raises(OSError, match="load error"):
        codec.decode_kernel(tmp_path / "missing.cubin", "k")
    del rng


def test_multi_device_context_shards_host_batches(oracle):
    """One process, two GPUs: host batches are cut into contiguous ranges, one per device, no exchange step."""
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    both = cubit_b200.Codec(devices=(0, 1))
    n = 300001
    words = oracle.synth(MIX_ZIPF, 13, n, noise_ppm=10000, records=False)
    d = both.decode_batch(words)
    od = oracle.decode_batch(words, threads=T)
    assert_records_equal(d[:3], od)
    assert d[3]["n_decoded"] + d[3]["n_rejected"] == n
    assert (both.encode_batch(*d[:3]) == oracle.encode_batch(*od, threads=T)).all()
    status, rc = both.roundtrip_batch(words)
    assert (status == oracle.roundtrip_batch(words, threads=T)).all()
    assert rc["n_exact"] + rc["n_mismatch"] + rc["n_rejected"] == n
    # a multi-kernel cubin is cut on the cumulative word count
    kernels = [(f"k{k:05d}", oracle.synth(MIX_FAMILY, 50 + k, 4000 + 37 * k, records=False).tobytes()) for k in range(9)]
    image = cubit_b200.build_cubin(kernels)
    sections, word_start, form, slots, ctrl, raw, counts = both.decode_elf(image)
    assert_records_equal((form, slots, ctrl), oracle.decode_batch(raw, threads=T))
    both.close()


def test_large_host_batch_crosses_chunk_and_stream_boundaries(codec, oracle):
    """Host batches above 4 Mi words are streamed in chunks over two staging halves and two streams:
    every plane must equal the device-path result, and the oracle on a strided sample and around the seams."""
    torch = pytest.importorskip("torch")
    n = 9 * 1024 * 1024 + 12345
    words, gform, gslots, gctrl = codec.synth(MIX_ZIPF, 3, n, noise_ppm=10000)
    form, slots, ctrl, counts = codec.decode_batch(words)
    dev = torch.device("cuda", 0)
    dw = torch.from_numpy(words.reshape(-1)).to(dev)
    dform = torch.empty(n, dtype=torch.int16, device=dev)
    dslots = torch.empty(8 * n, dtype=torch.int32, device=dev)
    dctrl = torch.empty(n, dtype=torch.int32, device=dev)
    dcounts = codec.decode_device(dw.data_ptr(), n, dform.data_ptr(), dslots.data_ptr(), dctrl.data_ptr(), want_counts=True)
    torch.cuda.synchronize()
    assert counts == dcounts
    assert (form == dform.cpu().numpy().view(np.uint16)).all()
    assert (slots == dslots.cpu().numpy().view(np.uint32).reshape(8, n)).all()
    assert (ctrl == dctrl.cpu().numpy().view(np.uint32)).all()
    chunk = 4 * 1024 * 1024
    idx = np.unique(np.concatenate([np.arange(0, n, 97), np.arange(chunk - 64, chunk + 64),
                                    np.arange(2 * chunk - 64, 2 * chunk + 64), np.arange(n - 64, n)]))
    of, os_, oc = oracle.decode_batch(words[idx], threads=T)
    assert (form[idx] == of).all() and (slots[:, idx] == os_).all() and (ctrl[idx] == oc).all()
    # encode and roundtrip through the host path at the same size
    enc = codec.encode_batch(gform, gslots, gctrl)
    keep = gform != 0xFFFF
    assert (enc[keep] == words[keep]).all() and not enc[~keep].any()
    status, rc = codec.roundtrip_batch(words)
    assert (status[idx] == oracle.roundtrip_batch(words[idx], threads=T)).all()
    assert rc["n_rejected"] == counts["n_rejected"] and rc["n_exact"] + rc["n_mismatch"] == counts["n_decoded"]
    # a cubin whose text crosses the chunk boundaries too: kernels of uneven length cut from the same words
    cuts = [0, 1000003, 1000003 + 2500007, 5 * 1024 * 1024 + 77, n - n % 8]
    image = cubit_b200.build_cubin([(f"k{k}", words[cuts[k]:cuts[k + 1]].tobytes()) for k in range(4)])
    sections, word_start, eform, eslots, ectrl, raw, ecounts = codec.decode_elf(image)
    assert len(sections) == 4 and int(word_start[-1]) == len(raw) >= cuts[-1]
    again = codec.decode_batch(raw)
    assert (eform == again[0]).all() and (eslots == again[1]).all() and (ectrl == again[2]).all() and ecounts == again[3]
    for k in range(4):                                   # each section starts with its kernel's words
        at, m = int(word_start[k]), cuts[k + 1] - cuts[k]
        assert (raw[at:at + m] == words[cuts[k]:cuts[k + 1]]).all()
        assert (eform[at:at + m] == form[cuts[k]:cuts[k + 1]]).all()


def test_infer_kernel_meta_matches_the_reference_algorithm(codec, oracle):
    """regcount / num_barriers / EXIT offsets of every kernel of a cubin from one launch, against the
    oracle's restatement of the reference's inference loop (decoded fields, and the raw-bits fallback
    for words that match nothing)."""
    kernels = []
    for k, (n, noise) in enumerate([(5000, 0), (37, 0), (4096, 300000), (8, 1000000), (20000, 20000), (150000, 5000)]):
        w = oracle.synth(MIX_FAMILY if k % 2 else MIX_UNIFORM, 60 + k, n, noise_ppm=noise, records=False)
        kernels.append((f"m{k:05d}", w.tobytes()))
    image = cubit_b200.build_cubin(kernels)
    got = codec.infer_kernel_meta(image)
    sections = oracle.elf_text_sections(image)
    assert [g["name"] for g in got] == [s[0] for s in sections]
    total_exits = 0
    for g, (name, off, size) in zip(got, sections):
        want = oracle.kernel_meta(image[off:off + size])      # padded section: NOPs and the self-branch count too
        for key in ("max_reg", "barrier_mask", "regcount", "num_barriers", "exit_offsets"):
            assert g[key] == want[key], (name, key)
        total_exits += len(want["exit_offsets"])
    assert total_exits > 10 and any(g["num_barriers"] for g in got)
    one = codec.infer_kernel_meta(image, "m00004")
    assert len(one) == 1 and one[0] == got[4]
    with pytest.raises(ValueError, match="not found"):
        codec.infer_kernel_meta(image, "zzz")


def test_host_injected_failures_come_back_as_errors(oracle, monkeypatch):
    """Failures made on the host (nothing on the GPU is faulted): a device worker that reports an error instead of
    running, and a staging buffer that cannot grow.  Each must come back as a return code with a message, leave
    nothing running, and leave the library usable: the next context works."""
    words = oracle.synth(MIX_ZIPF, 41, 50000, records=False, threads=T)
    want = oracle.decode_batch(words, threads=T)
    monkeypatch.setenv("CUBIT_TEST_FAIL_SLOT", "0")
    broken = cubit_b200.Codec(devices=(0,))
    monkeypatch.delenv("CUBIT_TEST_FAIL_SLOT")
    for call in (lambda: broken.decode_batch(words), lambda: broken.roundtrip_batch(words), lambda: broken.encode_batch(*want)):
        with pytest.raises(cubit_b200.CubitError) as e:
            call()
        assert e.value.code == -3 and "device slot 0 failed" in e.value.message
    broken.close()
    monkeypatch.setenv("CUBIT_TEST_FAIL_ALLOC", "1")
    starved = cubit_b200.Codec(devices=(0,))
    monkeypatch.delenv("CUBIT_TEST_FAIL_ALLOC")
    with pytest.raises(cubit_b200.CubitError) as e:
        starved.decode_batch(words)
    assert e.value.code == -7 and "allocation failed" in e.value.message
    # the paths that need no staging buffer still work in that context, and so does the built-in scratch
    assert_records_equal(starved.decode_batch_static(words)[:3], want)
    starved.close()
    healthy = cubit_b200.Codec(devices=(0,))
    assert_records_equal(healthy.decode_batch(words)[:3], want)
    healthy.close()


def test_the_reference_module_name_decodes_and_encodes(codec):
    """`import cubit` (reference src/python.rs:215-225) on the GPU: decode, to_sass and encode agree with the Codec."""
    import cubit
    lo, hi = codec.encode("IADD3 R5, PT, PT, R9, R4, R5")
    assert cubit.encode("IADD3 R5, PT, PT, R9, R4, R5") == (lo, hi)
    assert cubit.decode(lo, hi) == codec.decode(lo, hi)
    assert cubit.to_sass(lo, hi) == "IADD3 R5, PT, PT, R9, R4, R5"
