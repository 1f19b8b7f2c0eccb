"""The allocation-free decode entry point (cubit_decode_batch_static).

Who it is for: hosts that cannot allocate device memory once they are running.  Two kinds were in
mind — a process in which another component has already reserved the GPU's memory for itself, so a
cudaMalloc from this library would simply fail; and a thread with a latency budget, for which the
implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  The regular
host-buffer entry point grows a staging buffer with cudaMalloc; this one stages the batch through a
fixed array that is part of the library image instead (so every GPU that loads the library carries
it), which bounds the batch at STATIC_MAX_WORDS words.

What is checked: results equal the CPU oracle's and the regular entry point's on two calls in a row
(the calls share the array, so the second, smaller and different, batch would show anything left over
from the first); the calls leave the amount of free device memory unchanged; the limits are
refused with a clear message; and two contexts on one GPU can call it at the same time.
"""
import ctypes as C
import threading

import numpy as np
import pytest

import cubit_b200
from cubit_b200.codec import STATIC_MAX_WORDS

pytestmark = pytest.mark.gpu


def free_device_bytes():
    torch = pytest.importorskip("torch")
    return torch.cuda.mem_get_info(0)[0]


def assert_same(got, want):
    for name, g, w in zip(("form", "slots", "ctrl"), got, want):
        assert g.dtype == w.dtype and g.shape == w.shape and (g == w).all(), name


def test_static_entry_point_first_thing_in_a_fresh_context_allocates_nothing(oracle):
    """A context of its own, and the static call before any other: it may not lean on the staging buffer that the
    regular host path allocates.  Checked against the oracle, twice in a row, with free device memory watched."""
    fresh = cubit_b200.Codec(devices=(0,))
    try:
        first = oracle.synth(cubit_b200.MIX_ZIPF, 77, STATIC_MAX_WORDS, noise_ppm=20000, records=False)
        second = oracle.synth(cubit_b200.MIX_UNIFORM, 78, 4099, noise_ppm=300000, records=False)
        fresh.decode_batch_static(second)          # the one-time lookup of the array's address happens here
        before = free_device_bytes()
        for words in (first, second):
            got = fresh.decode_batch_static(words)
            assert_same(got[:3], oracle.decode_batch(words))
            assert got[3]["n_decoded"] + got[3]["n_rejected"] == len(words)
            assert got[3]["n_decoded"] == int((got[0] != 0xFFFF).sum())
            assert free_device_bytes() == before, "the call changed the amount of free device memory"
    finally:
        fresh.close()


def test_static_entry_point_matches_the_regular_one_twice_in_a_row(codec, oracle):
    first = oracle.synth(cubit_b200.MIX_ZIPF, 79, STATIC_MAX_WORDS, noise_ppm=20000, records=False)
    second = oracle.synth(cubit_b200.MIX_FAMILY, 80, 12345, noise_ppm=100000, records=False)
    for words in (first, second):
        want = codec.decode_batch(words)
        got = codec.decode_batch_static(words)
        assert_same(got[:3], want[:3])
        assert got[3] == want[3]


def test_static_entry_point_refuses_what_it_cannot_hold(codec):
    words = np.zeros((STATIC_MAX_WORDS + 1, 16), np.uint8)
    with pytest.raises(cubit_b200.CubitError) as e:
        codec.decode_batch_static(words)
    assert e.value.code == -1 and "CUBIT_STATIC_MAX_WORDS" in e.value.message
    with pytest.raises(cubit_b200.CubitError) as e:
        codec.decode_batch_static(np.zeros((4, 16), np.uint8), device_slot=1)
    assert e.value.code == -1 and "device_slot" in e.value.message
    form, slots, ctrl, counts = codec.decode_batch_static(np.zeros((0, 16), np.uint8))
    assert len(form) == 0 and counts["n_decoded"] == 0


def test_static_entry_point_without_counts_through_the_raw_abi(codec, oracle):
    words = oracle.synth(cubit_b200.MIX_UNIFORM, 81, 3000, records=False)
    n = len(words)
    form = np.empty(n, np.uint16); slots = np.empty((8, n), np.uint32); ctrl = np.empty(n, np.uint32)
    rc = codec._lib.cubit_decode_batch_static(codec._ctx, 0, words.ctypes.data_as(C.c_void_p), n, form.ctypes.data_as(C.c_void_p),
                                              slots.ctypes.data_as(C.c_void_p), ctrl.ctypes.data_as(C.c_void_p), None)
    assert rc == 0
    assert_same((form, slots, ctrl), oracle.decode_batch(words))


def test_two_contexts_on_one_gpu_share_the_array_safely(codec, oracle):
    """The array exists once per GPU, not once per context: calls from two contexts at the same time are serialised
    inside the library and both get their own results."""
    other = cubit_b200.Codec(devices=(0,))
    try:
        batches = [oracle.synth(cubit_b200.MIX_ZIPF, 90 + k, 20000 + 1000 * k, noise_ppm=50000, records=False) for k in range(2)]
        want = [oracle.decode_batch(b) for b in batches]
        errors = []

        def work(c, k):
            try:
                for _ in range(20):
                    assert_same(c.decode_batch_static(batches[k])[:3], want[k])
            except Exception as exc:   # noqa: BLE001 - reported below
                errors.append(exc)
        threads = [threading.Thread(target=work, args=(c, k)) for k, c in enumerate((codec, other))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert not errors, errors
    finally:
        other.close()
