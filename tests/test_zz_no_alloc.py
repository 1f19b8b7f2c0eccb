"""The allocation-free decode entry point (cubit_decode_batch_static) against the regular one.

It serves callers that may not allocate device memory while running — for instance when another
component of the process already holds the GPU's memory, or on a thread that cannot take the
implicit synchronisation of cudaMalloc — by staging the batch through a fixed array inside the
library.  Two calls in a row share that array, so the second (smaller, different) batch would show
anything left over from the first.
"""
import numpy as np
import pytest

import cubit_b200
from cubit_b200.codec import STATIC_MAX_WORDS

pytestmark = pytest.mark.gpu


def test_static_entry_point_matches_the_regular_one_twice_in_a_row(codec, oracle):
    first = oracle.synth(cubit_b200.MIX_ZIPF, 77, STATIC_MAX_WORDS, noise_ppm=20000, records=False)
    second = oracle.synth(cubit_b200.MIX_UNIFORM, 78, 4099, noise_ppm=300000, records=False)
    for words in (first, second):
        want = codec.decode_batch(words)
        got = codec.decode_batch_static(words)
        for name, g, w in zip(("form", "slots", "ctrl"), got[:3], want[:3]):
            assert g.dtype == w.dtype and g.shape == w.shape and (g == w).all(), name
        assert got[3] == want[3]
        assert got[3]["n_decoded"] + got[3]["n_rejected"] == len(words)


def test_static_entry_point_refuses_batches_beyond_its_scratch(codec):
    words = np.zeros((STATIC_MAX_WORDS + 1, 16), np.uint8)
    with pytest.raises(cubit_b200.CubitError) as e:
        codec.decode_batch_static(words)
    assert e.value.code == -1 and "CUBIT_STATIC_MAX_WORDS" in e.value.message
    form, slots, ctrl, counts = codec.decode_batch_static(np.zeros((0, 16), np.uint8))
    assert len(form) == 0 and counts["n_decoded"] == 0
