"""build() may be called by several processes at once (one rank per GPU under torchrun): exactly one compiles, into a
file of its own, and nobody ever loads a half-written library."""
import os
import subprocess
import sys

import cubit_b200


def test_a_stale_library_is_rebuilt_once_and_loads_in_every_process():
    source = cubit_b200.build.CSRC / "elf_text.cpp"
    os.utime(source)                      # make the library look older than a source
    assert cubit_b200.build.is_stale()
    code = ("import ctypes, cubit_b200.build as b; p = b.build(); ctypes.CDLL(str(p)); "
            "print(p.stat().st_mtime_ns)")
    root = str(cubit_b200.build.PKG.parent)
    procs = [subprocess.Popen([sys.executable, "-c", code], cwd=root, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for _ in range(4)]
    stamps = set()
    for p in procs:
        out, err = p.communicate(timeout=600)
        assert p.returncode == 0, err[-2000:]
        stamps.add(out.strip())
    assert len(stamps) == 1, "more than one process rebuilt the library"
    assert not cubit_b200.build.is_stale()
    leftovers = [f for f in os.listdir(cubit_b200.build.LIB_DIR) if f.startswith(".libcubit_b200.")]
    assert not leftovers
