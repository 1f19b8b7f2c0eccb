"""cubit — the reference's Python module name, served by the B200 codec.

The reference builds a PyO3 extension module called ``cubit`` with six functions (reference
src/python.rs:215-225).  This package gives the same six names, signatures and exceptions on
top of :mod:`cubit_b200`, so ``import cubit`` keeps working when the B200 library replaces the
Rust one: ``decode``, ``decode_kernel`` and ``to_sass`` run the decode kernel on the GPU,
``encode`` lowers the text on the host and encodes the record on the GPU, ``table_info``
answers from the table alone.  ``asm`` raises NotImplementedError: it runs the reference's
instruction-scheduling pass before encoding, which the B200 library does not contain.
"""
from cubit_b200 import asm, decode, decode_kernel, encode, table_info, to_sass

__all__ = ["encode", "decode", "decode_kernel", "table_info", "to_sass", "asm"]
