"""B200-native paged KV-cache path (append, quantised key append, sparse gather, page moves, page pool).

The product is the C-ABI library ``unholy_b200/lib/libunholy_pkv.so`` (sources in ``unholy_b200/csrc``, interface in
``include/unholy_pkv.h``). This package only loads it through ctypes for the tests and the benchmark; there is no
Python or CPU implementation of any operation behind it, and loading fails loudly when the library is missing.
"""
from .capi import PkvError, check, lib, library_path  # noqa: F401
