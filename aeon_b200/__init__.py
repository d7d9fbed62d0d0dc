"""aeon_b200: B200 implementation of aeon's per-record ETL hot path behind aeon's loader surface.

The work is done by ``libaeon_b200.so`` (CUDA kernels for sm_100a + host C++); this package is a
ctypes binding.  ``DataLoader`` mirrors ``aeon.DataLoader``; ``Provider`` and ``kernels`` expose the
lower levels of the C ABI.  Build the library with ``python -m aeon_b200.build``.
"""
from .dataloader import DataLoader, dict2json  # noqa: F401

__all__ = ["DataLoader", "dict2json"]
