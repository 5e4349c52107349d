"""B200-native decode path of the LFM2.5-1.2B runtime (sm_100a only).

``ops`` mirrors the reference's op surface (``src/ops``) over the C ABI of ``liblfm25_b200.so``;
``cache`` mirrors its paged KV store and block tables (``src/cache``); ``workloads`` builds the
seeded synthetic inputs of the benchmark configurations.
"""
from . import _abi  # noqa: F401
from ._abi import Lfm25Error, library  # noqa: F401

__all__ = ["Lfm25Error", "library"]
