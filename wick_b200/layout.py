"""Sizes that the Python side and the CUDA sources have to agree on.

``PAGE`` is the number of positions in one cache page.  The CUDA sources carry the
same number as ``wick::kPage`` (``csrc/common.cuh``); every library exports it
through ``wick_page_size()`` and the loader refuses a library whose number differs.
"""
PAGE = 64


def pages_for(n_tokens: int) -> int:
    """Pages that hold ``n_tokens`` positions."""
    return (n_tokens + PAGE - 1) // PAGE
