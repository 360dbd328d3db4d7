"""What the cache raises when pages or request slots run out.  The free lists themselves (LIFO
over page ids, as the reference's ``PageAllocator``, src/core/paging/paged_kv_cache.h:47-71, but
without reference counts: pages are never shared here) live in the C++ host runtime,
``csrc/host_runtime.cpp``.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    pass
