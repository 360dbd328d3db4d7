"""The cache manager's page bookkeeping against the reference project's own allocator.

``tests/golden/reference_allocator.json`` holds a seeded random sequence of create / append /
truncate / destroy operations and, after each, the free count and the touched sequence's block table
as fxslava/BlackwellLLM's ``paging::PageAllocator`` (src/core/paging/paged_kv_cache.h:47-71, compiled on
the CPU by ``tests/golden/make_allocator_golden.sh``) leaves them under its sequence manager's rules: a
new page exactly when the length reaches a page boundary, a LIFO free list that hands out page 0
first, destroy gives the pages back in table order, truncate from the back.  The same operations on
this cache manager (one group, the same page size and pool) must leave the same tables: the same
page ids in the same order.
"""
import json
import os

from blackwellllm_b200.cache.manager import CacheManager
from blackwellllm_b200.parts.base import PagedKVRequest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_same_operations_leave_the_same_block_tables():
    with open(os.path.join(HERE, "golden", "reference_allocator.json")) as f:
        gold = json.load(f)
    cm = CacheManager([PagedKVRequest(2, 16, None)], page_size=gold["page_size"], num_pages=gold["num_pages"],
                      max_requests=8)
    kinds = set()
    for n, op in enumerate(gold["ops"]):
        rid, arg = op["seq"], op["arg"]
        kinds.add(op["op"])
        if op["op"] == "create":
            cm.add_request(rid)
        elif op["op"] == "append":
            cm.append(rid, arg)
        elif op["op"] == "truncate":
            if arg < cm.length(rid):            # the reference's truncate never grows a sequence
                cm.truncate(rid, arg)
        else:
            cm.free_request(rid)
        what = f"operation {n}: {op}"
        assert cm.free_pages() == [op["free"]], what
        assert (cm.block_table(rid, 0) if cm.has(rid) else []) == op["table"], what
    assert kinds == {"create", "append", "truncate", "destroy"}
    assert min(op["free"] for op in gold["ops"]) == 0     # the pool ran dry on the way
    cm.check_invariants()
