"""The work lists of the tensor-core attention (``kernels.ops.plan_attention_work``) are host
arithmetic: which (request, token tile) a CTA of the prompt kernel takes, and into how many key
slices a decode row is cut.  Checked here without a GPU: every token of every request is covered
exactly once, slices and their result slots neither overlap nor leave holes, and a graph replay's
lists depend on the bound only."""
import random

import pytest

from blackwellllm_b200.kernels.ops import plan_attention_work


def random_batch(rng, R, G):
    q_len, q_start, kv_len = [], [], []
    for _ in range(R):
        kind = rng.choice(("decode", "portion", "few"))
        n = 1 if kind == "decode" else (rng.randint(2, 16 // G) if kind == "few" and 16 // G >= 2 else rng.randint(2, 700))
        start = rng.choice((0, 0, rng.randint(0, 9000)))
        q_len.append(n); q_start.append(start); kv_len.append(start + n)
    return q_len, q_start, kv_len


@pytest.mark.parametrize("G,nkv,hd,rows_tile,page", [(4, 8, 128, 128, 16), (3, 1, 32, 64, 8), (1, 5, 64, 128, 64),
                                                     (7, 4, 128, 128, 16), (16, 2, 80, 64, 16), (2, 2, 256, 128, 32)])
@pytest.mark.parametrize("window", (None, 48, 300))
def test_every_token_once_and_slices_without_holes(G, nkv, hd, rows_tile, page, window):
    rng = random.Random(G * 1000 + hd + (window or 0))
    for trial in range(40):
        R = rng.randint(1, 70)
        q_len, q_start, kv_len = random_batch(rng, R, G)
        rows, keys, merge, n_slots = plan_attention_work(q_len, q_start, kv_len, G, nkv, window, hd, rows_tile, page)
        tpt = rows_tile // G
        assert tpt >= 1
        # prompt portions: tiles of tpt tokens cover each long segment exactly once
        covered = {}
        for r, t0, a, b in rows:
            assert (a, b) == (0, 0) and q_len[r] * G > 16 and 0 <= t0 < q_len[r] and t0 % tpt == 0
            assert t0 not in covered.setdefault(r, set())
            covered[r].add(t0)
        for r in range(R):
            if q_len[r] * G > 16:
                assert covered.get(r) == set(range(0, q_len[r], tpt)), (r, q_len[r])
            else:
                assert r not in covered
        # longest first: the keys a tile walks never grow along the list
        walk = [q_start[r] + t0 for r, t0, _, _ in rows]
        assert walk == sorted(walk, reverse=True)
        # decode rows: slices 0..n-1 of each short segment, result slots contiguous and disjoint
        by_req = {}
        for r, s, n, first in keys:
            by_req.setdefault(r, []).append((s, n, first))
        slot = 0
        for r in range(R):
            if q_len[r] * G > 16:
                assert r not in by_req
                continue
            items = by_req[r]
            n = items[0][1]
            assert [s for s, _, _ in items] == list(range(n)) and all(it[1:] == (n, slot) for it in items)
            span = kv_len[r] if not window else min(kv_len[r], window + q_len[r])
            assert 1 <= n <= 64 and (n == 1 or 2 * n <= -(-span // 64))   # a slice has at least two key tiles
            assert ((r, 0, n, slot) in merge) == (n > 1)
            slot += n
        assert slot == n_slots and len(merge) == sum(1 for v in by_req.values() if v[0][1] > 1)


def test_a_graph_replay_depends_on_the_bound_only():
    q_len, q_start = [1] * 8, [100, 5000, 8191, 17, 0, 640, 4096, 77]
    a = plan_attention_work(q_len, q_start, [s + 1 for s in q_start], 4, 8, None, 128, 128, 16, static_bound=8192)
    b = plan_attention_work(q_len, [8191] * 8, [8192] * 8, 4, 8, None, 128, 128, 16, static_bound=8192)
    assert a == b and a[3] > 8          # cut into slices although some requests are short
    alone = plan_attention_work([1], [8191], [8192], 4, 8, None, 128, 128, 16)
    many = plan_attention_work([1] * 64, [8191] * 64, [8192] * 64, 4, 8, None, 128, 128, 16)
    assert alone[3] > many[3] // 64 >= 1   # fewer slices a request when more requests fill the GPU
