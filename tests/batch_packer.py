"""A step packed in Python, for tests that drive parts or kernels without the engine: the layout
that the host runtime's ``bwh_pack_step`` writes (token ids, positions, request of token, cu_q,
q_start, kv_len, slot, logit rows, one block table per group), built from explicit segments.
``tests/test_cache_scheduler.py`` checks the host runtime's packing against this one."""
import numpy as np


def pack_batch(builder, segments, logit_rows, block_rows, min_blocks=0, into=None):
    """``segments``: list of (rid, tokens, q_start, kv_len, slot).  ``block_rows``:
    group -> one block-table row (list of page ids) per segment.  ``into``: a device
    buffer of exactly this batch's size to overwrite (fixed addresses for a CUDA graph)."""
    R = len(segments)
    T = sum(len(s[1]) for s in segments)
    widths = {g: max([min_blocks, 1] + [len(r) for r in rows]) for g, rows in block_rows.items()}
    n_want = len(logit_rows)
    total = 3 * T + (R + 1) + 3 * R + n_want + sum(R * w for w in widths.values())
    host = builder.pinned(total)
    h = host[:total].numpy()
    off = 0

    def take(n):
        nonlocal off
        a = (off, off + n)
        off += n
        return a

    a_tok, a_pos, a_req = take(T), take(T), take(T)
    a_cu, a_qs, a_kv, a_sl = take(R + 1), take(R), take(R), take(R)
    a_lr = take(n_want)
    a_bt = {g: take(R * w) for g, w in widths.items()}
    q_lens = np.fromiter((len(sg[1]) for sg in segments), dtype=np.int32, count=R)
    q_starts = np.fromiter((sg[2] for sg in segments), dtype=np.int32, count=R)
    cu = np.zeros(R + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu[1:])
    h[a_cu[0]:a_cu[1]] = cu
    h[a_qs[0]:a_qs[1]] = q_starts
    h[a_kv[0]:a_kv[1]] = np.fromiter((sg[3] for sg in segments), dtype=np.int32, count=R)
    h[a_sl[0]:a_sl[1]] = np.fromiter((sg[4] for sg in segments), dtype=np.int32, count=R)
    if T == R:   # one token per request (a decode step): no per-segment loops
        h[a_tok[0]:a_tok[1]] = np.fromiter((sg[1][0] for sg in segments), dtype=np.int32, count=R)
        h[a_pos[0]:a_pos[1]] = q_starts
        h[a_req[0]:a_req[1]] = np.arange(R, dtype=np.int32)
    else:
        req = np.repeat(np.arange(R, dtype=np.int32), q_lens)
        h[a_req[0]:a_req[1]] = req
        h[a_pos[0]:a_pos[1]] = np.arange(T, dtype=np.int32) - cu[:-1][req] + q_starts[req]
        t = 0
        for sg in segments:
            n = len(sg[1])
            h[a_tok[0] + t: a_tok[0] + t + n] = sg[1]
            t += n
    if n_want:
        h[a_lr[0]:a_lr[1]] = logit_rows
    for g, rows in block_rows.items():
        w = widths[g]
        view = h[a_bt[g][0]:a_bt[g][1]].reshape(R, w)
        view[:] = -1
        for r, row in enumerate(rows):
            view[r, :len(row)] = row
    return builder.finish(host, T, R, n_want, widths, [sg[0] for sg in segments], into)

