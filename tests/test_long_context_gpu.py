"""The attention kernels at the lengths that are benchmarked: prompt portions of 2,048 and 8,192
tokens (also 2,048 new tokens on top of 6,144 cached ones) and decode rows over 8,192 keys at
batch 8 and 64 with the key bound of a graph replay, against the plain attention in float64; and
a negative control: with one block-table entry pointing at a page that is not the request's, the
error must EXCEED the bound the other tests allow (the bound can tell a wrong page from rounding).

The plain attention runs through torch on the GPU here (float64): the sequences are too long for
the CPU within the suite's minutes.  Keys and values lie on shuffled pages; pages no request owns
and the unused rest of every last page hold NaN.
"""
import pytest
import torch

from plain_model import plain_attention_tail
from test_kernels_gpu import ATT_TOL, FakeBatch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from blackwellllm_b200.kernels import ops as o
    return o


def paged_case_gpu(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=0, spare=5, width=None, spike=None):
    """As ``test_kernels_gpu.paged_case`` but made on the device: returns q [T, nh*hd], the pages,
    the block table and per request (q_tail, k, v) in the cache's dtype for the plain attention."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(q_lens)
    blocks = [-(-k // page) for k in kv_lens]
    num_pages = sum(blocks) + spare
    perm = torch.randperm(num_pages, generator=g, device=DEV)
    k_pages = torch.full((num_pages, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full_like(k_pages, float("nan"))
    table = torch.full((R, width or max(blocks) + 2), -1, dtype=torch.int32, device=DEV)
    qs, refs, at = [], [], 0
    for r in range(R):
        L, ql, nb = kv_lens[r], q_lens[r], blocks[r]
        k = torch.randn(L, nkv, hd, generator=g, device=DEV).to(dtype)
        v = torch.randn(L, nkv, hd, generator=g, device=DEV).to(dtype)
        q = torch.randn(ql, nh, hd, generator=g, device=DEV).to(dtype)
        if spike is not None:
            spike(r, q, k, v)
        ids = perm[at:at + nb]
        at += nb
        table[r, :nb] = ids.int()
        for src, pages in ((k, k_pages), (v, v_pages)):
            pad = torch.full((nb * page, nkv, hd), float("nan"), dtype=dtype, device=DEV)
            pad[:L] = src
            pages[ids] = pad.view(nb, page, nkv, hd).transpose(1, 2)
        qs.append(q)
        refs.append((q, k, v))
    return torch.cat(qs).reshape(-1, nh * hd).contiguous(), k_pages, v_pages, table, refs, perm[at:]


def plain_rows_gpu(refs, window=None):
    outs = [plain_attention_tail(q.double(), k.double(), v.double(), window=window).reshape(q.shape[0], -1)
            for q, k, v in refs]
    return torch.cat(outs)


def run(ops, dtype, q, kp, vp, table, batch, nh, window=None):
    hd = kp.shape[-1]
    if dtype == torch.float32:
        return ops.attention_simt(q, kp, vp, batch.positions, batch.req_of_token, table, nh, window, hd ** -0.5)
    return ops.attention_mma(q, kp, vp, batch, table, nh, window, hd ** -0.5)


def errors(out, ref):
    """(largest error over the largest value; largest error of a row over that row's largest value)."""
    d = (out.double() - ref).abs()
    per_row = d.amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-30)
    return float(d.max() / ref.abs().max()), float(per_row.max())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("q_len,kv_len", [(2048, 2048), (8192, 8192), (2048, 8192)])
def test_prompt_attention_at_benchmarked_lengths(ops, dtype, q_len, kv_len):
    """32 query / 8 kv heads' geometry (four query heads per kv head, head size 128, pages of 16) on two
    kv heads; every row is compared, each against its own largest value (late rows average thousands of
    values and are small: an error that the first rows' size would hide shows there)."""
    nh, nkv, hd, page = 8, 2, 128, 16
    far = 5

    def spike(r, q, k, v):   # the last query's score with key 5 dwarfs all others: its output is value 5
        k[far] = 0; k[far, :, 0] = 8.0
        q[-1] = 0; q[-1, :, 0] = 8.0 * hd ** 0.5
        v[far] = 5.0

    q, kp, vp, table, refs, _ = paged_case_gpu([q_len], [kv_len], nh, nkv, hd, page, dtype, seed=q_len + kv_len, spike=spike)
    out = run(ops, dtype, q, kp, vp, table, FakeBatch([q_len], [kv_len]), nh)
    assert not torch.isnan(out).any()
    ref = plain_rows_gpu(refs)
    whole, per_row = errors(out, ref)
    assert whole <= ATT_TOL[dtype] and per_row <= 2 * ATT_TOL[dtype], (whole, per_row)
    assert float((out[-1].float() - 5.0).abs().max()) < 0.05
    assert ops.attention_tc_status() == 0


@pytest.mark.parametrize("B", [8, 64])
def test_decode_rows_over_8192_keys_with_the_graphs_key_bound(ops, B):
    """What a decode graph at context 8,192 launches: one row per request, block tables 512 wide, the number
    of key slices fixed by the bound (not by the lengths), lengths from 1 to 8,192 in one batch."""
    nh, nkv, hd, page = 8, 2, 128, 16
    g = torch.Generator().manual_seed(B)
    kv_lens = [8192, 8191, 8177, 8192 - 16, 5000, 64, 1, 8192][:B]
    kv_lens += torch.randint(1, 8193, (B - len(kv_lens),), generator=g).tolist()
    q_lens = [1] * B
    q, kp, vp, table, refs, _ = paged_case_gpu(q_lens, kv_lens, nh, nkv, hd, page, torch.bfloat16, seed=B, width=512)
    ref = plain_rows_gpu(refs)
    bound = ops.attention_mma(q, kp, vp, FakeBatch(q_lens, kv_lens, static_bound=8192), table, nh, None, hd ** -0.5)
    free = ops.attention_mma(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, None, hd ** -0.5)
    for out in (bound, free):
        assert not torch.isnan(out).any()
        whole, per_row = errors(out, ref)
        assert whole <= ATT_TOL[torch.bfloat16] and per_row <= 2 * ATT_TOL[torch.bfloat16], (whole, per_row)


# ------------------------------------------------------------------ negative control

@pytest.mark.parametrize("kind", ["prompt_tcgen05", "prompt_mma", "decode_mma", "float32"])
def test_a_wrong_page_exceeds_the_bound(ops, kind, monkeypatch):
    """One block-table entry of one request is pointed at a page that belongs to nobody (filled with
    other finite numbers).  Every attention kernel must then miss the plain result by MORE than the
    bound the tests above allow; with the right table it stays within it."""
    dtype = torch.float32 if kind == "float32" else torch.bfloat16
    nh, nkv, hd, page = 8, 2, 128, 16
    if kind == "prompt_mma":
        monkeypatch.setenv("BW_ATTN_TC", "0")       # prompt portions on the mma.sync kernel
    q_lens, kv_lens = ([1, 1, 1], [300, 200, 77]) if kind == "decode_mma" else ([60, 140, 33], [300, 140, 97])
    q, kp, vp, table, refs, spare = paged_case_gpu(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=9)
    ref = plain_rows_gpu(refs)
    good = run(ops, dtype, q, kp, vp, table, FakeBatch(q_lens, kv_lens), nh)
    assert errors(good, ref)[0] <= ATT_TOL[dtype]
    stale = int(spare[0])
    gen = torch.Generator(device=DEV).manual_seed(1)
    kp[stale] = torch.randn(nkv, page, hd, generator=gen, device=DEV).to(dtype)
    vp[stale] = torch.randn(nkv, page, hd, generator=gen, device=DEV).to(dtype)
    rows_of = [0, q_lens[0], q_lens[0] + q_lens[1], sum(q_lens)]
    for r in range(3):
        wrong = table.clone()
        wrong[r, 1] = stale                          # keys 16..31 of request r come from the wrong page
        bad = run(ops, dtype, q, kp, vp, wrong, FakeBatch(q_lens, kv_lens), nh)
        rows = slice(rows_of[r], rows_of[r + 1])
        d = (bad.double() - ref).abs()
        assert float(d[rows].max() / ref[rows].abs().max()) > 2 * ATT_TOL[dtype], "the bound cannot see a wrong page"
        others = torch.ones(ref.shape[0], dtype=torch.bool, device=DEV)
        others[rows] = False
        assert float(d[others].max() / ref.abs().max()) <= ATT_TOL[dtype]   # nobody else is touched
