"""Each CUDA kernel alone against its plain restatement (tests/plain_ops.py), at sizes other than the
models' own: odd widths and vocabularies, head sizes in steps of 16, any number of heads and groups."""
import math

import pytest
import torch

import plain_ops as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from fms_b200.kernels import ops as o

    return o


@pytest.fixture
def own_product_for_some_rows(ops):
    """Every product of 9 to 256 rows through this library's own tcgen05 kernel (by default only the gated
    feed-forward product up to 128 rows takes it), and the own kernels for many rows whatever padding their tiles need."""
    saved = ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS, ops.TENSOR_CORE_MAX_PADDING, ops.TENSOR_CORE_ROWS_QKV
    ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS = True, ["linear", "glu", "qkv"], 256
    ops.TENSOR_CORE_MAX_PADDING, ops.TENSOR_CORE_ROWS_QKV = 10.0, 512
    yield
    ops.USE_MID_GEMM, ops.MID_OPS, ops.MID_ROWS, ops.TENSOR_CORE_MAX_PADDING, ops.TENSOR_CORE_ROWS_QKV = saved


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,dim", [(331, 240), (17, 16), (1000, 4096 + 48)])
def test_embed(ops, dtype, vocab, dim):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, dim, generator=g).to(dtype).cuda()
    tokens = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).cuda()
    got = ops.embed(table, tokens)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, P.embed(table, tokens), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gain_dtype", DTYPES)
@pytest.mark.parametrize("rows,dim,eps", [(5, 240, 1e-5), (3, 17, 1e-6), (2, 5000, 1e-3)])
def test_add_rmsnorm(ops, dtype, gain_dtype, rows, dim, eps):
    g = torch.Generator().manual_seed(1)
    res = (torch.randn(rows, dim, generator=g) * 3).cuda()
    delta = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    gain = (1 + 0.1 * torch.randn(dim, generator=g)).to(gain_dtype).cuda()
    res_ref = res.clone()
    want = P.add_rmsnorm(res_ref, delta, gain, eps, torch.float32)
    got = ops.add_rmsnorm(res, delta, gain, eps, dtype)
    torch.testing.assert_close(res, res_ref, atol=1e-6, rtol=1e-6)  # the stream itself, in float32
    torch.testing.assert_close(got.float(), want, **tol(dtype))
    # without a delta the stream is untouched
    before = res.clone()
    got2 = ops.add_rmsnorm(res, None, gain, eps, dtype)
    assert torch.equal(res, before)
    torch.testing.assert_close(got2.float(), P.add_rmsnorm(before.clone(), None, gain, eps, torch.float32), **tol(dtype))
    # gathered rows: only those rows, the stream untouched
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32).cuda()
    got3 = ops.add_rmsnorm(res, delta, gain, eps, dtype, rows=idx)
    assert torch.equal(res, before)
    torch.testing.assert_close(got3.float(), P.add_rmsnorm(before.clone(), delta, gain, eps, torch.float32, rows=idx),
                               **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_gated_activation(ops, dtype, act):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(7, 2 * 173, generator=g) * 2).to(dtype).cuda()
    got = ops.gated_activation(gu, act)
    want = P.gated_activation(gu.float(), act)
    torch.testing.assert_close(got.float(), want, **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 331, 240), (5, 64, 17), (70, 130, 328), (129, 257, 1000)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_float32_is_true_float32(ops, m, n, k, bias):
    g = torch.Generator().manual_seed(3)
    # values with many mantissa bits: a tf32 or bf16 product would miss the tolerance by orders of magnitude
    x = torch.randn(m, k, generator=g).cuda()
    w = torch.randn(n, k, generator=g).cuda()
    b = torch.randn(n, generator=g).cuda() if bias else None
    got = ops.linear(x, w, b)
    want = P.linear(x, w, b, torch.float64)
    err = (got.double() - want).abs().max().item()
    assert err < 2e-6 * math.sqrt(k) * 4, err
    # a row's result does not depend on the other rows of the batch
    alone = ops.linear(x[:1].contiguous(), w, b)
    assert torch.equal(alone[0], got[0])


@pytest.mark.parametrize("n,k", [(70, 4), (100, 68), (64, 2052), (333, 1024), (130, 30)])
@pytest.mark.parametrize("few", [1, 3, 8, 9, 16, 30, 64])
def test_linear_float32_few_rows_are_bit_for_bit_the_same_rows_among_many(ops, few, n, k):
    """Up to 64 rows go through a kernel of their own (one thread a column); its sums run in the same order as the
    tiled kernel's (which 70 rows take), so a token's logits do not depend on which of the two its step took."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(70, k, generator=g).cuda()
    w = torch.randn(n, k, generator=g).cuda()
    b = torch.randn(n, generator=g).cuda()
    many = ops.linear(x, w, b)
    got = ops.linear(x[:few].contiguous(), w, b)
    assert torch.equal(got, many[:few])
    want = P.linear(x[:few], w, b, torch.float64)
    assert (got.double() - want).abs().max().item() < 2e-6 * math.sqrt(k) * 4


@pytest.mark.parametrize("m,n,k", [(1, 331, 240), (8, 512, 96), (9, 331, 240), (16, 512, 96), (33, 1000, 328), (200, 384, 64)])
def test_linear_bfloat16(ops, m, n, k):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    want = P.linear(x, w, None, torch.float64)
    got = ops.linear(x, w)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.double(), want, atol=2e-2, rtol=2e-2)
    got32 = ops.linear(x, w, None, torch.float32)
    assert got32.dtype == torch.float32
    torch.testing.assert_close(got32.double(), want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k", [(331, 240), (40, 8), (4096 + 16, 1000), (16400, 96), (331, 256), (4099, 1152), (7, 128)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_bfloat16_few_rows(ops, m, n, k, out_dtype):
    """The weight-streaming kernel of decode steps: odd numbers of weight rows, K that is no multiple of 32,
    one to eight batch rows, with and without bias."""
    g = torch.Generator().manual_seed(40 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
    for bias in (None, b):
        got = ops.linear(x, w, bias, out_dtype)
        want = P.linear(x, w, bias, torch.float64)
        assert got.dtype == out_dtype and got.shape == (m, n)
        t = dict(atol=2e-2, rtol=2e-2) if out_dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-3)
        torch.testing.assert_close(got.double(), want, **t)
    # a row's result does not depend on how many other rows there are
    alone = ops.linear(x[:1].contiguous(), w, None, out_dtype)
    assert torch.equal(alone[0], ops.linear(x, w, None, out_dtype)[0])


@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("hidden,k", [(176, 64), (328, 240), (1000, 96), (14336, 128), (331, 384), (5, 1024)])
@pytest.mark.parametrize("act", [0, 2])
def test_gated_linear_few_rows(ops, m, hidden, k, act):
    g = torch.Generator().manual_seed(50 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * hidden, k, generator=g) * 0.1).to(torch.bfloat16).cuda()
    got = ops.gated_linear(x, w, None, act)
    want = P.gated_activation(P.linear(x, w, None, torch.float32), act)
    assert got.dtype == torch.bfloat16 and got.shape == (m, hidden)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    # many rows take the product and the activation as two kernels: the same values up to rounding
    x2 = torch.randn(40, k, generator=g).to(torch.bfloat16).cuda()
    torch.testing.assert_close(ops.gated_linear(x2, w, None, act).float(),
                               P.gated_activation(P.linear(x2, w, None, torch.float32), act), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("m", [9, 16, 17, 64, 100, 256])
@pytest.mark.parametrize("n,k", [(331, 240), (130, 64), (4096 + 16, 1000), (4096, 4096), (1000, 8), (256, 14336 + 8)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_bfloat16_some_rows(ops, own_product_for_some_rows, m, n, k, out_dtype):
    """9 to 256 rows: the tcgen05 kernel with the weights on the instruction's rows.  Numbers of weight rows that are
    no multiples of its tile, K that is no multiple of 64, few and many steps of K (one block a tile, or clusters of
    2, 4 and 8 that add their sums), with and without bias."""
    g = torch.Generator().manual_seed(70 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * (0.05 if k < 5000 else 0.01)).to(torch.bfloat16).cuda()
    b = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
    for bias in (None, b):
        got = ops.linear(x, w, bias, out_dtype)
        want = P.linear(x, w, bias, torch.float64)
        assert got.dtype == out_dtype and got.shape == (m, n)
        t = dict(atol=2e-2, rtol=2e-2) if out_dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-3)
        torch.testing.assert_close(got.double(), want, **t)
    ops.check_error_flag("cuda")
    # a row's result does not depend on how many other rows there are
    fewer = ops.linear(x[:9].contiguous(), w, None, out_dtype)
    assert torch.equal(fewer, ops.linear(x, w, None, out_dtype)[:9])


@pytest.mark.parametrize("m", [9, 40, 256])
@pytest.mark.parametrize("hidden,k", [(176, 64), (328, 240), (1000, 96), (14336, 128), (331, 384), (5, 1024), (64, 4096)])
@pytest.mark.parametrize("act", [0, 2])
def test_gated_linear_some_rows(ops, own_product_for_some_rows, m, hidden, k, act):
    g = torch.Generator().manual_seed(80 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * hidden, k, generator=g) * 0.1).to(torch.bfloat16).cuda()
    b = (torch.randn(2 * hidden, generator=g) * 0.3).to(torch.bfloat16).cuda()
    for bias in (None, b):
        got = ops.gated_linear(x, w, bias, act)
        want = P.gated_activation(P.linear(x, w, bias, torch.float32), act)
        assert got.dtype == torch.bfloat16 and got.shape == (m, hidden)
        torch.testing.assert_close(got.float(), want, atol=3e-2, rtol=2e-2)
    ops.check_error_flag("cuda")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 512, 256), (129, 331, 200), (1000, 777, 1000), (2048, 1024, 4096),
                                   (257, 4096 + 32, 72), (1024, 96, 4096), (640, 6144, 520), (100, 700, 136)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_bfloat16_tensor_core(ops, m, n, k, out_dtype):
    """The tcgen05 kernels of prefill steps (a pair of blocks per tile of 256 rows; one block per tile up to 128
    rows): sizes that are no multiples of the tiles, more and fewer tiles than multiprocessors."""
    g = torch.Generator().manual_seed(60 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
    for bias in (None, b):
        got = ops.linear_tensor_core(x, w, bias, out_dtype)
        want = P.linear(x, w, bias, torch.float64)
        ops.check_error_flag("cuda")
        t = dict(atol=3e-2, rtol=2e-2) if out_dtype == torch.bfloat16 else dict(atol=2e-3, rtol=1e-3)
        torch.testing.assert_close(got.double(), want, **t)


@pytest.mark.parametrize("m,hidden,k", [(128, 128, 64), (300, 328, 240), (513, 1000, 96), (1030, 14336, 264), (90, 331, 64)])
def test_gated_linear_tensor_core(ops, m, hidden, k):
    g = torch.Generator().manual_seed(70 + m)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * hidden, k, generator=g) * 0.1).to(torch.bfloat16).cuda()
    b = (torch.randn(2 * hidden, generator=g) * 0.1).to(torch.bfloat16).cuda()
    for bias in (None, b):
        got = ops.gated_linear_tensor_core(x, w, bias, 0)
        ops.check_error_flag("cuda")
        want = P.gated_activation(P.linear(x, w, bias, torch.float32), 0)
        torch.testing.assert_close(got.float(), want, atol=3e-2, rtol=2e-2)


def test_linear_float32_matrix_in_a_bfloat16_model(ops):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 96, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(50, 96, generator=g).cuda()
    got = ops.linear(x, w)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.double(), P.linear(x, w, None, torch.float64), atol=5e-2, rtol=2e-2)


class FakeBatch:
    pass


def make_cache_case(dtype, nheads, kvheads, hd, lens_before, num_new, seed, window=0, poison=True):
    """A cache with random contents for sequences of the given lengths, blocks handed out in a scrambled
    order, everything that is not a live position poisoned with NaN; the batch arrays of a step."""
    from fms_b200.cache import Cache, KVRequest
    from fms_b200.engine.batch import Batch

    g = torch.Generator().manual_seed(seed)
    n = len(lens_before)
    cache = Cache([KVRequest(kvheads, hd, window)], max_tokens=64 * (sum((a + b + 63) // 64 for a, b in zip(lens_before, num_new)) + 5),
                  max_positions=max(8192, 64 * ((max(a + b for a, b in zip(lens_before, num_new)) + 63) // 64)),
                  dtype=dtype, device="cuda")
    # scramble the free list so that block ids are not in order
    pool = cache.groups[0].pool
    perm = torch.randperm(len(pool._free), generator=g).tolist()
    pool._free = [pool._free[i] for i in perm]
    slots = cache.begin(n + 2)[2:]  # not slot 0, 1
    storage = cache.groups[0].storage
    if poison:
        storage.fill_(float("nan"))
    if any(lens_before):
        live = [(s, lb) for s, lb in zip(slots, lens_before) if lb]
        cache.prepare([s for s, _ in live], [lb for _, lb in live])
        cache.commit([s for s, _ in live], [lb for _, lb in live])
    cache.prepare(slots, num_new)
    view = cache.layer_view(0)
    # fill the positions that exist before the step with random keys and values
    table = cache.groups[0].table_host
    for s, lb in zip(slots, lens_before):
        lo = max(0, lb - window + 1) // 64 * 64 if window else 0
        for first in range(lo, lb, 64):  # block by block
            blk, count = int(table[s, first // 64]), min(64, lb - first)
            view.keys[blk, :, :count] = torch.randn(kvheads, count, hd, generator=g).to(dtype).cuda()
            view.values[blk, :, :count] = torch.randn(kvheads, count, hd, generator=g).to(dtype).cuda()
    tokens = [[0] * k for k in num_new]
    batch = Batch.from_lists(slots, lens_before, tokens, [[] for _ in tokens], "cuda")
    return cache, view, batch


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nheads,kvheads,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (12, 1, 64)])
def test_rope_store(ops, dtype, nheads, kvheads, hd):
    lens_before, num_new = [0, 70, 5], [3, 1, 66]
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens_before, num_new, 6)
    g = torch.Generator().manual_seed(7)
    n = sum(num_new)
    qkv = torch.randn(n, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
    inv = (1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))).cuda()
    keys0, values0 = view.keys.clone(), view.values.clone()

    class V:
        keys, values, table, block_tokens = keys0, values0, view.table, 64

    want_q = P.rope_store(qkv, inv, batch, V, nheads, kvheads, hd)
    got_q = ops.rope_store(qkv, inv, batch, view, nheads, kvheads, hd)
    t = tol(dtype)
    torch.testing.assert_close(got_q.float(), want_q.float(), **t)
    torch.testing.assert_close(view.keys.float(), keys0.float(), equal_nan=True, **t)
    torch.testing.assert_close(view.values.float(), values0.float(), equal_nan=True, **t)
    # without frequencies nothing is rotated; without cache writes nothing is written
    before = view.keys.clone()
    q2 = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd, writes_cache=False)
    assert torch.equal(q2, qkv[:, : nheads * hd].contiguous())
    assert torch.equal(torch.nan_to_num(view.keys.float()), torch.nan_to_num(before.float()))


@pytest.mark.parametrize("nheads,kvheads,hd,lens_before,num_new", [
    (4, 2, 16, [70, 0, 5], [1, 1, 1]),        # a decode step
    (3, 1, 32, [0, 63], [3, 2]),              # short prompts and a continuation across a block's edge
    (5, 5, 48, [130], [8]),                   # eight tokens of one sequence, odd head size
    (32, 8, 128, [100, 200, 300, 5, 64, 63, 1, 0], [1] * 8),  # the benchmark's head layout, batch 8
    # more than 8 rows: the tcgen05 kernel with the weights on the instruction's rows has the same epilogue
    (4, 2, 16, [70, 0, 5, 64, 63, 200, 1, 9, 10], [1] * 9),   # a decode step of nine
    (3, 1, 32, [0, 63], [30, 2]),                             # a short prompt and a continuation across a block's edge
    (5, 5, 48, [130], [100]),                                 # odd head size: tiles of 128 rows cut through heads
    (32, 8, 128, [100 + 7 * i for i in range(64)], [1] * 64), # the benchmark's head layout, batch 64
    (7, 1, 80, [5, 0], [120, 136]),                           # 256 rows
    # from 512 rows on: the tcgen05 kernel with the tokens on the instruction's rows has the epilogue too
    (32, 8, 128, [0, 100], [400, 112]),                       # the benchmark's head layout, 512 rows
    (5, 5, 48, [10, 0, 70], [300, 1, 219]),                   # odd head size, tiles that cut through heads, 520 rows
    (4, 1, 16, [0], [700]),                                   # the smallest head size
])
@pytest.mark.parametrize("with_bias", [False, True])
def test_projection_rotation_and_cache_write_in_one_kernel(ops, own_product_for_some_rows, nheads, kvheads, hd, lens_before,
                                                           num_new, with_bias):
    """bfloat16 rows: the product (weight-streaming mma.sync up to 8 rows, tcgen05 with the weights on the rows from
    9 to 256, tcgen05 with the tokens on the rows from 512 on) rotates q and k and writes k and v into the cache in its
    epilogue.  Against the plain product followed by the plain rotation and cache write (which round the product
    to bfloat16 in between; the fused kernel rotates the float32 sums)."""
    dtype, k = torch.bfloat16, 8 * 21
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens_before, num_new, 23)
    g = torch.Generator().manual_seed(24)
    n, rows = sum(num_new), (nheads + 2 * kvheads) * hd
    x = torch.randn(n, k, generator=g).to(dtype).cuda()
    w = (torch.randn(rows, k, generator=g) * 0.08).to(dtype).cuda()
    b = (torch.randn(rows, generator=g) * 0.3).to(dtype).cuda() if with_bias else None
    inv = (1.0 / (500000.0 ** (torch.arange(0, hd, 2).float() / hd))).cuda()
    keys0, values0 = view.keys.clone(), view.values.clone()

    class V:
        keys, values, table, block_tokens = keys0, values0, view.table, 64

    want_q = P.rope_store(P.linear(x, w, b, torch.float32), inv, batch, V, nheads, kvheads, hd)
    got_q = ops.qkv_rope_store(x, w, b, inv, batch, view, nheads, kvheads, hd)
    ops.check_error_flag("cuda")
    t = dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(got_q.float(), want_q.float(), **t)
    torch.testing.assert_close(view.keys.float(), keys0.float(), equal_nan=True, **t)
    torch.testing.assert_close(view.values.float(), values0.float(), equal_nan=True, **t)
    # nothing else of the cache was touched: what was NaN (no live position) is NaN still
    assert torch.equal(torch.isnan(view.keys), torch.isnan(keys0)) and torch.equal(torch.isnan(view.values), torch.isnan(values0))
    # the same values as the two kernels one after the other, up to the rounding of the product in between
    two = ops.rope_store(ops.linear(x, w, b), inv, batch, view, nheads, kvheads, hd)
    torch.testing.assert_close(got_q.float(), two.float(), **t)
    # without frequencies nothing is rotated; without cache writes the cache stays as it is
    before = view.keys.clone()
    q2 = ops.qkv_rope_store(x, w, b, None, batch, view, nheads, kvheads, hd, writes_cache=False)
    torch.testing.assert_close(q2.float(), P.linear(x, w, b, torch.float32)[:, : nheads * hd].float(), **t)
    assert torch.equal(torch.nan_to_num(view.keys.float()), torch.nan_to_num(before.float()))


@pytest.mark.parametrize("half,n", [(8, 5), (64, 700), (40, 33)])
@pytest.mark.parametrize("with_ids", [False, True])
def test_table_of_rotation_angles(ops, half, n, with_ids):
    """(sin, cos) of position * frequency in float32, once a step for all layers; with position ids, of those."""
    g = torch.Generator().manual_seed(half)
    inv = (1.0 / (10000.0 ** (torch.arange(half).float() / half))).cuda()

    class B:
        positions = torch.randint(0, 100000, (n,), generator=g, dtype=torch.int32).cuda()
        position_ids = torch.randint(0, 100000, (n,), generator=g, dtype=torch.int32).cuda() if with_ids else None
        scratch = {}

    got = ops.rotary_table(inv, B)
    seen = (B.position_ids if with_ids else B.positions).float()
    angles = (seen[:, None] * inv[None, :]).double()  # the float32 product, as the rotation kernels take it
    assert got.shape == (n, half, 2) and got.dtype == torch.float32
    torch.testing.assert_close(got[..., 0].double(), angles.sin(), atol=2e-7, rtol=0)
    torch.testing.assert_close(got[..., 1].double(), angles.cos(), atol=2e-7, rtol=0)
    assert ops.rotary_table(inv, B) is got  # kept with the batch until the next step empties it


ATTN_CASES = [
    # nheads, kvheads, hd, lens_before, num_new, window
    (4, 2, 16, [0, 0, 0], [5, 70, 17], 0),          # prompts from an empty cache
    (3, 1, 32, [100, 3, 64], [1, 1, 1], 0),         # decode, MQA
    (5, 5, 48, [130, 0], [40, 129], 0),             # continuation onto a cached prefix, odd head size
    (12, 1, 64, [300], [1], 0),                     # decode with 12 query heads on one kv head (two chunks)
    (4, 2, 16, [200, 10], [1, 1], 70),              # decode with a window
    (4, 2, 32, [90, 0], [50, 150], 33),             # prefill with a window
    (2, 2, 128, [513], [1], 0),                     # decode over three splits
    (2, 1, 256, [20], [30], 0),                     # the largest head size
    (8, 2, 128, [0, 100], [200, 77], 0),            # prefill, head size 128, four query heads a kv head
    (4, 4, 64, [64, 0], [130, 1], 0),               # prefill, head size 64, one query head a kv head
    (6, 2, 64, [10], [300], 50),                    # prefill, head size 64, window
    (3, 1, 128, [129], [64], 0),                    # three query heads a kv head: 42 positions a block, two rows idle
    (4, 2, 64, [500, 70], [100, 3], 50),            # prefill behind a window whose earlier blocks were given back
    (8, 2, 128, [300], [40], 64),                   # the same at head size 128
    (8, 2, 128, [300, 200], [1, 1], 64),            # decode behind a window
    (5, 5, 48, [130, 70], [1, 1], 0),               # decode, a head size whose 16-byte pieces do not divide a warp
    (4, 2, 80, [100, 200], [1, 1], 0),              # decode, head size 80 (a last k-step of 16 alone)
    (4, 2, 80, [10], [70], 0),                      # prefill, head size 80
    (2, 1, 64, [33000], [1], 0),                    # decode over more splits (129) than the merge stages in shared memory
    (4, 2, 16, [40000, 100], [1, 1], 3000),         # the same behind a window: the first 144 splits hold nothing
    (8, 8, 128, [33000, 100, 5000, 64], [1, 1, 1, 1], 0),  # the same with enough to read for the streaming kernel
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nheads,kvheads,hd,lens_before,num_new,window", ATTN_CASES)
def test_attention(ops, dtype, nheads, kvheads, hd, lens_before, num_new, window):
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens_before, num_new, 8, window)
    g = torch.Generator().manual_seed(9)
    n = sum(num_new)
    # the step's own keys and values
    qkv = torch.randn(n, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    scale = 1.0 / math.sqrt(hd)
    want = P.attention(q, batch, view, nheads, kvheads, hd, scale, window)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, window)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(ops, dtype):
    """One key among hundreds is scaled so that it takes nearly all the weight: its value must come out,
    wherever it lies (first position, a block edge, a split edge)."""
    nheads, kvheads, hd = 2, 1, 32
    for far in (0, 63, 64, 255, 256, 400):
        cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, [600], [1], 10)
        table = cache.groups[0].table_host
        slot = int(batch.slots[0])
        g = torch.Generator().manual_seed(11)
        qkv = torch.randn(1, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
        q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
        blk = int(table[slot, far // 64])
        view.keys[blk, 0, far % 64] = (q[0, :hd].float() * 8).to(dtype)  # a large score for head 0
        marker = torch.full((hd,), 3.0).to(dtype).cuda()
        view.values[blk, 0, far % 64] = marker
        got = ops.attention(q, batch, view, nheads, kvheads, hd, 1.0 / math.sqrt(hd), 0)
        torch.testing.assert_close(got[0, :hd].float(), marker.float(), atol=5e-2, rtol=0)
        want = P.attention(q, batch, view, nheads, kvheads, hd, 1.0 / math.sqrt(hd), 0)
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("hd,nheads,kvheads", [(128, 8, 2), (64, 4, 4), (48, 4, 2)])
def test_prefill_attention_with_keys_that_outgrow_the_running_maximum(ops, hd, nheads, kvheads):
    """Random scores are all alike, so a kernel's rescaling of what it has accumulated is never exercised by them.
    Here three cached keys are copies of one query row, scaled 2, 4 and 8 times: as the key blocks go by, that
    row's maximum grows in big steps (far past the 2^8 by which the tcgen05 kernel lets it lag), the last copy takes
    nearly all the weight, and its value must come out.  Head sizes 128 and 64 take the tcgen05 kernel, 48 mma.sync."""
    dtype = torch.bfloat16
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, [450], [70], 12)
    table = cache.groups[0].table_host
    slot = int(batch.slots[0])
    g = torch.Generator().manual_seed(13)
    qkv = torch.randn(70, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    row, head = 37, nheads - 1                       # a query in the middle of a tile, the last head of its group
    kvh = head // (nheads // kvheads)
    qv = q[row, head * hd:(head + 1) * hd].float()
    marker = torch.full((hd,), 3.0).to(dtype).cuda()
    for far, factor in ((10, 2.0), (100, 4.0), (300, 8.0)):
        blk = int(table[slot, far // 64])
        view.keys[blk, kvh, far % 64] = (qv * factor).to(dtype)
        view.values[blk, kvh, far % 64] = marker * (factor / 8.0)
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, 0)
    ops.check_error_flag("cuda")
    want = P.attention(q, batch, view, nheads, kvheads, hd, scale, 0)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got[row, head * hd:(head + 1) * hd].float(), marker.float(), atol=8e-2, rtol=0)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("n_seqs,kvheads", [(70, 8), (30, 8), (3, 2)])
def test_decode_attention_at_every_batch_size(ops, n_seqs, kvheads):
    """Decode attention picks the warps per block by the number of (sequence, kv head) pairs: one warp that walks
    four key blocks with a running maximum of its own (many pairs), two, or four with a block each (few).  Every
    variant against the plain implementation, with one key in the last block of a long sequence made large so that
    the running maximum jumps late."""
    dtype, hd = torch.bfloat16, 64
    nheads = kvheads * 4
    g = torch.Generator().manual_seed(14)
    lens = [int(v) for v in torch.randint(1, 520, (n_seqs,), generator=g)]
    lens[0] = 519
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens, [1] * n_seqs, 15, poison=False)
    qkv = torch.randn(n_seqs, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    table = cache.groups[0].table_host
    slot, far = int(batch.slots[0]), 500
    blk = int(table[slot, far // 64])
    view.keys[blk, 1, far % 64] = (q[0, 5 * hd:6 * hd].float() * 6).to(dtype)  # head 5 uses kv head 1
    view.values[blk, 1, far % 64] = torch.full((hd,), 2.0).to(dtype).cuda()
    scale = 1.0 / math.sqrt(hd)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, 0)
    want = P.attention(q, batch, view, nheads, kvheads, hd, scale, 0)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got[0, 5 * hd:6 * hd].float(), torch.full((hd,), 2.0).cuda(), atol=5e-2, rtol=0)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("n_seqs,nheads,kvheads,hd,window", [
    (70, 32, 8, 128, 0),     # the benchmark's head layout
    (40, 48, 16, 64, 100),   # a window: blocks behind it given back, first blocks cut on the left
    (66, 24, 8, 64, 0),      # three query heads a kv head: five of the tile's eight columns idle
    (33, 160, 16, 128, 0),   # ten query heads a kv head: two chunks of columns
    (600, 2, 1, 64, 0),      # more sequences than the persistent warps: several units each, unequal
])
def test_decode_attention_of_many_sequences_streams_the_cache(ops, n_seqs, nheads, kvheads, hd, window):
    """From 512 (sequence, kv head) pairs on, decode attention is a persistent kernel that streams whole cache
    blocks through shared memory with TMA.  Everything that is no live position is NaN: a block's rows beyond the
    sequence are copied too and must not reach the result.  One far key stands out in a long sequence."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(21)
    lens = [int(v) for v in torch.randint(1, 700, (n_seqs,), generator=g)]
    lens[0], lens[1], lens[2] = 699, 256, 1
    cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens, [1] * n_seqs, 16, window)
    qkv = torch.randn(n_seqs, (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
    q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
    group = nheads // kvheads
    head = nheads - 1
    far = 650 if window == 0 else 640
    table = cache.groups[0].table_host
    blk = int(table[int(batch.slots[0]), far // 64])
    view.keys[blk, head // group, far % 64] = (q[0, head * hd:(head + 1) * hd].float() * 6).to(dtype)
    view.values[blk, head // group, far % 64] = torch.full((hd,), 2.0).to(dtype).cuda()
    scale = 1.0 / math.sqrt(hd)
    before = ops.attention_stream_launches(hd)
    got = ops.attention(q, batch, view, nheads, kvheads, hd, scale, window)
    ops.check_error_flag("cuda")
    assert ops.attention_stream_launches(hd) == before + 1  # it was this kernel that ran
    want = P.attention(q, batch, view, nheads, kvheads, hd, scale, window)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got[0, head * hd:(head + 1) * hd].float(), torch.full((hd,), 2.0).cuda(), atol=5e-2, rtol=0)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


def test_kernels_report_what_the_host_should_have_prevented(ops):
    """A token id outside the vocabulary and a position without a cache block do not fault: the kernel leaves the
    row alone, sets the error flag, and the host's check raises (and clears the flag)."""
    from fms_b200.kernels.ops import KernelError

    ops.check_error_flag("cuda")
    table = torch.randn(10, 16).cuda()
    ops.embed(table, torch.tensor([3, 10, 2], dtype=torch.int32).cuda())  # 10 is one past the last row
    with pytest.raises(KernelError, match="vocabulary"):
        ops.check_error_flag("cuda")
    ops.check_error_flag("cuda")  # cleared

    for dtype, n_new in ((torch.float32, 2), (torch.bfloat16, 70)):  # the per-token and the many-token kernel
        cache, view, batch = make_cache_case(dtype, 4, 2, 16, [63], [n_new], 16, poison=False)
        view.table[int(batch.slots[0]), 1] = -1  # positions 64..127 have lost their block
        keys0 = view.keys.clone()
        qkv = torch.randn(n_new, 8 * 16).to(dtype).cuda()
        ops.rope_store(qkv, None, batch, view, 4, 2, 16)
        with pytest.raises(KernelError, match="cache block"):
            ops.check_error_flag("cuda")
        row = cache.groups[0].table_host[int(batch.slots[0])]
        still_there = sorted(int(row[i]) for i in range((63 + n_new + 63) // 64) if i != 1)
        changed = (view.keys != keys0).flatten(1).any(1).nonzero().flatten().tolist()
        assert changed == still_there  # only the blocks that exist were written

    # the same through the product that writes the cache itself (up to 8 bfloat16 rows)
    cache, view, batch = make_cache_case(torch.bfloat16, 4, 2, 16, [63], [2], 17, poison=False)
    view.table[int(batch.slots[0]), 1] = -1
    keys0 = view.keys.clone()
    x = torch.randn(2, 24).to(torch.bfloat16).cuda()
    w = torch.randn(8 * 16, 24).to(torch.bfloat16).cuda()
    ops.qkv_rope_store(x, w, None, None, batch, view, 4, 2, 16)
    with pytest.raises(KernelError, match="cache block"):
        ops.check_error_flag("cuda")
    changed = (view.keys != keys0).flatten(1).any(1).nonzero().flatten().tolist()
    assert changed == [int(cache.groups[0].table_host[int(batch.slots[0])][0])]  # position 63 was written, 64 was not


def test_attention_refuses_other_head_sizes():
    from fms_b200.kernels.build import KernelBuildError, _spec

    for hd in (8, 24, 272):
        with pytest.raises(KernelBuildError):
            _spec(f"attention_hd{hd}")


@pytest.mark.parametrize("vocab", [331, 1000, 128256])
def test_argmax(ops, vocab):
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(5, vocab, generator=g).cuda()
    logits[1, 7] = logits[1, vocab - 1] = 50.0  # equal maxima: the lower index
    logits[2, vocab - 1] = 60.0
    got = ops.argmax(logits)
    assert got.tolist() == torch.argmax(logits.cpu(), -1).tolist()
    assert got[1].item() == 7 and got[2].item() == vocab - 1


@pytest.mark.parametrize("vocab,top_k,temperature", [(331, 0, 0.8), (331, 10, 1.0), (1000, 1, 0.5), (128256, 50, 1.3),
                                                     (128256, 0, 0.7)])
def test_sample_equals_plain_inverse_cdf(ops, vocab, top_k, temperature):
    g = torch.Generator().manual_seed(13)
    rows = 24
    logits = (torch.randn(rows, vocab, generator=g) * 3).cuda()
    requests = torch.arange(100, 100 + rows, dtype=torch.int32).cuda()
    mismatches = 0
    for step in (0, 1, 17):
        got = ops.sample(logits, temperature, top_k, 77, requests, step).tolist()
        want = P.sample(logits.cpu(), temperature, top_k, 77, requests.cpu(), step).tolist()
        mismatches += sum(a != b for a, b in zip(got, want))
        # a request's draw does not depend on its row or on the other rows
        alone = ops.sample(logits[5:6].contiguous(), temperature, top_k, 77, requests[5:6].contiguous(), step)
        assert alone.item() == got[5]
    # float32 and float64 running sums may cross u at neighbouring tokens, rarely
    assert mismatches <= 1


def test_sample_distribution_and_top_k(ops):
    vocab, rows = 50, 4000
    g = torch.Generator().manual_seed(14)
    row = torch.randn(vocab, generator=g) * 2
    logits = row.repeat(rows, 1).cuda()
    requests = torch.arange(rows, dtype=torch.int32).cuda()
    got = ops.sample(logits, 1.0, 0, 5, requests, 0).long().cpu()
    freq = torch.bincount(got, minlength=vocab).double() / rows
    p = torch.softmax(row.double(), 0)
    assert (freq - p).abs().max() < 0.03
    got = ops.sample(logits, 1.0, 3, 5, requests, 1).long().cpu()
    assert set(got.tolist()) <= set(torch.topk(row, 3).indices.tolist())
    assert len(set(got.tolist())) == 3


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_long_context(ops, dtype):
    """Thousands of cached positions: many blocks, many decode splits, a prefill tile deep inside a sequence."""
    nheads, kvheads, hd = 8, 2, 64
    for lens_before, num_new in (([5000, 37], [1, 1]), ([4090], [20])):
        cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens_before, num_new, 90, poison=True)
        g = torch.Generator().manual_seed(91)
        qkv = torch.randn(sum(num_new), (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
        q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
        got = ops.attention(q, batch, view, nheads, kvheads, hd, 1.0 / math.sqrt(hd), 0)
        want = P.attention(q, batch, view, nheads, kvheads, hd, 1.0 / math.sqrt(hd), 0)
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
