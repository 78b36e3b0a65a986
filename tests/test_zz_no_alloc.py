"""Decode attention for callers that cannot allocate device memory (csrc/attention_no_alloc.h).

Some hosts of these kernels may not call cudaMalloc once they are running: a process with a fixed
memory budget, a loop that must not meet an allocation's synchronisation or failure, a plug-in whose host
owns the allocator.  ``fms_attention_decode_no_alloc`` keeps the scratch of the key splits in an array
inside the library.  This test calls it through its exported C symbol, exactly as such a host would, and
compares its output with the ordinary entry point's (which takes caller-allocated scratch), on two calls
in a row that share the built-in array.  It has a file of its own, collected last.
"""
import ctypes
import math

import pytest
import torch

import plain_ops as P

pytestmark = pytest.mark.gpu

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _no_alloc_entry(head_dim):
    from fms_b200.kernels.build import load_library

    lib = load_library(f"attention_hd{head_dim}")
    f = lib.fms_attention_decode_no_alloc
    f.argtypes = [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P]
    f.restype = _I
    return f, lib


def _call(f, q, out, view, batch, n_splits, nheads, kvheads, hd, scale, window):
    return f(q.data_ptr(), out.data_ptr(), 0 if q.dtype == torch.float32 else 1, view.keys.data_ptr(),
             view.values.data_ptr(), view.table.data_ptr(), view.table.shape[1], view.block_tokens,
             batch.slots.data_ptr(), batch.first_row.data_ptr(), batch.len_after.data_ptr(), batch.n_seqs, n_splits,
             nheads, kvheads, hd, scale, window, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_equals_the_ordinary_one_twice_in_a_row(dtype):
    from fms_b200.kernels import ops
    from test_kernels_gpu import make_cache_case

    nheads, kvheads, hd = 6, 2, 64
    f, lib = _no_alloc_entry(hd)
    scale = 1.0 / math.sqrt(hd)
    # two different batches, one after the other, through the same built-in scratch: the second has fewer
    # sequences and other lengths, so anything left over from the first would show
    for seed, lens in ((21, [700, 3, 256, 100]), (22, [90, 513])):
        cache, view, batch = make_cache_case(dtype, nheads, kvheads, hd, lens, [1] * len(lens), seed)
        g = torch.Generator().manual_seed(seed)
        qkv = torch.randn(len(lens), (nheads + 2 * kvheads) * hd, generator=g).to(dtype).cuda()
        q = ops.rope_store(qkv, None, batch, view, nheads, kvheads, hd)
        want = ops.attention(q, batch, view, nheads, kvheads, hd, scale, 0)  # caller-allocated scratch
        n_splits = (batch.max_len_after + 255) // 256
        out = torch.full_like(q, float("nan"))
        rc = _call(f, q, out, view, batch, n_splits, nheads, kvheads, hd, scale, 0)
        assert rc == 0, lib.fms_last_error().decode()
        torch.cuda.synchronize()
        tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out.float(), want.float(), **tol)
        assert torch.equal(out, want)  # the same kernels in the same order: the same bits
        # and against the plain restatement, so that this test stands without the ordinary entry point
        torch.testing.assert_close(out.float(), P.attention(q, batch, view, nheads, kvheads, hd, scale, 0).float(), **tol)


def test_no_alloc_entry_point_refuses_what_exceeds_its_scratch():
    from fms_b200.kernels import ops
    from test_kernels_gpu import make_cache_case

    nheads, kvheads, hd = 6, 2, 64
    f, lib = _no_alloc_entry(hd)
    cache, view, batch = make_cache_case(torch.float32, nheads, kvheads, hd, [10], [1], 23)
    q = torch.zeros(1, nheads * hd, device="cuda")
    out = torch.zeros_like(q)
    # 1 sequence x 6 heads x 60000 splits x 66 floats is far more than 8 MiB: refused on the host, nothing runs
    rc = _call(f, q, out, view, batch, 60000, nheads, kvheads, hd, 0.125, 0)
    assert rc != 0 and b"scratch" in lib.fms_last_error()
    rc = _call(f, q, out, view, batch, 1, nheads, kvheads, 32, 0.125, 0)  # another head size than the library's
    assert rc != 0 and b"head size" in lib.fms_last_error()
