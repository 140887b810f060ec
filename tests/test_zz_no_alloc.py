"""The decode-attention entry point that brings its own scratch memory.

Some hosts of the kernel library cannot allocate device memory at the moment they need attention
(all of it belongs to their own pool, or an allocation's device-wide synchronisation is not
acceptable there).  For them the library exports `hb_attention_decode_bf16_noalloc`, which uses a
fixed scratch array inside the library instead of scratch passed by the caller.  This test calls
it through its exported C symbol, twice in a row on different inputs (the second call finds the
first call's leftovers in the shared array), and checks both results against the ordinary entry
point's.  It runs last so that a run that stops at the first failure has seen every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, lens, nh, nkv, hd, page=64):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    P = max(-(-n // page) for n in lens)
    n_pages = B * P + 2
    k = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(B, nh * hd, generator=g).to(torch.bfloat16).cuda()
    table = torch.randperm(n_pages, generator=g)[: B * P].to(torch.int32).view(B, P).cuda()
    return q, k, v, table, torch.tensor(lens, dtype=torch.int32).cuda()


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from herbert_rs_b200 import ops
    from herbert_rs_b200.ops import lib as kernel_lib

    lib = kernel_lib.load()
    fn = lib.hb_attention_decode_bf16_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    nh, nkv, hd, scale = 8, 2, 128, 128 ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    # the second call has fewer sequences and fewer splits than the first: the first call's partial
    # results lie beyond what the second one writes, and must not be read
    for seed, lens, window, nsplit in [(1, [300, 65, 1, 129], 0, 4), (2, [500, 64, 17], 100, 2), (3, [700], 0, 1)]:
        q, k, v, table, seq_len = _case(seed, lens, nh, nkv, hd)
        want = torch.empty_like(q)
        scratch = torch.empty(ops.attention_decode_scratch_floats(len(lens), nh, hd, nsplit), device="cuda")
        ops.attention_decode(q, q.stride(0), want, k, v, seq_len, table, scratch, nh, nkv, hd, 64, nsplit, scale, window)
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), k.data_ptr(), v.data_ptr(), seq_len.data_ptr(),
                table.data_ptr(), table.stride(0), len(lens), nh, nkv, hd, 64, nsplit, scale, window, stream)
        assert rc == 0, kernel_lib.last_error()
        torch.cuda.synchronize()
        # the same kernels on the same inputs, and the splits are combined in a fixed order: the same bits
        assert torch.equal(got, want)
    # a request beyond the built-in array is refused with a message, and nothing runs
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), k.data_ptr(), v.data_ptr(), seq_len.data_ptr(),
            table.data_ptr(), table.stride(0), 4096, 64, 2, 128, 64, 64, scale, 0, stream)
    assert rc != 0 and "built-in array holds" in kernel_lib.last_error()
