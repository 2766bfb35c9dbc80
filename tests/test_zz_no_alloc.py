"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of this kernel cannot allocate device memory when they need it: a plug-in inside another
program's CUDA context with a fixed budget, a loop whose buffers are frozen after set-up, code inside
a stream capture.  For them ``qt_attention_decode_static`` keeps the split-KV scratch in a fixed array
inside the library.  The test calls it several times in a row (each later call finds the leftovers of the
one before in the shared scratch) and compares every result with a plain float32 statement of the
attention (so a wrong kernel fails here too) and, bit for bit, with the regular entry point, which runs
the same kernels on scratch from the caller.  It is collected last so that a failure here cannot hide another test's result, and
it sets up everything it needs itself, so it also passes alone in a fresh process.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
PAGE = 64


def _paged_case(seed, n_seqs, nq, nkv, d, lengths):
    generator = torch.Generator().manual_seed(seed)
    pages_per_seq = [math.ceil(n / PAGE) for n in lengths]
    total = sum(pages_per_seq) + 2
    order = torch.randperm(total, generator=generator).tolist()
    k_cache = (torch.randn(total, nkv, PAGE, d, generator=generator)).bfloat16().cuda()
    v_cache = (torch.randn(total, nkv, PAGE, d, generator=generator)).bfloat16().cuda()
    table = torch.zeros(n_seqs, max(pages_per_seq), dtype=torch.int32)
    cursor = 0
    for b, count in enumerate(pages_per_seq):
        table[b, :count] = torch.tensor(order[cursor:cursor + count], dtype=torch.int32)
        cursor += count
    q = torch.randn(n_seqs, nq, d, generator=generator).bfloat16().cuda()
    return q, k_cache, v_cache, table.cuda(), torch.tensor(lengths, dtype=torch.int32).cuda()


def _plain_attention(q, k_cache, v_cache, table, seq_len, nkv):
    """softmax(q k^T / sqrt(d)) v per sequence in float32, from the keys and values the page table names."""
    out = torch.empty(q.shape, dtype=torch.float32)
    n_seqs, nq, d = q.shape
    for b in range(n_seqs):
        n = int(seq_len[b])
        pages = table[b, :math.ceil(n / PAGE)].long().cpu()
        k = k_cache.cpu()[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n]      # [n, nkv, d]
        v = v_cache.cpu()[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n]
        k, v = k.repeat_interleave(nq // nkv, dim=1), v.repeat_interleave(nq // nkv, dim=1)
        scores = torch.einsum("hd,khd->hk", q[b].float().cpu(), k) * d ** -0.5
        out[b] = torch.einsum("hk,khd->hd", torch.softmax(scores, dim=-1), v)
    return out


def test_static_scratch_entry_point_matches_the_regular_one():
    from qwen_triton_b200.ops import _build, kernels

    lib = _build.load_library("attention_decode_static")
    fn = lib.qt_attention_decode_static
    c_int, c_ptr = ctypes.c_int, ctypes.c_void_p
    fn.argtypes = [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   ctypes.c_float, c_int, c_ptr]
    fn.restype = c_int
    stream = torch.cuda.current_stream().cuda_stream

    def call(q, k_cache, v_cache, table, seq_len, nkv, splits, window=0):
        out = torch.full_like(q, float("nan"))
        code = fn(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
                  seq_len.data_ptr(), q.shape[0], q.shape[1], nkv, q.shape[2], PAGE, 0, window, q.shape[2] ** -0.5, splits,
                  stream)
        return code, out

    def regular(q, k_cache, v_cache, table, seq_len, nkv, splits, window=None):
        out = torch.empty_like(q)
        n, nq, d = q.shape
        acc = torch.empty(n * nq * splits * d, device="cuda")
        ml = torch.empty(n * nq * splits * 2, device="cuda")
        kernels.attention_decode(q, k_cache, v_cache, out, table, seq_len, nkv, PAGE, 0, window, d ** -0.5, splits, acc, ml,
                                 impl="mma")
        return out

    # two calls in a row with different shapes and split counts: the second starts on the first one's leftovers
    first = _paged_case(1, 5, 8, 2, 128, [700, 1, 65, 129, 300])
    second = _paged_case(2, 3, 6, 3, 64, [64, 1000, 17])
    for case, nkv, splits in ((first, 2, 6), (second, 3, 3), (first, 2, 1)):
        code, out = call(*case, nkv, splits)
        assert code == 0, _build.last_error("attention_decode_static")
        torch.cuda.synchronize()
        # the tolerance of the bfloat16 kernel tests against the plain statement; the two entry points run the same
        # kernels in the same order, so their results are the same bits
        torch.testing.assert_close(out.float().cpu(), _plain_attention(*case, nkv), atol=2e-2, rtol=2e-2)
        assert torch.equal(out, regular(*case, nkv, splits))

    # a request beyond the built-in scratch is refused, and says so
    q, k_cache, v_cache, table, seq_len = _paged_case(3, 64, 32, 8, 128, [64] * 64)
    code, _ = call(q, k_cache, v_cache, table, seq_len, 8, 64)
    assert code != 0
    message = _build.last_error("attention_decode_static")
    assert "scratch" in message and str(64 * 32 * 64 * 130) in message
    # so are more (kv head, 16-head chunk) pairs than one launch takes
    q, k_cache, v_cache, table, seq_len = _paged_case(4, 1, 1, 1, 16, [64])
    code = fn(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q.data_ptr(), table.data_ptr(), 1, seq_len.data_ptr(),
              1, 70000, 70000, 16, PAGE, 0, 0, 0.25, 1, stream)
    assert code != 0 and "one launch" in _build.last_error("attention_decode_static")
