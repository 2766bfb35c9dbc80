"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same op, at sizes other
than the engine's tiny configurations (odd widths, head sizes in steps of 16, many groups, shuffled
pages), and with inputs made so that a fault shows: one far key that dominates, a key just outside
the window, stale data in reused pages."""
import math

import pytest
import torch

from qwen_triton_b200.ops import kernels
from qwen_triton_b200.ops.kernels import GemmOut

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# float32 1e-4/1e-4 and bfloat16 2e-2/2e-2: the reference's kernel bars (tests/test_kernels.py:28,150)
TOL = {torch.float32: dict(atol=1e-4, rtol=1e-4), torch.bfloat16: dict(atol=2e-2, rtol=2e-2)}
DTYPES = [torch.float32, torch.bfloat16]
PAGE = 64


def gen(seed=0):
    return torch.Generator(device="cpu").manual_seed(seed)


def rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    return (torch.randn(*shape, generator=gen(seed)) * scale).to(dtype).to(DEV)


def gate_act(name, g):
    """The gate activations the kernels offer, stated plainly."""
    return {"silu": lambda x: x * torch.sigmoid(x), "gelu": lambda x: torch.nn.functional.gelu(x),
            "gelu_tanh": lambda x: torch.nn.functional.gelu(x, approximate="tanh"), "relu": torch.relu}[name](g)


def rope_interleaved(x, cos, sin):
    """Rotation with neighbours as pairs: (x[2i], x[2i+1]) turns by angle i; dims beyond 2 * cos.shape[-1] pass."""
    rd = 2 * cos.shape[-1]
    even, odd = x[..., 0:rd:2], x[..., 1:rd:2]
    c, s = cos[:, None, :], sin[:, None, :]
    turned = torch.stack((even * c - odd * s, odd * c + even * s), dim=-1).flatten(-2)
    return torch.cat((turned, x[..., rd:]), dim=-1)


def close(actual, expected, dtype, what=""):
    torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), **TOL[dtype], msg=lambda m: f"{what}: {m}")


# ----------------------------------------------------------------------------- paged cache helpers
def paged(dense_k, dense_v, lengths, dtype, ring_tokens=0, seed=0, garbage=True):
    """Scatter per-sequence dense keys/values [len, nkv, d] into shuffled pages.  Unused room is filled
    with large garbage so that any read outside a sequence's valid range shows."""
    nkv, d = dense_k[0].shape[1:]
    per_seq = [min(math.ceil(n / PAGE), ring_tokens // PAGE) if ring_tokens else math.ceil(n / PAGE) for n in lengths]
    total = sum(per_seq) + 3
    order = torch.randperm(total, generator=gen(seed)).tolist()
    k_cache = torch.full((total, nkv, PAGE, d), 1e4 if garbage else 0.0)
    v_cache = torch.full((total, nkv, PAGE, d), -1e4 if garbage else 0.0)
    width = max(per_seq)
    table = torch.zeros((len(lengths), width), dtype=torch.int32)
    cursor = 0
    for b, n in enumerate(lengths):
        pages = order[cursor:cursor + per_seq[b]]
        cursor += per_seq[b]
        table[b, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        first = max(0, n - ring_tokens) if ring_tokens else 0
        for pos in range(first, n):
            idx = pos % ring_tokens if ring_tokens else pos
            k_cache[pages[idx // PAGE], :, idx % PAGE] = dense_k[b][pos]
            v_cache[pages[idx // PAGE], :, idx % PAGE] = dense_v[b][pos]
    return k_cache.to(dtype).to(DEV), v_cache.to(dtype).to(DEV), table.to(DEV)


def attention_reference(q, k, v, positions, scale, window):
    """q [n, nq, d] at absolute ``positions``; k/v [len, nkv, d] of the same sequence."""
    groups = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(groups, dim=1), v.repeat_interleave(groups, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    keys = torch.arange(k.shape[0])
    visible = keys[None, :] <= positions[:, None]
    if window:
        visible &= keys[None, :] > positions[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v)


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    table = rand(77, 200, seed=1, dtype=dtype)
    ids = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32, device=DEV)
    out = torch.full((5, 200), 9.0, device=DEV)
    kernels.embedding(out, table, ids)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, splits, rows", [(200, 1, 7), (96, 3, 7), (4100, 2, 7), (1024, 1, 7), (2048, 9, 9), (4100, 2, 300),
                                                  (9000, 2, 300), (36000, 1, 7), (16000, 9, 260)])
def test_add_rmsnorm(dtype, hidden, splits, rows):
    eps = 3e-6                                           # few rows of 1024 and more: a cluster of blocks per row
    residual = rand(rows, hidden, seed=2)
    delta_dtype = torch.float32 if splits > 1 else dtype
    delta = rand(splits, rows, hidden, seed=3, dtype=delta_dtype)
    weight = 1.0 + rand(hidden, seed=4, scale=0.1)
    expected_stream = residual + delta.float().sum(0)
    expected = expected_stream * torch.rsqrt(expected_stream.pow(2).mean(-1, keepdim=True) + eps) * weight
    stream = residual.clone()
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(stream, GemmOut(delta), weight, eps, out)
    close(stream, expected_stream, torch.float32, "stream")
    close(out, expected, dtype, "normed")
    # listed rows only: the stream stays as it was
    stream = residual.clone()
    picked = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(stream, GemmOut(delta), weight, eps, out, rows=picked)
    assert torch.equal(stream, residual)
    close(out, expected[picked.long()], dtype, "listed rows")
    # no pending delta
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(stream, None, weight, eps, out)
    close(out, residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps) * weight, dtype, "no delta")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, rotary, ring, splits, lengths", [
    (3, 3, 80, 40, 0, 1, [70, 3, 100]), (8, 2, 16, 16, 128, 2, [70, 3, 100]), (5, 1, 128, 128, 0, 1, [70, 3, 100]),
    # 256 tokens and more with every dimension rotating: the kernel that keeps rotation pairs in registers
    (5, 2, 128, 128, 0, 1, [200, 3, 150]), (3, 1, 64, 64, 0, 2, [200, 3, 150]), (2, 2, 256, 256, 512, 1, [200, 3, 150]),
    (7, 7, 128, 128, 0, 3, [190, 1, 99])])
@pytest.mark.parametrize("interleaved", [False, True])
def test_qk_norm_rope_write(dtype, nq, nkv, d, rotary, ring, splits, lengths, interleaved):
    import plain_qwen3 as plain
    rope = rope_interleaved if interleaved else plain.apply_rope
    past = [130, 0, 20]                                  # tokens before this step, per sequence; `lengths` are this step's
    tokens = sum(lengths)
    eps = 1e-5
    in_dtype = torch.float32 if splits > 1 else dtype
    qkv = rand(splits, tokens, (nq + 2 * nkv) * d, seed=5, dtype=in_dtype)
    qw, kw = 1.0 + rand(d, seed=6, scale=0.2), 1.0 + rand(d, seed=7, scale=0.2)
    max_pos = 400
    cos, sin = plain.rope_tables(torch.arange(max_pos), rotary, 50000.0, torch.float32)
    cos_sin = torch.cat((cos, sin), dim=-1).contiguous().to(DEV)
    token_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(lengths)).int().to(DEV)
    token_pos = torch.cat([torch.arange(p, p + n) for p, n in zip(past, lengths)]).int().to(DEV)
    totals = [p + n for p, n in zip(past, lengths)]
    zeros = [torch.zeros(t, nkv, d) for t in totals]
    k_cache, v_cache, table = paged(zeros, zeros, totals, dtype, ring_tokens=ring, seed=8, garbage=False)
    q_out = torch.empty(tokens, nq, d, dtype=dtype, device=DEV)
    kernels.qk_norm_rope_write(GemmOut(qkv), q_out, k_cache, v_cache, token_seq, token_pos, table, qw, kw, eps, cos_sin,
                               nq, nkv, d, PAGE, ring, interleaved=interleaved)
    x = qkv.float().sum(0).cpu().view(tokens, nq + 2 * nkv, d)
    pos = token_pos.cpu().long()
    q_ref = rope(plain.rms_norm(x[:, :nq], qw.cpu(), eps), cos[pos], sin[pos])
    k_ref = rope(plain.rms_norm(x[:, nq:nq + nkv], kw.cpu(), eps), cos[pos], sin[pos])
    v_ref = x[:, nq + nkv:]
    close(q_out, q_ref, dtype, "q")
    table_host, k_host, v_host = table.cpu(), k_cache.float().cpu(), v_cache.float().cpu()
    for t in range(tokens):
        b, p = int(token_seq[t]), int(pos[t])
        if ring and p < totals[b] - ring:
            continue                                      # overwritten by a later token of the ring
        idx = p % ring if ring else p
        page = int(table_host[b, idx // PAGE])
        close(k_host[page, :, idx % PAGE], k_ref[t], dtype, f"k of token {t}")
        close(v_host[page, :, idx % PAGE], v_ref[t], dtype, f"v of token {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, inter, group", [(5, 336, 0), (3, 301, 0), (300, 2056, 0), (5, 336, 16), (300, 2064, 16), (4, 300, 4)])
def test_swiglu(dtype, tokens, inter, group):      # vector form, scalar form, several blocks a row; gate and up rows interleaved
    for splits in (1, 3):
        in_dtype = torch.float32 if splits > 1 else dtype
        gate = rand(splits, tokens, inter, seed=9, scale=2.0, dtype=in_dtype)
        up = rand(splits, tokens, inter, seed=10, scale=2.0, dtype=in_dtype)
        if group:
            gate_up = torch.stack((gate.view(splits, tokens, inter // group, group), up.view(splits, tokens, inter // group, group)),
                                  dim=3).reshape(splits, tokens, 2 * inter).contiguous()
        else:
            gate_up = torch.cat((gate, up), dim=-1).contiguous()
        out = torch.empty(tokens, inter, dtype=dtype, device=DEV)
        kernels.swiglu(GemmOut(gate_up), out, group)
        close(out, torch.nn.functional.silu(gate.float().sum(0)) * up.float().sum(0), dtype, f"splits={splits}")
        for name in ("gelu", "gelu_tanh", "relu"):                  # the activation is a parameter of the part
            kernels.swiglu(GemmOut(gate_up), out, group, name)
            close(out, gate_act(name, gate.float().sum(0)) * up.float().sum(0), dtype, f"{name}, splits={splits}")
    with pytest.raises(kernels.KernelError, match="activation"):
        kernels.swiglu(GemmOut(gate_up), out, group, "softplus")


# ----------------------------------------------------------------------------- matrix product
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k", [(1, 503, 96), (37, 130, 257), (64, 64, 16), (129, 70, 1000)])
def test_gemm_simt(dtype, m, n, k):
    a, w = rand(m, k, seed=10, dtype=dtype), rand(n, k, seed=11, scale=0.1, dtype=dtype)
    expected = a.double() @ w.double().T
    for out_dtype in {dtype, torch.float32}:
        out = torch.empty(1, m, n, dtype=out_dtype, device=DEV)
        kernels.gemm_simt(a, w, GemmOut(out))
        close(out[0], expected, out_dtype, f"{m}x{n}x{k}")


def test_gemm_float32_is_true_float32():
    """Inputs that a reduced-precision matrix mode would round away: 1 + 2^-12 squared keeps the 2^-11 term."""
    a = torch.full((4, 64), 1.0 + 2.0 ** -12, device=DEV)
    w = torch.full((3, 64), 1.0 + 2.0 ** -12, device=DEV)
    out = torch.empty(1, 4, 3, device=DEV)
    kernels.gemm_simt(a, w, GemmOut(out))
    exact = 64 * (1.0 + 2.0 ** -12) ** 2
    assert abs(float(out[0, 0, 0]) - exact) < 1e-4 and abs(exact - 64.0) > 0.03


# ----------------------------------------------------------------------------- attention
def impls_for(dtype, d, prefill=False):
    if dtype != torch.bfloat16 or d % 16 or d > 128:
        return ["generic"]
    return ["generic", "mma"] + ((["tc"] if d in (64, 128) else []) if prefill else ["ws"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, window, ring", [(6, 2, 80, None, 0), (4, 4, 16, 40, 128), (8, 1, 128, None, 0), (2, 1, 256, 100, 0),
                                                      (3, 1, 48, 70, 192), (4, 2, 112, None, 0), (4, 2, 64, None, 0), (6, 3, 128, 90, 256),
                                                      (2, 2, 64, 50, 192), (32, 8, 128, None, 0)])
def test_attention_prefill(dtype, nq, nkv, d, window, ring):
    q_lens, past = [150, 1, 33, 64], [100, 0, 7, 64]
    if ring:
        q_lens = [min(n, ring - window + 1) for n in q_lens]       # a step never outruns the ring
    totals = [p + n for p, n in zip(past, q_lens)]
    k = [rand(t, nkv, d, seed=20 + i, dtype=dtype).float().cpu() for i, t in enumerate(totals)]
    v = [rand(t, nkv, d, seed=30 + i, dtype=dtype).float().cpu() for i, t in enumerate(totals)]
    k_cache, v_cache, table = paged(k, v, totals, dtype, ring_tokens=ring, seed=1)
    q = rand(sum(q_lens), nq, d, seed=40, dtype=dtype)
    out = torch.empty_like(q)
    seq_start = torch.tensor([0, *torch.tensor(q_lens).cumsum(0).tolist()], dtype=torch.int32, device=DEV)
    seq_past = torch.tensor(past, dtype=torch.int32, device=DEV)
    scale = d ** -0.5
    for impl in impls_for(dtype, d, prefill=True):
        out.fill_(float("nan"))
        kernels.attention_prefill(q, k_cache, v_cache, out, table, seq_start, seq_past, max(q_lens), nkv, PAGE, ring, window, scale, impl=impl)
        kernels.check_status(DEV)
        start = 0
        for b, n in enumerate(q_lens):
            ref = attention_reference(q[start:start + n].float().cpu(), k[b], v[b], torch.arange(past[b], past[b] + n), scale, window)
            close(out[start:start + n], ref, dtype, f"{impl}, sequence {b}")
            start += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, window, ring, splits", [
    (6, 2, 80, None, 0, 1), (6, 2, 80, None, 0, 5), (4, 4, 16, 40, 128, 2), (16, 1, 128, None, 0, 3),
    (32, 8, 128, None, 0, 4), (5, 5, 112, 300, 0, 7), (10, 2, 48, None, 0, 64), (40, 2, 64, None, 0, 2), (8, 2, 96, 130, 256, 3)])
def test_attention_decode(dtype, nq, nkv, d, window, ring, splits):
    lengths = [700, 1, 65, 129]
    k = [rand(t, nkv, d, seed=50 + i, dtype=dtype).float().cpu() for i, t in enumerate(lengths)]
    v = [rand(t, nkv, d, seed=60 + i, dtype=dtype).float().cpu() for i, t in enumerate(lengths)]
    k_cache, v_cache, table = paged(k, v, lengths, dtype, ring_tokens=ring, seed=2)
    q = rand(len(lengths), nq, d, seed=70, dtype=dtype)
    out = torch.empty_like(q)
    seq_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    part_acc = torch.full((len(lengths) * nq * splits * d,), float("nan"), device=DEV)
    part_ml = torch.full((len(lengths) * nq * splits * 2,), float("nan"), device=DEV)
    scale = d ** -0.5
    refs = [attention_reference(q[b:b + 1].float().cpu(), k[b], v[b], torch.tensor([n - 1]), scale, window) for b, n in enumerate(lengths)]
    for impl in impls_for(dtype, d):
        for warps in ((1, 3, 6) if impl == "ws" else (1,)):      # "ws": splits * warps key ranges
            out.fill_(float("nan"))
            kernels.attention_decode(q, k_cache, v_cache, out, table, seq_len, nkv, PAGE, ring, window, scale, splits, part_acc, part_ml,
                                     impl=impl, warps=warps)
            for b in range(len(lengths)):
                close(out[b:b + 1], refs[b], dtype, f"{impl} with {warps} warps, sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["decode", "prefill"])
def test_one_far_key_among_hundreds_wins(dtype, mode):
    """Key 3 of 700 gets a score far above the rest; the output must be its value row."""
    nq, nkv, d, n = 4, 2, 64, 700
    k = torch.randn(n, nkv, d, generator=gen(80)) * 0.1
    v = torch.randn(n, nkv, d, generator=gen(81))
    query = torch.randn(1, nq, d, generator=gen(82)) * 0.1
    for h in range(nq):
        k[3, h // 2] = 0.0
    k[3, :, 0] = 40.0
    query[0, :, 0] = 40.0
    k, v = k.to(dtype).float(), v.to(dtype).float()
    k_cache, v_cache, table = paged([k], [v], [n], dtype, seed=3)
    q = query.to(dtype).to(DEV)
    out = torch.empty_like(q)
    expected = v[3].repeat_interleave(2, dim=0)[None]
    for impl in impls_for(dtype, d, prefill=mode == "prefill"):
        out.fill_(float("nan"))
        if mode == "decode":
            kernels.attention_decode(q, k_cache, v_cache, out, table, torch.tensor([n], dtype=torch.int32, device=DEV), nkv, PAGE, 0,
                                     None, 1.0, 4, torch.empty(nq * 4 * d, device=DEV), torch.empty(nq * 4 * 2, device=DEV), impl=impl,
                                     warps=3 if impl == "ws" else 1)
        else:
            kernels.attention_prefill(q, k_cache, v_cache, out, table, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                      torch.tensor([n - 1], dtype=torch.int32, device=DEV), 1, nkv, PAGE, 0, None, 1.0, impl=impl)
        close(out, expected, dtype, f"far key, {impl}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["decode", "prefill"])
@pytest.mark.parametrize("d", [32, 64, 128])                 # 64 and 128: the tcgen05 prefill kernel among the others
def test_window_edge(dtype, mode, d):
    """The key just outside the window carries a huge score and a huge value: it must not be seen; the
    key just inside carries the second-largest score: it must dominate."""
    nq, nkv, n, window = 2, 1, 200, 37
    k = torch.randn(n, nkv, d, generator=gen(90)) * 0.05
    v = torch.randn(n, nkv, d, generator=gen(91))
    last = n - 1
    outside, inside = last - window, last - window + 1
    k[outside, :, 1] = 60.0
    v[outside] = 1000.0
    k[inside, :, 1] = 30.0
    query = torch.zeros(1, nq, d)
    query[0, :, 1] = 30.0
    k, v = k.to(dtype).float(), v.to(dtype).float()
    k_cache, v_cache, table = paged([k], [v], [n], dtype, seed=4)
    q = query.to(dtype).to(DEV)
    out = torch.empty_like(q)
    for impl in impls_for(dtype, d, prefill=mode == "prefill"):
        out.fill_(float("nan"))
        if mode == "decode":
            kernels.attention_decode(q, k_cache, v_cache, out, table, torch.tensor([n], dtype=torch.int32, device=DEV), nkv, PAGE, 0,
                                     window, 1.0, 3, torch.empty(nq * 3 * d, device=DEV), torch.empty(nq * 3 * 2, device=DEV), impl=impl,
                                     warps=2 if impl == "ws" else 1)
        else:
            kernels.attention_prefill(q, k_cache, v_cache, out, table, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                      torch.tensor([last], dtype=torch.int32, device=DEV), 1, nkv, PAGE, 0, window, 1.0, impl=impl)
        close(out, v[inside].expand(1, nq, d), dtype, f"window edge, {impl}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, window, ring", [(64, 37, 0), (64, 50, 192), (128, 100, 0), (128, 90, 256), (48, 30, 0)])
def test_both_edges_of_every_row_of_a_long_query_block(dtype, d, window, ring):
    """130 query rows after 150 earlier tokens, so that the window's edge and the causal edge of the rows wander through
    different 64-key tiles.  Key j carries 2 in dimension j mod d, and row i asks, with weights 30, 20 and 50, for
    the dimensions of the key just outside its window, the key just inside it and the key just after itself: the
    scores are 60 (must not be seen), 40 (must win: the row's output is that key's value) and 100 (must not be seen).
    With window < d no other key that the row sees shares one of these dimensions."""
    assert window < d - 1
    nq, nkv, past, rows = 4, 2, 150, 130
    if ring:
        rows = min(rows, ring - window + 1)
    total = past + rows
    k = torch.zeros(total + 1, nkv, d)
    k[torch.arange(total + 1), :, torch.arange(total + 1) % d] = 2.0
    v = torch.randn(total + 1, nkv, d, generator=gen(95))
    pos = torch.arange(past, past + rows)
    query = torch.zeros(rows, nq, d)
    query[torch.arange(rows), :, (pos - window) % d] = 30.0
    query[torch.arange(rows), :, (pos - window + 1) % d] = 20.0
    query[torch.arange(rows), :, (pos + 1) % d] = 50.0
    k, v = k.to(dtype).float(), v.to(dtype).float()
    # the cache holds the step's own keys and nothing later; the key after the last row exists only as the trap it is
    k_cache, v_cache, table = paged([k[:total]], [v[:total]], [total], dtype, ring_tokens=ring, seed=5)
    q = query.to(dtype).to(DEV)
    out = torch.empty_like(q)
    expected = v[pos - window + 1].repeat_interleave(nq // nkv, dim=1)
    for impl in impls_for(dtype, d, prefill=True):
        out.fill_(float("nan"))
        kernels.attention_prefill(q, k_cache, v_cache, out, table, torch.tensor([0, rows], dtype=torch.int32, device=DEV),
                                  torch.tensor([past], dtype=torch.int32, device=DEV), rows, nkv, PAGE, ring, window, 1.0, impl=impl)
        kernels.check_status(DEV)
        close(out, expected, dtype, f"edges of every row, {impl}")


# ----------------------------------------------------------------------------- sampling
def test_argmax_ties_go_to_the_lowest_id():
    logits = rand(5, 1500, seed=100)
    logits[0, 700] = logits[0, 1400] = 50.0
    logits[1, 0] = 50.0
    logits[2, 1499] = 50.0
    logits[3] = -float("inf")
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    kernels.argmax(logits, out)
    assert out.tolist() == [700, 0, 1499, 0, int(logits[4].argmax())]


def test_sample_follows_the_inverse_cdf():
    import plain_qwen3 as plain
    rows, vocab = 64, 5003
    logits = rand(rows, vocab, seed=101, scale=3.0)
    temps = torch.full((rows,), 0.8, device=DEV)
    uniforms = torch.rand(rows, generator=gen(102))
    uniforms[0] = 0.0
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    kernels.sample(logits, temps, uniforms.to(DEV), out)
    host = logits.cpu()
    for r in range(rows):
        assert plain.choice_is_consistent(host[r], 0.8, float(uniforms[r]), int(out[r])), r
    assert int(out[0]) == 0
    # the empirical distribution of many draws follows softmax(logits / T)
    small = rand(1, 7, seed=103).repeat(4000, 1).contiguous()
    draws = torch.empty(4000, dtype=torch.int32, device=DEV)
    kernels.sample(small, torch.full((4000,), 1.3, device=DEV), torch.rand(4000, generator=gen(104)).to(DEV), draws)
    freq = torch.bincount(draws.cpu().long(), minlength=7).float() / 4000
    assert (freq - torch.softmax(small[0].cpu() / 1.3, 0)).abs().max() < 0.03


def test_sample_draws_its_uniform_number_from_seed_request_and_step():
    """The kernel that makes the uniform number itself picks what the plain statement of that number picks, and a
    probe row whose logits make each token's share of the unit interval wide shows the number itself."""
    import plain_qwen3 as plain
    rows, vocab, seed = 40, 1009, (1 << 63) + 12345
    logits = rand(rows, vocab, seed=105, scale=2.0)
    keys = torch.stack([torch.arange(rows) * 7 - 3, torch.arange(rows) % 5], dim=1).int()      # a negative request number too
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    kernels.sample_keyed(logits, 0.7, seed, keys.to(DEV), out)
    host = logits.cpu()
    for r in range(rows):
        uniform = plain.uniform_for(seed, int(keys[r, 0]), int(keys[r, 1]))
        assert plain.choice_is_consistent(host[r], 0.7, uniform, int(out[r])), r
    # 4,096 tokens of equal weight: the chosen token is floor(uniform * 4096)
    flat = torch.zeros(rows, 4096, device=DEV)
    kernels.sample_keyed(flat, 1.0, seed, keys.to(DEV), out)
    expected = [int(plain.uniform_for(seed, int(keys[r, 0]), int(keys[r, 1])) * 4096) for r in range(rows)]
    assert all(abs(int(out[r]) - expected[r]) <= 1 for r in range(rows)), (out.tolist(), expected)


def _draws(logits_row, temperature, top_k, top_p, count=4000, seed=77):
    """``count`` draws from one row of logits, each with a request number of its own."""
    logits = logits_row.repeat(count, 1).contiguous()
    keys = torch.stack([torch.arange(count), torch.zeros(count, dtype=torch.long)], dim=1).int().to(DEV)
    out = torch.empty(count, dtype=torch.int32, device=DEV)
    kernels.sample_keyed(logits, temperature, seed, keys, out, top_k, top_p)
    return out.cpu().long()


@pytest.mark.parametrize("vocab, top_k, top_p", [(5003, 7, 1.0), (5003, 0, 0.6), (5003, 50, 0.8), (151936, 0, 0.9), (151936, 40, 0.95),
                                                 (300, 299, 0.999), (64, 1, 1.0)])
def test_sample_from_the_most_likely_tokens_only(vocab, top_k, top_p):
    """Many draws from one row: every drawn token is one that the sorted statement of top_k / top_p keeps, every kept
    token of some weight is drawn, and the frequencies follow the probabilities renormalised over the kept set."""
    import plain_qwen3 as plain
    temperature = 0.8
    row = rand(1, vocab, seed=140, scale=3.0)
    keep = plain.kept_tokens(row[0].cpu(), temperature, top_k, top_p)
    assert 0 < int(keep.sum()) < vocab
    draws = _draws(row, temperature, top_k, top_p)
    assert bool(keep[draws].all()), f"drawn outside the kept set: {sorted(set(draws[~keep[draws]].tolist()))[:10]}"
    probs = torch.where(keep, torch.softmax(row[0].cpu().double() / temperature, 0), torch.zeros(vocab, dtype=torch.float64))
    probs /= probs.sum()
    freq = torch.bincount(draws, minlength=vocab).double() / draws.numel()
    assert float((freq - probs).abs().max()) < 0.03
    assert bool((freq[probs > 0.01] > 0).all())
    # the same rows again: the same tokens (masses are summed as integers, so no order of additions shows)
    assert torch.equal(draws, _draws(row, temperature, top_k, top_p))


@pytest.mark.parametrize("top_k, top_p", [(300, 1.0), (0, 0.5), (12000, 0.3)])
def test_rows_of_nearly_equal_logits_are_cut_at_the_same_threshold(top_k, top_p):
    """20,000 logits within a few hundredths of each other: the threshold's neighbourhood holds more tokens than the
    kernel's short list, so it walks the whole row digit by digit instead; the kept set is the sorted statement's."""
    import plain_qwen3 as plain
    row = rand(1, 20000, seed=143, scale=0.01)
    keep = plain.kept_tokens(row[0].cpu(), 1.0, top_k, top_p)
    draws = _draws(row, 1.0, top_k, top_p, count=6000)
    assert bool(keep[draws].all())
    edge = row[0].cpu()[keep].min()                       # the least likely kept tokens are drawn as well
    near_edge = keep & (row[0].cpu() < edge + 0.002)
    assert int(near_edge.sum()) > 20 and bool(near_edge[draws].any())


def test_tokens_that_tie_with_the_last_kept_one_are_kept():
    """Ten tokens share the largest logit and top_k asks for four: all ten are drawn from.  Two tokens share the
    probability at which top_p is reached: both are kept."""
    row = rand(1, 700, seed=141, scale=0.5)
    tied = torch.tensor([3, 64, 65, 128, 300, 301, 511, 512, 640, 699])
    row[0, tied] = 6.0
    draws = _draws(row, 1.0, 4, 1.0, count=2000)
    assert sorted(set(draws.tolist())) == tied.tolist()
    row = torch.full((1, 500), -30.0, device=DEV)
    row[0, 10], row[0, 20], row[0, 400], row[0, 450] = 2.0, 1.0, 1.0, 0.0        # shares 0.55, 0.20, 0.20, 0.07 of the mass
    draws = _draws(row, 1.0, 0, 0.7, count=2000)                                   # 0.55 + 0.20 reaches 0.7: the other 0.20 ties
    assert sorted(set(draws.tolist())) == [10, 20, 400]
    draws = _draws(row, 1.0, 0, 0.5, count=500)
    assert set(draws.tolist()) == {10}
    # the two zeros are one value: a row of them is a row of ties, whatever their sign bits
    zeros = torch.zeros(1, 40, device=DEV)
    zeros[0, ::3] = -0.0
    for top_k, top_p in ((2, 1.0), (0, 0.1), (5, 0.5)):
        draws = _draws(zeros, 0.7, top_k, top_p, count=2000)
        assert sorted(set(draws.tolist())) == list(range(40)), (top_k, top_p)


def test_sample_of_distinct_rows_with_top_k_and_top_p():
    """64 different rows of the full vocabulary, each with the uniform number of its (request, step): the chosen token
    is the inverse-CDF choice over the kept set."""
    import plain_qwen3 as plain
    rows, vocab, seed = 64, 151936, 99
    logits = rand(rows, vocab, seed=142, scale=2.5)
    keys = torch.stack([torch.arange(rows) + 5, torch.arange(rows) % 3], dim=1).int()
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    for top_k, top_p in ((0, 0.9), (100, 1.0), (1000, 0.7)):
        kernels.sample_keyed(logits, 0.7, seed, keys.to(DEV), out, top_k, top_p)
        host = logits.cpu()
        for r in range(rows):
            uniform = plain.uniform_for(seed, int(keys[r, 0]), int(keys[r, 1]))
            assert plain.choice_is_consistent(host[r], 0.7, uniform, int(out[r]), top_k=top_k, top_p=top_p), (top_k, top_p, r)
    with pytest.raises(kernels.KernelError, match="top_p"):
        kernels.sample_keyed(logits, 0.7, seed, keys.to(DEV), out, 0, 0.0)


def test_kernels_refuse_what_they_cannot_run():
    with pytest.raises(kernels.KernelError, match="CUDA tensor"):
        kernels.argmax(torch.zeros(1, 4), torch.zeros(1, dtype=torch.int32))
    q = torch.zeros(1, 2, 272, device=DEV)
    cache = torch.zeros(1, 1, PAGE, 272, device=DEV)
    with pytest.raises(kernels.KernelError, match="head_dim"):
        kernels.attention_decode(q, cache, cache, torch.empty_like(q), torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                 torch.ones(1, dtype=torch.int32, device=DEV), 1, PAGE, 0, None, 1.0, 1, None, None)
    with pytest.raises(kernels.KernelError, match="do not fit"):
        kernels.gemm_simt(torch.zeros(2, 8, device=DEV), torch.zeros(4, 8, device=DEV), GemmOut(torch.zeros(2, 2, 4, device=DEV)))


@pytest.mark.parametrize("rows, cols", [(1, 7), (5, 130), (300, 4096), (2050, 257)])
def test_add_bias(rows, cols):
    out, bias = rand(rows, cols, seed=130), rand(cols, seed=131)
    expected = out + bias
    kernels.add_bias(out, bias)
    assert torch.equal(out, expected)
    with pytest.raises(kernels.KernelError):
        kernels.add_bias(out, bias[:-1].contiguous())


# ----------------------------------------------------------------------------- tensor-core matrix product
@pytest.mark.parametrize("m, n, k, splits, out_dtype", [
    (1, 503, 96, 1, torch.float32), (8, 640, 512, 2, torch.float32), (8, 6144, 4096, 3, torch.float32),
    (16, 130, 264, 1, torch.bfloat16), (37, 130, 264, 1, torch.bfloat16), (64, 4096, 1536, 4, torch.float32),
    (100, 200, 160, 1, torch.bfloat16), (300, 1000, 1024, 1, torch.bfloat16), (2048, 512, 4096, 1, torch.bfloat16),
    (513, 257, 72, 1, torch.float32), (5, 129, 8, 1, torch.float32),
    (1000, 5000, 256, 1, torch.bfloat16), (4096, 2560, 192, 1, torch.float32), (129, 19000, 64, 1, torch.bfloat16),
    (200, 384, 1024, 3, torch.float32), (256, 520, 2048, 4, torch.float32), (129, 130, 4096, 9, torch.float32)])   # split K over two token tiles
def test_gemm_tensor_cores(m, n, k, splits, out_dtype):
    a, w = rand(m, k, seed=110, dtype=torch.bfloat16), rand(n, k, seed=111, scale=0.1, dtype=torch.bfloat16)
    expected = a.double() @ w.double().T
    splits = kernels.tc_normalise_splits(k, splits)
    out = torch.full((splits, m, n), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_tc(a, w, GemmOut(out))
    kernels.check_status(DEV)
    close(GemmOut(out).value(), expected, out_dtype, f"{m}x{n}x{k} splits={splits}")


@pytest.mark.parametrize("m, n, k, out_dtype", [
    (1, 129, 8, torch.float32), (256, 256, 64, torch.float32), (300, 384, 200, torch.float32), (513, 257, 72, torch.float32),
    (1000, 1100, 4096, torch.bfloat16), (2048, 512, 4096, torch.bfloat16), (129, 19000, 64, torch.bfloat16),
    (777, 130, 264, torch.bfloat16), (4096, 24576, 192, torch.bfloat16), (5000, 7000, 448, torch.bfloat16)])   # the last two: several tiles per pair
def test_gemm_tensor_cores_block_pairs(m, n, k, out_dtype):
    """The cta_group::2 kernel: sizes that are no multiple of the pair's 256 x 256 tile, one K block and many."""
    a, w = rand(m, k, seed=114, dtype=torch.bfloat16), rand(n, k, seed=115, scale=0.1, dtype=torch.bfloat16)
    expected = a.double() @ w.double().T
    out = torch.full((1, m, n), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_tc_pair(a, w, GemmOut(out))
    kernels.check_status(DEV)
    close(out[0], expected, out_dtype, f"{m}x{n}x{k}")


@pytest.mark.parametrize("m, n, k, splits", [(300, 384, 1024, 2), (512, 4096, 4096, 2), (700, 1000, 3000, 4), (513, 257, 200, 3),
                                             (1100, 5000, 640, 3)])   # the last: more work items than resident pairs
def test_gemm_block_pairs_split_k(m, n, k, splits):
    """Work items of the pair kernel that are (tile, K range): each range's sums land in a float plane of their own,
    a last range shorter than the others included."""
    a, w = rand(m, k, seed=119, dtype=torch.bfloat16), rand(n, k, seed=120, scale=0.1, dtype=torch.bfloat16)
    splits = kernels.tc_normalise_splits(k, splits)
    assert splits > 1
    out = torch.full((splits, m, n), float("nan"), dtype=torch.float32, device=DEV)
    kernels.gemm_tc_pair(a, w, GemmOut(out))
    kernels.check_status(DEV)
    close(GemmOut(out).value(), a.double() @ w.double().T, torch.float32, f"{m}x{n}x{k} splits={splits}")
    per = -(-(-(-k // 64)) // splits) * 64
    close(out[0], a[:, :per].double() @ w[:, :per].double().T, torch.float32, "first K range")
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tc_pair(a, w, GemmOut(torch.empty(splits, m, n, dtype=torch.bfloat16, device=DEV)))


@pytest.mark.parametrize("m, inter, k", [(300, 48, 72), (1000, 560, 1024), (2048, 1536, 256), (513, 4096 + 16, 64)])
def test_gemm_block_pairs_with_the_silu_gate_in_the_epilogue(m, inter, k):
    """gate and up rows interleaved in groups of 16: the pair kernel stores silu(x G^T) * (x U^T)."""
    a = rand(m, k, seed=116, dtype=torch.bfloat16)
    gate, up = rand(inter, k, seed=117, scale=0.1, dtype=torch.bfloat16), rand(inter, k, seed=118, scale=0.1, dtype=torch.bfloat16)
    w = kernels.interleave_gate_up(gate, up, kernels.SWIGLU_GROUP).contiguous()
    assert torch.equal(w[:16], gate[:16]) and torch.equal(w[16:32], up[:16]) and torch.equal(w[32:48], gate[16:32])
    out = torch.full((1, m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc_pair(a, w, GemmOut(out), swiglu=True)
    kernels.check_status(DEV)
    expected = torch.nn.functional.silu(a.double() @ gate.double().T) * (a.double() @ up.double().T)
    close(out[0], expected, torch.bfloat16, f"{m} tokens, {inter} features, K={k}")
    kernels.gemm_tc_pair(a, w, GemmOut(out), swiglu=True, activation="gelu_tanh")
    close(out[0], gate_act("gelu_tanh", a.double() @ gate.double().T) * (a.double() @ up.double().T), torch.bfloat16, "gelu_tanh")
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tc_pair(a, w[:-8], GemmOut(out[:, :, :-4].contiguous()), swiglu=True)


@pytest.mark.parametrize("m, n, k, out_dtype, swiglu", [
    (300, 384, 2048, torch.bfloat16, False),       # 4 tiles over all pairs: a tile finished from many pairs' slots
    (2048, 4096, 4096, torch.bfloat16, False),     # 128 tiles: one whole wave, then 54 tiles by K ranges
    (1000, 1100, 4096, torch.float32, False),      # ragged edges in both directions
    (777, 5000, 1024, torch.bfloat16, False),      # 80 tiles: six of them over all pairs, a K block or two each
    (2048, 3072, 256, torch.bfloat16, True),       # the gated epilogue after the sums
    (4096, 24576, 448, torch.bfloat16, False)])    # many waves before the last
def test_gemm_block_pairs_last_wave_by_k_ranges(m, n, k, out_dtype, swiglu):
    """The pair kernel with the tiles of its last wave cut by K ranges (forced wherever the tiles do not divide by the
    pairs): pairs that do not finish a tile leave float sums in their slot, the finishing pair adds them.  Run
    twice: the flags that guard the slots must be down again after every launch."""
    a, w = rand(m, k, seed=121, dtype=torch.bfloat16), rand(n, k, seed=122, scale=0.1, dtype=torch.bfloat16)
    full = a.double() @ w.double().T
    if swiglu:
        gate, up = w[: n // 2], w[n // 2:]
        expected = torch.nn.functional.silu(a.double() @ gate.double().T) * (a.double() @ up.double().T)
        w = kernels.interleave_gate_up(gate, up, kernels.SWIGLU_GROUP).contiguous()
    else:
        expected = full
    slots, flags, pairs = kernels._pair_tail(a.device)
    tiles = -(-m // 256) * -(-n // 256)
    assert tiles % (kernels.sm_count(a.device) // 2) != 0, "this shape has no partly filled wave on this device"
    for attempt in range(2):
        slots.fill_(float("nan"))
        out = torch.full((1, m, expected.shape[1]), float("nan"), dtype=out_dtype, device=DEV)
        kernels.gemm_tc_pair(a, w, GemmOut(out), swiglu=swiglu, tail=1)
        kernels.check_status(DEV)
        close(out[0], expected, out_dtype, f"{m}x{n}x{k} attempt {attempt}")
        assert int(flags.abs().sum()) == 0
        assert not bool(torch.isnan(slots).all()), "no pair wrote a slot: the last wave was not cut"
    out = torch.full((1, m, expected.shape[1]), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_tc_pair(a, w, GemmOut(out), swiglu=swiglu, tail=0)       # and the same product with every tile whole
    close(out[0], expected, out_dtype, "whole tiles")


@pytest.mark.parametrize("m, inter, k", [(64, 1552, 256), (100, 560, 1024), (5, 48, 72), (33, 4096, 64), (200, 304, 448)])
def test_gemm_tensor_cores_with_the_gate_in_the_epilogue(m, inter, k):
    """The single-block product with gate and up rows interleaved in groups of 16: it stores act(x G^T) * (x U^T)."""
    a = rand(m, k, seed=160, dtype=torch.bfloat16)
    gate, up = rand(inter, k, seed=161, scale=0.1, dtype=torch.bfloat16), rand(inter, k, seed=162, scale=0.1, dtype=torch.bfloat16)
    w = kernels.interleave_gate_up(gate, up, kernels.SWIGLU_GROUP).contiguous()
    out = torch.full((1, m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(a, w, GemmOut(out), swiglu=True)
    kernels.check_status(DEV)
    g, u = a.double() @ gate.double().T, a.double() @ up.double().T
    close(out[0], torch.nn.functional.silu(g) * u, torch.bfloat16, f"{m} tokens, {inter} features, K={k}")
    kernels.gemm_tc(a, w, GemmOut(out), swiglu=True, activation="relu")
    close(out[0], torch.relu(g) * u, torch.bfloat16, "relu")
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tc(a, w, GemmOut(torch.empty(2, m, inter, dtype=torch.float32, device=DEV)), swiglu=True)


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_gemm_tensor_cores_every_token_tile(tile):
    m, n, k = 70, 384, 448
    a, w = rand(m, k, seed=112, dtype=torch.bfloat16), rand(n, k, seed=113, scale=0.1, dtype=torch.bfloat16)
    for stages in (0, 3):           # the default ring depth for the tile, and a forced one
        out = torch.full((1, m, n), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemm_tc(a, w, GemmOut(out), token_tile=tile, stages=stages)
        kernels.check_status(DEV)
        close(out[0], a.double() @ w.double().T, torch.float32, f"token tile {tile}, stages {stages}")


def test_gemm_dispatch_is_static():
    a = rand(4, 100, seed=114, dtype=torch.bfloat16)          # K = 100: rows do not start on 16-byte boundaries
    w = rand(9, 100, seed=115, dtype=torch.bfloat16)
    assert not kernels.gemm_tc_supported(a, w)
    out = torch.empty(1, 4, 9, dtype=torch.bfloat16, device=DEV)
    kernels.gemm(a, w, GemmOut(out))                           # goes to the FMA kernel
    close(out[0], a.double() @ w.double().T, torch.bfloat16, "unaligned K")
    with pytest.raises(kernels.KernelError, match="multiple of 8"):
        kernels.gemm_tc(a, w, GemmOut(out))
    assert kernels.tc_normalise_splits(320, 4) == 3 and kernels.tc_normalise_splits(4096, 3) == 3
    assert kernels.tc_normalise_splits(64, 8) == 1
