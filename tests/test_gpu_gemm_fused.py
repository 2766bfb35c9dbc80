"""The fused product of a decode step (csrc/gemm_fused.cu) alone: every epilogue against a plain float statement of
the product followed by the op it absorbs, at sizes other than the engine's: widths that are no multiple of the
128-row tile, every token tile, every cluster size, a deferred norm factor, partial rotation, a ring cache."""
import pytest
import torch

import plain_qwen3 as plain
from qwen_triton_b200.ops import kernels
from qwen_triton_b200.ops.kernels import ScaledRows
from test_gpu_kernels import DEV, PAGE, close, gate_act, paged, rand, rope_interleaved

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def product(x, w):
    return x.float().cpu() @ w.float().cpu().T


def scaled_rows(rows, k, seed, eps=2e-5):
    """A stream r, a norm weight g, and what a producer would hand on: bf16(r g) with per-tile sums of squares."""
    r = rand(rows, k, seed=seed, scale=1.5)
    g = 1.0 + rand(k, seed=seed + 1, scale=0.2)
    tiles = -(-k // 128)
    sq = torch.stack([r[:, i * 128:(i + 1) * 128].pow(2).sum(-1) for i in range(tiles)])
    handed = ScaledRows((r * g).to(BF16), sq.contiguous(), k, eps)
    factor = torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps).cpu()
    return handed, factor


@pytest.mark.parametrize("rows, n, k, splits", [(1, 503, 96, 1), (8, 4096, 1024, 4), (16, 130, 512, 8), (17, 640, 2048, 3),
                                                (64, 384, 1000, 2), (65, 256, 4096, 8), (128, 1000, 264, 1), (5, 128, 64, 1)])
@pytest.mark.parametrize("out_dtype", [torch.float32, BF16])
def test_store(rows, n, k, splits, out_dtype):
    x, w = rand(rows, k, seed=1, dtype=BF16), rand(n, k, seed=2, scale=0.05, dtype=BF16)
    out = torch.full((rows, n), float("nan"), dtype=out_dtype, device=DEV)
    kernels.gemm_fused_store(x, w, out, splits)
    kernels.check_status(DEV)
    close(out, product(x, w), BF16, "plain product")
    handed, factor = scaled_rows(rows, k, seed=3)
    kernels.gemm_fused_store(handed, w, out, splits)
    close(out, product(handed.tensor, w) * factor, BF16, "with the deferred norm factor")


@pytest.mark.parametrize("rows, n, k, splits", [(1, 96, 160, 1), (8, 4096, 12288, 8), (16, 136, 512, 4), (33, 1024, 3072, 5),
                                                (128, 320, 256, 2)])
def test_residual_add_and_norm_preparation(rows, n, k, splits):
    x, w = rand(rows, k, seed=4, dtype=BF16), rand(n, k, seed=5, scale=0.05, dtype=BF16)
    stream = rand(rows, n, seed=6)
    expected = stream.cpu() + product(x, w)
    # the sum alone
    residual = stream.clone()
    assert kernels.gemm_fused_residual(x, w, residual, splits=splits) is None
    torch.testing.assert_close(residual.cpu(), expected, atol=2e-3, rtol=2e-3)          # float sums of bfloat16 products
    # with the next norm prepared
    residual = stream.clone()
    g = 1.0 + rand(n, seed=7, scale=0.2)
    xw = torch.full((rows, n), float("nan"), dtype=BF16, device=DEV)
    sq = torch.full((-(-n // 128), rows), float("nan"), device=DEV)
    handed = kernels.gemm_fused_residual(x, w, residual, g, 3e-6, xw, sq, splits=splits)
    kernels.check_status(DEV)
    torch.testing.assert_close(residual.cpu(), expected, atol=2e-3, rtol=2e-3)
    close(handed.tensor, residual.cpu() * g.cpu(), BF16, "weighted stream")
    torch.testing.assert_close(handed.sq.sum(0).cpu(), residual.pow(2).sum(-1).cpu(), atol=1e-3, rtol=1e-4)
    assert handed.width == n and handed.eps == 3e-6
    # handed to the next product, the pair equals norm-then-product
    w2 = rand(200, n, seed=8, scale=0.05, dtype=BF16)
    out = torch.empty(rows, 200, device=DEV)
    kernels.gemm_fused_store(handed, w2, out, 1)
    normed = plain.rms_norm(residual.cpu(), g.cpu(), 3e-6)
    close(out, normed @ w2.float().cpu().T, BF16, "norm then product")


@pytest.mark.parametrize("rows, inter, k, splits", [(1, 48, 72, 1), (8, 12288 // 4, 1024, 3), (16, 560, 512, 2), (40, 64, 4096, 8),
                                                    (128, 176, 128, 1)])
def test_silu_gate(rows, inter, k, splits):
    gate, up = rand(inter, k, seed=9, scale=0.1, dtype=BF16), rand(inter, k, seed=10, scale=0.1, dtype=BF16)
    w = kernels.interleave_gate_up(gate, up, kernels.SWIGLU_GROUP)
    handed, factor = scaled_rows(rows, k, seed=11)
    out = torch.full((rows, inter), float("nan"), dtype=BF16, device=DEV)
    kernels.gemm_fused_swiglu(handed, w, out, splits)
    kernels.check_status(DEV)
    g, u = product(handed.tensor, gate) * factor, product(handed.tensor, up) * factor
    close(out, g * torch.sigmoid(g) * u, BF16, "silu(gate) * up")
    for name in ("gelu", "relu"):
        kernels.gemm_fused_swiglu(handed, w, out, splits, activation=name)
        close(out, gate_act(name, g) * u, BF16, f"{name}(gate) * up")


@pytest.mark.parametrize("nq, nkv, d, rotary, ring, splits, lengths, own_kv", [
    (8, 2, 16, 16, 128, 2, [1, 1, 1], True), (5, 1, 128, 128, 0, 4, [1, 1, 1], True), (3, 3, 64, 32, 0, 1, [20, 3, 41], True),
    (6, 2, 32, 24, 0, 8, [1, 1, 1], True), (4, 2, 128, 0, 0, 2, [1, 1, 1], True), (7, 1, 64, 64, 0, 3, [1, 1, 1], False)])
@pytest.mark.parametrize("interleaved", [False, True])
def test_qkv_with_norm_rotation_and_cache_write(nq, nkv, d, rotary, ring, splits, lengths, own_kv, interleaved):
    past = [130, 0, 20]
    tokens, k, eps = sum(lengths), 512, 1e-5
    n = (nq + (2 * nkv if own_kv else 0)) * d
    w = rand(n, k, seed=12, scale=0.08, dtype=BF16)
    handed, factor = scaled_rows(tokens, k, seed=13)
    qw, kw = 1.0 + rand(d, seed=14, scale=0.2), 1.0 + rand(d, seed=15, scale=0.2)
    max_pos = 400
    cos_sin = None
    if rotary:
        cos, sin = plain.rope_tables(torch.arange(max_pos), rotary, 50000.0, torch.float32)
        cos_sin = torch.cat((cos, sin), dim=-1).contiguous().to(DEV)
    token_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(lengths)).int().to(DEV)
    token_pos = torch.cat([torch.arange(p, p + m) for p, m in zip(past, lengths)]).int().to(DEV)
    totals = [p + m for p, m in zip(past, lengths)]
    zeros = [torch.zeros(t, nkv, d) for t in totals]
    k_cache, v_cache, table = paged(zeros, zeros, totals, BF16, ring_tokens=ring, seed=16, garbage=False)
    q_out = torch.full((tokens, nq, d), float("nan"), dtype=BF16, device=DEV)
    kernels.gemm_fused_qkv(handed, w, q_out, k_cache, v_cache, token_seq, token_pos, table, qw, kw, eps, cos_sin, nq, nkv, d,
                           PAGE, ring, write_kv=own_kv, splits=splits, interleaved=interleaved)
    kernels.check_status(DEV)
    x = (product(handed.tensor, w) * factor).view(tokens, -1, d)
    pos = token_pos.cpu().long()

    def rotated(heads, weight):
        normed = plain.rms_norm(heads, weight.cpu(), eps)
        if not rotary:
            return normed
        return rope_interleaved(normed, cos[pos], sin[pos]) if interleaved else plain.apply_rope(normed, cos[pos], sin[pos])

    close(q_out, rotated(x[:, :nq], qw), BF16, "q")
    if not own_kv:
        assert float(k_cache.float().abs().max()) == 0.0
        return
    k_ref, v_ref = rotated(x[:, nq:nq + nkv], kw), x[:, nq + nkv:]
    table_host, k_host, v_host = table.cpu(), k_cache.float().cpu(), v_cache.float().cpu()
    for t in range(tokens):
        b, p = int(token_seq[t]), int(pos[t])
        if ring and p < totals[b] - ring:
            continue
        idx = p % ring if ring else p
        page = int(table_host[b, idx // PAGE])
        close(k_host[page, :, idx % PAGE], k_ref[t], BF16, f"k of token {t}")
        close(v_host[page, :, idx % PAGE], v_ref[t], BF16, f"v of token {t}")


def test_what_the_fused_product_refuses():
    x, w = rand(4, 64, seed=1, dtype=BF16), rand(256, 64, seed=2, dtype=BF16)
    out = torch.empty(4, 256, device=DEV)
    with pytest.raises(kernels.KernelError, match="rank without K blocks|splits"):
        kernels.gemm_fused_store(x, w, out, splits=2)                       # one K block cannot be shared
    with pytest.raises(kernels.KernelError, match="tokens"):
        kernels.gemm_fused_store(rand(129, 64, seed=1, dtype=BF16), w, torch.empty(129, 256, device=DEV), 1)
    with pytest.raises(kernels.KernelError, match="head_dim"):
        kernels.gemm_fused_qkv(x, rand(3 * 48, 64, seed=3, dtype=BF16), torch.empty(4, 1, 48, dtype=BF16, device=DEV), None, None,
                               torch.zeros(4, dtype=torch.int32, device=DEV), torch.zeros(4, dtype=torch.int32, device=DEV), None,
                               None, None, 1e-6, None, 1, 1, 48, PAGE, 0, write_kv=False)
