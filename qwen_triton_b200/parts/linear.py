"""y = x W^T for a weight kept as [out_features, in_features] (qwen_triton/modules/linear.py:11-34).

The weight stays in the layout the checkpoint stores, which is the K-major operand the kernels
read; nothing is transposed per call (the reference re-materialises W^T every call,
qwen_triton/kernels/matmul.py:140).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from .base import Runtime


_SM_COUNT = 148
_MAX_SPLITS = 16
# (most rows, blocks wanted in flight) for products bound by reading the weight.  Up to 16 rows the kernel's ring is
# three stages deep and four blocks share an SM, which also lets the next product's blocks move in and fetch their
# first weight tiles while this one drains; up to 64 rows two blocks with deeper rings measured better.  Up to 256
# rows (a large decode batch, a short prompt) the weight still bounds the product: blocks of 128 tokens, split
# (alone, 256 rows of the 8B shapes: 16.6 us against 54 us for q/k/v, 32 against 158 us for the down projection).
_SPLIT_PLANS = ((16, 4 * _SM_COUNT), (64, 2 * _SM_COUNT), (128, 2 * _SM_COUNT), (256, 2 * _SM_COUNT))


def pick_splits(out_features: int, in_features: int, target_blocks: int = 2 * _SM_COUNT, rows: int = 16) -> int:
    """Split count for a product with few rows, by a cost in bytes: the weight, read at the rate its blocks
    (128-row weight tiles x token tiles of at most 128 x splits) keep ``target_blocks`` slots busy (a second token
    tile reads it again, from L2), plus the float partial sums of ``rows`` rows, written once and read once.  Each split keeps at least four 64-wide K blocks; fewer splits win near-ties.
    (Filling waves alone would cut a product that already has blocks for several waves into many splits, whose
    partial sums then cost more than the weight: 14 splits for a 51,200 x 5,120 weight at 64 rows.)"""
    token_tiles = -(-rows // kernels.TC_MAX_BLOCK_TOKENS)
    tiles = -(-out_features // 128) * token_tiles
    blocks_k = -(-in_features // 64)
    weight_bytes = 2.0 * out_features * in_features * (1.0 + 0.3 * (token_tiles - 1))
    best, best_cost = 1, float("inf")
    for splits in range(1, _MAX_SPLITS + 1):
        if splits > 1 and blocks_k // splits < 4:
            break
        if kernels.tc_normalise_splits(in_features, splits) != splits:
            continue
        waves = tiles * splits / target_blocks
        fill = waves if waves <= 1.0 else waves / (waves + 0.35)     # under one wave: idle slots; over: a tail of about a third of a wave
        partial_bytes = 2.0 * 4 * splits * rows * out_features if splits > 1 else 0.0
        cost = weight_bytes / fill + partial_bytes
        if cost < best_cost * 0.99:
            best, best_cost = splits, cost
    return best


_PAIRS = _SM_COUNT // 2                # pairs of blocks the pair kernel keeps resident (one per TPC)
_PAIR_TILE = 256                       # weight rows and tokens of one pair tile


def pick_pair_splits(out_features: int, in_features: int, rows: int) -> int:
    """Split count for a product of a few hundred rows by the pair kernel, whose 256 x 256 tiles alone leave TPCs
    idle or end in a nearly empty wave: waves of work items (tiles x splits over 74 pairs) times the time of one item at the pair's share of the
    tensor throughput plus a fixed cost per item, plus the float partial sums written and read once (they stay
    in L2); the constants are fitted to products of 300 to 768 rows timed alone.  Every split keeps at least eight 64-wide K blocks; fewer splits win near-ties."""
    tiles = -(-out_features // _PAIR_TILE) * -(-rows // _PAIR_TILE)
    blocks_k = -(-in_features // 64)
    pair_flops, first_overhead, later_overhead, partial_rate = 1.45e15 / _PAIRS, 2e-6, 0.5e-6, 2e13
    best, best_cost = 1, float("inf")
    for splits in range(1, 5):
        if splits > 1 and blocks_k // splits < 8:
            break
        if kernels.tc_normalise_splits(in_features, splits) != splits:
            continue
        item = 2.0 * _PAIR_TILE * _PAIR_TILE * in_features / splits / pair_flops
        waves = -(-tiles * splits // _PAIRS)                  # a pair's later items start under the epilogue of the one before
        partial = 2.0 * 4 * splits * rows * out_features / partial_rate if splits > 1 else 0.0
        cost = waves * item + first_overhead + (waves - 1) * later_overhead + partial
        if cost < best_cost * 0.97:
            best, best_cost = splits, cost
    return best


class Linear:
    def __init__(self, key: str, out_features: int, in_features: int, runtime: Runtime, max_rows: int | None = None,
                 float_out: bool = False) -> None:
        self.key = key
        self.out_features = out_features
        self.in_features = in_features
        self.runtime = runtime
        self.float_out = float_out
        self.weight: torch.Tensor | None = None
        self.max_rows = runtime.max_step_tokens if max_rows is None else max_rows
        self.out_dtype = torch.float32 if float_out else runtime.dtype
        runtime.workspace.declare(f"{key}.out", self.max_rows * out_features, self.out_dtype)
        # few rows (decode): split K over more blocks so that every SM streams weights; partial sums are float
        self.split_plans: list[tuple[int, int]] = []          # (most rows, splits), fewest rows first
        if runtime.dtype == torch.bfloat16 and in_features % 8 == 0:
            self.split_plans = [(rows, pick_splits(out_features, in_features, target, rows)) for rows, target in _SPLIT_PLANS]
            # a few hundred rows: the pair kernel with split K where its tiles alone would not fill the TPCs
            if not float_out and self.max_rows > _PAIR_TILE:
                for tiles_x in range(2, -(-self.max_rows // _PAIR_TILE) + 1):
                    rows = min(tiles_x * _PAIR_TILE, self.max_rows)
                    if rows > self.split_plans[-1][0]:
                        self.split_plans.append((rows, pick_pair_splits(out_features, in_features, rows)))
                    if -(-out_features // _PAIR_TILE) * tiles_x >= 4 * _PAIRS:      # several waves of tiles: no split pays
                        break
        words = max((rows * splits for rows, splits in self.split_plans if splits > 1), default=0)
        if words:
            runtime.workspace.declare(f"{key}.partial", words * out_features, torch.float32)

    def set_weight(self, weight: torch.Tensor) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"{self.key}: weight {tuple(weight.shape)} is not [{self.out_features}, {self.in_features}]")
        self.weight = weight.to(device=self.runtime.device, dtype=self.runtime.dtype).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None) -> GemmOut:
        rows = x.shape[0]
        splits = next((n for most, n in self.split_plans if rows <= most), 1)
        if out is None and splits > 1:
            partial = self.runtime.workspace.view(f"{self.key}.partial", splits, rows, self.out_features)
            result = GemmOut(partial)
            kernels.gemm(x, self.weight, result)
            return result
        if out is None:
            out = self.runtime.workspace.view(f"{self.key}.out", 1, rows, self.out_features)
        else:
            out = out.view(1, rows, self.out_features)
        result = GemmOut(out)
        kernels.gemm(x, self.weight, result)
        return result
