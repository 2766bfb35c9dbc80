"""y = x W^T for a weight kept as [out_features, in_features] (qwen_triton/modules/linear.py:11-34).

The weight stays in the layout the checkpoint stores, which is the K-major operand the kernels
read; nothing is transposed per call (the reference re-materialises W^T every call,
qwen_triton/kernels/matmul.py:140).
"""
from __future__ import annotations

import os

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut, ScaledRows
from .base import Runtime


_MAX_SPLITS = 16
# Ring depths of the fused product that are tried in turn, deepest first (see Linear._fused_stages), and the blocks of
# the 16-token tile that share an SM at each depth (18 KB a stage).
_FUSED_STAGES = {"qkv": (4,), "attn_out": (4,), "gate": (4,), "mlp_out": (5, 4)}
_FUSED_BLOCKS_PER_SM = {3: 4, 4: 3, 5: 2}
# Most rows that take the fused product.  What a fused launch adds to the plain product is its tail (park, cluster
# barrier, the peers' sums); it grows with the rows, and beyond 16 it costs more than the small kernels it replaces
# (8B shapes, 64 rows, replayed alone: q/k/v 15.8 us fused against 10.4 + 2.7 us, down 23.0 against 19.9 + 3.5 us).
_FUSED_ROWS = int(os.environ.get("QT_B200_FUSED_ROWS", "16"))
# (most rows, blocks wanted in flight) for products bound by reading the weight.  Up to 16 rows the kernel's ring is
# three stages deep and four blocks share an SM, which also lets the next product's blocks move in and fetch their
# first weight tiles while this one drains; up to 64 rows two blocks with deeper rings measured better.  Up to 256
# rows (a large decode batch, a short prompt) the weight still bounds the product: blocks of 128 tokens, split
# (alone, 256 rows of the 8B shapes: 16.6 us against 54 us for q/k/v, 32 against 158 us for the down projection).
_SPLIT_PLANS = ((16, 4), (64, 2), (128, 2), (256, 2))      # (most rows, blocks per SM)


def pick_splits(out_features: int, in_features: int, target_blocks: int, rows: int = 16, most: int = _MAX_SPLITS,
                partial_cost: float = 2.0, sms: int = 0) -> int:
    """Split count for a product with few rows, by a cost in bytes: the weight, read at the rate its blocks
    (128-row weight tiles x token tiles of at most 128 x splits) keep ``target_blocks`` slots busy (a second token
    tile reads it again, from L2), plus the float partial sums of ``rows`` rows, written once and read once.  Each
    split keeps at least four 64-wide K blocks (two in the fused product, whose sums never leave the chip: the 0.6B
    shape at batch 8, 1.18 ms a step against 1.21); fewer splits win near-ties.
    (Filling waves alone would cut a product that already has blocks for several waves into many splits, whose
    partial sums then cost more than the weight: 14 splits for a 51,200 x 5,120 weight at 64 rows.)
    ``partial_cost`` is 2 for partial sums written to and read from global memory, 1 for the fused product, whose
    blocks (at most ``most`` = 8 of a cluster) park them in shared memory and read each other's.
    A weight whose tiles alone give every one of the ``sms`` SMs a block is not cut beyond the ``target_blocks`` that
    are resident at once: its blocks already draw what the memory gives, and a second wave of them only adds a ramp
    and partial sums (the gated product of the 8B shape at 64 rows, alone: 39.1 us unsplit, 43.1 / 41.2 us in two /
    three ranges; in the model at batch 48 / 64 / 96 / 128: 3 % shorter steps; the 32B shape's gated product, 400
    tiles, at batch 8: 16 layers and the head in 3.22 ms against 3.53 ms with eight ranges)."""
    token_tiles = -(-rows // kernels.TC_MAX_BLOCK_TOKENS)
    tiles = -(-out_features // 128) * token_tiles
    blocks_k = -(-in_features // 64)
    weight_bytes = 2.0 * out_features * in_features * (1.0 + 0.3 * (token_tiles - 1))
    best, best_cost = 1, float("inf")
    clustered = most <= kernels.FUSED_MAX_SPLITS         # the fused product: the K ranges of a tile are a thread-block cluster
    for splits in range(1, most + 1):
        if splits > 1 and blocks_k // splits < (2 if clustered else 4):
            break
        if kernels.tc_normalise_splits(in_features, splits) != splits:
            continue
        if clustered and splits == 7:
            continue            # clusters of seven pack the SMs of a GPC worst (32B q/k/v at batch 8: 3.23 ms a step
                                # against 3.15 with 4, 5, 6 or 8)
        if splits > 1 and sms and tiles >= sms and tiles * splits > target_blocks:
            break
        waves = tiles * splits / target_blocks
        fill = waves if waves <= 1.0 else waves / (waves + 0.35)     # under one wave: idle slots; over: a tail of about a third of a wave
        partial_bytes = partial_cost * 4 * splits * rows * out_features if splits > 1 else 0.0
        cost = weight_bytes / fill + partial_bytes
        if cost < best_cost * 0.99:
            best, best_cost = splits, cost
    return best


_PAIR_TILE = 256                       # weight rows and tokens of one pair tile


def pick_pair_splits(out_features: int, in_features: int, rows: int, pairs: int) -> int:
    """Split count for a product of a few hundred rows by the pair kernel, whose 256 x 256 tiles alone leave TPCs
    idle or end in a nearly empty wave: waves of work items (tiles x splits over ``pairs`` resident pairs, one per
    TPC) times the time of one item at the pair's share of the tensor throughput plus a fixed cost per item, plus
    the float partial sums written and read once (they stay in L2); the constants are fitted to products of 300 to
    768 rows timed alone.  Every split keeps at least eight 64-wide K blocks; fewer splits win near-ties."""
    tiles = -(-out_features // _PAIR_TILE) * -(-rows // _PAIR_TILE)
    blocks_k = -(-in_features // 64)
    pair_flops, first_overhead, later_overhead, partial_rate = 1.45e15 / pairs, 2e-6, 0.5e-6, 2e13
    best, best_cost = 1, float("inf")
    for splits in range(1, 5):
        if splits > 1 and blocks_k // splits < 8:
            break
        if kernels.tc_normalise_splits(in_features, splits) != splits:
            continue
        item = 2.0 * _PAIR_TILE * _PAIR_TILE * in_features / splits / pair_flops
        waves = -(-tiles * splits // pairs)                   # a pair's later items start under the epilogue of the one before
        partial = 2.0 * 4 * splits * rows * out_features / partial_rate if splits > 1 else 0.0
        cost = waves * item + first_overhead + (waves - 1) * later_overhead + partial
        if cost < best_cost * 0.97:
            best, best_cost = splits, cost
    return best


class Linear:
    def __init__(self, key: str, out_features: int, in_features: int, runtime: Runtime, max_rows: int | None = None,
                 float_out: bool = False, role: str = "", bias: bool = False) -> None:
        self.key = key
        self.role = role                   # which of the fused products of a decode step this one is, if any
        self.out_features = out_features
        self.in_features = in_features
        self.runtime = runtime
        # a bias is added to the float sums (the first plane of a product split over K), so such a product stays float
        # up to its consumer, and it keeps to the plain kernels: the fused products have no bias operand
        self.has_bias = bias
        float_out = float_out or bias
        self.float_out = float_out
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.max_rows = runtime.max_step_tokens if max_rows is None else max_rows
        self.out_dtype = torch.float32 if float_out else runtime.dtype
        runtime.workspace.declare(f"{key}.out", self.max_rows * out_features, self.out_dtype)
        # few rows (decode): split K over more blocks so that every SM streams weights; partial sums are float
        sms = runtime.sm_count
        pairs = max(1, sms // 2)               # pairs of blocks the pair kernel keeps resident (one per TPC)
        self.split_plans: list[tuple[int, int]] = []          # (most rows, splits), fewest rows first
        self.fused_plans: list[tuple[int, int]] = []          # the same for the fused product (its blocks add up in shared memory)
        if runtime.dtype == torch.bfloat16 and in_features % 8 == 0:
            self.split_plans = [(rows, pick_splits(out_features, in_features, per_sm * sms, rows, sms=sms)) for rows, per_sm in _SPLIT_PLANS]
            self.fused_plans = [(rows, pick_splits(out_features, in_features, (3 if role == "gate" else per_sm) * sms, rows,
                                                   kernels.FUSED_MAX_SPLITS, 1.0, sms=sms))
                                for rows, per_sm in _SPLIT_PLANS if rows <= kernels.FUSED_MAX_ROWS]
            # a few hundred rows: the pair kernel with split K where its tiles alone would not fill the TPCs
            if not float_out and self.max_rows > _PAIR_TILE:
                for tiles_x in range(2, -(-self.max_rows // _PAIR_TILE) + 1):
                    rows = min(tiles_x * _PAIR_TILE, self.max_rows)
                    if rows > self.split_plans[-1][0]:
                        self.split_plans.append((rows, pick_pair_splits(out_features, in_features, rows, pairs)))
                    if -(-out_features // _PAIR_TILE) * tiles_x >= 4 * pairs:      # several waves of tiles: no split pays
                        break
        words = max((rows * splits for rows, splits in self.split_plans if splits > 1), default=0)
        if words:
            runtime.workspace.declare(f"{key}.partial", words * out_features, torch.float32)
        if self.fused_plans and not float_out:
            runtime.workspace.declare(f"{key}.wide", min(self.max_rows, kernels.FUSED_MAX_ROWS) * out_features, torch.float32)

    def set_weight(self, weight: torch.Tensor) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"{self.key}: weight {tuple(weight.shape)} is not [{self.out_features}, {self.in_features}]")
        self.weight = weight.to(device=self.runtime.device, dtype=self.runtime.dtype).contiguous()

    def set_bias(self, bias: torch.Tensor) -> None:
        if not self.has_bias or tuple(bias.shape) != (self.out_features,):
            raise ValueError(f"{self.key}: bias {tuple(bias.shape)} for a projection "
                             f"{'of ' + str(self.out_features) + ' features' if self.has_bias else 'built without bias'}")
        self.bias = bias.to(device=self.runtime.device, dtype=torch.float32).contiguous()

    # ------------------------------------------------------------------ the fused product of a decode step
    @property
    def fused_capable(self) -> bool:
        """Whether this product has a fused form at all (known before the weight is loaded)."""
        return bool(self.fused_plans) and bool(self.role) and kernels.fused_enabled(self.role) and not self.has_bias

    def fusable(self, rows: int) -> bool:
        """Whether ``rows`` tokens take the fused product (a static choice: element type, sizes, row count), in which
        what follows the product (residual add and norm preparation, SiLU gate, q/k-norm + rotation + cache write)
        runs in its epilogue.  ``QT_B200_FUSED=0`` in the environment turns it off."""
        return self.fused_capable and 0 < rows <= _FUSED_ROWS and self.weight is not None \
            and kernels.fused_supported(self.weight)

    def _fused_splits(self, rows: int) -> int:
        return next(n for most, n in self.fused_plans if rows <= most)

    def _fused_stages(self, rows: int) -> int:
        """Depth of the fused product's ring (0: the kernel's default of three stages, four blocks per SM): the deepest of
        this product's candidates at which all its blocks are still resident at once.  Timed in the model (8B shape,
        batch 8, 36 layers): 3.55 ms a step with three stages for q/k/v, o and down, 3.43 ms with four for each (three
        blocks per SM), 3.41 ms with five for down (whose K is the longest); two stages or five for q/k/v are slower
        (3.56, 3.58 ms).  Where the deeper ring would push blocks into a second wave it costs more than it brings (32B
        shape, 16 layers at batch 8: 3.35 ms with four stages for the 480 blocks of q/k/v against 3.13 ms with three).
        The gated product has blocks for every slot of the machine at two or three splits; with four stages three of
        them share an SM and the next product's blocks find room beside them (alone, 8 rows: 33.4 us against 39.6 us
        with three; five or six in the model: 3.72 ms)."""
        blocks = -(-self.out_features // 128) * self._fused_splits(rows)
        for stages in _FUSED_STAGES.get(self.role, ()):
            if self.role == "gate" or blocks <= _FUSED_BLOCKS_PER_SM[stages] * self.runtime.sm_count:
                return stages
        return 0

    def into_residual(self, x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor | None = None, eps: float = 0.0,
                      xw: torch.Tensor | None = None, sq: torch.Tensor | None = None) -> "ScaledRows | None":
        """residual += x W^T, and the norm behind it prepared (see ``kernels.gemm_fused_residual``)."""
        return kernels.gemm_fused_residual(x, self.weight, residual, norm_weight, eps, xw, sq, splits=self._fused_splits(x.shape[0]), stages=self._fused_stages(x.shape[0]))

    def into_swiglu(self, x, out: torch.Tensor, activation: str = "silu") -> None:
        kernels.gemm_fused_swiglu(x, self.weight, out, splits=self._fused_splits(x.shape[0]), stages=self._fused_stages(x.shape[0]),
                                  activation=activation)

    def into_qkv(self, x, *args, **kwargs) -> None:
        kernels.gemm_fused_qkv(x, self.weight, *args, splits=self._fused_splits(x.shape[0]), stages=self._fused_stages(x.shape[0]), **kwargs)

    def plan_splits(self, rows: int) -> int:
        """The number of K ranges that ``rows`` tokens are cut into by the plain products."""
        return next((n for most, n in self.split_plans if rows <= most), 1)

    def __call__(self, x, out: torch.Tensor | None = None) -> GemmOut:
        rows = x.shape[0]
        if isinstance(x, ScaledRows):
            # rows whose norm factor is still to be applied: the fused product's plain store applies it
            if out is None:
                out = self.runtime.workspace.view(f"{self.key}.wide", rows, self.out_features)
            kernels.gemm_fused_store(x, self.weight, out.view(rows, self.out_features), splits=self._fused_splits(rows))
            return GemmOut(out.view(1, rows, self.out_features))
        splits = self.plan_splits(rows)
        if out is None and splits > 1:
            result = GemmOut(self.runtime.workspace.view(f"{self.key}.partial", splits, rows, self.out_features))
        elif out is None:
            result = GemmOut(self.runtime.workspace.view(f"{self.key}.out", 1, rows, self.out_features))
        else:
            result = GemmOut(out.view(1, rows, self.out_features))
        kernels.gemm(x, self.weight, result)
        if self.has_bias and rows:
            if self.bias is None:
                raise ValueError(f"{self.key}: the bias was not loaded")
            kernels.add_bias(result.tensor[0], self.bias)
        return result
