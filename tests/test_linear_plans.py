"""The split plans of ``Linear`` (host decisions, no device): every plan is one the kernels accept."""
import itertools

import pytest
import torch

from qwen_triton_b200.ops import kernels
from qwen_triton_b200.parts import linear


class _Workspace:
    def __init__(self):
        self.declared = {}

    def declare(self, name, numel, dtype):
        self.declared[name] = (numel, dtype)


class _Runtime:
    def __init__(self, dtype, max_step_tokens):
        self.dtype, self.max_step_tokens, self.workspace, self.device = dtype, max_step_tokens, _Workspace(), "cpu"
        self.sm_count = 148


SHAPES = [(6144, 4096), (4096, 12288), (24576, 4096), (151936, 4096), (1024, 2048), (130, 72), (5003, 1000), (200, 8), (51200, 5120)]


@pytest.mark.parametrize("out_features, in_features", SHAPES)
def test_every_split_count_leaves_no_split_without_k_blocks(out_features, in_features):
    for rows, per_sm in linear._SPLIT_PLANS:
        splits = linear.pick_splits(out_features, in_features, per_sm * 148, rows)
        assert 1 <= splits <= 16 and kernels.tc_normalise_splits(in_features, splits) == splits
        fused = linear.pick_splits(out_features, in_features, per_sm * 148, rows, kernels.FUSED_MAX_SPLITS, 1.0)
        assert 1 <= fused <= kernels.FUSED_MAX_SPLITS and kernels.tc_normalise_splits(in_features, fused) == fused
    for rows in (257, 300, 512, 1000, 2048, 4096):
        splits = linear.pick_pair_splits(out_features, in_features, rows, 74)
        assert 1 <= splits <= 4 and kernels.tc_normalise_splits(in_features, splits) == splits
        blocks = -(-in_features // 64)
        assert (splits - 1) * -(-blocks // splits) < blocks


def test_a_weight_whose_tiles_fill_the_machine_is_not_cut_into_a_second_wave():
    """192 tiles of the 8B shape's gate/up weight: three ranges up to 16 rows (576 blocks of 592 resident), none beyond
    (two blocks per SM: 384 blocks would be a second wave); the fused form (three blocks per SM for this product)
    keeps two ranges there and gives the 32B shape's 400 tiles none."""
    assert [linear.pick_splits(24576, 4096, per_sm * 148, rows, sms=148) for rows, per_sm in linear._SPLIT_PLANS] == [3, 1, 1, 1]
    assert linear.pick_splits(24576, 4096, 3 * 148, 16, kernels.FUSED_MAX_SPLITS, 1.0, sms=148) == 2
    assert linear.pick_splits(51200, 5120, 3 * 148, 16, kernels.FUSED_MAX_SPLITS, 1.0, sms=148) == 1
    # a weight with fewer tiles than SMs is cut as before
    assert linear.pick_splits(6144, 4096, 2 * 148, 64, sms=148) == linear.pick_splits(6144, 4096, 2 * 148, 64) == 6


def test_a_product_with_many_tiles_is_not_split():
    assert linear.pick_splits(151936, 4096, 296, 64) == 1
    assert linear.pick_pair_splits(24576, 4096, 2048, 74) == 1
    assert linear.pick_pair_splits(4096, 4096, 512, 74) > 1          # 32 tiles on 74 pairs


@pytest.mark.parametrize("max_rows", [40, 256, 300, 4096])
def test_plans_are_sorted_and_the_partial_buffer_holds_every_plan(max_rows):
    runtime = _Runtime(torch.bfloat16, max_rows)
    layer = linear.Linear("x", 4096, 12288, runtime)
    most = [rows for rows, _ in layer.split_plans]
    assert most == sorted(set(most))
    words = max((rows * splits for rows, splits in layer.split_plans if splits > 1), default=0)
    assert runtime.workspace.declared["x.partial"][0] == words * 4096
    for rows, splits in layer.split_plans:
        assert kernels.tc_normalise_splits(12288, splits) == splits
    # float32 models and rows that TMA cannot address take no split plan at all
    assert linear.Linear("y", 4096, 12288, _Runtime(torch.float32, max_rows)).split_plans == []
    assert linear.Linear("z", 4096, 12284, _Runtime(torch.bfloat16, max_rows)).split_plans == []


def test_the_fused_ring_is_as_deep_as_keeps_every_block_resident():
    """8B shapes: four stages for q/k/v and o (384 and 256 blocks of the 444 that three to an SM give), five for down
    (256 of 296); the 32B shape's q/k/v has 480 blocks and keeps the default three stages, its down takes four."""
    runtime = _Runtime(torch.bfloat16, 64)
    def stages(out_features, in_features, role):
        return linear.Linear(f"t.{role}.{out_features}", out_features, in_features, runtime, role=role)._fused_stages(8)
    assert [stages(6144, 4096, "qkv"), stages(4096, 4096, "attn_out"), stages(24576, 4096, "gate"), stages(4096, 12288, "mlp_out")] == [4, 4, 4, 5]
    assert [stages(10240, 5120, "qkv"), stages(5120, 8192, "attn_out"), stages(5120, 25600, "mlp_out")] == [0, 4, 4]
    assert stages(4096, 4096, "") == 0
