"""Choices the product path makes on the host, checked without a GPU: which products may take the
engine's own kernels, and when a position part offers a table for the step."""
import types

import torch

from litellmengine_b200.config.specs import PositionSpec
from litellmengine_b200.csrc import ops
from litellmengine_b200.parts.position import NoPosition, RotaryPosition


def test_the_paired_product_is_never_chosen_for_host_tensors_or_other_types():
    x = torch.zeros(300, 64, dtype=torch.bfloat16)
    w = torch.zeros(128, 64, dtype=torch.bfloat16)
    for kind in ("plain", "silu", "into"):
        assert ops._pair_takes(x, w, 64, kind) is False
    assert ops._pair_takes(x.float(), w.float(), 64, "silu") is False
    assert ops.linear_into(x, w, torch.zeros(300, 128)) is False


def test_only_the_gate_up_product_takes_the_paired_kernel_by_default():
    assert ops._PAIR_NEEDS["silu"] is not None
    assert ops._PAIR_NEEDS["plain"] is None and ops._PAIR_NEEDS["into"] is None


def test_a_position_part_offers_its_table_only_for_steps_its_kernel_reads_it_in():
    rope = RotaryPosition(PositionSpec(kind="rope", theta=10000.0, rotary_dim=None), 128, "cpu")
    small = types.SimpleNamespace(num_tokens=8, tables={}, positions=None)
    large = types.SimpleNamespace(num_tokens=4096, tables={}, positions=None)
    assert rope.angles(small) is None
    assert rope.angles(large) is None                      # tables live on the GPU only
    assert NoPosition(PositionSpec(kind="none"), 128, "cpu").rotation(large) is None
    assert rope.rotation(large).inv_freq is rope.inv_freq and rope.rotation(large).angles is None
    odd = RotaryPosition(PositionSpec(kind="rope", theta=10000.0, rotary_dim=32), 48, "cpu")
    assert odd._table_ok is False and rope._table_ok is True


def test_partial_sums_add_up_and_round_once():
    parts = torch.tensor([[[1.0, 2.0]], [[0.5, 0.25]], [[1e-3, 0.0]]])
    total = ops.as_tensor(ops.PartialSum(parts, None))
    assert torch.equal(total, (parts[0] + parts[1]) + parts[2])
    rounded = ops.as_tensor(ops.PartialSum(parts, torch.bfloat16))
    assert rounded.dtype == torch.bfloat16 and torch.equal(rounded, total.to(torch.bfloat16))
