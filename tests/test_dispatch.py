"""Choices the product path makes on the host, checked without a GPU: which products may take the
engine's own kernels, and when a position part offers a table for the step."""
import types

import pytest

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


def test_decode_key_splits_follow_the_length_and_the_wave_fill():
    """On a device of 148 SMs (296 CTA slots).  Few rows: the square-root rule, in steps, never under
    64 keys a split.  More rows: the fewest splits that fill 0.85 of the waves they start."""
    from litellmengine_b200.parts import attention
    dev = torch.device("cpu")
    attention._slots[dev] = 296
    attention._split_choice.clear()
    try:
        pick = lambda rows, kv, nkv=8: attention.decode_key_splits(dev, rows, nkv, kv)
        assert [pick(1, kv) for kv in (1, 64, 65, 300, 1024, 2304, 4096, 8192, 32768)] == [1, 1, 2, 4, 8, 12, 16, 16, 32]
        assert [pick(rows, 4096) for rows in (2, 4, 8, 12, 16, 20, 24, 32, 40, 48, 64, 128)] == [16, 8, 4, 3, 2, 5, 3, 1, 4, 2, 1, 1]
        assert pick(40, 100) == 1 and pick(40, 1000) == 1 and pick(40, 2048) == 4   # evening out the waves pays from 512 keys a split
        assert pick(4, 100) == 2 and pick(4, 64) == 1                   # fewer CTAs than slots: a short context caps the splits
        assert pick(1, 1300, nkv=2) == 8 and pick(1, 201, nkv=2) == 4
    finally:
        del attention._slots[dev]
        attention._split_choice.clear()


@pytest.mark.gpu
def test_small_products_take_the_streaming_kernel_up_to_32_rows():
    """On the GPU (the rule reads the device's SM count): the products of a 0.6B-sized layer are small,
    those of an 8B-sized layer and an output head are not; `linear` follows."""
    assert all(ops.skinny_small(n, k) for n, k in ((4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)))
    assert not any(ops.skinny_small(n, k) for n, k in ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 1024)))
    before = ops.launch_count
    x = torch.randn(24, 1024, device="cuda:0").bfloat16()
    w = (torch.randn(4096, 1024, device="cuda:0") * 0.05).bfloat16()
    y = ops.linear(x, w, out_dtype=torch.float32)
    assert ops.launch_count > before                              # the engine's own kernel ran, not the library's
    assert float((y - x.float() @ w.float().t()).abs().max()) < 1e-4
