"""The position-encoding parts alone, on the host: the rotary tables of the product path against the plain
implementation's and against the formula in 64-bit, partial rotation, sharing between layers, refusals."""
import math

import pytest
import torch

from plain import qwen3_plain as plain


def _part(head_dim, rotary_dim, theta, n_positions):
    from prelude_b200.config.spec import RopeSpec
    from prelude_b200.parts.registry import RunContext, make_part
    import prelude_b200.parts.rope  # noqa: F401 - registers the kinds
    part = make_part("position", RopeSpec(head_dim, rotary_dim, theta, n_positions), "unused")
    part.load(None, RunContext(torch.device("cpu"), torch.float32))
    return part


@pytest.mark.parametrize("head_dim,theta,n_positions", [(16, 10000.0, 128), (32, 1000000.0, 256), (48, 500000.0, 100), (128, 1000000.0, 4096)])
def test_rotary_tables(head_dim, theta, n_positions):
    part = _part(head_dim, head_dim, theta, n_positions)
    assert part.tensors() == {} and part.rotary_dim == head_dim
    assert part.cos.dtype == torch.float32 and part.cos.shape == (n_positions, head_dim // 2) == part.sin.shape
    cos, sin = plain.rope_tables(head_dim, n_positions, theta)
    assert torch.equal(part.cos, cos) and torch.equal(part.sin, sin)
    # the formula itself, in 64-bit: angle = p / theta^(2 j / D); the 32-bit angle is off by its own rounding
    for p, j in [(0, 0), (1, 0), (n_positions - 1, 0), (n_positions - 1, head_dim // 2 - 1), (n_positions // 2, head_dim // 4)]:
        ang = p / math.pow(theta, 2 * j / head_dim)
        bound = 2e-7 * max(1.0, ang) + 1e-6
        assert abs(float(part.cos[p, j]) - math.cos(ang)) <= bound and abs(float(part.sin[p, j]) - math.sin(ang)) <= bound
    assert torch.equal(part.cos[0], torch.ones(head_dim // 2)) and torch.equal(part.sin[0], torch.zeros(head_dim // 2))


def test_partial_rotation_has_tables_for_its_own_width():
    part = _part(64, 32, 10000.0, 50)
    assert part.rotary_dim == 32 and part.cos.shape == (50, 16)
    cos, _ = plain.rope_tables(32, 50, 10000.0)           # the angles depend on the rotated width, not on the head's
    assert torch.equal(part.cos, cos)


def test_layers_share_one_pair_of_tables():
    a, b = _part(32, 32, 10000.0, 64), _part(32, 32, 10000.0, 64)
    assert a.cos.data_ptr() == b.cos.data_ptr() and a.sin.data_ptr() == b.sin.data_ptr()
    c = _part(32, 32, 20000.0, 64)
    assert c.cos.data_ptr() != a.cos.data_ptr() and not torch.equal(c.cos, a.cos)


def test_refusals_and_no_position():
    from prelude_b200.config.spec import NoPositionSpec
    from prelude_b200.parts.registry import make_part
    for rotary in (0, 7, 34):
        with pytest.raises(ValueError, match="rotary_dim"):
            _part(32, rotary, 10000.0, 8)
    none = make_part("position", NoPositionSpec(), "unused")
    assert none.cos is None and none.sin is None and none.rotary_dim == 0 and none.tensors() == {}
