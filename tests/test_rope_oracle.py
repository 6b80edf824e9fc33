"""The oracle's RoPE against the reference's own known answers (src/attention/rope.rs:167-185) - runs on the CPU."""
import numpy as np
import pytest

from oracle import oracle as orc


def test_split_half_known_answer():
    out = orc.rope(np.array([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32), 1, 4, 0, [0.0, 0.0], [1.0, 1.0], layout=0, placement=0)
    assert out.tolist() == [[-3.0, -4.0, 1.0, 2.0]]


def test_interleaved_known_answer():
    out = orc.rope(np.array([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32), 1, 4, 0, [0.0, 0.0], [1.0, 1.0], layout=1, placement=0)
    assert out.tolist() == [[-2.0, 1.0, -4.0, 3.0]]


def test_short_table_is_rejected():
    with pytest.raises(Exception):
        orc.rope(np.zeros((1, 4), dtype=np.float32), 1, 4, 1, [1.0, 1.0], [0.0, 0.0], layout=0, placement=1)


def test_suffix_leaves_the_head_prefix_alone_and_matches_a_plain_restatement():
    rng = np.random.default_rng(0)
    rows, heads, head_dim, rotary, pos = 3, 2, 16, 8, 5
    x = rng.standard_normal((rows, heads * head_dim)).astype(np.float32)
    cos = rng.standard_normal((pos + rows, rotary // 2)).astype(np.float32)
    sin = rng.standard_normal((pos + rows, rotary // 2)).astype(np.float32)
    out = orc.rope(x, heads, rotary, pos, cos, sin, layout=0, placement=1)
    for r in range(rows):
        for h in range(heads):
            s = h * head_dim + head_dim - rotary
            assert np.array_equal(out[r, h * head_dim:s], x[r, h * head_dim:s])
            re, im = x[r, s:s + rotary // 2], x[r, s + rotary // 2:s + rotary]
            c, sn = cos[pos + r], sin[pos + r]
            assert np.array_equal(out[r, s:s + rotary // 2], (re * c).astype(np.float32) - (im * sn).astype(np.float32))
            assert np.array_equal(out[r, s + rotary // 2:s + rotary], (im * c).astype(np.float32) + (re * sn).astype(np.float32))
