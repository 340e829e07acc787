"""The plain implementation against outputs of NKKdev/TFFinfer's own device code.

tests/golden/reference_outputs.npz holds what the reference's kernels computed on a B200 for the
inputs of tests/golden/golden_inputs.py (tests/golden/make_reference_golden.py made it; it cuts the
kernels out of a checkout of the reference at run time).  Here each function of tests/plain_qwen3.py
that restates one of those kernels is run in float64 on the same inputs.

Tolerances are set by the arithmetic of the reference's kernels, not by what the comparison gives:
  * RMSNorm (src/kernel/cuda/norm.cu:9-51) and SiLU-times-up (unary.cu:10-27) are float32 throughout:
    a few float32 roundings of the result;
  * the rotation table (rope_table.cu:10-40) forms the exponent -(2i/d)*ln(theta) in float32 (three
    roundings of a number up to ln(theta) ~ 14 in size, i.e. ~2.5e-6 of the frequency) and then takes
    cos/sin of a float32 angle: the angle may be off by 4e-6 of itself, plus float32 cos/sin;
  * the attention kernel (paged_flash_attention.cu:877-1055) rounds the table to half precision, rotates
    in half precision, and keeps its output accumulator in half precision, rescaled at every block of 32
    keys: 2e-2 of the largest value of the row, the tolerance the reference itself checks its
    half-precision kernels with being 0.01 absolute (src/kernel/include/kernel_util.cu:10-60).
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import golden_inputs as gi  # noqa: E402
import plain_qwen3 as plain  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "reference_outputs.npz")


@pytest.fixture(scope="module")
def golden():
    assert os.path.isfile(GOLDEN), "tests/golden/reference_outputs.npz is part of the repository"
    return np.load(GOLDEN)


@pytest.mark.parametrize("name", list(gi.NORM_CASES))
def test_rms_norm_follows_the_reference_kernel(golden, name):
    c = gi.NORM_CASES[name]
    x, w = gi.norm_inputs(c)
    want = golden[name].astype(np.float64)
    got = plain.rms_norm(torch.from_numpy(x).double(), torch.from_numpy(w).double(), c["eps"]).numpy()
    assert want.shape == got.shape
    assert np.abs(got - want).max() <= 4 * 2.0 ** -24 * np.abs(want).max()


@pytest.mark.parametrize("name", list(gi.ROPE_CASES))
def test_rotation_angles_follow_the_reference_table(golden, name):
    c = gi.ROPE_CASES[name]
    table = golden[name].astype(np.float64)                     # [kept positions, dim/2, (cos, sin)]
    ang = plain.rope_angles(c["keep"], c["dim"], c["theta"]).double().numpy()
    slack = 4e-6 * np.abs(ang) + 3e-7
    assert (np.abs(np.cos(ang) - table[..., 0]) <= slack).all()
    assert (np.abs(np.sin(ang) - table[..., 1]) <= slack).all()
    # position 0 is the identity; position 1 carries the frequencies themselves
    assert (table[0, :, 0] == 1).all() and (table[0, :, 1] == 0).all()
    i = np.arange(c["dim"] // 2)
    assert np.abs(np.arctan2(table[1, :, 1], table[1, :, 0]) - c["theta"] ** (-2.0 * i / c["dim"])).max() < 5e-6


def test_silu_times_up_follows_the_reference_kernel(golden):
    gate, up = gi.silu_inputs(gi.SILU_CASE)
    want = golden["silu_mul"].astype(np.float64)
    got = (plain.silu(torch.from_numpy(gate).double()) * torch.from_numpy(up).double()).numpy()
    assert np.abs(got - want).max() <= 4 * 2.0 ** -24 * np.abs(want).max()
    assert (np.abs(got - want) <= 8 * 2.0 ** -24 * np.abs(want) + 1e-12).all()


@pytest.mark.parametrize("name", list(gi.ATTENTION_CASES))
def test_rotation_and_attention_follow_the_reference_kernel(golden, name):
    """Rotate-half rotation of queries and keys, the grouping of query heads on key/value heads, the
    1/sqrt(d) scale, the causal mask and the softmax, all in one: the reference's attention kernel takes
    un-rotated q and k and the table."""
    c = gi.ATTENTION_CASES[name]
    g = gi.ATTENTION_GEOMETRY
    q, k, v = (torch.from_numpy(a.astype(np.float64)) for a in gi.attention_inputs(c))
    total = c["start"] + c["new"]
    ang = plain.rope_angles(range(total), g["head_dim"], g["theta"])
    kr = plain.rope_rotate_half(k, ang)
    # the plain attention works on whole sequences: give it empty query rows for the cached positions
    q_all = torch.zeros(total, g["heads"], g["head_dim"], dtype=torch.float64)
    q_all[c["start"]:] = q
    qr = plain.rope_rotate_half(q_all, ang)
    got = plain.causal_attention(qr, kr, v)[c["start"]:][c["keep_rows"]].numpy()
    want = golden[name].astype(np.float64)
    assert want.shape == got.shape
    scale = np.abs(want).max(axis=-1, keepdims=True)
    err = np.abs(got - want) / scale
    assert err.max() <= 2e-2, f"largest difference {err.max():.3e} of the row's largest value"
    # the comparison can tell a wrong convention from rounding: the same outputs without the rotation,
    # with adjacent-pair rotation in its place, or with the heads grouped the other way, are far off
    no_rot = plain.causal_attention(q_all, k, v)[c["start"]:][c["keep_rows"]].numpy()
    assert (np.abs(no_rot - want) / scale).max() > 0.2
    other_grouping = plain.causal_attention(qr, kr.flip(1), v.flip(1))[c["start"]:][c["keep_rows"]].numpy()
    assert (np.abs(other_grouping - want) / scale).max() > 0.2
