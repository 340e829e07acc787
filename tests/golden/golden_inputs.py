"""Inputs of the golden cases, made by integer arithmetic alone so that the script that runs
the reference's kernels and the test that reads their outputs build the very same arrays on
any machine and any version of numpy."""
from __future__ import annotations

import numpy as np


def det_uniform(n: int, seed: int) -> np.ndarray:
    """n float64 values in [-0.5, 0.5), a fixed function of (index, seed): a 64-bit mix
    (multiply, xor-shift) of the index, its top 24 bits taken."""
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64) * np.uint64(6364136223846793005) \
            + np.uint64(seed) * np.uint64(1442695040888963407) + np.uint64(1)
        x ^= x >> np.uint64(33)
        x *= np.uint64(0xFF51AFD7ED558CCD)
        x ^= x >> np.uint64(33)
        x *= np.uint64(0xC4CEB9FE1A85EC53)
        x ^= x >> np.uint64(33)
    return (x >> np.uint64(40)).astype(np.float64) / float(1 << 24) - 0.5


# name -> sizes.  rms_norm: x [rows, heads, dim] normalised over dim with one weight vector [dim].
NORM_CASES = {
    "norm_wide": dict(rows=37, heads=1, dim=96, eps=1e-5, scale=3.0, seed=11),
    "norm_heads": dict(rows=19, heads=4, dim=32, eps=1e-6, scale=0.7, seed=12),
}
# rotation tables: (cos, sin) of pos * theta^(-2i/dim); only the listed positions are kept
ROPE_CASES = {
    "rope_small": dict(max_pos=300, dim=32, theta=1e4, keep=[0, 1, 2, 3, 17, 100, 299]),
    "rope_head128": dict(max_pos=2048, dim=128, theta=1e6, keep=[0, 1, 5, 64, 1000, 2047]),
}
SILU_CASE = dict(n=1000, span=24.0, seed=21)
# attention of 32 query heads on 8 key/value heads of 128 (the one geometry the reference's kernel is built
# for): M new tokens after ``start`` cached ones; queries, keys and values un-rotated, as the kernel takes them
ATTENTION_GEOMETRY = dict(heads=32, kv_heads=8, head_dim=128, theta=1e6)
ATTENTION_CASES = {
    "attention_prompt": dict(start=0, new=64, keep_rows=[0, 1, 7, 8, 31, 32, 33, 63], seed=31),
    "attention_continued": dict(start=56, new=8, keep_rows=[0, 1, 2, 3, 4, 5, 6, 7], seed=32),
}


def norm_inputs(c):
    x = (det_uniform(c["rows"] * c["heads"] * c["dim"], c["seed"]) * 2 * c["scale"]).astype(np.float32)
    w = (1.0 + 0.2 * det_uniform(c["dim"], c["seed"] + 1000)).astype(np.float32)
    return x.reshape(c["rows"], c["heads"], c["dim"]), w


def silu_inputs(c):
    gate = (det_uniform(c["n"], c["seed"]) * c["span"]).astype(np.float32)
    up = (det_uniform(c["n"], c["seed"] + 1) * 4).astype(np.float32)
    return gate, up


def attention_inputs(c):
    g = ATTENTION_GEOMETRY
    total = c["start"] + c["new"]
    q = (det_uniform(c["new"] * g["heads"] * g["head_dim"], c["seed"]) * 8).astype(np.float16)
    k = (det_uniform(total * g["kv_heads"] * g["head_dim"], c["seed"] + 1) * 8).astype(np.float16)
    v = (det_uniform(total * g["kv_heads"] * g["head_dim"], c["seed"] + 2) * 2).astype(np.float16)
    return (q.reshape(c["new"], g["heads"], g["head_dim"]), k.reshape(total, g["kv_heads"], g["head_dim"]),
            v.reshape(total, g["kv_heads"], g["head_dim"]))
