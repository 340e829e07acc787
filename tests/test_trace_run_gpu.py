"""bin/trace_run itself, as a user runs it: the steps of a trace on its standard input, one at a time,
each sent only after ``done <step>`` of the one before; the ``<step>.f32`` files it writes are
compared with the plain implementation, in the four ways of cutting the same requests, in 32-bit
and in bfloat16.  The tool drives the engine's own step function; this test is what keeps the tool
itself (its reading of the steps, the order of the wanted rows, the files, the give-back at ``end``) right."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import (make_model_dir, make_requests, tiny_config, PROMPT_LENS, trace_whole, trace_tail_decode,
                     trace_portions, trace_mixed, steps_to_jsonl, first_bad)
from plain_qwen3 import PlainModel

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def _round64(n):
    return -(-n // 64) * 64


def _max_tokens(reqs, steps):
    """The most tokens that live requests hold at any time, each request rounded up to a multiple of 64."""
    live, most = set(), 0
    for entries, end in steps:
        live |= {r for r, _, _ in entries}
        most = max(most, sum(_round64(len(reqs[r])) for r in live))
        live -= set(end)
    return most


def _replay(model_dir, dtype, max_tokens, lines, out_dir):
    """Runs the tool, one step at a time.  Returns its exit code."""
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=str(out_dir))
    try:
        for i, line in enumerate(lines):
            proc.stdin.write(line + "\n")
            proc.stdin.flush()
            answer = proc.stdout.readline().strip()
            assert answer == f"done {i}", f"step {i}: the tool answered {answer!r}"
        proc.stdin.close()
        return proc.wait(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("trace_models")
    out = {}
    for name in ("A", "B"):
        d = make_model_dir(tmp, name)
        reqs = make_requests(name)
        pm = PlainModel(d)
        out[name] = (d, reqs, {r: pm.logits(t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_the_tool_replays_the_four_cuts(cases, tmp_path, name, dtype):
    d, reqs, want = cases[name]
    vocab = tiny_config(name).vocab_size
    longest = max(_round64(len(t)) for t in reqs.values())
    traces = {
        "whole": trace_whole(reqs),
        "tail": trace_tail_decode(reqs),
        "portions": trace_portions(reqs),
        # a pool of one and a half of the longest request, in the tool's own rounding: later requests get the
        # pages of finished ones
        "mixed": trace_mixed(reqs, PROMPT_LENS[name], max_live=4, page_size=64, pool_tokens=longest + longest // 2 // 64 * 64 + 64,
                             chunk=5 if name == "A" else 7),
    }
    for mode, steps in traces.items():
        out_dir = tmp_path / f"{mode}"
        out_dir.mkdir()
        max_tokens = _max_tokens(reqs, steps)
        if mode == "mixed":
            assert max_tokens < sum(_round64(len(t)) for t in reqs.values()), "the pool must not hold all requests at once"
        rc = _replay(d, dtype, max_tokens, steps_to_jsonl(reqs, steps), str(out_dir))
        assert rc == 0
        got = {r: [None] * len(t) for r, t in reqs.items()}
        for i, (entries, _) in enumerate(steps):
            path = out_dir / f"{i}.f32"
            rows = sum(n for _, _, n in entries)
            arr = np.fromfile(str(path), dtype="<f4")
            assert arr.size == rows * vocab, f"{mode}: step {i} wrote {arr.size} values for {rows} rows"
            arr = torch.from_numpy(arr.reshape(rows, vocab))
            row = 0
            for r, start, n in entries:
                for k in range(n):
                    got[r][start + k] = arr[row]
                    row += 1
        for r in reqs:
            bad = first_bad(torch.stack(got[r]), want[r], TOL[dtype])
            assert bad is None, f"{name}/{mode}/{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e})"


def test_the_tool_writes_only_wanted_rows_in_order_and_no_file_when_nothing_is_wanted(cases, tmp_path):
    d, reqs, want = cases["B"]
    a, b = "r1", "r2"
    lines = [
        json.dumps({"step": 0, "entries": [{"id": a, "tokens": reqs[a][:6], "want": []},
                                           {"id": b, "tokens": reqs[b][:9], "want": [8, 2]}], "end": []}),
        json.dumps({"step": 1, "entries": [{"id": a, "tokens": reqs[a][6:8], "want": []}], "end": []}),
        json.dumps({"step": 2, "entries": [{"id": b, "tokens": reqs[b][9:10], "want": [0]},
                                           {"id": a, "tokens": reqs[a][8:11], "want": [2, 0]}], "end": [a, b]}),
    ]
    assert _replay(d, "float32", 128, lines, str(tmp_path)) == 0
    vocab = tiny_config("B").vocab_size
    assert not (tmp_path / "1.f32").exists()
    s0 = torch.from_numpy(np.fromfile(str(tmp_path / "0.f32"), dtype="<f4").reshape(2, vocab))
    s2 = torch.from_numpy(np.fromfile(str(tmp_path / "2.f32"), dtype="<f4").reshape(3, vocab))
    for got, (r, pos) in zip(list(s0) + list(s2), [(b, 8), (b, 2), (b, 9), (a, 10), (a, 8)]):
        assert first_bad(got[None], want[r][pos][None], 2e-5) is None, (r, pos)
