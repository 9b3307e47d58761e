"""The Pazenex model on the real kernels, in float32 and bfloat16, against the plain implementation: the cases of
tests/pazenex_suite.py, and trace replay as a child process."""

import numpy as np
import pytest

from tests import pazenex_suite as suite
from tests.plain import pazenex_plain as plain
from tests.util import TraceRun

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, dtype, tmp_path):
    case(tmp_path, "cuda:0", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_with_four_state_slots(dtype, tmp_path):
    """bin/trace_run on a schedule of six requests, four live at most, in a pool that holds three of them."""
    cfg = suite.CONFIGS["mixed_loop"]
    w = suite.make_model(tmp_path / "m", cfg, seed=41)
    seqs = {f"r{i}": suite.tokens_for(cfg, n, seed=80 + i) for i, n in enumerate((40, 33, 21, 38, 27, 30))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    run = TraceRun(tmp_path / "m", dtype, tmp_path / "out", max_tokens=4 * 64, page_size=8)
    at = {r: 0 for r in seqs}
    order = list(seqs)
    live, step = [], 0
    try:
        while order or live:
            while order and len(live) < 4:
                live.append(order.pop(0))
            entries, end = [], []
            for j, r in enumerate(live):
                n = min(len(seqs[r]) - at[r], (13, 1, 2, 5)[(step + j) % 4])
                entries.append((r, seqs[r][at[r] : at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == len(seqs[r]):
                    end.append(r)
            got = run.step(entries, end)
            row = 0
            for r, toks, _ in entries:
                n = len(toks)
                lo = at[r] - n
                suite.close(got[row : row + n].astype(np.float64), want[r][lo : lo + n], dtype, f"{r} at {lo}")
                row += n
            live = [r for r in live if r not in end]
            step += 1
    finally:
        run.close()
