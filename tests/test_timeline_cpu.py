"""Host logic of the per-launch timeline: names of the launches of a step, and the table made from the kernels'
timestamp marks (synthetic marks here: no device involved)."""

from __future__ import annotations

import torch

from deltaforge_b200 import timeline as TL


def test_launch_names_follow_the_layer_kinds():
    names = TL.launch_names(["linear_attention", "full_attention"], 14)
    assert names == ["embed", "L0.in_proj", "L0.deltanet", "L0.out_proj", "L0.gate_up", "L0.down",
                     "L1.in_proj", "L1.attention", "L1.out_proj", "L1.gate_up", "L1.down", "head", "argmax", "advance"]  # fmt: skip
    assert TL.launch_names(["linear_attention"], 3) == ["embed", "L0.in_proj", "L0.deltanet"]
    assert TL.launch_names([], 5)[-1] == "launch4"


def test_summary_gives_boundary_and_chain_per_launch():
    # three launches, two CTAs each, marks in nanoseconds; launch 0 records nothing (like the embedding gather)
    t = torch.zeros((3, 4, len(TL.MARKS)), dtype=torch.int64)
    base = 1_000_000
    for cta, skew in enumerate((0, 200)):
        # launch 1: enters at 0, wait returns at 1000, activation ready 2000, dots 4000, barrier 4500, exit 5000 (+skew)
        t[1, cta] = torch.tensor([base + 0, base + 1000, base + 2000 + skew, base + 4000 + skew, base + 2500, base + 4500 + skew,
                                  base + 5000 + skew, base + 100])
        # launch 2: enters while launch 1 runs, its wait returns 600 ns after launch 1's last exit
        t[2, cta] = torch.tensor([base + 1500, base + 5800, base + 6800, base + 8000 + skew, base + 7200, base + 8300,
                                  base + 9000 + skew, base + 1600])
    rows = TL.summarise(t, ["embed", "L0.in_proj", "L0.deltanet"])
    assert [r["name"] for r in rows] == ["L0.in_proj", "L0.deltanet"] and rows[0]["ctas"] == 2
    first, second = rows
    assert "boundary" not in first and abs(first["chain"] - (5.2 - 1.0)) < 1e-9
    assert abs(first["exit_last"] - 5.2) < 1e-9 and abs(first["dots_done_last"] - 4.2) < 1e-9
    assert abs(second["boundary"] - 0.6) < 1e-9  # 5800 - 5200
    assert abs(second["chain"] - (9.2 - 5.8)) < 1e-9
    text = TL.render(rows)
    assert "L0.deltanet" in text and "boundary us (mean)" in text
    assert TL.summarise(torch.zeros((2, 2, len(TL.MARKS)), dtype=torch.int64), ["a", "b"]) == []
