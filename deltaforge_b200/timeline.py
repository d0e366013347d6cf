"""Per-launch timeline of the graph-of-kernels decode step, from the device timestamps the kernels record.

``DecodeEngine.set_trace()`` makes one thread of every CTA of every launch store the global nanosecond timer
at up to eight marks (``dfb_engine_set_trace`` in include/dfb200.h lists them). ``summarise`` turns the buffer
of the last step into one row per launch: when its CTAs entered, when the wait for the previous kernel
returned, when the activation was ready, when the dot products were done, when the cluster barrier passed and
when the last CTA left, all in microseconds from the first mark of the step, plus the two figures that
matter for a chain of dependent kernels: how long after the previous launch's last exit this launch's wait
returned (the boundary), and how long the launch then took (the chain inside it).
"""

from __future__ import annotations

import torch

MARKS = ("entry", "wait_ret", "x_ready", "dots_done", "unit1_done", "barrier", "exit", "issued")


def launch_names(layer_kinds: list[str], launches: int) -> list[str]:
    """Names of the launches of one batch-1 step in order (embed; five per layer; head, argmax, advance)."""
    names = ["embed"]
    for i, kind in enumerate(layer_kinds):
        mixer = "deltanet" if kind == "linear_attention" else "attention"
        names += [f"L{i}.in_proj", f"L{i}.{mixer}", f"L{i}.out_proj", f"L{i}.gate_up", f"L{i}.down"]
    names += ["head", "argmax", "advance"]
    return (names + [f"launch{j}" for j in range(len(names), launches)])[:launches]


def summarise(trace: torch.Tensor, names: list[str]) -> list[dict]:
    """One dict per traced launch (launches without marks, e.g. the embedding gather, are left out)."""
    t = trace.detach().cpu().to(torch.float64)
    live = t[..., 0] > 0
    if not bool(live.any()):
        return []
    t0 = float(t[..., 0][live].min())
    rows: list[dict] = []
    prev_exit = None
    for l in range(t.shape[0]):
        m = live[l]
        if not bool(m.any()):
            continue
        marks = t[l][m]  # (ctas, 8)

        def col(j, how):
            v = marks[:, j]
            v = v[v > 0]
            if v.numel() == 0:
                return None
            x = {"min": v.min(), "max": v.max(), "med": v.median()}[how]
            return (float(x) - t0) / 1e3

        row = {
            "launch": l,
            "name": names[l] if l < len(names) else f"launch{l}",
            "ctas": int(m.sum()),
            "entry_first": col(0, "min"),
            "entry_last": col(0, "max"),
            "issued": col(7, "med"),
            "wait_ret": col(1, "med"),
            "x_ready": col(2, "med"),
            "unit1_done": col(4, "med"),
            "dots_done": col(3, "med"),
            "dots_done_last": col(3, "max"),
            "barrier": col(5, "med"),
            "exit_last": col(6, "max"),
        }
        if row["wait_ret"] is not None and prev_exit is not None:
            row["boundary"] = row["wait_ret"] - prev_exit
        if row["wait_ret"] is not None and row["exit_last"] is not None:
            row["chain"] = row["exit_last"] - row["wait_ret"]
        if row["exit_last"] is not None:
            prev_exit = row["exit_last"]
        rows.append(row)
    return rows


def render(rows: list[dict]) -> str:
    cols = ("launch", "name", "ctas", "entry_first", "entry_last", "issued", "wait_ret", "x_ready", "unit1_done", "dots_done", "dots_done_last",
            "barrier", "exit_last", "boundary", "chain")  # fmt: skip
    out = [" ".join(f"{c:>14}" for c in cols)]
    for r in rows:
        cells = []
        for c in cols:
            v = r.get(c)
            cells.append(f"{v:>14.2f}" if isinstance(v, float) else f"{str(v) if v is not None else '-':>14}")
        out.append(" ".join(cells))
    # totals by kind of launch
    kinds: dict[str, list[dict]] = {}
    for r in rows:
        kinds.setdefault(r["name"].split(".")[-1], []).append(r)
    out.append("")
    out.append(f"{'kind':>12} {'launches':>9} {'boundary us (mean)':>20} {'chain us (mean)':>17} {'sum us':>9}")
    for k, rs in kinds.items():
        b = [r["boundary"] for r in rs if "boundary" in r]
        c = [r["chain"] for r in rs if "chain" in r]
        if not c:
            continue
        mb = sum(b) / len(b) if b else float("nan")
        out.append(f"{k:>12} {len(rs):>9} {mb:>20.2f} {sum(c) / len(c):>17.2f} {sum(b) + sum(c):>9.1f}")
    return "\n".join(out)
