"""Prints the schedule candidates of a tensor-parallel linear and the one the cost model picks.

    python examples/select_schedule.py --op gemm_rs --tokens 8192 --n 8192 --k 3584 --tp 8

Runs on any host (the selector is integer host code in the native library); each candidate is
an EDM graph, shown with the ordinary EDM-IR printing and exposure analysis.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from edmir_b200 import graph_json, lowering  # noqa: E402
from edmir_b200.calibration import Calibration  # noqa: E402
from edmir_b200.ir.printing import format_summary, format_uops  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm_rs", choices=lowering.OPS)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--allow-unfused", action="store_true", help="let the library collective win if it scores best")
    ap.add_argument("--show-graphs", action="store_true")
    ap.add_argument("--save-graph", metavar="PATH", help="write the chosen candidate's EDM graph as JSON")
    args = ap.parse_args()

    spec = lowering.TPLinearSpec(args.op, args.tokens, args.n, args.k, args.tp)
    sel = lowering.select_schedule(spec, Calibration.load(), allow_unfused=args.allow_unfused)
    print(f"{spec}")
    for s, c in zip(sel.schedules, sel.costs):
        mark = "*" if s.index == sel.chosen else " "
        print(f"{mark} [{s.index:2d}] {s.label():22s} makespan={c.makespan / 1e3:9.1f} us "
              f"exposed_comm={c.exposed_comm / 1e3:8.1f} us total_comm={c.total_comm / 1e3:8.1f} us")
    if args.show_graphs:
        g = sel.graphs[sel.chosen]
        print(format_uops(g, highlight=g.critical_path()[0]))
        print(format_summary(g))
    if args.save_graph:
        graph_json.save(sel.graphs[sel.chosen], args.save_graph)


if __name__ == "__main__":
    main()
