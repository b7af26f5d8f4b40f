"""How well did the cost model rank?  Reads the standard output of the tuning CLIs.

    python -m deca_b200.cli.rank_report gemm.log fa.log ... [--within 0.01]

For every tuned shape the CLIs print one record per measured config, in the cost model's order
(best-ranked first), followed by the final record.  This tool reports, per shape: how many configs were
measured, the best measured throughput, the position of that config in the model's order, the
throughput of the model's first choice relative to the best ("top-1"), and whether one of the model's
first three choices is within ``--within`` (default 1 %) of the best ("top-3 hit"), which is the fair
form of "the best is among the first three" when several configs differ by less than the timing noise
(the tile orders of one tile shape usually do).  Output is a Markdown table per input file.
"""

from __future__ import annotations

import argparse
import re

RECORD = re.compile(r"cost time: ([0-9.]+) ms, throughput: ([0-9.]+) (TFLOPS|GB/s)")
HEADER = re.compile(r"^(GEMMTC|FlashAttention|Softmax|RMSNorm)\(.*\)\s*$")
FOUND = re.compile(r"^Find (\d+) \S+ configs, measuring (\d+)")


def parse(path: str):
    """[(description, unit, [throughput in the model's order])] per tuned shape."""
    shapes, cur = [], None
    with open(path, errors="replace") as f:
        lines = f.read().splitlines()
    for i, line in enumerate(lines):
        if FOUND.match(line):
            cur = {"desc": None, "unit": None, "tp": []}
            shapes.append(cur)
            continue
        if cur is None:
            continue
        if HEADER.match(line.strip()) and cur["desc"] is None:
            cur["desc"] = line.strip()
        m = RECORD.search(line)
        if m:
            cur["tp"].append(float(m.group(2)))
            cur["unit"] = m.group(3)
    return [(s["desc"], s["unit"], s["tp"]) for s in shapes if s["tp"]]


def report(path: str, within: float) -> str:
    rows, hits, n = [], 0, 0
    out = [f"### {path}", "", "| shape | measured | best | rank of best | model's top-1 / best | top-3 hit |", "|---|---|---|---|---|---|"]
    for desc, unit, tp in parse(path):
        best = max(tp)
        rank = tp.index(best) + 1
        top3 = max(tp[:3])
        hit = top3 >= (1.0 - within) * best
        hits += hit
        n += 1
        out.append(f"| {desc} | {len(tp)} | {best:.1f} {unit} | {rank} | {tp[0] / best:.3f} | {'yes' if hit else f'no ({top3 / best:.3f})'} |")
    out.append("")
    out.append(f"{hits} of {n} shapes: one of the model's first three choices is within {100 * within:.0f} % of the measured best.")
    return "\n".join(out)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--within", type=float, default=0.01)
    args = ap.parse_args(argv)
    for p in args.logs:
        print(report(p, args.within))
        print()


if __name__ == "__main__":
    main()
