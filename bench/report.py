#!/usr/bin/env python
"""Turns the JSON lines that ``bench.py`` and the ``bench/*.py`` programs print into one HTML (or Markdown) report
(role of the reference's benchmark reporting, ``crates/torsh-benches/src``: HTML / CI reports): one row per run with
the metric, throughput, step time, end-to-end figure, clocks and configuration, plus scaling efficiency when runs of the
same metric exist for several GPU counts.

  python bench.py > n1.json; torchrun ... bench.py --gpus 2 > n2.json
  python bench/report.py n1.json n2.json --out report.html"""
from __future__ import annotations

import argparse
import html
import json
import sys


def load(paths) -> list[dict]:
    runs = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        d = json.loads(line)
                    except json.JSONDecodeError:
                        continue
                    if "metric" in d or "unavailable" in d:
                        d["_file"] = p
                        runs.append(d)
    return runs


def scaling(runs: list[dict]) -> dict:
    """metric → {n_gpus: efficiency vs the smallest GPU count present} (weak scaling: value / (n x value at n0) x n0)."""
    out = {}
    by_metric: dict[str, dict[int, float]] = {}
    for r in runs:
        if "value" in r and "n_gpus" in r:
            by_metric.setdefault(r["metric"] + "|" + str(r.get("impl", "ours")), {})[int(r["n_gpus"])] = float(r["value"])
    for m, vals in by_metric.items():
        if len(vals) > 1:
            n0 = min(vals)
            out[m] = {n: v / (vals[n0] * n / n0) for n, v in sorted(vals.items())}
    return out


def rows(runs):
    for r in runs:
        if "unavailable" in r:
            yield [r.get("impl", "reference"), "unavailable", "", "", "", "", r["unavailable"]]
            continue
        e2e, clk = r.get("e2e", {}), r.get("clocks", {})
        yield [r.get("impl", "ours"), r["metric"], str(r.get("n_gpus", "")), f"{r['value']:,.0f} {r.get('unit', '')}",
               f"{r.get('ms_per_step', 0):.2f}", f"{e2e.get('value', 0):,.0f}" if e2e else "",
               f"{clk.get('sm_mhz')} / {clk.get('sm_max_mhz')} MHz {','.join(clk.get('reasons', []))}; "
               + json.dumps(r.get("config", {}))]


HEAD = ["impl", "metric", "GPUs", "value", "ms / step", "end to end", "clocks; config"]


def to_html(runs) -> str:
    cell = lambda c: f"<td>{html.escape(str(c))}</td>"
    body = "\n".join("<tr>" + "".join(cell(c) for c in row) + "</tr>" for row in rows(runs))
    sc = scaling(runs)
    extra = "".join(f"<p>{html.escape(m.split('|')[0])}: " + ", ".join(f"{n} GPUs {e:.1%}" for n, e in eff.items()) + "</p>"
                    for m, eff in sc.items())
    return ("<html><head><meta charset='utf-8'><title>torsh_b200 benchmarks</title><style>td,th{border:1px solid #999;"
            "padding:4px;font:12px monospace}</style></head><body><table><tr>" + "".join(f"<th>{h}</th>" for h in HEAD)
            + f"</tr>\n{body}</table><h3>Weak-scaling efficiency</h3>{extra}</body></html>")


def to_markdown(runs) -> str:
    out = ["| " + " | ".join(HEAD) + " |", "|" + "---|" * len(HEAD)]
    out += ["| " + " | ".join(str(c).replace("|", "/") for c in row) + " |" for row in rows(runs)]
    for m, eff in scaling(runs).items():
        out.append(f"\n{m.split('|')[0]}: " + ", ".join(f"{n} GPUs {e:.1%}" for n, e in eff.items()))
    return "\n".join(out)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--out", default=None, help=".html or .md; default: Markdown on stdout")
    a = ap.parse_args(argv)
    runs = load(a.files)
    text = to_html(runs) if a.out and a.out.endswith(".html") else to_markdown(runs)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text + "\n")
    return runs


if __name__ == "__main__":
    main()
