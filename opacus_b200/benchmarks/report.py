"""Pivot the JSON files written by ``benchmarks.layers --json`` into one table and gate on a threshold.

    python -m opacus_b200.benchmarks.layers --impl ours --json ours.json
    python -m opacus_b200.benchmarks.layers --impl reference --json ref.json
    python -m opacus_b200.benchmarks.report ours.json ref.json [--max-ratio 1.0] [--csv out.csv]
    python -m opacus_b200.benchmarks.report ours_b16.json,ours_b64.json ref_b16.json,ref_b64.json     # a batch sweep

Prints, per (layer, dtype, mode, batch), both times, ``ours / reference`` and both peak-memory figures with their ratio;
with ``--max-ratio`` (runtime) or ``--max-memory-ratio`` the exit code is 1 if any ratio exceeds it (the role of ``benchmarks/generate_report.py`` and ``benchmarks/check_threshold.py:44-48`` in
the reference, whose gate compares a DP mode against the non-private baseline).
"""
import argparse
import json
import sys


def load(paths):
    """Rows of one or several result files (comma separated, e.g. one per batch size), keyed by
    (layer, dtype, mode, batch)."""
    out = {}
    for path in paths.split(","):
        with open(path) as f:
            for r in json.load(f):
                out[(r["layer"], r["dtype"], r["mode"], int(r.get("batch", 64)))] = r
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("ours")
    ap.add_argument("reference")
    ap.add_argument("--max-ratio", type=float, default=None)
    ap.add_argument("--max-memory-ratio", type=float, default=None)
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    a, b = load(args.ours), load(args.reference)
    rows, worst, worst_mem = [], 0.0, 0.0
    print(f"{'layer':13s} {'dtype':9s} {'mode':6s} {'batch':>5s} {'ours ms':>10s} {'ref ms':>10s} {'ours/ref':>9s}"
          f" {'ours MB':>10s} {'ref MB':>10s} {'ours/ref':>9s}")
    for key in sorted(set(a) | set(b)):
        x, y = a.get(key, {}).get("ms"), b.get(key, {}).get("ms")
        ratio = x / y if x and y else None
        if ratio is not None:
            worst = max(worst, ratio)
        mx, my = a.get(key, {}).get("peak_mb"), b.get(key, {}).get("peak_mb")
        mratio = mx / my if mx and my else None
        if mratio is not None:
            worst_mem = max(worst_mem, mratio)
        fmt = lambda v: f"{v:10.3f}" if v is not None else f"{'-':>10s}"
        rat = lambda v: f"{v:9.2f}" if v else f"{'-':>9s}"
        print(f"{key[0]:13s} {key[1]:9s} {key[2]:6s} {key[3]:5d} {fmt(x)} {fmt(y)} {rat(ratio)} {fmt(mx)} {fmt(my)} "
              f"{rat(mratio)}")
        rows.append((*key, x, y, ratio, mx, my, mratio))
    if args.csv:
        with open(args.csv, "w") as f:
            f.write("layer,dtype,mode,batch,ours_ms,reference_ms,ratio,ours_peak_mb,reference_peak_mb,memory_ratio\n")
            for r in rows:
                f.write(",".join("" if v is None else str(v) for v in r) + "\n")
    if args.max_ratio is not None and worst > args.max_ratio:
        print(f"FAILED: worst ratio {worst:.2f} exceeds {args.max_ratio}")
        return 1
    if args.max_memory_ratio is not None and worst_mem > args.max_memory_ratio:
        print(f"FAILED: worst memory ratio {worst_mem:.2f} exceeds {args.max_memory_ratio}")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
