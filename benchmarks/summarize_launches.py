"""Summarise an `ncu --metrics gpu__time_duration.sum --csv` launch list by kernel.

    python benchmarks/summarize_launches.py launches.csv [top_n]
"""
import collections
import csv
import re
import sys


def main():
    path = sys.argv[1]
    top = int(sys.argv[2]) if len(sys.argv) > 2 else 25
    with open(path) as f:
        lines = [ln for ln in f if not ln.startswith("==")]
    tot, cnt = collections.Counter(), collections.Counter()
    for row in csv.DictReader(lines):
        try:
            v = float(row["Metric Value"].replace(",", ""))
        except (KeyError, ValueError):
            continue
        unit = row.get("Metric Unit", "")
        v *= {"us": 1e3, "ms": 1e6, "s": 1e9}.get(unit, 1.0)
        key = re.sub(r"\(.*$", "", row["Kernel Name"])[:100]
        tot[key] += v
        cnt[key] += 1
    total = sum(tot.values())
    print(f"{sum(cnt.values())} launches, {total / 1e6:.2f} ms of kernel time (serialised, cold caches: compare shares)")
    for k, v in tot.most_common(top):
        print(f"{v / 1e6:8.3f} ms {100 * v / total:5.1f}% n={cnt[k]:4d} {k}")


if __name__ == "__main__":
    main()
