"""Per-kernel time of the LAST step in an `ncu --metrics gpu__time_duration.sum --csv` launch list of profiles/tools/mapedra_step.py
(a step starts at its embedding launch): `python profiles/tools/mapedra_step_summary.py launches.csv "title"`."""
import collections
import csv
import re
import sys


def main(path, title):
    rows = []
    with open(path) as f:
        lines = [l for l in f if not l.startswith("==")]
    for x in csv.DictReader(lines):
        if x.get("Metric Name") == "gpu__time_duration.sum":
            v, u = float(x["Metric Value"].replace(",", "")), x["Metric Unit"]
            us = v / 1000 if u in ("ns", "nsecond") else v if u in ("us", "usecond") else v * 1000
            rows.append((x["Kernel Name"], us, x.get("Grid Size", "")))
    starts = [i for i, (k, _, _) in enumerate(rows) if "embed_rows" in k]
    step = rows[starts[-1]:]
    agg = collections.OrderedDict()
    for k, us, g in step:
        m = re.search(r"(\w+_kernel)", k)
        kk = m.group(1) if m else k[:40]
        if "gemm" in kk:
            kk += " grid" + g
        a = agg.setdefault(kk, [0, 0.0])
        a[0] += 1
        a[1] += us
    tot = sum(a[1] for a in agg.values())
    print(f"{title}: {len(step)} launches, {tot:.1f} us (ncu launch list: cold caches, serialised; compare shares)")
    for k, (c, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"  {k:62s} n={c:3d} {us:9.1f} us {us / c:8.1f} avg {100 * us / tot:5.1f}%")


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else "step")
