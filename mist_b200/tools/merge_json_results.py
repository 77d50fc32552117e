"""Merges the record lists written by several calibration runs into one file for fitting.

    python -m mist_b200.tools.merge_json_results calib_n2.json calib_n8.json -o bandwidth-merged.json
    python -m mist_b200.tools.comm_model bandwidth-merged.json

Each input is the JSON list ``mist_b200.tools.profile_interference`` writes (one run per group
size or per node count); duplicates (same sizes and layout) are kept once, the later file
winning (reference: mist/tools/merge_json_results.py, used by
mist/tools/scripts/profile_interference_multinode.sh to combine per-node files).
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List


def _key(rec: Dict):
    return (rec.get("intra"), rec.get("inter"), round(rec.get("g2g_gbytes", 0.0), 6), round(rec.get("c2g_gbytes", 0.0), 6),
            round(rec.get("g2c_gbytes", 0.0), 6), round(rec.get("C", 0.0), 5))


def merge(lists: List[List[Dict]]) -> List[Dict]:
    out: Dict = {}
    for recs in lists:
        for r in recs:
            out[_key(r)] = r
    return list(out.values())


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("-o", "--out", default="bandwidth-merged.json")
    args = ap.parse_args(argv)
    lists = []
    for p in args.inputs:
        with open(p) as f:
            lists.append(json.load(f))
    merged = merge(lists)
    with open(args.out, "w") as f:
        json.dump(merged, f)
    print(f"merged {sum(len(x) for x in lists)} records from {len(lists)} files into {len(merged)} -> {args.out}")
    return merged


if __name__ == "__main__":
    main()
