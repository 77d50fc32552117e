"""Summarises a CUDA caching-allocator snapshot written by the exec entry point with
``memory_debug=true`` (``torch.cuda.memory._dump_snapshot``).

    python -m mist_b200.tools.parse_memory_snapshot memory_snapshot_rank0.pickle --top 15

Prints reserved / allocated / fragmented bytes per segment class and the largest live
blocks with the innermost Python frames that allocated them (reference:
mist/tools/parse_memory_snapshot.py, which walks the same pickle).
"""
from __future__ import annotations

import argparse
import pickle
from collections import defaultdict
from typing import Dict, List


def summarise(snapshot: Dict, top: int = 10) -> Dict:
    segments = snapshot.get("segments", [])
    reserved = sum(s.get("total_size", 0) for s in segments)
    allocated = sum(s.get("allocated_size", 0) for s in segments)
    active = sum(s.get("active_size", 0) for s in segments)
    by_kind = defaultdict(lambda: [0, 0, 0])        # kind -> [segments, reserved, allocated]
    blocks: List[Dict] = []
    largest_free = 0
    for s in segments:
        k = by_kind[s.get("segment_type", "?")]
        k[0] += 1
        k[1] += s.get("total_size", 0)
        k[2] += s.get("allocated_size", 0)
        for b in s.get("blocks", []):
            if b.get("state") == "active_allocated":
                blocks.append(b)
            elif b.get("state") == "inactive":
                largest_free = max(largest_free, b.get("size", 0))
    blocks.sort(key=lambda b: -b.get("size", 0))

    def frames(b):
        fr = b.get("frames") or (b.get("history") or [{}])[-1].get("frames") or []
        keep = [f for f in fr if str(f.get("filename", "")).endswith(".py")][:3]
        return " <- ".join(f"{f.get('filename', '?').split('/')[-1]}:{f.get('line', '?')} {f.get('name', '')}" for f in keep)

    return {"reserved": reserved, "allocated": allocated, "active": active,
            "fragmentation": 1.0 - allocated / reserved if reserved else 0.0, "largest_free_block": largest_free,
            "by_kind": {k: tuple(v) for k, v in by_kind.items()},
            "top_blocks": [(b.get("size", 0), b.get("requested_size", b.get("size", 0)), frames(b)) for b in blocks[:top]]}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("snapshot")
    ap.add_argument("--top", type=int, default=10)
    args = ap.parse_args(argv)
    with open(args.snapshot, "rb") as f:
        snap = pickle.load(f)
    r = summarise(snap, args.top)
    mb = 1 << 20
    print(f"reserved {r['reserved'] / mb:.1f} MB, allocated {r['allocated'] / mb:.1f} MB, active {r['active'] / mb:.1f} MB, "
          f"unused in segments {100 * r['fragmentation']:.1f} %, largest free block {r['largest_free_block'] / mb:.1f} MB")
    for kind, (n, res, alloc) in sorted(r["by_kind"].items()):
        print(f"  {kind:>6} pool: {n} segments, reserved {res / mb:.1f} MB, allocated {alloc / mb:.1f} MB")
    print(f"largest {len(r['top_blocks'])} live blocks:")
    for size, req, where in r["top_blocks"]:
        print(f"  {size / mb:10.1f} MB (requested {req / mb:.1f})  {where}")
    return r


if __name__ == "__main__":
    main()
