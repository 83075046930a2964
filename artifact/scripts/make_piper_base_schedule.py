"""Generate a base schedule (place / replicate / shard directives) for a pp x dp [x ep] layout.

``python artifact/scripts/make_piper_base_schedule.py --pp 4 --dp 2 --zero 1 --out sched.json``

Device ids are global ranks; data-parallel replicas of stage ``s`` are ranks ``s + pp*d`` (pipeline inner), or
``s*dp + d`` with ``--pp-outer``.  ``--zero`` 0/1 = all-reduce, 2 = shard_grads, 3 = shard_grads + shard_params
(the naming of the reference's generator, ``artifact/scripts/make_piper_base_schedule.py:57-66``);
``--virtual-stages v`` places ``v*pp`` stages round-robin, ``--v-placement`` folds them back (DualPipeV).
"""
from __future__ import annotations

import argparse
import json


def make_schedule(pp: int, dp: int, zero: int = 0, ep: bool = False, virtual_stages: int = 1,
                  v_placement: bool = False, pp_outer: bool = False, bucket_size: int | None = None,
                  comm_stream: str = "dp_stream") -> list[dict]:
    def devices(rank: int) -> list[int]:
        return [rank * dp + d for d in range(dp)] if pp_outer else [rank + pp * d for d in range(dp)]

    n_stages = pp * virtual_stages
    out: list[dict] = []
    stage_rank = []
    for s in range(n_stages):
        r = s % pp
        if v_placement and (s // pp) % 2 == 1:
            r = pp - 1 - r
        stage_rank.append(r)
        out.append({"op": "place", "filter": {"PP": s}, "devices": devices(r), "stream": "pp_stream"})
    if dp > 1:
        for s in range(n_stages):
            d = {"op": "replicate", "filter": {"PP": s}, "devices": devices(stage_rank[s]), "reduce_stream": comm_stream}
            if zero >= 2:
                d["shard_grads"] = True
            if zero >= 3:
                d["shard_params"] = True
                d["gather_stream"] = comm_stream
            if bucket_size:
                d["bucket_size"] = int(bucket_size)
            out.append(d)
        if ep:
            for s in range(n_stages):
                out.append({"op": "shard", "filter": {"PP": s, "EP": "*"}, "devices": devices(stage_rank[s]),
                            "stream": "ep_stream" if zero < 2 else comm_stream})
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--pp", type=int, required=True)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--zero", type=int, default=0, choices=(0, 1, 2, 3))
    ap.add_argument("--ep", action="store_true")
    ap.add_argument("--virtual-stages", type=int, default=1)
    ap.add_argument("--v-placement", action="store_true")
    ap.add_argument("--pp-outer", action="store_true")
    ap.add_argument("--bucket-size", type=int, default=None)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    sched = make_schedule(a.pp, a.dp, a.zero, a.ep, a.virtual_stages, a.v_placement, a.pp_outer, a.bucket_size)
    with open(a.out, "w", encoding="utf-8") as f:
        json.dump(sched, f, indent=2)
        f.write("\n")
    print(a.out)


if __name__ == "__main__":
    main()
