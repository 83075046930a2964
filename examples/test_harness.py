"""Build a schedule JSON and run a model test with it.

``python examples/test_harness.py --test-file examples/test_llama.py --base-schedule examples/base-schedules/dp2.json
--schedule 1f1b --ranks 1 --mbs 4 [test args...]``

The harness appends generated ``order`` directives (1f1b, interleaved_1f1b, zerobubble, dualpipev) to a base
schedule (or keeps a ``custom`` one untouched), writes it to ``out/<timestamp>/<stem>.json``, starts one
process per device id named in the schedule, runs the selected test module's ``main(args, pg)`` in each,
and writes ``out/<timestamp>/results.csv`` with one row per data-parallel rank.  Unknown arguments are
forwarded to the test module; ``--schedule-directives-file`` is always overridden with the generated file.
The flag surface is the reference's (``examples/test_harness.py:37-129``); ``--address/--port/--ray-namespace``
are accepted and ignored because there is no Ray cluster.
"""
from __future__ import annotations

import argparse
import csv
import importlib.util
import json
import os
import statistics
import sys
from datetime import datetime
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from piper_b200.compiler.builders import (build_1f1b_schedule, build_dualpipev_schedule,  # noqa: E402
                                          build_interleaved_1f1b_schedule, build_zerobubble_schedule)
from piper_b200.compiler.schedule import load_schedule_directives  # noqa: E402
from piper_b200.compiler.viz import visualize_order_directives  # noqa: E402


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="Build a full schedule JSON from a base schedule and generated "
                                                 "order directives, then run a model test with it.")
    parser.add_argument("--test-file", "--test", required=True, help="example file to run, e.g. examples/test_qwen.py")
    parser.add_argument("--base-schedule", required=True, type=Path, help="input JSON schedule without order directives")
    parser.add_argument("--schedule", "--schedule-name", dest="schedule", required=True,
                        choices=("1f1b", "interleaved_1f1b", "zerobubble", "dualpipev", "custom"))
    parser.add_argument("--ranks", type=int, default=None, help="number of PP ranks; required unless --schedule custom")
    parser.add_argument("--mbs", type=int, default=None, help="number of microbatches; required unless --schedule custom")
    parser.add_argument("--virtual-stages", type=int, default=None, help=argparse.SUPPRESS)
    parser.add_argument("--keep-existing-order", action="store_true")
    parser.add_argument("--dry-run", action="store_true",
                        help="write the generated schedule and print the test command without running it")
    parser.add_argument("--viz", action="store_true")
    parser.add_argument("--pytorch-profiler", action="store_true")
    parser.add_argument("--address", default="", help="ignored (no Ray cluster)")
    parser.add_argument("--port", type=int, default=4567, help="ignored (no Ray cluster)")
    parser.add_argument("--temp-dir", default="/tmp/piper/tmp")
    parser.add_argument("--ray-namespace", default=None, help="ignored (no Ray cluster)")
    parser.add_argument("--out-root", default="out")
    parser.add_argument("--hang-timeout", type=float, default=None,
                        help="report a rank as hung when its per-step heartbeat is older than this many seconds")
    args, test_args = parser.parse_known_args(argv)

    if args.schedule != "custom":
        missing = [f for f, v in (("--ranks", args.ranks), ("--mbs", args.mbs)) if v is None]
        if missing:
            parser.error(f"the following arguments are required unless --schedule custom: {', '.join(missing)}")
        if args.virtual_stages is not None:
            parser.error("--virtual-stages is internal; it is 2 for interleaved_1f1b/dualpipev and 1 otherwise")
        args.virtual_stages = 2 if args.schedule in ("interleaved_1f1b", "dualpipev") else 1

    run_dir = Path(args.out_root) / datetime.now().strftime("%Y%m%d_%H%M%S")
    run_dir.mkdir(parents=True, exist_ok=True)
    generated, viz_path = build_schedule_file(args, run_dir)
    forwarded = _replace_arg(test_args, "--schedule-directives-file", str(generated))
    if args.viz:
        forwarded.append("--viz")
    profile_dir = None
    if args.pytorch_profiler and not args.dry_run:
        profile_dir = (run_dir / "pytorch_profiles").resolve()
        profile_dir.mkdir(parents=True, exist_ok=True)
        for stale in profile_dir.glob("dp*_pp*.json"):
            stale.unlink()

    if args.dry_run:
        dry = list(forwarded) + (["--pytorch-profiler"] if args.pytorch_profiler else [])
        _, mod = _load_test_file(args.test_file)
        mod.parse_args(dry)
        cmd = [sys.executable, str(Path(__file__).resolve()), "--test-file", args.test_file, "--base-schedule",
               str(args.base_schedule), "--schedule", args.schedule]
        if args.ranks is not None:
            cmd += ["--ranks", str(args.ranks)]
        if args.mbs is not None:
            cmd += ["--mbs", str(args.mbs)]
        print(" ".join(cmd + dry))
        print(f"generated_schedule={generated}")
        if viz_path is not None:
            print(f"schedule_viz={viz_path}")
        return

    if args.pytorch_profiler:
        forwarded.append("--pytorch-profiler")
    metrics = _run_test_module(args, forwarded, profile_dir)
    if metrics:
        rows = _metrics_rows(metrics)
        out_csv = run_dir / "results.csv"
        _write_results_csv(out_csv, rows)
        print(f"metrics written to {out_csv}")
    if profile_dir is not None:
        from piper_b200.runtime.profiler import combine_profiles
        combine_profiles(str(profile_dir), str(run_dir), schedule=args.schedule,
                         pp=args.ranks if args.ranks is not None else "X", mbs=args.mbs if args.mbs is not None else "X")


def _rank_main(payload, pg=None):
    """Runs in every rank: import the test module by path and call its main."""
    test_file, test_args, extras = payload
    _, mod = _load_test_file(test_file)
    ns = mod.parse_args(test_args)
    for k, v in extras.items():
        setattr(ns, k, v)
    if hasattr(mod, "_derive_num_stages"):
        ns.num_stages = mod._derive_num_stages(ns.schedule_directives_file)
    return mod.main(ns, pg)


def _run_test_module(args, test_args, profile_dir) -> list:
    from piper_b200.runtime.launcher import Coordinator

    _, mod = _load_test_file(args.test_file)
    ns = mod.parse_args(test_args)
    coord = Coordinator(schedule_directives_file=ns.schedule_directives_file, hang_timeout=args.hang_timeout,
                        kill_on_hang=args.hang_timeout is not None, nsight=bool(getattr(ns, "nsight", False)),
                        nsight_dir=str(Path(args.out_root) / "nsight_reports"))
    extras = {"temp_dir": args.temp_dir, "profile_dir": str(profile_dir) if profile_dir else ""}
    job = coord.run_program(_rank_main, (str(Path(args.test_file).resolve()), list(test_args), extras))
    return [r for r in job.results if r]


def _metrics_rows(rank_metrics: list) -> list:
    """One CSV row per data-parallel rank: timing from the replica's slowest pipeline rank, peak memory per stage."""
    by_dp: dict[int, list[dict]] = {}
    for m in rank_metrics:
        by_dp.setdefault(int(m.get("dp_rank", 0)), []).append(m)
    rows = []
    for dp in sorted(by_dp):
        ms = sorted(by_dp[dp], key=lambda m: int(m.get("pp_rank", 0)))
        m0 = ms[0]
        per_iter = [max(m["iter_times_s"][i] for m in ms if len(m["iter_times_s"]) > i)
                    for i in range(len(m0.get("iter_times_s") or []))]
        mean = statistics.fmean(per_iter) if per_iter else float("nan")
        std = statistics.pstdev(per_iter) if len(per_iter) > 1 else 0.0
        tokens = (m0.get("batch_size") or 0) * (m0.get("num_microbatches") or 1) * (m0.get("seq_len") or 0)
        row = {"dp_rank": dp, "model": m0.get("model"), "schedule": m0.get("schedule"), "pp": m0.get("pp"),
               "dp": m0.get("dp"), "batch_size": m0.get("batch_size"), "num_microbatches": m0.get("num_microbatches"),
               "seq_len": m0.get("seq_len"), "samples": len(per_iter), "iter_time_mean_s": mean,
               "iter_time_std_s": std, "throughput_tokens_per_s": tokens / mean if per_iter and mean else float("nan")}
        peak = {}
        for m in ms:
            peak.update(m.get("peak_memory_by_rank") or {})
        for stage, rank in enumerate(sorted(peak, key=int)):
            row[f"peak_memory_pp{stage}_gb"] = float(peak[rank]) / (1024 ** 3)
        rows.append(row)
    return rows


def _write_results_csv(path: Path, rows: list) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fields: list = []
    for r in rows:
        for k in r:
            if k not in fields:
                fields.append(k)
    with path.open("w", newline="", encoding="utf-8") as f:
        w = csv.DictWriter(f, fieldnames=fields, restval="")
        w.writeheader()
        w.writerows(rows)


def build_schedule_file(args, run_dir: Path):
    base = load_schedule_directives(str(args.base_schedule))
    if args.schedule == "custom":
        schedule = list(base)
        order = [d for d in schedule if d.get("op") == "order"]
    else:
        schedule = list(base) if args.keep_existing_order else [d for d in base if d.get("op") != "order"]
        _set_num_microbatches(schedule, args.mbs)
        if args.schedule == "1f1b":
            order = build_1f1b_schedule(args.ranks, args.mbs)
        elif args.schedule == "zerobubble":
            order = build_zerobubble_schedule(args.ranks, args.mbs)
        elif args.schedule == "dualpipev":
            order = build_dualpipev_schedule(args.ranks, args.mbs)
        else:
            order = build_interleaved_1f1b_schedule(args.ranks, args.mbs, args.virtual_stages)
        _validate_generated_order_placement(schedule, order, schedule_name=args.schedule, ranks=args.ranks)
        schedule.extend(order)
    stem = _schedule_stem(args.schedule, args.ranks, args.mbs, args.virtual_stages, args.base_schedule)
    out = run_dir / f"{stem}.json"
    with out.open("w", encoding="utf-8") as f:
        json.dump(schedule, f, indent=2)
        f.write("\n")
    viz = visualize_order_directives(order, run_dir / f"{stem}.png") if args.viz and order else None
    return out, viz


def _schedule_stem(name, ranks, mbs, virtual_stages, base_schedule=None) -> str:
    if name == "custom":
        return f"custom_{Path(base_schedule).stem}" if base_schedule is not None else "custom"
    stem = f"{name}_pp{ranks}_mbs{mbs}"
    return stem + (f"_v{virtual_stages}" if name == "interleaved_1f1b" else "")


def _set_num_microbatches(schedule: list, n: int) -> None:
    found = False
    for d in schedule:
        if d.get("op") == "split":
            d["num_microbatches"] = n
            found = True
    if not found:
        schedule.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": n})


def _validate_generated_order_placement(base: list, order: list, *, schedule_name: str, ranks) -> None:
    """Generated rows are per physical rank: every stage a row (or a slot) names must sit on one device set."""
    stage_dev = {}
    for d in base:
        if d.get("op") == "place":
            pp = (d.get("filter") or {}).get("PP")
            devs = d.get("devices", d.get("device"))
            if pp is not None and pp != "*" and isinstance(devs, list):
                stage_dev[int(pp)] = tuple(sorted(int(x) for x in devs))
    if not stage_dev:
        return
    errors = []
    for ri, d in enumerate(order):
        row_devs = set()
        for si, slot in enumerate(d.get("filters", [])):
            devs, pps = set(), []
            for flt in slot:
                pp = flt.get("PP")
                if pp is None or pp == "*":
                    continue
                pps.append(int(pp))
                if int(pp) not in stage_dev:
                    errors.append(f"row {ri} slot {si} references PP{pp}, but no matching place directive exists")
                else:
                    devs.add(stage_dev[int(pp)])
            if len(devs) > 1:
                errors.append(f"row {ri} slot {si} groups stages {pps} across devices {sorted(devs)}")
            row_devs |= devs
        if len(row_devs) > 1:
            errors.append(f"row {ri} orders stages across devices {sorted(row_devs)}")
    if errors:
        hint = ""
        if schedule_name == "dualpipev" and ranks is not None:
            hint = (" DualPipeV uses V-layout virtual stages; each pair "
                    f"{[(r, 2 * ranks - 1 - r) for r in range(ranks)]} must be placed on the same physical device set.")
        raise ValueError("generated order directives are not compatible with the base placement: "
                         + "; ".join(errors[:4]) + hint)


def _replace_arg(test_args: list, flag: str, value: str) -> list:
    out, skip = [], False
    for a in test_args:
        if skip:
            skip = False
            continue
        if a == flag:
            skip = True
            continue
        if a.startswith(flag + "="):
            continue
        out.append(a)
    return out + [flag, value]


def _load_test_file(test_file: str):
    path = Path(test_file)
    if path.suffix != ".py":
        raise ValueError(f"--test-file must be a Python file path, got: {test_file}")
    if not path.is_absolute():
        path = Path.cwd() / path
    if not path.exists():
        raise FileNotFoundError(f"test file does not exist: {path}")
    sys.path.insert(0, str(path.parent))
    name = path.stem
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return name, mod


if __name__ == "__main__":
    main()
