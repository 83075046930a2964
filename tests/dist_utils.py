"""Helpers for multi-process CPU (gloo) tests: spawn ranks, run a worker, collect results or the first failure."""
from __future__ import annotations

import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, out_dir):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    try:
        res = fn(rank, world, *args)
        torch.save({"ok": True, "res": res}, os.path.join(out_dir, f"r{rank}.pt"))
    except BaseException:
        torch.save({"ok": False, "err": traceback.format_exc()}, os.path.join(out_dir, f"r{rank}.pt"))
        raise


def run_ranks(world: int, fn, args=(), tmp_path=None, timeout: float = 300.0, expect_failure: bool = False):
    """Runs ``fn(rank, world, *args)`` in ``world`` processes; returns the list of per-rank results."""
    out_dir = str(tmp_path)
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, out_dir)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    results = []
    for r in range(world):
        f = os.path.join(out_dir, f"r{r}.pt")
        results.append(torch.load(f, weights_only=False) if os.path.exists(f) else {"ok": False, "err": "no result"})
    if expect_failure:
        return results
    if alive:
        raise AssertionError(f"{len(alive)} rank(s) did not finish within {timeout}s: "
                             + "; ".join(str(x.get("err")) for x in results if not x["ok"]))
    bad = [x["err"] for x in results if not x["ok"]]
    if bad:
        raise AssertionError("rank failure:\n" + bad[0])
    return [x["res"] for x in results]
