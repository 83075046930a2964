"""Process launcher and job coordinator.

One OS process per GPU replaces the reference's Ray actors and per-DP-rank driver tasks
(``src/coordinator.py``).  ``Coordinator.run_program(fn, args)`` starts ``world_size`` ranks with the
``torchrun`` environment (``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``, ``MASTER_ADDR=127.0.0.1``, ``MASTER_PORT``)
plus ``PIPER_DP_RANK / PIPER_DP_DEGREE / PIPER_PP_DEGREE / PIPER_WORLD_SIZE`` derived from the schedule,
runs ``fn(args, None)`` in each, and collects what they return.

Health monitoring keeps the reference's semantics (``docs/health_monitoring.md``): the first rank that fails
ends the job (fail fast) unless ``PIPER_STANDBY_ENABLED=1``, in which case the coordinator keeps waiting until
every rank has finished or failed.  In addition every rank touches a heartbeat file once per training step;
a rank whose heartbeat is older than ``hang_timeout`` seconds while its process is alive is reported as
hung, and the job is ended when ``kill_on_hang`` is set - the bounded hang detection that the reference
names as its next milestone.  All failures are produced and observed on the host.

Nsight Systems: with ``nsight`` set (``True`` or a dict of ``nsys profile`` options) every rank is started as
``nsys profile -o <dir>/piper_rank<r> ... python -m piper_b200.runtime.launcher <payload>`` instead of a spawned
child, one report per rank, as the reference does per Ray actor (``src/actor.py:57-64,81``).  The executor's
NVTX ranges (one per DAG node) label the timeline.  A missing ``nsys`` binary is an error, not a silent no-op.
"""
from __future__ import annotations

import os
import shutil
import socket
import subprocess
import sys
import tempfile
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch
import torch.multiprocessing as mp

from ..compiler.schedule import load_schedule_directives, stage_device_map
from ..state import LOG_LEVEL, create_logger
from .layout import make_layout

logger = create_logger("piper_coordinator", LOG_LEVEL)
STANDBY_ENV = "PIPER_STANDBY_ENABLED"
HEARTBEAT_ENV = "PIPER_HEARTBEAT_DIR"


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def heartbeat(step: int) -> None:
    """Called by the step driver: records that this rank finished ``step``."""
    d = os.environ.get(HEARTBEAT_ENV)
    if not d:
        return
    path = os.path.join(d, f"hb_rank{os.environ.get('RANK', '0')}")
    with open(path, "w", encoding="utf-8") as f:
        f.write(f"{step} {time.time()}\n")


def _rank_entry(rank: int, world: int, port: int, env: dict, fn: Callable, args: Any, out_dir: str) -> None:
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), HEARTBEAT_ENV: out_dir})
    os.environ.update(env)
    os.environ.setdefault("TORCH_LOGS", "+graph_breaks")
    try:
        res = fn(args, None)
        torch.save({"ok": True, "res": res}, os.path.join(out_dir, f"result_rank{rank}.pt"))
    except BaseException:
        torch.save({"ok": False, "err": traceback.format_exc()}, os.path.join(out_dir, f"result_rank{rank}.pt"))
        raise


NSIGHT_DEFAULTS = {"t": "cuda,nvtx,osrt,cublas,cudnn", "cuda-memory-usage": "true", "cuda-graph-trace": "node",
                   "force-overwrite": "true"}


def nsight_prefix(rank: int, report_dir: str, options: Optional[dict] = None, nsys: str = "nsys") -> list:
    """``nsys profile`` command prefix of one rank; ``options`` override or extend the defaults (a one-letter key
    becomes ``-k value``, a longer one ``--key=value``; ``None`` drops a default)."""
    opts = dict(NSIGHT_DEFAULTS)
    opts.update(options or {})
    opts.setdefault("o", os.path.join(report_dir, f"piper_rank{rank}"))
    cmd = [nsys, "profile"]
    for k, v in opts.items():
        if v is None:
            continue
        cmd += [f"-{k}", str(v)] if len(k) == 1 else [f"--{k}={v}"]
    return cmd


class _CommandRank:
    """A rank started as a command (under ``nsys``), with the part of ``multiprocessing.Process`` the watch loop uses."""

    def __init__(self, cmd: list, log_path: str) -> None:
        self._log = open(log_path, "w", encoding="utf-8")
        self._p = subprocess.Popen(cmd, stdout=self._log, stderr=subprocess.STDOUT)

    def start(self) -> None:
        pass

    def is_alive(self) -> bool:
        return self._p.poll() is None

    @property
    def exitcode(self):
        return self._p.poll()

    def terminate(self) -> None:
        self._p.terminate()

    def join(self, timeout: Optional[float] = None) -> None:
        try:
            self._p.wait(timeout)
        except subprocess.TimeoutExpired:
            self._p.kill()
        self._log.close()


@dataclass
class JobResult:
    ok: bool
    results: list = field(default_factory=list)          # per rank, None where a rank produced nothing
    failures: dict = field(default_factory=dict)         # rank -> traceback / reason
    hung: list = field(default_factory=list)


class JobFailed(RuntimeError):
    def __init__(self, result: JobResult) -> None:
        first = next(iter(result.failures.items()), (None, "unknown"))
        super().__init__(f"{len(result.failures)} rank(s) failed; first: rank {first[0]}:\n{first[1]}")
        self.result = result


class Coordinator:
    """Starts the ranks of one job and watches over them."""

    def __init__(self, schedule_directives_file: Optional[str] = None, world_size: Optional[int] = None,
                 hang_timeout: Optional[float] = None, kill_on_hang: bool = False, poll_s: float = 0.2,
                 nsight=None, nsight_dir: Optional[str] = None) -> None:
        self.schedule_file = schedule_directives_file
        self.stage_devices = None
        if schedule_directives_file is not None:
            self.stage_devices = stage_device_map(load_schedule_directives(schedule_directives_file))
            world_size = len({d for t in self.stage_devices.values() for d in t})
        if world_size is None:
            raise ValueError("Coordinator needs a schedule file or a world size")
        self.world_size = int(world_size)
        self.hang_timeout = hang_timeout
        self.kill_on_hang = kill_on_hang
        self.poll_s = poll_s
        self.standby = os.environ.get(STANDBY_ENV, "0") == "1"
        self.nsight = ({} if nsight is True else dict(nsight)) if nsight else None
        self.nsight_dir = nsight_dir

    def _rank_env(self, rank: int) -> dict:
        env = {"PIPER_WORLD_SIZE": str(self.world_size)}
        if self.stage_devices is not None:
            lay = make_layout(self.stage_devices, rank, self.world_size)
            env.update({"PIPER_DP_RANK": str(lay.dp_rank), "PIPER_DP_DEGREE": str(lay.dp_degree),
                        "PIPER_PP_DEGREE": str(lay.pp_degree), "PIPER_PP_RANK": str(lay.pp_rank)})
        return env

    def run_program(self, fn: Callable, args: Any = None, timeout: Optional[float] = None,
                    raise_on_failure: bool = True) -> JobResult:
        ctx = mp.get_context("spawn")
        out_dir = tempfile.mkdtemp(prefix="piper_job_")
        port = free_port()
        if self.nsight is not None:
            procs = self._nsight_ranks(fn, args, port, out_dir)
        else:
            procs = [ctx.Process(target=_rank_entry,
                                 args=(r, self.world_size, port, self._rank_env(r), fn, args, out_dir))
                     for r in range(self.world_size)]
        for p in procs:
            p.start()
        t0 = time.time()
        failed: dict[int, str] = {}
        hung: list[int] = []
        done: set[int] = set()
        while len(done) < len(procs):
            time.sleep(self.poll_s)
            for r, p in enumerate(procs):
                if r in done or p.is_alive():
                    continue
                done.add(r)
                if p.exitcode != 0:
                    failed[r] = self._failure_text(out_dir, r, p.exitcode)
                    logger.error(f"a rank failed ({len(failed)}/{len(procs)}): rank {r} exit code {p.exitcode}")
            if failed and not self.standby:
                logger.error("failing fast: stopping the remaining ranks")
                break
            if self.hang_timeout is not None:
                for r, p in enumerate(procs):
                    if r in done or r in hung:
                        continue
                    age = self._heartbeat_age(out_dir, r)
                    if age is not None and age > self.hang_timeout:
                        hung.append(r)
                        logger.error(f"rank {r} heartbeat overdue by {age:.1f}s (limit {self.hang_timeout:.1f}s)")
                if hung and self.kill_on_hang:
                    for r in hung:
                        failed.setdefault(r, "hung: heartbeat overdue")
                    break
            if timeout is not None and time.time() - t0 > timeout:
                for r, p in enumerate(procs):
                    if p.is_alive():
                        failed.setdefault(r, f"job timeout after {timeout}s")
                break
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(10)
        results = []
        for r in range(self.world_size):
            f = os.path.join(out_dir, f"result_rank{r}.pt")
            rec = torch.load(f, weights_only=False) if os.path.exists(f) else None
            results.append(rec["res"] if rec and rec.get("ok") else None)
            if rec and not rec.get("ok"):
                failed[r] = rec["err"]
        job = JobResult(ok=not failed, results=results, failures=failed, hung=hung)
        if failed and raise_on_failure:
            raise JobFailed(job)
        return job

    def _nsight_ranks(self, fn: Callable, args: Any, port: int, out_dir: str) -> list:
        import cloudpickle

        nsys = shutil.which(str(self.nsight.pop("nsys", "nsys")))
        if nsys is None:
            raise RuntimeError("nsight was requested but no `nsys` binary is on PATH")
        report_dir = self.nsight_dir or os.path.join(os.getcwd(), "nsight_reports")
        os.makedirs(report_dir, exist_ok=True)
        procs = []
        for r in range(self.world_size):
            payload = os.path.join(out_dir, f"payload_rank{r}.pkl")
            with open(payload, "wb") as f:
                cloudpickle.dump((r, self.world_size, port, self._rank_env(r), fn, args, out_dir), f)
            cmd = nsight_prefix(r, report_dir, self.nsight, nsys) + [sys.executable, "-m", __name__, payload]
            procs.append(_CommandRank(cmd, os.path.join(report_dir, f"piper_rank{r}.log")))
        logger.info(f"ranks run under nsys; reports in {report_dir}")
        return procs

    @staticmethod
    def _failure_text(out_dir: str, rank: int, code) -> str:
        f = os.path.join(out_dir, f"result_rank{rank}.pt")
        if os.path.exists(f):
            rec = torch.load(f, weights_only=False)
            if not rec.get("ok"):
                return rec["err"]
        return f"process exited with code {code}"

    @staticmethod
    def _heartbeat_age(out_dir: str, rank: int) -> Optional[float]:
        f = os.path.join(out_dir, f"hb_rank{rank}")
        if not os.path.exists(f):
            return None
        return time.time() - os.path.getmtime(f)


# name kept for code written against the reference
PiperProgramCoordinator = Coordinator


if __name__ == "__main__":           # one rank started as a command (under nsys): the payload names everything
    import pickle

    with open(sys.argv[1], "rb") as _f:
        _rank_entry(*pickle.load(_f))
