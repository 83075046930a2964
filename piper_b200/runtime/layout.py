"""Rank layout and process groups of one training job.

Device ids in a schedule's ``place`` directives are global ranks (on a single
box: CUDA ordinals).  The sorted distinct device tuples are the physical
pipeline ranks; a process's data-parallel rank is its index inside its tuple
(the reference derives the same two numbers, ``src/directives.py:405-411``,
``src/runtime.py:150-154``, but then maps ranks to GPUs through Ray).

Process groups, all created in the same deterministic order on every rank:

* one data-parallel group per device tuple, plus a second communicator over
  the same ranks for expert-parallel traffic so that it can overlap the
  gradient traffic (``src/actor.py:267-280`` does the same);
* expert-parallel sub-groups when a ``shard`` directive lists nested groups;
* one two-rank group per pipeline *channel* ``(sender stage, receiver stage,
  pass)`` and data-parallel index.  Messages of one channel are produced and
  consumed in microbatch order on both sides, so a channel is FIFO even when
  several virtual stages share a pair of GPUs (the reference keys its two
  communicators on direction only, ``src/actor.py:282-294``).  With the gloo
  backend channels are message tags on the world group instead.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class RankLayout:
    world_size: int
    global_rank: int
    device_tuples: list            # sorted distinct device tuples (index = pp rank)
    pp_rank: int
    dp_rank: int
    dp_ranks: tuple                # global ranks of this rank's data-parallel group
    stage_devices: dict            # PP stage index -> device tuple (as written)

    @property
    def pp_degree(self) -> int:
        return len(self.device_tuples)

    @property
    def dp_degree(self) -> int:
        return len(self.dp_ranks)

    def peer_rank(self, peer_pp_rank: int) -> int:
        """Global rank of the process with the same data-parallel index in another pipeline rank."""
        return self.peer_tuple(peer_pp_rank)[self.dp_rank]

    def peer_tuple(self, peer_pp_rank: int) -> tuple:
        return self._tuples_as_written[peer_pp_rank]

    _tuples_as_written: list = field(default_factory=list)


def make_layout(stage_devices: dict, global_rank: int, world_size: Optional[int] = None) -> RankLayout:
    written = []
    for _st, devs in sorted(stage_devices.items()):
        if tuple(devs) not in written:
            written.append(tuple(devs))
    written.sort(key=lambda t: tuple(sorted(t)))
    sorted_tuples = [tuple(sorted(t)) for t in written]
    all_ranks = sorted({d for t in written for d in t})
    ws = len(all_ranks) if world_size is None else world_size
    mine = [i for i, t in enumerate(written) if global_rank in t]
    if len(mine) != 1:
        raise ValueError(f"rank {global_rank} must appear in exactly one device set, found {mine} in {written}")
    pp = mine[0]
    return RankLayout(world_size=ws, global_rank=global_rank, device_tuples=sorted_tuples, pp_rank=pp,
                      dp_rank=written[pp].index(global_rank), dp_ranks=written[pp], stage_devices=dict(stage_devices),
                      _tuples_as_written=written)


class ProcessGroups:
    """Creates and hands out the communicators described in the module docstring."""

    def __init__(self, layout: RankLayout, backend: str, timeout_s: float = 1800.0) -> None:
        self.layout = layout
        self.backend = backend
        self.timeout = datetime.timedelta(seconds=timeout_s)
        self.dp_group = None
        self.ep_group = None
        self.ep_ranks: tuple = layout.dp_ranks
        self._channels: dict = {}
        self._channel_tags: dict = {}
        self._ep_subgroups: dict = {}
        self.expert_replica_group = None      # ranks that hold the same expert shard (EP groups nested in DP)
        self.expert_replica_ranks: tuple = ()
        for t in layout._tuples_as_written:
            if len(t) > 1:
                g = dist.new_group(ranks=list(t), backend=backend, timeout=self.timeout)
                e = dist.new_group(ranks=list(t), backend=backend, timeout=self.timeout)
            else:
                g = e = None
            if t == layout.dp_ranks:
                self.dp_group, self.ep_group = g, e

    def ensure_ep_subgroups(self, groups: list) -> None:
        """``shard`` with nested device lists: every rank creates every sub-group, in list order."""
        key = tuple(tuple(g) for g in groups)
        if key in self._ep_subgroups:
            return
        mine = None
        for g in groups:
            pg = dist.new_group(ranks=list(g), backend=self.backend, timeout=self.timeout) if len(g) > 1 else None
            if self.layout.global_rank in g:
                mine = (pg, tuple(g))
        self._ep_subgroups[key] = mine
        if mine is not None:
            self.ep_group, self.ep_ranks = mine
        # Experts are partitioned inside a sub-group and replicated across sub-groups: the ranks at the same
        # position of every sub-group hold the same experts and must sum their gradients.
        if len(groups) > 1:
            if len({len(g) for g in groups}) != 1:
                raise ValueError(f"shard.devices: expert-parallel groups must have equal sizes, got {groups}")
            for i in range(len(groups[0])):
                ranks = [g[i] for g in groups]
                pg = dist.new_group(ranks=ranks, backend=self.backend, timeout=self.timeout)
                if self.layout.global_rank in ranks:
                    self.expert_replica_group, self.expert_replica_ranks = pg, tuple(ranks)

    def declare_channels(self, channels: list) -> None:
        """``channels``: sorted list of (rank_a, rank_b, from_stage, to_stage, pass) over the whole job."""
        for i, ch in enumerate(channels):
            self._channel_tags[ch] = 1000 + i
            if self.backend == "nccl":
                a, b = ch[0], ch[1]
                # A posted receive waits on the GPU for its peer.  Keep the footprint of these kernels small: every
                # SM they hold is an SM the persistent GEMM and attention kernels cannot use while they wait.
                opts = dist.ProcessGroupNCCL.Options()
                try:
                    opts.config.max_ctas = int(os.environ.get("PIPER_P2P_MAX_CTAS", "8"))
                    opts.config.min_ctas = 1
                except (AttributeError, TypeError, ValueError):
                    pass   # a torch build whose NCCL options lack these fields: run with NCCL's defaults
                pg = dist.new_group(ranks=sorted((a, b)), backend=self.backend, timeout=self.timeout, pg_options=opts)
                if self.layout.global_rank in (a, b):
                    self._channels[ch] = pg

    def channel(self, ch: tuple):
        """Returns (group, tag) to use for a pipeline message on channel ``ch``."""
        if self.backend == "nccl":
            return self._channels[ch], 0
        return None, self._channel_tags[ch]


def init_distributed(device_type: str, timeout_s: float = 1800.0) -> tuple[int, int, str]:
    """Initialise ``torch.distributed`` from the launcher's environment; returns (rank, world, backend)."""
    rank = int(os.environ.get("RANK", os.environ.get("PIPER_GLOBAL_RANK", "0")))
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("PIPER_WORLD_SIZE", "1")))
    backend = "nccl" if device_type == "cuda" else "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if device_type == "cuda":
            local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, backend
