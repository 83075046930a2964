"""Fused compute+collective paths used by the executor instead of NCCL calls.

``FusedCollectives`` moves a data-parallel bucket's fp32 gradient buffer and bf16 parameter buffer into
symmetric memory and replaces ``all_reduce(grads)`` + ``Adam`` by one kernel per bucket
(``csrc/fused_collectives.cu``): reduce-scatter over peer loads, sharded Adam, all-gather by peer stores.
The optimizer state of such a bucket is sharded over the data-parallel group (each rank keeps fp32 master
weights and moments for 1/dp of the bucket), which is what cuts the update's HBM traffic and memory by dp.

The NCCL lowering (``ParamStorage.all_reduce_grads`` + the flat Adam kernel) stays available as the
baseline; ``PIPER_FUSED=0`` or ``piper_setup(fused_collectives=False)`` selects it.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import core as ops_core
from ..ops import native
from ..runtime.storage import ParamStorage
from ..state import LOG_LEVEL, create_logger
from .symm import SymmetricBuffer

logger = create_logger("piper_fused", LOG_LEVEL)


class _FusedBucket:
    def __init__(self, st: ParamStorage, buf: SymmetricBuffer, grads_off: int, flags_off: int) -> None:
        self.buf = buf
        self.peer_params = buf.offset_ptrs(0)
        self.peer_grads = buf.offset_ptrs(grads_off)
        self.peer_flags = buf.offset_ptrs(flags_off)
        self.counter = torch.zeros(1, dtype=torch.int32, device=st.device)
        self.epoch = 0


class FusedCollectives:
    def __init__(self, actor, timeout_s: float, num_ctas: int) -> None:
        self.actor = actor
        self.timeout_s = timeout_s
        self.num_ctas = num_ctas
        self.buckets: dict[str, _FusedBucket] = {}

    @classmethod
    def create(cls, actor) -> Optional["FusedCollectives"]:
        if actor.device.type != "cuda" or actor.groups is None or actor.layout.dp_degree <= 1:
            return None
        self = cls(actor, float(os.environ.get("PIPER_PEER_TIMEOUT_S", "30")),
                   int(os.environ.get("PIPER_F1_CTAS", "128")))
        for b in actor.buckets.values():
            st = b.storage
            if st is not None and st.mode == "allreduce" and st.numel > 0 and st.dtype == torch.bfloat16:
                self._adopt(st)
        return self

    def _adopt(self, st: ParamStorage) -> None:
        """Re-home the bucket's parameter and gradient buffers in symmetric memory and shard its Adam state."""
        lay = self.actor.layout
        p_bytes = st.numel * 2
        g_off = (p_bytes + 255) // 256 * 256
        f_off = g_off + st.numel * 4
        buf = SymmetricBuffer.create(f_off + 2 * 8 * lay.dp_degree, list(lay.dp_ranks), self.actor.groups.dp_group)
        new_params = buf.view(torch.bfloat16, st.numel, 0)
        new_grads = buf.view(torch.float32, st.numel, g_off)
        new_params.copy_(st.flat_params)
        st._unregister_sinks()
        st.flat_params = new_params
        st.flat_grads = new_grads
        st._bind(new_params)
        st._register_sinks()
        lo, hi = lay.dp_rank * st.shard_numel, (lay.dp_rank + 1) * st.shard_numel
        st.master = st.master[lo:hi].clone()
        st.m = st.m[lo:hi].clone()
        st.v = st.v[lo:hi].clone()
        st.shard_params = new_params[lo:hi]
        st.fused_shard = (lo, hi)
        self.buckets[st.key] = _FusedBucket(st, buf, g_off, f_off)
        torch.cuda.synchronize()
        dist.barrier(group=self.actor.groups.dp_group)

    def supports(self, st: ParamStorage) -> bool:
        return st.key in self.buckets

    def reduce_scatter_adam(self, st: ParamStorage, grad_scale: float) -> None:
        fb = self.buckets[st.key]
        fb.epoch += 1
        st.step_count += 1
        a = st.adam
        lay = self.actor.layout
        native.lib().f1_rs_adam_ag(fb.peer_grads, fb.peer_params, fb.peer_flags, st.master, st.m, st.v, lay.dp_rank,
                                   lay.dp_degree, fb.epoch, a.lr, a.betas[0], a.betas[1], a.eps, a.weight_decay,
                                   st.step_count, grad_scale, fb.counter, native.status_tensor(st.device),
                                   self.timeout_s, self.num_ctas)
