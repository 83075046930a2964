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


# --------------------------------------------------------------------------------------------------
# F2: ZeRO-3 all-gather fused into the consuming GEMM
# --------------------------------------------------------------------------------------------------
class ShardedWeight:
    """A weight ``[N, K]`` sharded by rows over a group, each shard in symmetric memory.

    ``linear(x)`` computes ``x @ W^T`` with one kernel.  With ``keep_full=True`` gather warps inside the GEMM
    pull every remote weight row once over NVLink into a local ``[N, K]`` buffer while the tensor cores start on
    the rows this rank owns; the GEMM reads remote rows from that buffer as they arrive, and the backward GEMMs
    use it afterwards.  With ``keep_full=False`` each CTA loads the weight tiles it needs straight from their
    owners (more NVLink traffic, no extra memory).
    """

    def __init__(self, full_weight: torch.Tensor, ranks: list, group, keep_full: bool = True) -> None:
        N, K = full_weight.shape
        dp = len(ranks)
        me = list(ranks).index(dist.get_rank())
        rows = (N + dp - 1) // dp
        rows = (rows + 63) // 64 * 64
        self.N, self.K, self.rows_per_shard, self.dp, self.index = N, K, rows, dp, me
        self.buf = SymmetricBuffer.create(rows * K * 2, list(ranks), group)
        self.shard = self.buf.view(torch.bfloat16, rows * K).view(rows, K)
        lo, hi = me * rows, min((me + 1) * rows, N)
        self.shard.zero_()
        if hi > lo:
            self.shard[:hi - lo].copy_(full_weight[lo:hi])
        self.full = torch.empty((N, K), dtype=torch.bfloat16, device=full_weight.device) if keep_full else None
        # gather bookkeeping of the kernel (next chunk, per-block arrival counters); cleared by every launch
        self.scratch = torch.zeros((N + 255) // 256 + 2, dtype=torch.int32, device=full_weight.device) \
            if keep_full else None
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def linear(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, self.K).contiguous()
        y = torch.empty((x2.shape[0], self.N), dtype=torch.bfloat16, device=x.device)
        native.lib().ag_gemm(x2, [int(p) for p in self.buf.ptrs], self.index, self.full, self.scratch, y, self.N,
                             self.rows_per_shard, native.status_tensor(x.device))
        return y.view(*x.shape[:-1], self.N)


# --------------------------------------------------------------------------------------------------
# F3: expert-parallel dispatch / combine over peer memory
# --------------------------------------------------------------------------------------------------
class FusedExpertExchange:
    """Symmetric buffers and epochs of one expert-parallel group for the fused dispatch and combine kernels.

    ``dispatch(x, idx, counts)`` scatters token rows into the expert owners' receive regions with peer stores
    (permutation + all-to-all in one pass) and returns the owner-side view: the local receive buffer, its group
    table and the flat count vector, valid once the kernel that waits for all sources has run on the stream.
    ``combine(out_rows, pos, weights)`` publishes the local expert outputs and gathers each token's ``k`` outputs
    from their owners with peer loads while applying the router weights.
    """

    def __init__(self, ranks: list, group, tokens: int, dim: int, experts: int, k: int, timeout_s: float = 30.0,
                 num_ctas: int = 128) -> None:
        from ..ops.moe import row_capacity
        self.ranks, self.group = list(ranks), group
        self.ep = len(ranks)
        self.me = self.ranks.index(dist.get_rank()) if self.ep > 1 else 0
        self.T, self.D, self.E, self.k = tokens, dim, experts, k
        self.El = experts // self.ep
        self.cap = row_capacity(tokens, k, self.El)
        self.timeout_s, self.num_ctas = timeout_s, num_ctas
        rows = self.ep * self.cap
        self.recv = SymmetricBuffer.create(rows * dim * 2, self.ranks, group)
        self.out = SymmetricBuffer.create(rows * dim * 2, self.ranks, group)
        self.meta = SymmetricBuffer.create(self.ep * self.El * 4, self.ranks, group)
        self.flags = SymmetricBuffer.create(2 * self.ep * 8, self.ranks, group)
        dev = self.recv.local.device
        self.recv_rows = self.recv.view(torch.bfloat16, rows * dim).view(rows, dim)
        self.out_rows = self.out.view(torch.bfloat16, rows * dim).view(rows, dim)
        self.meta_local = self.meta.view(torch.int32, self.ep * self.El)
        self.flags_local = self.flags.view(torch.int64, 2 * self.ep)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = 0
        torch.cuda.synchronize()
        if self.ep > 1:
            dist.barrier(group=group)

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor):
        lib = native.lib()
        dev = x.device
        self.epoch += 1
        seg_off = torch.empty(self.E, dtype=torch.int32, device=dev)
        cursor = torch.zeros(self.E, dtype=torch.int32, device=dev)
        pos = torch.empty(x.shape[0] * self.k, dtype=torch.int32, device=dev)
        lib.ep_dispatch_push(x.contiguous(), idx, counts, seg_off, cursor, pos, self.recv.peer_ptrs, self.meta.peer_ptrs,
                             self.flags.peer_ptrs, self.counter, self.me, self.ep, self.cap, self.epoch, self.num_ctas)
        G = self.ep * self.El
        g_start = torch.empty(G, dtype=torch.int32, device=dev)
        g_len = torch.empty(G, dtype=torch.int32, device=dev)
        recv_counts = torch.empty(G, dtype=torch.int32, device=dev)
        lib.ep_wait_table(self.flags_local, self.meta_local, g_start, g_len, recv_counts, self.ep, self.cap, self.epoch,
                          self.timeout_s, native.status_tensor(dev))
        return self.recv_rows, pos, g_start, g_len, recv_counts

    def combine(self, pos: torch.Tensor, weights: torch.Tensor, tokens: int) -> torch.Tensor:
        """Call after the expert outputs of this epoch have been written to ``self.out_rows``."""
        lib = native.lib()
        dev = weights.device
        lib.ep_signal(self.flags.peer_ptrs, self.ep, self.me, self.ep, self.epoch)
        out = torch.empty((tokens, self.D), dtype=torch.bfloat16, device=dev)
        lib.ep_combine_pull(self.out.peer_ptrs, pos, weights.contiguous(), out, self.flags_local[self.ep:], self.ep,
                            self.cap, self.epoch, self.timeout_s, native.status_tensor(dev), self.num_ctas)
        return out
