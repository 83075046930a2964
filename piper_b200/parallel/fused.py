"""Fused compute+collective paths used by the executor instead of NCCL calls.

``FusedCollectives`` adopts every data-parallel bucket of the actor (plain ``replicate``, ``shard_grads``,
``shard_params``) and replaces the collectives of its gradient and parameter life cycle by kernels that read and
write the peers' memory (``csrc/zero_fused.cu``, ``csrc/ag_gemm_sm100.cu``):

============================ ============================================== ==================================
reference call site           NCCL lowering (``PIPER_FUSED=0``)              fused lowering
============================ ============================================== ==================================
``all_reduce(grad)`` per      ``all_reduce`` of the flat bucket + local Adam  one kernel: reduce-scatter by peer
tensor, ``src/executors.py``  on the whole bucket                             loads, Adam on this rank's rows,
``:125-127``                                                                  new bf16 rows stored into every
                                                                              rank's parameter buffer
``reduce_scatter_tensor`` +   the same two calls + Adam on the shard at the   the same kernel per gradient chain,
``add_``, ``:150-154``        end of the step (+ all-gather for ZeRO-2)       accumulating into the fp32 shard;
                                                                              Adam fused into the last one
``all_gather_into_tensor``,   ``all_gather_into_tensor`` into the full        pull kernel over the peers' shards;
``src/runtime.py:443``        buffer                                          the first weight a forward segment
                                                                              multiplies by is gathered inside
                                                                              that GEMM (``ag_gemm``)
============================ ============================================== ==================================

Buckets are sharded by parameter rows (``ParamStorage.row_layout``): rank ``p`` keeps fp32 master weights, Adam
moments and a gradient accumulator for piece ``p`` of every parameter, which cuts the update's memory and HBM
traffic by ``dp`` also for plain ``replicate`` buckets.  Gradient buffers (and, unless parameters are sharded,
the parameter buffers) live in symmetric memory.

Neither kernel spins: each is bracketed by one-thread kernels that publish and wait for flag words (READY: "my
gradients of this reduction are final"; DONE: "I have read everybody's gradients and stored my update";
PARAMS: "my shard holds version v").  A wait that runs out records ``kStatusPeerTimeout``, the kernel behind it
does nothing, and the step driver raises ``PiperCommTimeout`` at the next step.
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

READY_OFF, DONE_OFF, PARAMS_OFF = 0, 1, 2          # flag blocks of dp words each


def first_linear_slot(gm, slot_positions: list) -> int:
    """Index (into ``slot_positions``) of the weight that the segment's first ``piper::linear`` multiplies by, if
    that call is also the first use of the weight; -1 otherwise."""
    phs = [n for n in gm.graph.nodes if n.op == "placeholder"]
    pos_of = {n: i for i, n in enumerate(phs)}
    for n in gm.graph.nodes:
        if n.op != "call_function" or "piper.linear" not in str(n.target).replace("::", "."):
            continue
        w = n.args[1] if len(n.args) > 1 else None
        if w in pos_of and pos_of[w] in slot_positions:
            users = sorted(w.users, key=lambda u: list(gm.graph.nodes).index(u))
            if users and users[0] is n and len(users) == 1:
                return slot_positions.index(pos_of[w])
        return -1
    return -1


class _FusedBucket:
    def __init__(self, st: ParamStorage, ranks: list, group, dp: int) -> None:
        dev = st.device
        self.st = st
        table, shard = ParamStorage.row_layout(st.slots, dp)
        self.shard_numel = shard
        self.bufs: dict[str, SymmetricBuffer] = {}

        def symm(name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
            esz = torch.empty((), dtype=dtype).element_size()
            self.bufs[name] = SymmetricBuffer.create(numel * esz, ranks, group)
            return self.bufs[name].view(dtype, numel)

        self.flags_local = symm("flags", 3 * dp, torch.int64)
        self.full_grads = symm("grads", st.numel, torch.float32)
        self.full_params = None if st.params_sharded else symm("params", st.numel, st.dtype)
        self.alloc = symm
        if any(stride >= 2 ** 33 for _, stride in table):
            raise ValueError(f"bucket {st.key}: a parameter piece of 2^33 elements or more exceeds the kernels' 32-bit "
                             "vector index")
        t = torch.tensor([[s.offset for s in st.slots], [sh for sh, _ in table], [stride for _, stride in table],
                          [(s.numel + 63) // 64 * 64 for s in st.slots]], dtype=torch.int64)
        self.table = t.to(dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.abort = torch.zeros(2, dtype=torch.int32, device=dev)      # [reduce, gather]
        self.scratch: Optional[torch.Tensor] = None                      # bookkeeping of the gather GEMM
        self.use = 0
        self.version = 0
        self.first_slot = -1

    def ptrs(self, name: str) -> torch.Tensor:
        return self.bufs[name].peer_ptrs


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
        if not _same_host(actor.groups.dp_group):
            logger.warning("data-parallel group spans hosts: peer memory is unavailable, using the NCCL lowering")
            return None
        self = cls(actor, float(os.environ.get("PIPER_PEER_TIMEOUT_S", "30")),
                   int(os.environ.get("PIPER_F1_CTAS", "128")))
        for b in actor.buckets.values():
            st = b.storage
            if st is not None and st.mode in ("allreduce", "zero2", "zero3") and st.numel > 0 \
                    and st.dtype == torch.bfloat16:
                self._adopt(st, b)
        return self

    def _adopt(self, st: ParamStorage, bucket) -> None:
        """Re-home the bucket's gradient (and parameter) buffers in symmetric memory and re-shard its state by rows."""
        lay = self.actor.layout
        fb = _FusedBucket(st, list(lay.dp_ranks), self.actor.groups.dp_group, lay.dp_degree)
        st.convert_to_rows(fb.alloc)                    # reads the current parameters (gathers them if sharded)
        st._unregister_sinks()
        if fb.full_params is not None:
            fb.full_params.copy_(st.flat_params)
            st.flat_params = fb.full_params
            st._bind(fb.full_params)
        st.flat_grads = fb.full_grads
        st.persistent_grads = True
        if st.params_live:
            st._register_sinks()
        slot_pos = [s.pos for s in st.slots]
        fb.first_slot = first_linear_slot(bucket.gm, slot_pos) if st.params_sharded else -1
        if fb.first_slot >= 0:
            n_rows = st.slots[fb.first_slot].shape[0]
            fb.scratch = torch.zeros((n_rows + 255) // 256 + 2, dtype=torch.int32, device=st.device)
        self.buckets[st.key] = fb
        torch.cuda.synchronize()
        dist.barrier(group=self.actor.groups.dp_group)

    def supports(self, st: ParamStorage) -> bool:
        return st is not None and st.key in self.buckets

    def close(self) -> None:
        """Collective: unmap the peers' buffers everywhere before any rank frees its own."""
        torch.cuda.synchronize()
        for fb in self.buckets.values():
            for b in fb.bufs.values():
                b.close()
        dist.barrier(group=self.actor.groups.dp_group)

    # ------------------------------------------------------------------ gradients
    def reduce(self, st: ParamStorage, final: bool, grad_scale: float) -> None:
        """Reduce-scatter the group's gradient buckets into this rank's shard; with ``final`` also the optimizer
        step and the publication of the new parameters.  Runs on the current stream."""
        fb = self.buckets[st.key]
        lib, lay, a = native.lib(), self.actor.layout, st.adam
        dp, me = lay.dp_degree, lay.dp_rank
        status = native.status_tensor(st.device)
        fb.use += 1
        flags = fb.ptrs("flags")
        lib.ep_signal(flags, READY_OFF * dp, me, dp, fb.use)
        lib.ep_wait(fb.flags_local, READY_OFF * dp, dp, fb.use, self.timeout_s, status, 11, fb.abort[0:1])
        if final:
            st.step_count += 1
        accumulate = st.mode != "allreduce"
        lib.zero_reduce(fb.ptrs("grads"), st.shard_grads if accumulate else None, st.master, st.m, st.v,
                        st.shard_params, None if st.params_sharded else fb.ptrs("params"), fb.table, me, dp,
                        accumulate, final, a.lr, a.betas[0], a.betas[1], a.eps, a.weight_decay, a.decoupled,
                        max(st.step_count, 1), grad_scale, flags, DONE_OFF * dp, fb.use, fb.counter, fb.abort[0:1],
                        self.num_ctas)
        # nobody reads this rank's gradients any more once every peer is done: clear them for the next chain
        lib.ep_wait(fb.flags_local, DONE_OFF * dp, dp, fb.use, self.timeout_s, status, 12, None)
        lib.zero_clear_others(st.flat_grads, fb.table, me, dp, self.num_ctas)
        if final:
            st.fused_stepped = True
            if st.params_sharded:
                fb.version += 1
                lib.ep_signal(flags, PARAMS_OFF * dp, me, dp, fb.version)

    # ----------------------------------------------------------------- parameters
    def gather(self, st: ParamStorage, fuse_first: bool) -> None:
        """ZeRO-3 parameter materialisation on the current stream: pull every peer's rows into the full buffer;
        with ``fuse_first`` the first linear weight of the segment is left to the GEMM that multiplies by it."""
        if st.numel == 0:
            return
        st.param_users += 1
        fb = self.buckets[st.key]
        lib, lay = native.lib(), self.actor.layout
        dp = lay.dp_degree
        if st.params_live:
            # another chain shares the buffer; if its first weight is still waiting for the GEMM that gathers it,
            # this user may run first: fetch that weight now
            if fb.first_slot >= 0:
                w = st.param_views[st.slots[fb.first_slot].pos]
                if ops_core.gather_gemms.pop(w.data_ptr(), None) is not None:
                    lib.zero_gather(fb.ptrs("shard_params"), st.flat_params, fb.table, dp, -1, fb.first_slot,
                                    fb.abort[1:2], self.num_ctas)
            return
        st.flat_params.untyped_storage().resize_(st.numel * st.flat_params.element_size())
        status = native.status_tensor(st.device)
        lib.ep_wait(fb.flags_local, PARAMS_OFF * dp, dp, fb.version, self.timeout_s, status, 13, fb.abort[1:2])
        skip = fb.first_slot if (fuse_first and fb.first_slot >= 0) else -1
        lib.zero_gather(fb.ptrs("shard_params"), st.flat_params, fb.table, dp, skip, -1, fb.abort[1:2], self.num_ctas)
        st.params_live = True
        st._register_sinks()
        if skip >= 0:
            s = st.slots[skip]
            w = st.param_views[s.pos]
            sh, stride = st.row_table[skip]
            k = s.numel // s.shape[0]
            shard_ptrs = [int(p) + sh * 2 for p in fb.bufs["shard_params"].ptrs]
            w_full = st.flat_params[s.offset:s.offset + s.numel].view(s.shape[0], k)

            def run(x2: torch.Tensor, y: torch.Tensor, fb=fb, me=lay.dp_rank, rows=stride // k, n=s.shape[0]) -> None:
                lib.ag_gemm(x2, shard_ptrs, me, w_full, fb.scratch, y, n, rows, native.status_tensor(x2.device))

            ops_core.gather_gemms[w.data_ptr()] = run

    def release(self, st: ParamStorage) -> None:
        """The full buffer is about to be freed: a gather GEMM that never ran must not fire on a later tensor."""
        fb = self.buckets.get(st.key)
        if fb is not None and fb.first_slot >= 0 and st.params_live:
            w = st.param_views[st.slots[fb.first_slot].pos]
            ops_core.gather_gemms.pop(w.data_ptr(), None)


def _same_host(group) -> bool:
    import socket
    names: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(names, socket.gethostname(), group=group)
    return len(set(names)) == 1


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
