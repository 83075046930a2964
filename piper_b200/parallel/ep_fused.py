"""Fused lowering of the expert-parallel exchanges (the A2A tasks of a ``shard`` directive).

The reference issues ``all_to_all_single`` on ``ep_stream`` before and after every expert region, forward and
backward (``src/executors.py:102-106,654-691``; nodes inserted by ``src/directives.py:957-1156``).  Here the four
transfers of a mixture-of-experts layer are kernels that read and write the peers' memory directly
(``csrc/ep_exchange.cu``):

========== ======================================= =====================================================
task        reference                               this lowering
========== ======================================= =====================================================
dispatch    local permute, then all-to-all          ``moe_dispatch`` gathers rows by router index straight into
                                                    the expert owners' receive regions (no local permute)
experts     grouped compute on the received copy    grouped tcgen05 GEMMs read the receive region in place
return      all-to-all of the outputs               owner copies each (source, expert) segment into the source's
                                                    buffer in that source's own padded layout; ``moe_combine``
                                                    applies the router weights there
backward    the two mirrors                         the same two kernels with the roles swapped
========== ======================================= =====================================================

Row counts never visit the host: senders publish them with the rows, the owner builds its group table on the
device, and every buffer has a static shape.  A receive region holds ``cap_src`` rows per source, by default
the worst case (every row of a source lands on one owner); ``PIPER_EP_CAPACITY_FACTOR`` shrinks it to that
multiple of the balanced share, in which case a dispatch that would overflow a region is not sent and the step
fails with ``PiperKernelError`` instead of corrupting memory.

Buffers.  The receive region of an exchange is read again by the weight-gradient GEMMs of its backward pass,
and the returned outputs are read again by the backward of ``moe_combine``, so both live in *slots* that stay
occupied from an exchange's forward to its backward; the number of slots is the largest number of exchanges
that are in flight at once in this rank's dispatch order.  Incoming and returned gradients are transient and
use two buffers each, alternately.  Reuse of any buffer is guarded by a pair of flag words per peer, READY
(writer to reader) and FREE (reader to writer), that carry the buffer's use number; the kernels wait on them
with a deadline and record ``kStatusPeerTimeout`` when it passes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..compiler.dag import A2A, COMPUTE
from ..ops import moe as moe_ops
from ..ops import native
from ..state import LOG_LEVEL, create_logger
from .symm import SymmetricBuffer

logger = create_logger("piper_ep_fused", LOG_LEVEL)

READY, FREE = 0, 1


def source_capacity(tokens: int, k: int, experts_local: int, ep: int, factor: Optional[float]) -> int:
    """Rows of one source's region in an owner's receive buffer (a multiple of 128)."""
    worst = tokens * k
    share = worst if factor is None else min(worst, int(-(-tokens * k * factor // ep)))
    return (share + experts_local * (moe_ops.PAD - 1) + moe_ops.PAD - 1) // moe_ops.PAD * moe_ops.PAD


@dataclass
class _Exchange:
    """Static description of the exchanges of one (microbatch, stage, layer) and its per-step state."""
    key: tuple
    slot: int = -1
    first: int = 0                       # positions in the dispatch order between which the slot is occupied
    last: int = 0
    split_backward: bool = False         # the expert region's backward is BWD_I + BWD_W
    gin_buf: int = 0                     # transient gradient buffers of this exchange (see _plan)
    gret_buf: int = 0
    gin_span: tuple = (0, 0)             # dispatch-order positions between which each is occupied
    gret_span: tuple = (0, 0)
    # per step
    saved: Optional[tuple] = None        # outputs of the fused moe_dispatch (for an activation-checkpoint replay)
    seg_off: Any = None
    g_start_loc: Any = None
    g_len_loc: Any = None
    table: Optional[tuple] = None        # owner side: (g_start, g_len, recv_counts)
    recv_use: int = 0
    ret_use: int = 0
    gin_use: int = 0
    gret_use: int = 0


class _Pool:
    """Symmetric buffers of one expert-parallel group for one problem shape."""

    def __init__(self, ranks: list, group, me: int, slots: int, tokens: int, dim: int, experts: int, k: int,
                 factor: Optional[float], device: torch.device, n_gin: int = 2, n_gret: int = 2) -> None:
        lib = native.lib()
        self.ep, self.me, self.S = len(ranks), me, slots
        self.T, self.D, self.E, self.k = tokens, dim, experts, k
        self.El = experts // self.ep
        self.cap_src = source_capacity(tokens, k, self.El, self.ep, factor)
        self.cap_own = self.ep * self.cap_src
        self.cap_loc = moe_ops.row_capacity(tokens, k, experts)
        row = dim * 2
        self.n_gin, self.n_gret = n_gin, n_gret
        self.nbuf = 2 * slots + n_gin + n_gret
        sizes = {"recv": slots * self.cap_own * row, "ret": slots * self.cap_loc * row, "gin": n_gin * self.cap_own * row,
                 "gret": n_gret * self.cap_loc * row, "meta": slots * 2 * self.ep * self.El * 4,
                 "flags": self.nbuf * 2 * self.ep * 8}
        self.bufs = {n: SymmetricBuffer.create(b, ranks, group) for n, b in sizes.items()}
        self.bytes = sum(sizes.values())
        self.flags_local = self.bufs["flags"].view(torch.int64, self.nbuf * 2 * self.ep)
        self.flags_ptrs = self.bufs["flags"].peer_ptrs
        self.counters = torch.zeros(self.nbuf, dtype=torch.int32, device=device)
        self.aborts = torch.zeros(self.nbuf, dtype=torch.int32, device=device)
        self.uses = [0] * self.nbuf

        def ptrs(name, i, stride):
            return self.bufs[name].offset_ptrs(i * stride)

        def local(name, i, rows):
            base = self.bufs[name].local.data_ptr() + i * rows * row
            return lib.symm_tensor_bf16(base, rows, dim)

        self.recv_ptrs = [ptrs("recv", s, self.cap_own * row) for s in range(slots)]
        self.ret_ptrs = [ptrs("ret", s, self.cap_loc * row) for s in range(slots)]
        self.gin_ptrs = [ptrs("gin", r, self.cap_own * row) for r in range(n_gin)]
        self.gret_ptrs = [ptrs("gret", r, self.cap_loc * row) for r in range(n_gret)]
        self.meta_ptrs = [ptrs("meta", s, 2 * self.ep * self.El * 4) for s in range(slots)]
        self.recv = [local("recv", s, self.cap_own) for s in range(slots)]
        self.ret = [local("ret", s, self.cap_loc) for s in range(slots)]
        self.gin = [local("gin", r, self.cap_own) for r in range(n_gin)]
        self.gret = [local("gret", r, self.cap_loc) for r in range(n_gret)]
        G2 = 2 * self.ep * self.El
        meta_all = self.bufs["meta"].view(torch.int32, slots * G2)
        self.meta = [meta_all[s * G2:(s + 1) * G2] for s in range(slots)]
        torch.cuda.synchronize()
        if self.ep > 1:
            dist.barrier(group=group)

    # buffer numbering: recv slots, ret slots, incoming-gradient buffers, returned-gradient buffers
    def buf_id(self, kind: str, i: int) -> int:
        return {"recv": 0, "ret": self.S, "gin": 2 * self.S, "gret": 2 * self.S + self.n_gin}[kind] + i

    def off(self, b: int, which: int) -> int:
        return (b * 2 + which) * self.ep

    def next_use(self, b: int) -> int:
        self.uses[b] += 1
        return self.uses[b]


class FusedExpertRuntime:
    """Plans slots from the actor's dispatch order and runs the exchanges of its A2A nodes."""

    def __init__(self, actor, ranks: list, group, timeout_s: float, num_ctas: int, factor: Optional[float]) -> None:
        self.actor = actor
        self.ranks, self.group = list(ranks), group
        self.ep = len(ranks)
        self.me = self.ranks.index(actor.layout.global_rank) if self.ep > 1 else 0
        self.timeout_s, self.num_ctas, self.factor = timeout_s, num_ctas, factor
        self.exchanges: dict[tuple, _Exchange] = {}
        self.role: dict[str, tuple] = {}          # A2A uid -> (kind, key)
        self.dispatch_of: dict[str, tuple] = {}   # forward node that ends in moe_dispatch -> key
        self.region_of: dict[str, tuple] = {}     # forward node of the expert region -> key
        self.after: dict[str, list] = {}          # compute uid -> [(action, key)] run after the node
        self.pool: Optional[_Pool] = None
        self.slots = self.n_gin = self.n_gret = 0
        self.active: Optional[_Exchange] = None   # exchange whose moe_dispatch the running segment contains
        self.replay = False
        self._plan()

    # ------------------------------------------------------------------ planning
    @classmethod
    def create(cls, actor) -> Optional["FusedExpertRuntime"]:
        if actor.device.type != "cuda":
            return None
        a2a = [n for n in actor.dag.nodes.values() if n.node_kind == A2A]
        if not a2a:
            return None
        mode = os.environ.get("PIPER_FUSED_EP", "1")
        if mode == "0":
            return None
        ep = a2a[0].node_meta.get("ep_shard") or {}
        ranks = None
        for g in ep.get("groups") or []:
            if actor.layout.global_rank in g:
                ranks = list(g)
        if ranks is None:
            ranks = list(ep.get("devices") or actor.layout.dp_ranks)
        if len(ranks) == 1 and mode != "force":
            return None
        group = actor.groups.ep_group if (actor.groups is not None and len(ranks) > 1) else None
        if len(ranks) > 1 and not _same_host(group):
            logger.warning("expert-parallel group spans hosts: peer memory is unavailable, using the NCCL lowering")
            return None
        f = os.environ.get("PIPER_EP_CAPACITY_FACTOR")
        return cls(actor, ranks, group, float(os.environ.get("PIPER_PEER_TIMEOUT_S", "30")),
                   int(os.environ.get("PIPER_EP_CTAS", "64")), float(f) if f else None)

    def _plan(self) -> None:
        dag, order = self.actor.dag, self.actor.order
        index = {uid: i for i, uid in enumerate(order)}

        def compute_neighbour(uid: str, preds: bool):
            ids = dag.data_preds(uid) if preds else dag.data_succs(uid)
            for u in ids:
                if dag.nodes[u].node_kind == COMPUTE:
                    return dag.nodes[u]
            return None

        for n in dag.nodes.values():
            if n.node_kind != A2A:
                continue
            key = (n.tag.get("MB"), n.tag.get("PP"), n.tag.get("EP"))
            x = self.exchanges.setdefault(key, _Exchange(key))
            fwd = n.tag.get("PASS") == "F"
            incoming = n.node_meta["direction"] == "incoming"
            pred, succ = compute_neighbour(n.uid, True), compute_neighbour(n.uid, False)
            if pred is None or succ is None:
                raise RuntimeError(f"{n.uid}: an expert exchange needs a compute node on both sides")
            if fwd and incoming:
                self.role[n.uid] = ("F_in", key)
                self.dispatch_of[pred.uid] = key
                self.region_of[succ.uid] = key
                x.first = index[pred.uid]
            elif fwd:
                self.role[n.uid] = ("F_out", key)
            elif incoming:
                # gradients of the returned outputs travel to the expert owners
                self.role[n.uid] = ("B_in", key)
                self.after.setdefault(pred.uid, []).append(("free_ret", key))
                x.last = max(x.last, index[pred.uid])
                last = succ
                if succ.compute_subkind == "BWD_I":
                    x.split_backward = True
                    for u in dag.data_succs(succ.uid):
                        if dag.nodes[u].node_kind == COMPUTE and dag.nodes[u].compute_subkind == "BWD_W":
                            last = dag.nodes[u]
                self.after.setdefault(last.uid, []).append(("free_recv", key))
                x.last = max(x.last, index[last.uid])
                # a split backward copies the incoming gradients out at once, so their buffer is free again
                x.gin_span = (index[n.uid], index[n.uid] if x.split_backward else index[succ.uid])
            else:
                self.role[n.uid] = ("B_out", key)
                self.after.setdefault(succ.uid, []).append(("free_gret", key))
                x.gret_span = (index[n.uid], index[succ.uid])
        # Buffers are handed out by greedy colouring of the occupancy intervals in dispatch order (identical on
        # every rank of the group, because they replay the same order).  A buffer is reused only by an exchange
        # that starts after the node that frees it, so every FREE flag a kernel waits for is set by work that this
        # rank (and, by the common order, every peer) enqueued earlier: no wait depends on a later launch.
        xs = list(self.exchanges.values())
        for x in xs:
            if x.last <= x.first:
                x.last = len(order)            # forward-only plan: the slot is never handed back within a step
        self.slots = _colour([(x.first, x.last) for x in xs], lambda i, c: setattr(xs[i], "slot", c))
        back = [x for x in xs if x.gin_span != (0, 0)]
        self.n_gin = max(1, _colour([x.gin_span for x in back], lambda i, c: setattr(back[i], "gin_buf", c)))
        back = [x for x in xs if x.gret_span != (0, 0)]
        self.n_gret = max(1, _colour([x.gret_span for x in back], lambda i, c: setattr(back[i], "gret_buf", c)))

    # --------------------------------------------------------------- segment hooks
    def enter(self, node, replay: bool = False) -> None:
        """Called by the executor before it runs forward node ``node`` (or re-runs it for a checkpoint)."""
        key = self.dispatch_of.get(node.uid)
        self.active = self.exchanges[key] if key is not None else None
        self.replay = replay
        rk = self.region_of.get(node.uid)
        table = self.exchanges[rk].table if rk is not None else None
        moe_ops.set_ep_context(self if (self.active is not None or table is not None) else None,
                               table[:2] if table is not None else None)

    def leave(self) -> None:
        self.active = None
        moe_ops.set_ep_context(None, None)

    def close(self) -> None:
        """Collective: unmap the peers' buffers everywhere before any rank frees its own."""
        torch.cuda.synchronize()
        if self.pool is not None:
            for b in self.pool.bufs.values():
                b.close()
        if self.ep > 1:
            dist.barrier(group=self.group)

    def after_node(self, node) -> None:
        """Hands buffers back once the node that read them last has been enqueued."""
        for action, key in self.after.get(node.uid, ()):
            x, p = self.exchanges[key], self.pool
            if p is None:
                continue
            if action == "free_ret":
                self._signal(p.buf_id("ret", x.slot), x.ret_use)
            elif action == "free_recv":
                self._signal(p.buf_id("recv", x.slot), x.recv_use)
                if not x.split_backward:
                    self._signal(p.buf_id("gin", x.gin_buf), x.gin_use)
            elif action == "free_gret":
                self._signal(p.buf_id("gret", x.gret_buf), x.gret_use)

    def _signal(self, b: int, value: int) -> None:
        p = self.pool
        native.lib().ep_signal(p.flags_ptrs, p.off(b, FREE), self.me, self.ep, value)

    # ------------------------------------------------------------------- dispatch
    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor):
        """Body of ``piper::moe_dispatch`` inside a segment whose rows go to expert owners."""
        ex = self.active
        if self.replay and ex.saved is not None:
            return tuple(t.detach() for t in ex.saved)      # fresh tensor objects over the same memory
        lib = native.lib()
        dev = x.device
        T, D = x.shape
        k, E = idx.shape[1], counts.numel()
        if self.pool is None:
            self.pool = _Pool(self.ranks, self.group, self.me, self.slots, T, D, E, k, self.factor, dev, self.n_gin,
                              self.n_gret)
            logger.info("expert exchange: %d slots, %d + %d gradient buffers, %d rows per source region, %.2f GB of "
                        "symmetric memory", self.slots, self.n_gin, self.n_gret, self.pool.cap_src,
                        self.pool.bytes / 2 ** 30)
        p = self.pool
        if (T, D, E, k) != (p.T, p.D, p.E, p.k):
            raise ValueError(f"expert exchange buffers were sized for tokens={p.T} dim={p.D} experts={p.E} k={p.k}, "
                             f"got tokens={T} dim={D} experts={E} k={k}")
        if idx.dtype != torch.int32 or counts.dtype != torch.int32 or idx.shape[0] != T:
            raise ValueError("moe_dispatch expects int32 idx [T, k] and int32 counts [E]")
        g_start = torch.empty_like(counts)
        g_len = torch.empty_like(counts)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        lib.moe_group_table(counts, E, None, g_start, g_len, total)
        scratch = torch.zeros(2 * E + 1 + self.ep, dtype=torch.int32, device=dev)
        seg_off, cursor, ctl = scratch[:E], scratch[E:2 * E], scratch[2 * E:]
        pos = torch.empty(T * k, dtype=torch.int32, device=dev)
        b = p.buf_id("recv", ex.slot)
        use = p.next_use(b)
        lib.ep_dispatch_push(x.contiguous(), idx, counts, g_start, seg_off, ctl, cursor, pos, p.recv_ptrs[ex.slot],
                             p.meta_ptrs[ex.slot], p.flags_ptrs, p.flags_local, p.off(b, FREE), use - 1,
                             p.off(b, READY), use, p.counters[b:b + 1], self.me, self.ep, p.cap_src, self.timeout_s,
                             native.status_tensor(dev), self.num_ctas)
        ex.recv_use, ex.seg_off, ex.g_start_loc, ex.g_len_loc = use, seg_off, g_start, g_len
        ex.saved = (p.ret[ex.slot], pos, g_start, g_len, counts.clone())
        return tuple(t.detach() for t in ex.saved)

    # ------------------------------------------------------------------ exchanges
    def supports(self, node) -> bool:
        return node.uid in self.role

    def exchange(self, node, vals: list) -> tuple:
        kind, key = self.role[node.uid]
        ex, p = self.exchanges[key], self.pool
        m = node.node_meta
        ti, ci = m["a2a_tensor_idx"], m.get("a2a_counts_idx")
        out = list(vals)
        if p is None or vals[ti] is None:
            return tuple(out)
        lib = native.lib()
        dev = self.actor.device
        status = native.status_tensor(dev)
        G = self.ep * p.El
        if kind == "F_in":
            g_start = torch.empty(G, dtype=torch.int32, device=dev)
            g_len = torch.empty(G, dtype=torch.int32, device=dev)
            rc = torch.empty(G, dtype=torch.int32, device=dev)
            b = p.buf_id("recv", ex.slot)
            lib.ep_wait_table(p.flags_local, p.off(b, READY), p.meta[ex.slot], g_start, g_len, rc, self.ep, p.cap_src,
                              ex.recv_use, self.timeout_s, status)
            # the senders' own segment starts travel in the slot's meta block, which the next exchange in this
            # slot overwrites: keep a copy for the two returns of this exchange
            ex.table = (g_start, g_len, rc, p.meta[ex.slot][G:2 * G].clone())
            out[ti] = p.recv[ex.slot]
            if ci is not None:
                out[ci] = rc
            return tuple(out)
        rows = vals[ti].contiguous()
        if kind in ("F_out", "B_out"):
            # expert owner -> token owners: segment (source, local expert) goes home to the source's own layout
            name, i = ("ret", ex.slot) if kind == "F_out" else ("gret", ex.gret_buf)
            b = p.buf_id(name, i)
            use = p.next_use(b)
            dst = p.ret_ptrs[i] if kind == "F_out" else p.gret_ptrs[i]
            g_start, g_len, _, home = ex.table
            lib.ep_block_push(rows, g_start, g_len, home, p.El, 0, p.cap_loc, dst, p.flags_ptrs,
                              p.flags_local, p.off(b, FREE), self._free_needed(b, use), p.off(b, READY), use,
                              p.counters[b:b + 1], p.aborts[b:b + 1], self.me, self.ep, self.timeout_s, status, self.num_ctas)
            lib.ep_wait(p.flags_local, p.off(b, READY), self.ep, use, self.timeout_s, status, 4 if kind == "F_out" else 6, None)
            if kind == "F_out":
                ex.ret_use = use
                out[ti] = p.ret[i]
            else:
                ex.gret_use = use
                out[ti] = p.gret[i]
            return tuple(out)
        # B_in: token owner -> expert owners, the local padded segments land where the forward rows landed
        i = ex.gin_buf
        b = p.buf_id("gin", i)
        use = p.next_use(b)
        lib.ep_block_push(rows, ex.g_start_loc, ex.g_len_loc, ex.seg_off, p.El, self.me * p.cap_src, p.cap_own,
                          p.gin_ptrs[i], p.flags_ptrs, p.flags_local, p.off(b, FREE), self._free_needed(b, use),
                          p.off(b, READY), use, p.counters[b:b + 1], p.aborts[b:b + 1], self.me, self.ep,
                          self.timeout_s, status, self.num_ctas)
        lib.ep_wait(p.flags_local, p.off(b, READY), self.ep, use, self.timeout_s, status, 5, None)
        ex.gin_use = use
        if ex.split_backward:
            # the deferred weight-gradient GEMMs read these rows long after the ring has moved on
            out[ti] = p.gin[i].clone()
            out[ti].record_stream(torch.cuda.default_stream(dev))    # allocated on this stream, read by compute kernels
            self._signal(b, use)
        else:
            out[ti] = p.gin[i]
        return tuple(out)

    @staticmethod
    def _free_needed(b: int, use: int) -> int:
        return use - 1


def _colour(spans: list, assign) -> int:
    """Greedy interval colouring: span i gets the lowest colour whose previous span ended before it starts."""
    free: list[int] = []
    busy: list[tuple] = []
    n = 0
    for i in sorted(range(len(spans)), key=lambda j: spans[j][0]):
        lo, hi = spans[i]
        for item in sorted(busy):
            if item[0] < lo:
                busy.remove(item)
                free.append(item[1])
        if free:
            c = min(free)
            free.remove(c)
        else:
            c = n
            n += 1
        assign(i, c)
        busy.append((hi, c))
    return n


def _same_host(group) -> bool:
    import socket
    if group is None:
        return True
    names: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(names, socket.gethostname(), group=group)
    return len(set(names)) == 1
