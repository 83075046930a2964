"""Parameter, gradient and optimizer-state storage of one parameter bucket.

A bucket is the set of trainable parameters read by one compute node of the
training DAG (a model segment, or one slice of it after ``replicate.bucket_size``).
All of them live in one flat buffer each for

* ``flat_params``  model dtype (bf16 in production), parameters are views into it;
* ``flat_grads``   fp32, the sink that weight-gradient kernels accumulate into;
* ``master / m / v`` fp32 optimizer state over the range this rank *owns*.

The owned range is the whole bucket for ``local`` (no data parallelism) and
``allreduce`` (replicated update) buckets, and the rank's 1/dp slice for
``zero2`` / ``zero3`` buckets and for the fused reduce-scatter + Adam path.
With ``zero3`` the full ``flat_params`` buffer exists only between an
all-gather and the free that the lifetime planner placed after the last
consumer (the reference implements the same life cycle with
``untyped_storage().resize_`` and a host thread for deferred frees,
``src/runtime.py:202-495``; here the caching allocator's stream-ordered free
plus ``record_stream`` does that job without a host thread).

Parameter initialisation is a pure function of the parameter's module-qualified
name, so every data-parallel replica, every pipeline layout and a plain
single-process model start from identical weights.
"""
from __future__ import annotations

import os
import zlib
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from ..ops import core as ops_core
from ..ops import native

# PIPER_DEBUG_POISON=1: fill gathered ZeRO-3 parameters with NaN right before their storage is released
_POISON_FREED = os.environ.get("PIPER_DEBUG_POISON", "0") == "1"

ALIGN = 64  # elements; keeps every parameter view 128-byte aligned in bf16


def init_tensor(fqn: str, shape, dtype, device, seed: int = 0, std: float = 0.02) -> torch.Tensor:
    """Deterministic initial value of parameter ``fqn``: ones for 1-D tensors (norm gains), N(0, std) otherwise."""
    shape = tuple(shape)
    if len(shape) <= 1:
        return torch.ones(shape, dtype=dtype, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed((zlib.crc32(fqn.encode()) + 1000003 * seed) & 0x7FFFFFFF)
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


def materialize_module(module: torch.nn.Module, seed: int = 0, std: float = 0.02) -> torch.nn.Module:
    """Initialise a plain module with the same name-keyed rule the runtime uses (for single-process oracles)."""
    with torch.no_grad():
        for name, p in module.named_parameters():
            p.copy_(init_tensor(name, p.shape, p.dtype, p.device, seed, std))
    return module


@dataclass
class ParamSlot:
    pos: int                 # placeholder position in the bucket's GraphModule
    fqn: str
    shape: tuple
    dtype: torch.dtype
    requires_grad: bool
    offset: int = -1         # element offset in the flat buffers (trainable float params only)
    numel: int = 0
    ep_sharded: bool = False
    full_shape: Optional[tuple] = None
    ep_index: int = 0
    ep_degree: int = 1


@dataclass
class AdamConfig:
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    decoupled: bool = False     # True: AdamW (decay shrinks the weight); False: torch.optim.Adam's L2 term in the gradient


class ParamStorage:
    """Flat buffers of one bucket plus its (possibly sharded) Adam state."""

    def __init__(self, key: str, slots: list[ParamSlot], device: torch.device, dtype: torch.dtype, mode: str,
                 dp_rank: int, dp_degree: int, dp_group, adam: AdamConfig, seed: int = 0) -> None:
        self.key = key
        self.slots = [s for s in slots if s.requires_grad]
        self.device = device
        self.dtype = dtype
        self.mode = mode                 # local | allreduce | zero2 | zero3
        self.dp_rank, self.dp_degree, self.dp_group = dp_rank, max(dp_degree, 1), dp_group
        self.adam = adam
        self.step_count = 0
        self.replica_group = None        # expert shards replicated over expert-parallel groups: summed before the step
        off = 0
        for s in self.slots:
            s.offset = off
            s.numel = 1
            for d in s.shape:
                s.numel *= int(d)
            off += (s.numel + ALIGN - 1) // ALIGN * ALIGN
        quantum = ALIGN * self.dp_degree
        self.numel = (off + quantum - 1) // quantum * quantum if off else 0
        self.shard_numel = self.numel // self.dp_degree
        self.sharded_state = mode in ("zero2", "zero3")
        self.params_sharded = mode == "zero3"
        self.flat_params: Optional[torch.Tensor] = None
        self.flat_grads: Optional[torch.Tensor] = None
        self.shard_grads: Optional[torch.Tensor] = None
        self.param_views: dict[int, torch.Tensor] = {}
        self.params_live = False
        self.param_users = 0
        self.grad_users = 0
        # row sharding (the fused data-parallel paths): per slot (offset of this rank's piece in the shard buffers,
        # elements per piece); None = the shard is the contiguous range owned_range() of the flat layout
        self.row_table: Optional[list] = None
        self.persistent_grads = False      # the full gradient buffer is never freed (it lives in symmetric memory)
        self.fused_stepped = False
        if self.numel == 0:
            return
        full = torch.zeros(self.numel, dtype=dtype, device=device)
        for s in self.slots:
            full[s.offset:s.offset + s.numel].copy_(self._init_slot(s, seed).reshape(-1))
        lo, hi = self.owned_range()
        self.master = full[lo:hi].to(torch.float32) if dtype != torch.float32 else None
        self.m = torch.zeros(hi - lo, dtype=torch.float32, device=device)
        self.v = torch.zeros(hi - lo, dtype=torch.float32, device=device)
        self.flat_params = full
        self.params_live = True
        self._bind(full)
        if self.params_sharded:
            self.shard_params = full[lo:hi].clone()
        else:
            self.shard_params = full[lo:hi]
        if self.sharded_state:
            self.shard_grads = torch.zeros(hi - lo, dtype=torch.float32, device=device)
        if not self.params_sharded:
            self.flat_grads = torch.zeros(self.numel, dtype=torch.float32, device=device)
            self._register_sinks()
        else:
            self.free_params()

    # ------------------------------------------------------------ helpers
    def _init_slot(self, s: ParamSlot, seed: int) -> torch.Tensor:
        if s.ep_sharded and s.full_shape is not None:
            # expert-parallel parameter: initialise the full tensor, keep this rank's experts
            full = init_tensor(s.fqn, s.full_shape, self.dtype, self.device, seed)
            per = s.full_shape[0] // s.ep_degree
            return full[s.ep_index * per:(s.ep_index + 1) * per].contiguous()
        return init_tensor(s.fqn, s.shape, self.dtype, self.device, seed)

    def owned_range(self) -> tuple[int, int]:
        if self.mode in ("zero2", "zero3"):
            return self.dp_rank * self.shard_numel, (self.dp_rank + 1) * self.shard_numel
        return 0, self.numel

    def owned_pieces(self) -> list:
        """``(slot, a, e, sh)``: this rank keeps optimizer state (and, when parameters are sharded, the
        parameters) of elements ``[a, e)`` of the flat layout at ``[sh, sh + e - a)`` of its shard buffers."""
        out = []
        if self.row_table is not None:
            for s, (sh, stride) in zip(self.slots, self.row_table):
                a = s.offset + self.dp_rank * stride
                e = min(s.offset + s.numel, a + stride)
                if a < e:
                    out.append((s, a, e, sh))
            return out
        lo, hi = self.owned_range()
        for s in self.slots:
            a, e = max(s.offset, lo), min(s.offset + s.numel, hi)
            if a < e:
                out.append((s, a, e, a - lo))
        return out

    @staticmethod
    def row_layout(slots: list, dp: int) -> tuple[list, int]:
        """Row sharding of a bucket: parameter ``[N, K]`` is cut into ``dp`` pieces of ``R = ceil(N / dp)`` rows
        rounded up to 64; returns ([(offset of the piece in a shard, elements per piece)], shard length)."""
        table, sh = [], 0
        for s in slots:
            n_rows = int(s.shape[0]) if len(s.shape) >= 1 else 1
            k = 1
            for d in s.shape[1:]:
                k *= int(d)
            rows = ((n_rows + dp - 1) // dp + 63) // 64 * 64
            table.append((sh, rows * k))
            sh += rows * k
        return table, sh

    def convert_to_rows(self, alloc: Callable) -> None:
        """Re-shard the optimizer state (and parameter shard) of this bucket by parameter rows.

        ``alloc(name, numel, dtype)`` returns the zeroed buffer for ``shard_params`` / ``shard_grads`` (the fused
        paths pass symmetric memory).  Must run before training or right after a checkpoint was loaded into the
        full parameters: master weights are re-derived from the current parameters, moments restart at zero.
        """
        full = self.full_param_tensor()
        table, shard = self.row_layout(self.slots, self.dp_degree)
        self.row_table = table
        self.shard_numel = shard
        self.master = torch.zeros(shard, dtype=torch.float32, device=self.device)
        self.m = torch.zeros(shard, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(shard, dtype=torch.float32, device=self.device)
        self.shard_params = alloc("shard_params", shard, self.dtype)
        self.shard_grads = alloc("shard_grads", shard, torch.float32)
        for s, a, e, sh in self.owned_pieces():
            self.master[sh:sh + e - a].copy_(full[a:e].to(torch.float32))
            self.shard_params[sh:sh + e - a].copy_(full[a:e])

    def _bind(self, flat: torch.Tensor) -> None:
        """Create the parameter tensors once: leaves over ``flat``'s storage with their own version counters,
        so collectives and the optimizer writing through ``flat`` never invalidate tensors autograd saved."""
        self.param_views = {}
        base = flat.data
        for s in self.slots:
            v = base[s.offset:s.offset + s.numel].view(s.shape)
            v.requires_grad_(True)
            self.param_views[s.pos] = v

    def _register_sinks(self) -> None:
        if self.flat_grads is None:
            return
        for s in self.slots:
            p = self.param_views.get(s.pos)
            if p is not None:
                ops_core.grad_sinks.register(p, self.flat_grads[s.offset:s.offset + s.numel])

    def _unregister_sinks(self) -> None:
        for p in self.param_views.values():
            ops_core.grad_sinks.unregister(p)

    # -------------------------------------------------- zero-3 life cycle
    def params_ready(self) -> bool:
        return self.numel == 0 or self.params_live

    def all_gather_params(self) -> None:
        """Materialise the full parameter buffer from the shards (zero3).

        The buffer keeps its tensor and storage objects across free/gather cycles (only the allocation behind the
        storage comes and goes), so parameter tensors saved by autograd in a forward pass are valid again in
        the backward pass after the next gather (``src/runtime.py:312-352`` uses the same device).
        """
        if self.numel == 0:
            return
        # lifetimes of chains that the schedule interleaves overlap: count users, gather once
        self.param_users += 1
        if self.params_live:
            return
        self.flat_params.untyped_storage().resize_(self.numel * self.flat_params.element_size())
        if self.row_table is not None:
            # row-sharded bucket outside a step (checkpoint load, inspection): the step itself gathers with the
            # peer-memory kernels
            self.flat_params.copy_(self._rebuild_from_rows())
        elif self.dp_degree > 1:
            dist.all_gather_into_tensor(self.flat_params, self.shard_params, group=self.dp_group)
        else:
            self.flat_params.copy_(self.shard_params)
        self.params_live = True
        self._register_sinks()

    def _rebuild_from_rows(self) -> torch.Tensor:
        """Full parameters of a row-sharded bucket: every rank contributes its pieces (a collective)."""
        mine = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        for _s, a, e, sh in self.owned_pieces():
            mine[a:e].copy_(self.shard_params[sh:sh + e - a])
        if self.dp_degree > 1:
            dist.all_reduce(mine, group=self.dp_group)
        return mine

    def free_params(self, consumer_stream=None) -> None:
        if self.numel == 0 or not self.params_sharded or not self.params_live:
            return
        self.param_users = max(self.param_users - 1, 0)
        if self.param_users > 0:
            return
        self._unregister_sinks()
        if consumer_stream is not None and self.flat_params.is_cuda:
            self.flat_params.record_stream(consumer_stream)
        if _POISON_FREED:
            # debug aid: a kernel that still reads these parameters after the free (a missing event or a wrong
            # ZeRO lifetime in the plan) then produces NaNs instead of silently using stale weights
            self.flat_params.fill_(float("nan"))
        self.flat_params.untyped_storage().resize_(0)
        self.params_live = False

    def alloc_grads(self) -> None:
        """Full-size fp32 gradient buffer of one ZeRO gradient chain (shared by chains that overlap in time)."""
        if self.numel == 0:
            return
        self.grad_users += 1
        if self.flat_grads is not None:
            return
        self.flat_grads = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self._register_sinks()

    def release_grads(self) -> bool:
        """A gradient chain ended.  Returns True when it was the last one using the buffer, i.e. when the
        reduce-scatter has to run now; an earlier chain's reduction is simply deferred to that point."""
        self.grad_users = max(self.grad_users - 1, 0)
        return self.grad_users == 0

    def free_grads(self, consumer_stream=None) -> None:
        if self.numel == 0 or not self.params_sharded or self.flat_grads is None or self.persistent_grads:
            return
        for p in self.param_views.values():
            ops_core.grad_sinks.unregister(p)
        if consumer_stream is not None and self.flat_grads.is_cuda:
            self.flat_grads.record_stream(consumer_stream)
        self.flat_grads = None

    # ------------------------------------------------------ grad handling
    def absorb_autograd_grads(self) -> None:
        """Fold ``.grad`` tensors that autograd produced (ops without a sink) into the flat buffer."""
        for s in self.slots:
            p = self.param_views.get(s.pos)
            if p is None or p.grad is None:
                continue
            sink = self.flat_grads[s.offset:s.offset + s.numel]
            g = p.grad.reshape(-1)
            if g.is_cuda and g.dtype == torch.bfloat16:
                native.lib().accum_bf16_into_f32(g.contiguous(), sink)
            else:
                sink.add_(g.to(torch.float32))
            p.grad = None

    def all_reduce_grads(self, per_tensor: bool = False) -> None:
        if self.numel == 0 or self.dp_degree <= 1:
            return
        if per_tensor:   # one call per parameter tensor, as the reference issues them
            for s in self.slots:
                dist.all_reduce(self.flat_grads[s.offset:s.offset + s.numel], group=self.dp_group)
        else:
            dist.all_reduce(self.flat_grads, group=self.dp_group)

    def reduce_scatter_grads(self) -> None:
        """shard_grads += reduce_scatter(flat_grads); the full buffer is zeroed or freed by the caller."""
        if self.numel == 0:
            return
        if self.dp_degree > 1:
            tmp = torch.empty(self.shard_numel, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(tmp, self.flat_grads, group=self.dp_group)
            self.shard_grads.add_(tmp)
        else:
            self.shard_grads.add_(self.flat_grads)

    # ------------------------------------------------------------- update
    def step(self, grad_scale: float) -> None:
        if self.numel == 0:
            return
        if self.row_table is not None:
            raise RuntimeError(f"bucket {self.key}: a row-sharded bucket is stepped by the fused reduction kernel")
        self.step_count += 1
        lo, hi = self.owned_range()
        grads = self.shard_grads if self.sharded_state else self.flat_grads[lo:hi]
        target = self.shard_params if (self.sharded_state or self.params_sharded) else self.flat_params[lo:hi]
        a = self.adam
        if grads.is_cuda and self.dtype == torch.bfloat16:
            native.lib().adam_flat(self.master, self.m, self.v, grads, target, a.lr, a.betas[0], a.betas[1], a.eps,
                                   a.weight_decay, self.step_count, grad_scale, a.decoupled)
        else:
            _adam_reference(self.master if self.master is not None else target, self.m, self.v, grads,
                            target if self.master is not None else None, a, self.step_count, grad_scale)
        if self.mode == "zero2" and self.dp_degree > 1 and self.params_live:
            # the reference never re-synchronises parameters after a sharded step
            # (``src/runtime.py:462-473``); replicas would drift, so gather them here
            dist.all_gather_into_tensor(self.flat_params, self.shard_params.contiguous(), group=self.dp_group)
        if self.shard_grads is not None:
            self.shard_grads.zero_()
        if self.flat_grads is not None:
            self.flat_grads.zero_()

    def snapshot_grads(self, scale: float) -> dict:
        """fqn -> scaled copy of the gradient this rank holds (full tensors, or its ZeRO shard as a flat range)."""
        out = {}
        if self.sharded_state:
            g = self.shard_grads * scale
            for s, a, e, sh in self.owned_pieces():
                out[s.fqn] = (a - s.offset, g[sh:sh + e - a].clone())
        elif self.flat_grads is not None:
            for s in self.slots:
                out[s.fqn] = (self.flat_grads[s.offset:s.offset + s.numel] * scale).view(s.shape).clone()
        return out

    # --------------------------------------------------------- checkpoint
    def full_param_tensor(self) -> torch.Tensor:
        if self.params_live:
            return self.flat_params
        flat = torch.empty(self.numel, dtype=self.dtype, device=self.device)
        if self.row_table is not None:
            return self._rebuild_from_rows()
        if self.dp_degree > 1:
            dist.all_gather_into_tensor(flat, self.shard_params, group=self.dp_group)
        else:
            flat.copy_(self.shard_params)
        return flat


def _adam_reference(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
                    param_out: Optional[torch.Tensor], a: AdamConfig, step: int, grad_scale: float) -> None:
    """The math of the flat Adam kernel in PyTorch ops (CPU runs and fp32 parameters)."""
    with torch.no_grad():
        g = grad * grad_scale
        if a.weight_decay and not a.decoupled:
            g = g + a.weight_decay * master
        m.mul_(a.betas[0]).add_(g, alpha=1 - a.betas[0])
        v.mul_(a.betas[1]).addcmul_(g, g, value=1 - a.betas[1])
        bc1 = 1 - a.betas[0] ** step
        bc2 = 1 - a.betas[1] ** step
        denom = (v / bc2).sqrt_().add_(a.eps)
        upd = (m / bc1) / denom
        if a.weight_decay and a.decoupled:
            upd = upd + a.weight_decay * master
        master.add_(upd, alpha=-a.lr)
        if param_out is not None:
            param_out.copy_(master)
