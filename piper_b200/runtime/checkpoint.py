"""Checkpoint / resume in a torch ``state_dict`` layout.

The reference has no checkpointing.  Layout written here, one file per rank plus metadata::

    <dir>/step_<N>/rank<r>.pt   {"model": {fqn: tensor}, "optimizer": {"state": {fqn: {"step", "exp_avg",
                                 "exp_avg_sq", "master"}}, "param_groups": [...]}, "shards": {fqn: (offset, numel,
                                 shape)}, "step": N, "layout": {...}}
    <dir>/step_<N>/meta.json    {"step": N, "world_size": W, "schedule": <directive JSON>}
    <dir>/latest                "step_<N>"

Keys are module-qualified parameter names recovered from the trace, so ``consolidate`` produces a dict that
``model.load_state_dict`` of the un-annotated model accepts, whatever pipeline / data / expert layout wrote
it.  Each rank writes only what it owns: full tensors for parameters it holds whole, its flat range for
optimizer state that is sharded over the data-parallel group, its expert slice for expert-parallel
weights.  Loading re-shards by name under the current schedule.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch
import torch.distributed as dist


def _rank_state(actor) -> dict:
    model, opt_state, shards = {}, {}, {}
    for b in actor.buckets.values():
        st = b.storage
        if st is None or st.numel == 0:
            continue
        flat = st.full_param_tensor()
        for s in st.slots:
            model[s.fqn] = flat[s.offset:s.offset + s.numel].view(s.shape).detach().cpu().clone()
        for s, a, e, sh in st.owned_pieces():
            key = s.fqn
            sl = slice(sh, sh + e - a)
            entry = {"step": st.step_count, "exp_avg": st.m[sl].cpu().clone(), "exp_avg_sq": st.v[sl].cpu().clone()}
            if getattr(st, "master", None) is not None:
                entry["master"] = st.master[sl].cpu().clone()
            opt_state[key] = entry
            shards[key] = {"offset": a - s.offset, "numel": e - a, "shape": tuple(s.shape),
                           "ep_index": s.ep_index, "ep_degree": s.ep_degree,
                           "full_shape": tuple(s.full_shape) if s.full_shape else tuple(s.shape)}
    a = actor.adam
    return {"model": model,
            "optimizer": {"state": opt_state, "param_groups": [{"lr": a.lr, "betas": tuple(a.betas), "eps": a.eps,
                                                                "weight_decay": a.weight_decay}]},
            "shards": shards}


def save_checkpoint(actor, directory: str, step: int, schedule: Optional[list] = None) -> str:
    d = os.path.join(directory, f"step_{step}")
    os.makedirs(d, exist_ok=True)
    state = _rank_state(actor)
    lay = actor.layout
    state.update({"step": step, "layout": {"global_rank": lay.global_rank, "pp_rank": lay.pp_rank,
                                           "dp_rank": lay.dp_rank, "world_size": lay.world_size}})
    torch.save(state, os.path.join(d, f"rank{lay.global_rank}.pt"))
    if dist.is_initialized():
        dist.barrier()
    if lay.global_rank == min(r for t in lay._tuples_as_written for r in t):
        with open(os.path.join(d, "meta.json"), "w", encoding="utf-8") as f:
            json.dump({"step": step, "world_size": lay.world_size, "schedule": schedule}, f)
        with open(os.path.join(directory, "latest"), "w", encoding="utf-8") as f:
            f.write(f"step_{step}")
    return d


def _resolve(directory: str) -> str:
    latest = os.path.join(directory, "latest")
    if os.path.exists(latest):
        with open(latest, encoding="utf-8") as f:
            return os.path.join(directory, f.read().strip())
    return directory


def consolidate(directory: str) -> dict:
    """Merge all rank files into {"model": {fqn: full tensor}, "optimizer": {...}, "step": N}."""
    d = _resolve(directory)
    model: dict = {}
    opt: dict = {}
    step = 0
    groups = None
    for name in sorted(os.listdir(d)):
        if not (name.startswith("rank") and name.endswith(".pt")):
            continue
        st = torch.load(os.path.join(d, name), map_location="cpu", weights_only=False)
        step = st.get("step", step)
        groups = st["optimizer"]["param_groups"]
        for k, t in st["model"].items():
            sh = st["shards"].get(k)
            if sh and sh["ep_degree"] > 1:
                full = model.setdefault(k, torch.zeros(sh["full_shape"], dtype=t.dtype))
                per = sh["full_shape"][0] // sh["ep_degree"]
                full[sh["ep_index"] * per:(sh["ep_index"] + 1) * per] = t
            else:
                model[k] = t
        for k, e in st["optimizer"]["state"].items():
            sh = st["shards"][k]
            numel = 1
            for x in sh["full_shape"]:
                numel *= x
            base = 0
            if sh["ep_degree"] > 1:
                base = sh["ep_index"] * (numel // sh["ep_degree"])
            dst = opt.setdefault(k, {"step": e["step"], "exp_avg": torch.zeros(numel), "exp_avg_sq": torch.zeros(numel),
                                     "master": torch.zeros(numel)})
            sl = slice(base + sh["offset"], base + sh["offset"] + sh["numel"])
            dst["exp_avg"][sl] = e["exp_avg"]
            dst["exp_avg_sq"][sl] = e["exp_avg_sq"]
            if "master" in e:
                dst["master"][sl] = e["master"]
            else:
                dst["master"][sl] = model[k].reshape(-1).float()[sl] if k in model else 0
    for k, e in opt.items():
        shape = model[k].shape
        for f in ("exp_avg", "exp_avg_sq", "master"):
            e[f] = e[f].view(shape)
    return {"model": model, "optimizer": {"state": opt, "param_groups": groups}, "step": step}


def load_checkpoint(actor, directory: str) -> int:
    """Load parameters and optimizer state by name into the actor's (possibly differently sharded) storage."""
    full = consolidate(directory)
    for b in actor.buckets.values():
        st = b.storage
        if st is None or st.numel == 0:
            continue
        pieces = {id(s): (a, z, sh) for s, a, z, sh in st.owned_pieces()}
        was_live = st.params_live
        if not was_live:
            st.all_gather_params()
        for s in st.slots:
            if s.fqn not in full["model"]:
                raise KeyError(f"checkpoint has no parameter {s.fqn!r}")
            t = full["model"][s.fqn]
            e = full["optimizer"]["state"].get(s.fqn)
            if s.ep_sharded:
                per = t.shape[0] // s.ep_degree
                sel = slice(s.ep_index * per, (s.ep_index + 1) * per)
                t = t[sel]
                if e is not None:
                    e = {k: (v[sel] if isinstance(v, torch.Tensor) else v) for k, v in e.items()}
            st.flat_params[s.offset:s.offset + s.numel].copy_(t.reshape(-1).to(st.dtype))
            if id(s) in pieces:
                a, z, sh = pieces[id(s)]
                own = slice(sh, sh + z - a)
                src = slice(a - s.offset, z - s.offset)
                if st.params_sharded or st.sharded_state or st.row_table is not None:
                    st.shard_params[own].copy_(t.reshape(-1)[src].to(st.dtype))
                if e is not None:
                    st.m[own].copy_(e["exp_avg"].reshape(-1)[src])
                    st.v[own].copy_(e["exp_avg_sq"].reshape(-1)[src])
                    if getattr(st, "master", None) is not None:
                        st.master[own].copy_(e["master"].reshape(-1)[src])
                    st.step_count = int(e["step"])
        if not was_live:
            st.free_params()
    actor.iteration = int(full["step"])
    return actor.iteration
