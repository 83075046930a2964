"""JSON (de)serialisation of segment ``GraphModule`` s.

Every rank of this runtime traces and compiles for itself, so graphs never have to travel; the serialiser
exists for debug dumps (``--viz`` writes each segment's graph next to the DAG) and for tools that want to
inspect or replay a compiled plan offline.  The reference ships its graphs through Ray with the same kind of
encoding (``src/fx.py:17-329``): nodes in order, targets by kind, arguments with explicit encodings for node
references, dtypes, devices, slices and nested containers.
"""
from __future__ import annotations

import importlib
import json
import operator
from typing import Any

import torch
import torch.fx as fx


def _encode_target(node: fx.Node) -> dict:
    t = node.target
    if isinstance(t, str):
        return {"kind": "string", "value": t}
    if isinstance(t, torch._ops.OpOverload):
        return {"kind": "torch_op", "value": f"{t.namespace}::{t._schema.name.split('::')[-1]}", "overload": t._overloadname}
    if isinstance(t, torch._ops.OpOverloadPacket):
        ns, name = t._qualified_op_name.split("::")
        return {"kind": "torch_op", "value": f"{ns}::{name}", "overload": None}
    mod, qual = getattr(t, "__module__", None), getattr(t, "__qualname__", getattr(t, "__name__", None))
    if mod and qual:
        return {"kind": "py_func", "module": mod, "qualname": qual}
    raise TypeError(f"cannot serialise call target {t!r} of node {node.name}")


def _decode_target(d: dict):
    k = d["kind"]
    if k == "string":
        return d["value"]
    if k == "torch_op":
        ns, name = d["value"].split("::")
        packet = getattr(getattr(torch.ops, ns), name)
        return getattr(packet, d["overload"]) if d.get("overload") else packet
    if k == "py_func":
        mod = d["module"]
        if mod in ("_operator", "operator"):
            return getattr(operator, d["qualname"])
        obj: Any = importlib.import_module(mod if not mod.startswith("torch._C") else "torch")
        for part in d["qualname"].split("."):
            obj = getattr(obj, part)
        return obj
    raise ValueError(f"unknown target kind {k}")


def _encode_arg(a: Any) -> Any:
    if isinstance(a, fx.Node):
        return {"__node__": a.name}
    if isinstance(a, (list, tuple)):
        return {"__seq__": "tuple" if isinstance(a, tuple) else "list", "items": [_encode_arg(x) for x in a]}
    if isinstance(a, dict):
        return {"__dict__": {k: _encode_arg(v) for k, v in a.items()}}
    if isinstance(a, torch.dtype):
        return {"__dtype__": str(a).split(".")[-1]}
    if isinstance(a, torch.device):
        return {"__device__": str(a)}
    if isinstance(a, slice):
        return {"__slice__": [_encode_arg(a.start), _encode_arg(a.stop), _encode_arg(a.step)]}
    if isinstance(a, torch.memory_format):
        return {"__memory_format__": str(a).split(".")[-1]}
    if a is None or isinstance(a, (bool, int, float, str)):
        return a
    if a is Ellipsis:
        return {"__ellipsis__": True}
    raise TypeError(f"cannot serialise argument {a!r}")


def _decode_arg(a: Any, env: dict) -> Any:
    if isinstance(a, dict):
        if "__node__" in a:
            return env[a["__node__"]]
        if "__seq__" in a:
            items = [_decode_arg(x, env) for x in a["items"]]
            return tuple(items) if a["__seq__"] == "tuple" else items
        if "__dict__" in a:
            return {k: _decode_arg(v, env) for k, v in a["__dict__"].items()}
        if "__dtype__" in a:
            return getattr(torch, a["__dtype__"])
        if "__device__" in a:
            return torch.device(a["__device__"])
        if "__slice__" in a:
            return slice(*[_decode_arg(x, env) for x in a["__slice__"]])
        if "__memory_format__" in a:
            return getattr(torch, a["__memory_format__"])
        if "__ellipsis__" in a:
            return Ellipsis
    return a


def serialize_graphmodule(gm: fx.GraphModule) -> dict:
    nodes = []
    for n in gm.graph.nodes:
        rec = {"op": n.op, "name": n.name, "args": _encode_arg(tuple(n.args)), "kwargs": _encode_arg(dict(n.kwargs))}
        if n.op in ("call_function", "call_method", "call_module", "get_attr", "placeholder"):
            rec["target"] = _encode_target(n) if n.op in ("call_function",) else {"kind": "string", "value": str(n.target)}
        if n.meta.get("piper_fqn"):
            rec["fqn"] = n.meta["piper_fqn"]
        nodes.append(rec)
    state = {k: {"dtype": str(v.dtype).split(".")[-1], "shape": list(v.shape), "data": v.detach().cpu().tolist()}
             for k, v in gm.state_dict().items()}
    return {"nodes": nodes, "state_dict": state}


def deserialize_graphmodule(data: dict) -> fx.GraphModule:
    g = fx.Graph()
    env: dict = {}
    for rec in data["nodes"]:
        op = rec["op"]
        args = _decode_arg(rec["args"], env)
        kwargs = _decode_arg(rec["kwargs"], env)
        if op == "placeholder":
            node = g.placeholder(rec["name"])
            if rec.get("fqn"):
                node.meta["piper_fqn"] = rec["fqn"]
        elif op == "output":
            node = g.output(args[0])
        elif op == "get_attr":
            node = g.get_attr(rec["target"]["value"])
        elif op == "call_function":
            node = g.call_function(_decode_target(rec["target"]), args, kwargs)
        elif op == "call_method":
            node = g.call_method(rec["target"]["value"], args, kwargs)
        else:
            raise ValueError(f"cannot rebuild node kind {op}")
        node.name = rec["name"]
        env[rec["name"]] = node
    root = torch.nn.Module()
    for k, v in data.get("state_dict", {}).items():
        root.register_buffer(k.replace(".", "_"), torch.tensor(v["data"], dtype=getattr(torch, v["dtype"])).reshape(v["shape"]))
    g.lint()
    return fx.GraphModule(root, g)


def dumps(gm: fx.GraphModule) -> str:
    return json.dumps(serialize_graphmodule(gm))


def loads(text: str) -> fx.GraphModule:
    return deserialize_graphmodule(json.loads(text))


_serialize_graphmodule = serialize_graphmodule
_deserialize_graphmodule = deserialize_graphmodule
