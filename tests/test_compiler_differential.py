"""Differential test against the reference compiler, when its source tree is present.

The reference's compiler modules (``src/{fx,dag,directives,ordering,zero,piper}.py``) run without Ray once a
``ray`` module can be imported (the stand-in under ``baseline/ray_shim`` is enough: nothing of Ray is called at
compile time).  Both compilers get the same annotated toy mixture-of-experts model and the same directive
programs; for every pipeline rank the test compares the dispatch sequence (node kind, tags, devices, stream) and
the edge set with node identities replaced by dispatch positions, so uid spelling does not matter.
"""
import importlib
import importlib.util
import json
import os
import sys

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: named explicitly, installed for the comparison arm, or a sibling of this repository
CANDIDATES = [os.environ.get("PIPER_REFERENCE_DIR", ""), os.path.join(os.path.dirname(ROOT), "reference"),
              os.path.join(ROOT, "baseline", "_ref")]


def _reference_root():
    for c in CANDIDATES:
        if c and os.path.isfile(os.path.join(c, "src", "directives.py")):
            return c
    return None


REF = _reference_root()
pytestmark = pytest.mark.skipif(REF is None, reason="the reference source tree is not available")


def _load_reference():
    """Import the reference's ``src`` package under another name (this repository has its own ``src``)."""
    from piper_b200 import api  # noqa: F401  (registers this framework's Dynamo backend first)
    import torch._dynamo.backends.registry as reg

    if "refsrc" in sys.modules:
        return sys.modules["refsrc"]
    if importlib.util.find_spec("ray") is None:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "ray_shim"))
    # both packages register a Dynamo backend called "piper": park ours while the reference registers its own
    tables = [getattr(reg, k) for k in ("_COMPILER_FNS", "_BACKENDS") if isinstance(getattr(reg, k, None), dict)]
    parked = [t.pop("piper", None) for t in tables]
    src = os.path.join(REF, "src")
    spec = importlib.util.spec_from_file_location("refsrc", os.path.join(src, "__init__.py"),
                                                  submodule_search_locations=[src])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["refsrc"] = mod
    spec.loader.exec_module(mod)
    importlib.import_module("refsrc.piper")
    for t, v in zip(tables, parked):
        if v is not None:
            t["piper"] = v
    return mod


def _make_model(annotate, stages: int):
    class Block(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.a = nn.Linear(d, d, bias=False)
            self.e = nn.Linear(d, d, bias=False)
            self.o = nn.Linear(d, d, bias=False)

        def forward(self, x):
            x = x + torch.relu(self.a(x))
            r = torch.relu(self.a(x)) * 0.5
            with annotate("EP"):
                r = torch.relu(self.e(r))
            return x + self.o(r)

    class Net(nn.Module):
        def __init__(self, d=16):
            super().__init__()
            self.blocks = nn.ModuleList(Block(d) for _ in range(stages))
            self.head = nn.Linear(d, d, bias=False)

        def forward(self, x):
            for i, b in enumerate(self.blocks):
                with annotate("PP"):
                    x = b(x)
                    if i == stages - 1:
                        x = self.head(x)
            return x

    return Net


def _canon(dag, order):
    pos = {n.uid: i for i, n in enumerate(order)}
    seq = []
    for n in order:
        tag = {k: v for k, v in sorted(n.tag.items()) if v is not None}
        seq.append((n.compute_subkind or n.node_kind, tuple(tag.items()),
                    tuple(sorted(n.device)) if n.device is not None else None, n.stream))
    edges = sorted((pos[e.src_uid], pos[e.dst_uid], e.dep_kind) for e in dag.edges
                   if e.src_uid in pos and e.dst_uid in pos)
    # a forward node and its own backward node: this framework records that dependency (saved activations) as
    # a data edge for every pair, the reference only for the last forward segment of the last stage
    pairs = {(pos[e.src_uid], pos[e.dst_uid], e.dep_kind) for e in dag.edges
             if e.src_uid in pos and e.dst_uid in pos
             and (dag.nodes[e.dst_uid].node_meta or {}).get("fwd_uid") == e.src_uid}
    return seq, edges, pairs


def _compile_reference(ref, path, stages):
    rp = importlib.import_module("refsrc.piper")
    meta = importlib.import_module("refsrc.state").piper_metadata
    sched = importlib.import_module("refsrc.schedule")
    order_of = importlib.import_module("refsrc.ordering")._serial_topological_order
    d = sched.load_schedule_directives(path)
    meta.schedule_directives, meta.schedule_info, meta.visualize_dag = d, sched.derive_schedule_info(d, path), False
    torch._dynamo.reset()
    rp._reset_annotation_state()
    with torch.device("meta"):
        m = _make_model(rp.annotate, stages)()
    torch.compile(m, backend=rp.piper, fullgraph=True)(torch.empty(4, 16, device="meta"))
    return [_canon(dag, [dag.nodes[u] for u in order_of(dag)]) for dag in meta.per_pp_training_dags]


def _compile_ours(path, stages):
    from piper_b200 import api
    from piper_b200.compiler.ordering import serial_topological_order
    from piper_b200.compiler.schedule import derive_schedule_info, load_schedule_directives
    from piper_b200.state import piper_metadata as meta

    d = load_schedule_directives(path)
    meta.schedule_directives, meta.schedule_info = d, derive_schedule_info(d, path)
    torch._dynamo.reset()
    api._reset_annotation_state()
    with torch.device("meta"):
        m = _make_model(api.annotate, stages)()
    with torch.no_grad():
        torch.compile(m, backend=api.piper, fullgraph=True)(torch.empty(4, 16, device="meta"))
    return [_canon(dag, [dag.nodes[u] for u in serial_topological_order(dag)]) for dag in meta.per_pp_training_dags]


def _schedule(tmp_path, base, builder, ranks, mbs, **kw):
    sys.path.insert(0, os.path.join(REF, "examples"))
    try:
        bs = importlib.import_module("build_schedule")
    finally:
        sys.path.pop(0)
    src = os.path.join(REF, "examples", "base-schedules", base)
    if not os.path.isfile(src):          # an installed copy has no data files: this repository ships the same names
        src = os.path.join(ROOT, "examples", "base-schedules", base)
    with open(src) as f:
        prog = json.load(f)
    if builder is not None:              # otherwise the file's own split and order rows are the program
        prog = [d for d in prog if d.get("op") not in ("order", "split")]
        prog.append({"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": mbs})
        prog += getattr(bs, builder)(ranks, mbs, **kw)
    path = tmp_path / f"{builder}_{base}"
    path.write_text(json.dumps(prog))
    return str(path)


CASES = [
    ("pp2_dp2_ep2.json", "build_1f1b_schedule", 2, 2, 2, {}),
    ("pp2_dp2_ep2.json", "build_zerobubble_schedule", 2, 2, 4, {}),
    ("pp2_dp2_ep2_zero2.json", "build_1f1b_schedule", 2, 2, 2, {}),
    ("pp2_dp2_ep2_zero3.json", "build_1f1b_schedule", 2, 2, 2, {}),
    ("pp4_dp2_ep2_interleaved.json", "build_interleaved_1f1b_schedule", 4, 2, 4, {"n_virtual_stages": 2}),
    ("pp4_dp2_ep2_v_placement.json", "build_dualpipev_schedule", 4, 2, 4, {}),
    ("pp2_dp2_ep2_bucket100.json", "build_1f1b_schedule", 2, 2, 2, {}),
    ("dp2.json", "build_1f1b_schedule", 1, 1, 2, {}),
    ("pp2_dp2_ep2_custom_order.json", None, 2, 2, 0, {}),
]


@pytest.mark.parametrize("base,builder,stages,ranks,mbs,kw", CASES)
def test_same_plans_as_the_reference_compiler(tmp_path, base, builder, stages, ranks, mbs, kw):
    ref = _load_reference()
    path = _schedule(tmp_path, base, builder, ranks, mbs, **kw)
    theirs = _compile_reference(ref, path, stages)
    ours = _compile_ours(path, stages)
    assert len(ours) == len(theirs) == ranks
    for r, ((seq_o, edges_o, pairs), (seq_t, edges_t, _)) in enumerate(zip(ours, theirs)):
        assert len(seq_o) == len(seq_t), (r, len(seq_o), len(seq_t))
        assert seq_o == seq_t, (r, [i for i, (a, b) in enumerate(zip(seq_o, seq_t)) if a != b][:5])
        assert set(edges_t) <= set(edges_o), (r, sorted(set(edges_t) - set(edges_o))[:10])
        assert set(edges_o) - pairs == set(edges_t) - pairs, (r, sorted(set(edges_o) ^ set(edges_t))[:10])


def test_golden_dispatch_trace_of_rank_zero(tmp_path):
    """29 nodes: 6 FWD, 6 BWD, 8 exchanges, 4 all-reduces, 2 sends, 2 receives, 1 update, in the recorded order."""
    path = _schedule(tmp_path, "pp2_dp2_ep2.json", "build_1f1b_schedule", 2, 2)
    _load_reference()
    seq, _, _ = _compile_ours(path, 2)[0]
    kinds = [(k, dict(t).get("MB")) for k, t, _d, _s in seq]
    want = ("FWD0 A2A_COMM0 FWD0 A2A_COMM0 FWD0 SEND_COMM0 FWD1 A2A_COMM1 FWD1 A2A_COMM1 FWD1 SEND_COMM1 "
            "RECV_COMM0 BWD0 RECV_COMM1 A2A_COMM0 REDUCE_COMM0 BWD0 A2A_COMM0 BWD0 REDUCE_COMM0 "
            "BWD1 A2A_COMM1 REDUCE_COMM1 BWD1 A2A_COMM1 BWD1 REDUCE_COMM1 UPDNone").split()
    assert [f"{k}{mb}" for k, mb in kinds] == want
    streams = [s for _k, _t, _d, s in seq]
    assert (streams.count("default_stream"), streams.count("ep_stream"), streams.count("pp_stream"),
            streams.count("dp_stream")) == (13, 8, 4, 4)
