"""Compiler behaviour: graph split, directive engine, schedule loader, builders, ordering."""
import json

import pytest
import torch
import torch.fx as fx
import torch.nn as nn

from piper_b200.api import _reset_annotation_state, annotate, compile_training_dags
from piper_b200.compiler import directives as D
from piper_b200.compiler.builders import (build_1f1b_schedule, build_dualpipev_schedule,
                                          build_interleaved_1f1b_schedule, build_zerobubble_schedule, format_rows)
from piper_b200.compiler.dag import TrainingDAG, TrainingDAGEdge, TrainingDAGNode
from piper_b200.compiler.fxsplit import split_gm_by_annotations
from piper_b200.compiler.ordering import serial_topological_order
from piper_b200.compiler.schedule import load_schedule_directives, load_schedule_info


class _Net(nn.Module):
    def __init__(self, dim=8):
        super().__init__()
        self.fc1 = nn.Linear(dim, dim, bias=False)
        self.fc2 = nn.Linear(dim, dim, bias=False)
        self.fc3 = nn.Linear(dim, dim, bias=False)

    def forward(self, x):
        with annotate("PP"):
            x = torch.relu(self.fc1(x))
            with annotate("EP"):
                x = torch.relu(self.fc2(x))
        with annotate("PP"):
            return self.fc3(x)


def _capture(model, x):
    got = {}

    def backend(gm, example_inputs):
        got["gm"], got["inputs"] = gm, list(example_inputs)
        return gm.forward

    _reset_annotation_state()
    torch._dynamo.reset()
    with torch.no_grad():
        ref = torch.compile(model, backend=backend, fullgraph=True)(x).detach().clone()
    return got["gm"], got["inputs"], ref


def test_split_nested_annotations_and_reexecution():
    torch.manual_seed(0)
    model, x = _Net(), torch.randn(2, 8)
    gm, inputs, ref = _capture(model, x)
    _, segs = split_gm_by_annotations(gm)
    assert [s.tag for s in segs] == [{"PP": 0}, {"PP": 0, "EP": 0}, {"PP": 1}]
    assert [s.stage_id for s in segs] == [0, 0, 1]
    assert [s.a2a_boundary_after["from_tag"] for s in segs[:-1]] == [{"PP": 0}, {"PP": 0, "EP": 0}]
    assert [s.a2a_boundary_after["to_tag"] for s in segs[:-1]] == [{"PP": 0, "EP": 0}, {"PP": 1}]
    # the model input is a runtime input of segment 0, parameters are parameter slots with module FQNs
    assert len(segs[0].input_idxs) == 1 and len(segs[0].param_idxs) == 1
    assert [f for f in segs[0].param_fqns if f] == ["fc1.weight"]
    vals = {n.name: v for n, v in zip([n for n in gm.graph.nodes if n.op == "placeholder"], inputs)}
    prev = None
    for s in segs:
        acts = iter(() if prev is None else (prev if isinstance(prev, tuple) else (prev,)))
        args = [vals[p.name] if p.name in vals else next(acts) for p in s.gm.graph.nodes if p.op == "placeholder"]
        with torch.no_grad():
            prev = s.gm(*args)
    out = prev[0] if isinstance(prev, (tuple, list)) else prev
    assert torch.allclose(ref, out, atol=1e-6)


def test_split_ignores_foreign_custom_metadata_and_rejects_bare_compute():
    gm = fx.symbolic_trace(nn.Sequential(nn.ReLU()))
    next(n for n in gm.graph.nodes if n.op == "call_module").meta["custom"] = {"name": "PP", "index": 0}
    assert split_gm_by_annotations(gm)[1] == []
    gm2, _, _ = _capture(_Net(), torch.randn(2, 8))
    next(n for n in gm2.graph.nodes if n.op not in ("placeholder", "get_attr", "output")).meta.pop("custom", None)
    with pytest.raises(ValueError, match="without Piper annotations"):
        split_gm_by_annotations(gm2)


def _compute(uid, tag, kind="FWD", device=(0,), meta=None):
    return TrainingDAGNode(uid, "COMPUTE", kind, tag, list(device), "default_stream", dict(meta or {}))


def test_order_parsing_and_stencil():
    nested = {"op": "order", "filters": [[{"PP": 0, "MB": 0, "PASS": "F"}, {"PP": 0, "MB": 1, "PASS": "F"}],
                                         [{"PP": 0, "MB": 0, "PASS": "B"}]]}
    assert D.parse_order_directive(nested) == nested["filters"]
    with pytest.raises(ValueError, match="must be a non-empty list"):
        D.parse_order_directive({"op": "order", "filters": [{"PP": 0}, {"PP": 1}]})
    keys = D.validate_split_backward_order_stencil([{"op": "order", "filters": [
        [{"PP": 0, "MB": 0, "PASS": "BI"}, {"PP": 0, "MB": 0, "PASS": "BW"}], [{"PP": 0, "MB": 1, "PASS": "F"}]]}])
    assert keys == {(("MB", 0), ("PP", 0))}
    with pytest.raises(ValueError, match="exactly one BI and one BW"):
        D.validate_split_backward_order_stencil([{"op": "order", "filters": [[{"PP": 0, "PASS": "BI"}], [{"PP": 1, "PASS": "F"}]]}])


def test_mixed_fused_and_split_backward_microbatches():
    directive = {"op": "order", "filters": [[{"PP": 0, "MB": 0, "PASS": "B"}], [{"PP": 0, "MB": 1, "PASS": "BI"}],
                                            [{"PP": 0, "MB": 1, "PASS": "BW"}]]}
    dag = TrainingDAG()
    dag.add_node(_compute("fwd", {"PP": 0, "PASS": "F"}))
    dag.add_node(_compute("bwd", {"PP": 0, "PASS": "B"}, "BWD", meta={"fwd_uid": "fwd", "bucket_key": "fwd"}))
    dag.add_edge(TrainingDAGEdge("fwd", "bwd", "data"))
    keys = D.validate_split_backward_order_stencil([directive])
    D.apply_split_directive(dag, {}, "MB", 2)
    D.apply_split_backward_stencil(dag, keys)
    assert dag.nodes["bwd"].compute_subkind == "BWD" and dag.nodes["bwd"].tag["PASS"] == "B"
    assert dag.nodes["bwd.splitMB1"].compute_subkind == "BWD_I" and dag.nodes["bwd.splitMB1"].tag["PASS"] == "BI"
    assert dag.nodes["bwd.splitMB1.bw"].compute_subkind == "BWD_W"
    assert dag.nodes["bwd.splitMB1"].node_meta["fwd_uid"] == "fwd.splitMB1"


def _dummy_gm():
    g = fx.Graph()
    g.output(g.placeholder("x"))
    return fx.GraphModule({}, g)


def test_bucket_rewrite_follows_split_microbatches():
    dag = TrainingDAG()
    dag.add_node(_compute("fwd", {"PP": 0, "PASS": "F"}, meta={
        "stage_id": 0, "segment_id": 0, "gm": _dummy_gm(), "graphargs": [], "input_idxs": [], "param_idxs": []}))
    dag.add_node(_compute("bwd", {"PP": 0, "PASS": "B"}, "BWD", meta={"fwd_uid": "fwd", "bucket_key": "fwd"}))
    dag.add_edge(TrainingDAGEdge("fwd", "bwd", "data"))
    D.apply_split_directive(dag, {}, "MB", 2)
    D.bucket_matched_fwd_nodes(dag, [{"PP": 0}], 25,
                               lambda *a, **k: [(_dummy_gm(), [], [], []), (_dummy_gm(), [], [], [])])
    for uid in ("fwd.bucket0", "fwd.bucket0.bwd", "fwd.splitMB1.bucket0", "fwd.splitMB1.bucket1.bwd"):
        assert uid in dag.nodes
    assert dag.has_edge("fwd.bucket0", "fwd.bucket1", "data") and dag.has_edge("fwd.bucket1.bwd", "fwd.bucket0.bwd", "data")
    assert dag.has_edge("fwd.bucket1", "fwd.bucket1.bwd", "data")


def test_order_groups_use_dummy_source_and_sink():
    dag = TrainingDAG()
    for n in (_compute("prev", {"slot": 0}), _compute("lane0.first", {"slot": 1, "lane": 0}),
              _compute("lane0.last", {"slot": 1, "lane": 0}), _compute("lane1", {"slot": 1, "lane": 1}),
              _compute("next", {"slot": 2})):
        dag.add_node(n)
    dag.add_edge(TrainingDAGEdge("lane0.first", "lane0.last", "data"))
    D.apply_order_directive(dag, [[{"slot": 0}], [{"slot": 1, "lane": 0}, {"slot": 1, "lane": 1}], [{"slot": 2}]],
                            directive_idx=7)
    src, snk = "order.7.group1.source", "order.7.group1.sink"
    assert dag.nodes[src].node_kind == "ORDER_DUMMY" and dag.nodes[snk].node_kind == "ORDER_DUMMY"
    temporal = {(e.src_uid, e.dst_uid) for e in dag.edges if e.dep_kind == "temporal"}
    assert temporal == {("prev", src), (src, "lane0.first"), (src, "lane1"), ("lane0.last", snk), ("lane1", snk),
                        (snk, "next")}
    order = serial_topological_order(dag)
    assert order.index("prev") < order.index(src) < order.index("lane1") < order.index(snk) < order.index("next")


def test_order_rejects_dataflow_reversal_and_cross_device():
    dag = TrainingDAG()
    dag.add_node(_compute("producer", {"slot": 0}))
    dag.add_node(_compute("consumer", {"slot": 1}))
    dag.add_edge(TrainingDAGEdge("producer", "consumer", "data"))
    with pytest.raises(ValueError, match="violates model dataflow"):
        D.apply_order_directive(dag, [[{"slot": 1}], [{"slot": 0}]], directive_idx=3)
    dag2 = TrainingDAG()
    dag2.add_node(_compute("rank0", {"slot": 0}))
    dag2.add_node(_compute("rank1", {"slot": 1}, device=(1,)))
    with pytest.raises(ValueError, match="crosses device placement"):
        D.apply_order_directive(dag2, [[{"slot": 0}], [{"slot": 1}]], directive_idx=4)


def test_shard_drops_reduce_scatter_and_zero_metadata():
    dag = TrainingDAG()
    n = _compute("expert.bwd", {"PP": 0, "EP": 0, "PASS": "B"}, "BWD", (0, 2), {"bucket_key": "expert", "fwd_uid": "expert.fwd"})
    dag.add_node(n)
    D.insert_reduce_scatter_comm_nodes(dag, [{"PP": 0, "EP": 0}], [0, 2])
    assert n.node_meta["zero_alloc_full_grads_before"] is True
    assert any(x.node_kind == "REDUCE_SCATTER_COMM" for x in dag.nodes.values())
    D.insert_shard_a2a_comm_nodes(dag, [{"PP": 0, "EP": 0}], [0, 2])
    assert "zero_alloc_full_grads_before" not in n.node_meta
    assert not any(x.node_kind == "REDUCE_SCATTER_COMM" for x in dag.nodes.values())


def test_tag_validation_and_unmatched_place():
    dag = TrainingDAG()
    dag.add_node(_compute("fwd", {"PP": 0, "PASS": "F"}))
    with pytest.raises(ValueError, match="not found in model annotations"):
        D.validate_schedule_tags_exist(dag, [{"op": "place", "filter": {"TP": 0}, "devices": [0]}])
    D.validate_schedule_tags_exist(dag, [{"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2},
                                         {"op": "order", "filters": [[{"PP": 0, "MB": 0, "PASS": "F"}]]}])
    with pytest.raises(ValueError, match="matched zero nodes"):
        D.apply_schedule_directives(dag, [{"op": "place", "filter": {"PP": 1}, "devices": [0]}])


def test_schedule_loader(tmp_path):
    p = tmp_path / "qwen_example.json"
    p.write_text(json.dumps([{"op": "place", "filter": {"PP": 0}, "devices": [0, 1]},
                             {"op": "place", "filter": {"PP": 1}, "devices": [2, 3]},
                             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4}]))
    assert load_schedule_info(str(p)) == {"name": "qwen_example", "path": str(p), "num_stages": 2, "pp_degree": 2,
                                          "dp_degree": 2, "num_microbatches": 4}
    assert load_schedule_directives(str(p))[0]["filter"] == {"PP": 0}
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps([{"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": "__MBS__"}]))
    with pytest.raises(ValueError, match="__MBS__"):
        load_schedule_directives(str(bad))


def test_builder_golden_rows():
    assert format_rows(build_1f1b_schedule(2, 4)) == [
        "F0.0 F0.1 B0.0 F0.2 B0.1 F0.3 B0.2 B0.3", "F1.0 B1.0 F1.1 B1.1 F1.2 B1.2 F1.3 B1.3"]
    assert format_rows(build_zerobubble_schedule(2, 4)) == [
        "F0.0 F0.1 BI0.0 BW0.0 F0.2 BI0.1 BW0.1 F0.3 BI0.2 BW0.2 BI0.3 BW0.3",
        "F1.0 BI1.0 F1.1 BI1.1 BW1.0 F1.2 BI1.2 BW1.1 F1.3 BI1.3 BW1.2 BW1.3"]
    assert format_rows(build_interleaved_1f1b_schedule(2, 4, 2)) == [
        "F0.0 F0.1 F2.0 F2.1 F0.2 B2.0 F0.3 B2.1 F2.2 B0.0 F2.3 B0.1 B2.2 B2.3 B0.2 B0.3",
        "F1.0 F1.1 F3.0 B3.0 F3.1 B3.1 F1.2 B1.0 F1.3 B1.1 F3.2 B3.2 F3.3 B3.3 B1.2 B1.3"]
    assert format_rows(build_dualpipev_schedule(2, 4)) == [
        "F0.0 F0.1 F0.2 F3.0 BI3.0 BW3.0 F3.1 F0.3+B3.1 F3.2+B0.0 B3.2 F3.3+B0.1 B3.3 BI0.2 BW0.2 BI0.3 BW0.3",
        "F1.0 F2.0 F1.1 F2.1 F1.2 B2.0 F2.2+B1.0 F1.3+B2.1 F2.3+B1.1 B2.2 B1.2 BI2.3 BI1.3 BW2.3 BW1.3"]
    with pytest.raises(ValueError):
        build_dualpipev_schedule(2, 3)


class _TwoStage(nn.Module):
    def __init__(self, dim=8):
        super().__init__()
        self.a = nn.Linear(dim, dim, bias=False)
        self.b = nn.Linear(dim, dim, bias=False)

    def forward(self, x):
        with annotate("PP"):
            x = torch.relu(self.a(x))
        with annotate("PP"):
            return self.b(x)


def test_full_pipeline_pp2_dp2_1f1b_plan_shape():
    """PP2 x DP2 with all-reduce, 1F1B over 4 microbatches: 21 nodes per rank (4 F, 4 B, 4 SEND, 4 RECV, 4 AR, UPD)."""
    gm, _, _ = _capture(_TwoStage(), torch.randn(2, 8))
    directives = [
        {"op": "place", "filter": {"PP": 0}, "devices": [0, 2], "stream": "pp_stream"},
        {"op": "place", "filter": {"PP": 1}, "devices": [1, 3], "stream": "pp_stream"},
        {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 2], "reduce_stream": "dp_stream"},
        {"op": "replicate", "filter": {"PP": 1}, "devices": [1, 3], "reduce_stream": "dp_stream"},
        {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4},
        *build_1f1b_schedule(2, 4),
    ]
    dag, per_dev, _ = compile_training_dags(gm, directives)
    assert len(per_dev) == 2
    for sub in per_dev:
        kinds = [n.node_kind for n in sub.nodes.values()]
        assert len(kinds) == 21
        assert kinds.count("SEND_COMM") == 4 and kinds.count("RECV_COMM") == 4 and kinds.count("REDUCE_COMM") == 4
        order = serial_topological_order(sub)
        assert sub.nodes[order[-1]].node_kind == "UPD"
    r0 = [u for u in serial_topological_order(per_dev[0]) if per_dev[0].nodes[u].node_kind == "COMPUTE"]
    seq = [f"{per_dev[0].nodes[u].tag['PASS']}{per_dev[0].nodes[u].tag['MB']}" for u in r0]
    assert seq == ["F0", "F1", "B0", "F2", "B1", "F3", "B2", "B3"]


class _FourLinear(nn.Module):
    def __init__(self, dim=64):
        super().__init__()
        self.fcs = nn.ModuleList(nn.Linear(dim, dim, bias=False) for _ in range(4))

    def forward(self, x):
        with annotate("PP"):
            for fc in self.fcs:
                x = torch.relu(fc(x))
            return x


def test_bucket_stage_splits_by_parameter_bytes_and_reexecutes():
    from piper_b200.compiler.bucket import bucket_stage

    torch.manual_seed(0)
    model, x = _FourLinear(), torch.randn(2, 64)
    gm, inputs, ref = _capture(model, x)
    _, segs = split_gm_by_annotations(gm)
    seg = segs[0]
    one = 64 * 64 * 4
    buckets = bucket_stage(seg.gm, seg.graphargs, seg.input_idxs, seg.param_idxs, bucket_size_bytes=2 * one)
    assert len(buckets) == 2
    fqns = [[f for f in b[4] if f] for b in buckets]
    assert fqns == [["fcs.0.weight", "fcs.1.weight"], ["fcs.2.weight", "fcs.3.weight"]]
    vals = {n.name: v for n, v in zip([n for n in gm.graph.nodes if n.op == "placeholder"], inputs)}
    prev = None
    for bgm, b_in, b_par, _args, _f in buckets:
        phs = [n for n in bgm.graph.nodes if n.op == "placeholder"]
        acts = iter(() if prev is None else (prev if isinstance(prev, tuple) else (prev,)))
        args = [vals[p.name] if p.name in vals else next(acts) for p in phs]
        with torch.no_grad():
            prev = bgm(*args)
    out = prev[0] if isinstance(prev, (tuple, list)) else prev
    assert torch.allclose(out, ref, atol=1e-6)
    assert len(bucket_stage(seg.gm, seg.graphargs, seg.input_idxs, seg.param_idxs, bucket_size_bytes=100 * one)) == 1


def test_replicate_bucket_size_produces_bucket_chains_with_one_reduce_each():
    gm, _, _ = _capture(_FourLinear(), torch.randn(2, 64))
    directives = [
        {"op": "place", "filter": {"PP": 0}, "devices": [0, 1]},
        {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1], "reduce_stream": "dp_stream", "bucket_size": 1},
        {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2},
    ]
    # bucket_size is in MB: make the four 16 KiB weights exceed it by patching the limit through a tiny size
    from piper_b200.compiler import directives as DD
    import piper_b200.compiler.bucket as B
    orig = B.bucket_stage
    try:
        B.bucket_stage = lambda *a, **k: orig(*a, **{**k, "bucket_size_bytes": 2 * 64 * 64 * 4})
        dag, per_dev, _ = compile_training_dags(gm, directives)
    finally:
        B.bucket_stage = orig
    sub = per_dev[0]
    fwd = [u for u, n in sub.nodes.items() if n.node_kind == "COMPUTE" and n.compute_subkind == "FWD"]
    assert sorted(fwd) == sorted(f"s0.seg0{mb}.bucket{i}" for mb in ("", ".splitMB1") for i in (0, 1))
    reduces = [n for n in sub.nodes.values() if n.node_kind == "REDUCE_COMM"]
    assert len(reduces) == 4 and {n.node_meta["bucket_key"] for n in reduces} == {"s0.seg0.bucket0", "s0.seg0.bucket1"}


def test_fx_json_roundtrip_of_traced_segments():
    """Segments of the tiny Llama survive JSON serialisation and compute the same outputs."""
    from piper_b200.compiler import fxserial
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.runtime.storage import materialize_module

    cfg = LLAMA_CONFIGS["tiny"]
    model = Transformer(cfg, 32, 2)
    model.load_const_attrs(32)
    materialize_module(model)
    x = torch.randint(0, cfg.vocab_size, (2, 32))
    gm, inputs, ref = _capture(model, x)
    _, segs = split_gm_by_annotations(gm)
    vals = {n.name: v for n, v in zip([n for n in gm.graph.nodes if n.op == "placeholder"], inputs)}
    prev = None
    for s in segs:
        clone = fxserial.loads(fxserial.dumps(s.gm))
        phs = [p for p in clone.graph.nodes if p.op == "placeholder"]
        acts = iter(() if prev is None else (prev if isinstance(prev, tuple) else (prev,)))
        args = [vals[p.name] if p.name in vals else next(acts) for p in phs]
        with torch.no_grad():
            prev = clone(*args)
    out = prev[0] if isinstance(prev, (tuple, list)) else prev
    assert torch.allclose(out, ref, atol=1e-5)


# ------------------------------------------------------------------ plan checker
def _plan(nodes, edges):
    """nodes: (uid, kind, stream, meta); edges: (src, dst, dep_kind)."""
    dag = TrainingDAG()
    for uid, kind, stream, meta in nodes:
        dag.add_node(TrainingDAGNode(uid=uid, node_kind=kind, compute_subkind="FWD" if kind == "COMPUTE" else None,
                                     tag={}, device=[0], stream=stream, node_meta=dict(meta)))
    for s, d, k in edges:
        dag.add_edge(TrainingDAGEdge(s, d, k))
    return dag


def test_plan_checker_accepts_compiled_schedules_and_finds_defects():
    from piper_b200.compiler.check import PlanError, check_plans
    from piper_b200.engine import assign_pipeline_channels

    gm, _, _ = _capture(_TwoStage(), torch.randn(2, 8))
    for order_rows in (build_1f1b_schedule(2, 4), build_zerobubble_schedule(2, 4)):
        directives = [
            {"op": "place", "filter": {"PP": 0}, "devices": [0], "stream": "pp_stream"},
            {"op": "place", "filter": {"PP": 1}, "devices": [1], "stream": "pp_stream"},
            {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4},
            *order_rows,
        ]
        dag, per_dev, _ = compile_training_dags(gm, directives)
        assign_pipeline_channels(dag, per_dev, [(0,), (1,)])
        stats = check_plans(per_dev)
        assert stats["ranks"] == 2 and stats["messages"] == 8
    # swapped receives of one channel on rank 1: messages would be delivered to the wrong microbatch
    order1 = serial_topological_order(per_dev[1])
    recvs = [u for u in order1 if per_dev[1].nodes[u].node_kind == "RECV_COMM"
             and per_dev[1].nodes[u].node_meta["channel_base"][4] == per_dev[1].nodes[
                 next(v for v in order1 if per_dev[1].nodes[v].node_kind == "RECV_COMM")].node_meta["channel_base"][4]]
    i, j = order1.index(recvs[0]), order1.index(recvs[1])
    swapped = list(order1)
    swapped[i], swapped[j] = swapped[j], swapped[i]
    with pytest.raises(PlanError):
        check_plans(per_dev, [serial_topological_order(per_dev[0]), swapped])

    # hand-built deadlock: each rank queues, on its compute stream, the consumer of the peer's message in front of
    # the producer of its own message
    ch_a, ch_b = ((0,), (1,), 0, 1, "F"), ((1,), (0,), 1, 0, "F")
    r0 = _plan([("x0", "COMPUTE", "default_stream", {}), ("f0", "COMPUTE", "default_stream", {}),
                ("send_a", "SEND_COMM", "pp", {"channel_base": ch_a, "pair_uid": "recv_a"}),
                ("recv_b", "RECV_COMM", "pp", {"channel_base": ch_b})],
               [("f0", "send_a", "data"), ("recv_b", "x0", "data")])
    r1 = _plan([("x1", "COMPUTE", "default_stream", {}), ("f1", "COMPUTE", "default_stream", {}),
                ("send_b", "SEND_COMM", "pp", {"channel_base": ch_b, "pair_uid": "recv_b"}),
                ("recv_a", "RECV_COMM", "pp", {"channel_base": ch_a})],
               [("f1", "send_b", "data"), ("recv_a", "x1", "data")])
    good = [["f0", "send_a", "recv_b", "x0"], ["f1", "send_b", "recv_a", "x1"]]
    assert check_plans([r0, r1], good)["messages"] == 2
    bad = [["recv_b", "x0", "f0", "send_a"], ["recv_a", "x1", "f1", "send_b"]]
    with pytest.raises(PlanError, match="deadlock"):
        check_plans([r0, r1], bad)
    with pytest.raises(PlanError, match="dispatched before"):
        check_plans([r0, r1], [["send_a", "f0", "recv_b", "x0"], good[1]])
