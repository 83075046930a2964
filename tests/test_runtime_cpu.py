"""Harness, coordinator / health monitoring, checkpointing, visualisation and trace merging on CPU."""
import importlib.util
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
SEQ = 64


# ----------------------------------------------------------------- harness
def test_harness_dry_run_writes_schedule_and_prints_command(tmp_path):
    cmd = [sys.executable, str(ROOT / "examples" / "test_harness.py"), "--test-file", str(ROOT / "examples" / "test_qwen.py"),
           "--base-schedule", str(ROOT / "examples" / "base-schedules" / "pp4_dp2_ep2_v_placement.json"),
           "--schedule", "dualpipev", "--ranks", "2", "--mbs", "4", "--dry-run", "--viz", "--out-root", str(tmp_path),
           "--model", "9M"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    gen = [l for l in out.stdout.splitlines() if l.startswith("generated_schedule=")][0].split("=", 1)[1]
    sched = json.load(open(gen))
    assert Path(gen).name == "dualpipev_pp2_mbs4.json"
    assert sum(1 for d in sched if d["op"] == "order") == 2
    assert [d for d in sched if d["op"] == "split"][0]["num_microbatches"] == 4
    assert any(l.startswith("schedule_viz=") for l in out.stdout.splitlines())
    # a generated order that crosses the placement is rejected
    bad = cmd.copy()
    bad[bad.index(str(ROOT / "examples" / "base-schedules" / "pp4_dp2_ep2_v_placement.json"))] = \
        str(ROOT / "examples" / "base-schedules" / "pp4_dp2_ep2_interleaved.json")
    out2 = subprocess.run(bad, capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert out2.returncode != 0 and "not compatible with the base placement" in out2.stderr


# ------------------------------------------------------- health monitoring
def _train_fn(args, pg):
    """Two data-parallel CPU ranks training a tiny Llama; honours PIPER_FAULT."""
    import torch
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.models.llama3 import LlamaConfig, Transformer
    from piper_b200.nn import cross_entropy_loss

    cfg = LlamaConfig(dim=64, n_layers=2, n_heads=2, n_kv_heads=2, vocab_size=128, ffn_hidden=128, max_seq_len=SEQ)
    x = torch.randint(0, 128, (4, SEQ))
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0, 1]},
             {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1], "reduce_stream": "dp_stream"},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    piper_setup(Transformer, (cfg, SEQ, 1), optim_fn=torch.optim.Adam, example_inputs=[x], example_outputs=x,
                model_dtype=torch.float32, const_attrs=Transformer.const_attrs(cfg, SEQ), schedule_directives=sched,
                device="cpu")
    losses = []
    for _ in range(args["steps"]):
        losses.append(float(piper_exec_dag(cross_entropy_loss, step_timeout=args.get("step_timeout"))[0]))
    return losses


def test_fault_injection_fails_fast_and_names_the_rank(monkeypatch):
    from piper_b200.runtime.launcher import Coordinator, JobFailed

    monkeypatch.setenv("PIPER_FAULT", "bwd:1:1")
    coord = Coordinator(world_size=2)
    t0 = time.time()
    with pytest.raises(JobFailed) as ei:
        coord.run_program(_train_fn, {"steps": 50}, timeout=240)
    assert 1 in ei.value.result.failures and "PIPER_FAULT fired" in ei.value.result.failures[1]
    assert time.time() - t0 < 200      # the healthy rank was stopped, not left waiting in a collective


def test_healthy_job_returns_results_and_heartbeats():
    from piper_b200.runtime.launcher import Coordinator

    job = Coordinator(world_size=2, hang_timeout=120).run_program(_train_fn, {"steps": 2}, timeout=240)
    assert job.ok and all(len(r) == 2 for r in job.results) and not job.hung
    assert job.results[0][1] < job.results[0][0] + 0.5


def test_sleeping_rank_is_reported_as_hung(monkeypatch):
    from piper_b200.runtime.launcher import Coordinator

    monkeypatch.setenv("PIPER_FAULT", "bwd:1:0:sleep:60")
    coord = Coordinator(world_size=2, hang_timeout=8, kill_on_hang=True)
    job = coord.run_program(_train_fn, {"steps": 3, "step_timeout": 2.0}, timeout=240, raise_on_failure=False)
    assert not job.ok and job.hung, job


def test_fault_spec_parsing():
    from piper_b200.runtime.faults import FaultInjector, InjectedFault, parse_fault_spec

    s = parse_fault_spec("bwd:3:1:sleep:2.5")
    assert (s.point, s.iteration, s.dp_rank, s.action, s.seconds) == ("bwd", 3, 1, "sleep", 2.5)
    assert parse_fault_spec("") is None
    with pytest.raises(ValueError):
        parse_fault_spec("fwd:1:0")
    inj = FaultInjector(1, parse_fault_spec("bwd:2:1"))
    inj.maybe_fire("bwd", 1)
    with pytest.raises(InjectedFault):
        inj.maybe_fire("bwd", 2)
    inj.maybe_fire("bwd", 2)        # latched: fires once


# ------------------------------------------------------------- checkpoint
def _ckpt_worker(rank, world, schedule, dp, ckpt_dir, mode):
    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.compiler.schedule import stage_device_map
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime.checkpoint import load_checkpoint, save_checkpoint
    from piper_b200.runtime.layout import make_layout

    cfg = LLAMA_CONFIGS["tiny"]
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, 129), generator=g)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    lay = make_layout(stage_device_map(schedule), rank, world)
    per = 4 // dp
    xs, ys = x[lay.dp_rank * per:(lay.dp_rank + 1) * per], y[lay.dp_rank * per:(lay.dp_rank + 1) * per]
    actor = piper_setup(Transformer, (cfg, 128, len(stage_device_map(schedule))), optim_fn=torch.optim.Adam,
                        example_inputs=[xs], example_outputs=ys, model_dtype=torch.float32,
                        const_attrs=Transformer.const_attrs(cfg, 128), schedule_directives=schedule, device="cpu")
    out = []
    if mode == "save":
        for _ in range(2):
            out.append(sum(float(v) for v in piper_exec_dag(cross_entropy_loss)))
        save_checkpoint(actor, ckpt_dir, step=2, schedule=schedule)
        out.append(sum(float(v) for v in piper_exec_dag(cross_entropy_loss)))     # step 3 of the original run
    else:
        assert load_checkpoint(actor, ckpt_dir) == 2
        out.append(sum(float(v) for v in piper_exec_dag(cross_entropy_loss)))     # step 3 after resume
    return out


def test_checkpoint_resume_under_a_different_layout(tmp_path):
    """Save from DP2 with ZeRO-3, resume on PP2: the third step's loss is the same."""
    from tests.dist_utils import run_ranks
    from piper_b200.compiler.builders import build_1f1b_schedule
    from piper_b200.runtime.checkpoint import consolidate

    ck = str(tmp_path / "ckpt")
    zero3 = [{"op": "place", "filter": {"PP": 0}, "devices": [0, 1]},
             {"op": "replicate", "filter": {"PP": 0}, "devices": [0, 1], "gather_stream": "dp_stream",
              "reduce_stream": "dp_stream", "shard_grads": True, "shard_params": True},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    (tmp_path / "a").mkdir()
    saved = run_ranks(2, _ckpt_worker, (zero3, 2, ck, "save"), tmp_path / "a")
    full = consolidate(ck)
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    model = Transformer(LLAMA_CONFIGS["tiny"], 128, 1)
    missing, unexpected = model.load_state_dict(full["model"], strict=False)
    assert not unexpected and all("rope" in m for m in missing)
    assert set(full["optimizer"]["state"]) == set(full["model"]) and full["step"] == 2
    pp2 = [{"op": "place", "filter": {"PP": 0}, "devices": [0], "stream": "pp_stream"},
           {"op": "place", "filter": {"PP": 1}, "devices": [1], "stream": "pp_stream"},
           {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4}, *build_1f1b_schedule(2, 4)]
    (tmp_path / "b").mkdir()
    resumed = run_ranks(2, _ckpt_worker, (pp2, 1, ck, "load"), tmp_path / "b")
    step3_saved = (saved[0][2] + saved[1][2]) / 4          # 2 ranks x 2 microbatch losses
    step3_resumed = sum(r[0] for r in resumed if r) / 4     # 4 microbatch losses on the last stage
    assert abs(step3_saved - step3_resumed) < 2e-4, (step3_saved, step3_resumed)


# ------------------------------------------------------------ viz / traces
def test_viz_outputs_and_trace_relabel(tmp_path):
    from piper_b200.compiler.builders import build_dualpipev_schedule
    from piper_b200.compiler.dag import TrainingDAG, TrainingDAGNode
    from piper_b200.compiler.viz import (compute_columns, print_training_dag_order, render_training_dag,
                                         visualize_order_directives)
    from piper_b200.runtime.profiler import relabel_gpu_events

    order = build_dualpipev_schedule(2, 4)
    path = visualize_order_directives(order, tmp_path / "grid.png")
    text = open(path if path.endswith(".dot") else str(tmp_path / "grid.dot")).read()
    assert "F0.3<BR/>B3.1" in text and "rank 1" in text
    cols = compute_columns([d["filters"] for d in order])
    assert all(c == sorted(c) for c in cols) and cols[1][0] > cols[0][0]      # stage 1 starts after stage 0
    dag = TrainingDAG()
    for u in ("a", "b"):
        dag.add_node(TrainingDAGNode(u, "COMPUTE", "FWD", {"PP": 0, "PASS": "F"}, [0], "default_stream", {}))
    dag.connect("a", "b", "data")
    out = render_training_dag(dag, str(tmp_path / "training_dag_pp0"))
    assert os.path.exists(out) and '"a" -> "b"' in open(str(tmp_path / "training_dag_pp0.dot")).read()
    lines = print_training_dag_order(dag, label="pp0", rank=0, out_dir=str(tmp_path))
    assert "FWD:PASS=F,PP=0:uida" in lines[1] and (tmp_path / "training_dag_order_rank0").exists()
    events = [
        {"ph": "X", "cat": "user_annotation", "name": "FWD:MB=0,PP=0:uids0.seg0", "ts": 100, "dur": 50, "tid": 1},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "ts": 110, "dur": 2, "tid": 1, "args": {"External id": 7}},
        {"ph": "X", "cat": "kernel", "name": "gemm_kernel", "ts": 300, "dur": 20, "args": {"External id": 7}},
        {"ph": "X", "cat": "kernel", "name": "other", "ts": 400, "dur": 20, "args": {"External id": 9}},
    ]
    assert relabel_gpu_events(events) == 1
    assert events[2]["name"] == "FWD:MB=0,PP=0:uids0.seg0::gemm_kernel" and events[3]["name"] == "other"


def test_artifact_dry_run_and_schedule_generator(tmp_path):
    sys.path.insert(0, str(ROOT / "artifact" / "scripts"))
    from make_piper_base_schedule import make_schedule
    from piper_b200.compiler.schedule import derive_schedule_info

    s = make_schedule(2, 2, zero=3, ep=True, virtual_stages=2, v_placement=True)
    places = {d["filter"]["PP"]: d["devices"] for d in s if d["op"] == "place"}
    assert places == {0: [0, 2], 1: [1, 3], 2: [1, 3], 3: [0, 2]}
    assert all(d.get("shard_params") for d in s if d["op"] == "replicate")
    info = derive_schedule_info(s + [{"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 4}], "x.json")
    assert (info["num_stages"], info["pp_degree"], info["dp_degree"]) == (4, 2, 2)
    out = subprocess.run([sys.executable, str(ROOT / "artifact" / "e2e_eval.py"), "--sweeps", "schedule", "--dry-run",
                          "--systems", "piper,megatron", "--out", str(tmp_path)], capture_output=True, text=True,
                         timeout=300, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-1500:]
    assert out.stdout.count("test_harness.py") == 4 and "pretrain_gpt.py" in out.stdout
    rows = list(__import__("csv").DictReader(open(next(tmp_path.glob("*/results.csv")))))
    assert len(rows) == 8 and {r["schedule"] for r in rows} == {"1f1b", "interleaved_1f1b", "zerobubble", "dualpipev"}


def test_artifact_backends_and_log_parsers(tmp_path, monkeypatch):
    """ssh backend: one command per node for a baseline, one on the head node for this framework; log parsers
    of the three baselines and of the harness CSV."""
    spec = importlib.util.spec_from_file_location("e2e_eval_mod", ROOT / "artifact" / "e2e_eval.py")
    ev = importlib.util.module_from_spec(spec)
    sys.modules["e2e_eval_mod"] = ev
    spec.loader.exec_module(ev)
    for k, v in {"SSH_KEY": "k.pem", "HEAD_PUBLIC_IP": "1.2.3.4", "HEAD_PRIVATE_IP": "10.0.0.1",
                 "WORKER1_PRIVATE_IP": "10.0.0.2"}.items():
        monkeypatch.setenv(k, v)
    be = ev.SshBackend(gpus_per_node=4)
    exp = ev.Experiment("scalability", "pp4_dp2", "9B", pp=4, dp=2, micro_batch=4, num_microbatches=8)
    assert be.layout(exp) == (2, 4)
    lines = be.dry_run_lines("megatron", exp, ev.baseline_command("megatron", exp))
    assert len(lines) == 2 and "NODE_RANK=1" in lines[1] and "ProxyCommand" in lines[1] and "--node-rank=1" in lines[1]
    assert "--master-addr=10.0.0.1" in lines[0] and "--nnodes=2" in lines[0]
    assert len(be.dry_run_lines("piper", exp, ["python", "x.py"])) == 1
    big = ev.Experiment("scalability", "pp8_dp4", "9B", pp=8, dp=4)
    with pytest.raises(RuntimeError):
        be.dry_run_lines("megatron", big, ev.baseline_command("megatron", big))
    docker = ev.LocalBackend(image="img:1", cuda_visible_devices="0,1")
    line = docker.dry_run_lines("megatron", exp, ev.baseline_command("megatron", exp))[0]
    assert line.startswith("docker run") and "device=0,1" in line and "img:1" in line

    log = tmp_path / "m.log"
    log.write_text(" elapsed time per iteration (ms): 1000.0 | x\n elapsed time per iteration (ms): 3000.0 |\n"
                   "[Rank 0] (after 2 iterations) memory (MB) | allocated: 1 | max allocated: 2048.0 |\n")
    r = ev.parse_log("megatron", log)
    assert r["iter_time_mean_s"] == pytest.approx(2.0) and r["iter_time_std_s"] == pytest.approx(1.0)
    assert r["peak_memory_gb"] == "2.00" and not r["oom"]
    log.write_text("\x1b[32m[rank0] step: 1  loss: 9.0  memory: 10.50GiB(13%)  tps: 1,000  mfu: 1%\x1b[0m\n"
                   "[rank1] step: 1  loss: 9.0  memory: 11.00GiB(13%)  tps: 1,000\n")
    r = ev.parse_log("torchtitan", log, tokens_per_iter=4000)
    assert r["iter_time_mean_s"] == pytest.approx(2.0) and r["peak_memory_gb"] == "10.50/11.00"
    log.write_text("[step 0] loss=1 time=0.500s\npeak memory rank 0: 3.0 GB\ntorch.OutOfMemoryError: CUDA out of memory\n")
    r = ev.parse_log("deepspeed", log)
    assert r["iter_time_mean_s"] == pytest.approx(0.5) and r["oom"] and r["peak_memory_gb"] == "3.00"
    m = tmp_path / "results.csv"
    m.write_text("dp_rank,iter_time_mean_s,iter_time_std_s,peak_memory_pp0_gb\n0,0.4,0.01,5.0\n1,0.5,0.02,5.5\n")
    r = ev.parse_log("piper", tmp_path / "none.log", m)
    assert r["iter_time_mean_s"] == pytest.approx(0.5) and "0:5.50" in r["peak_memory_gb"]
    rows = [ev.Result(system="piper", sweep="s", name="a", model="9M", schedule="1f1b", pp=1, dp=1, ep=False, zero=0,
                      micro_batch=1, num_microbatches=1, seq_len=8, gpus=1, global_batch=1, tokens_per_s=10.0)]
    out = ev.write_results(tmp_path, rows)
    assert out.is_file() and (tmp_path / "s.svg").is_file()


def _nsight_job(args, pg=None):
    return {"rank": int(os.environ["RANK"]), "profiled": os.environ.get("FAKE_NSYS_OUT", "")}


def test_coordinator_runs_ranks_under_nsys(tmp_path, monkeypatch):
    """With nsight set, every rank is started as `nsys profile ... python -m piper_b200.runtime.launcher payload`;
    a stand-in `nsys` records its options and runs the command."""
    from piper_b200.runtime.launcher import Coordinator, nsight_prefix

    fake = tmp_path / "bin" / "nsys"
    fake.parent.mkdir()
    fake.write_text("#!/bin/bash\n[ \"$1\" = profile ] || exit 9\nshift\nopts=()\n"
                    "while [[ \"$1\" == -* ]]; do if [[ \"$1\" == --* ]]; then opts+=(\"$1\"); shift; "
                    "else opts+=(\"$1 $2\"); out=\"$2\"; shift 2; fi; done\n"
                    "printf '%s\\n' \"${opts[@]}\" > \"$out.opts\"\nFAKE_NSYS_OUT=\"$out\" exec \"$@\"\n")
    fake.chmod(0o755)
    monkeypatch.setenv("PATH", f"{fake.parent}:{os.environ['PATH']}")
    reports = tmp_path / "reports"
    job = Coordinator(world_size=2, nsight={"t": "cuda,nvtx", "cuda-graph-trace": None}, nsight_dir=str(reports)
                      ).run_program(_nsight_job, None, timeout=120)
    assert job.ok and [r["rank"] for r in job.results] == [0, 1]
    assert job.results[1]["profiled"] == str(reports / "piper_rank1")
    opts = (reports / "piper_rank0.opts").read_text()
    assert "-t cuda,nvtx" in opts and "--force-overwrite=true" in opts and "cuda-graph-trace" not in opts
    assert nsight_prefix(3, "/r")[:2] == ["nsys", "profile"] and "/r/piper_rank3" in nsight_prefix(3, "/r")
    monkeypatch.setenv("PATH", "/nonexistent")
    with pytest.raises(RuntimeError, match="nsys"):
        Coordinator(world_size=1, nsight=True).run_program(_nsight_job, None)


def test_baseline_runners_dry_run_and_padded_bmm_hook():
    """Megatron runner builds its command without Megatron; DeepSpeed runner reports the missing package; the
    TorchTitan hook's padded batched-matmul experts equal a per-expert loop."""
    import importlib.util
    import subprocess

    import torch.nn.functional as F

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "artifact", "run_megatron.py"), "--nnodes", "1",
                          "--nproc-per-node", "8", "--pp", "4", "--dp", "2", "--model", "qwen3_9b", "--dry-run"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "--pipeline-model-parallel-size 4" in out.stdout and "--num-experts 64" in out.stdout
    bad = subprocess.run([sys.executable, os.path.join(root, "artifact", "run_megatron.py"), "--nnodes", "1",
                          "--nproc-per-node", "8", "--pp", "4", "--dp", "1", "--dry-run"],
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "does not match" in bad.stderr
    if importlib.util.find_spec("deepspeed") is None:
        ds = subprocess.run([sys.executable, os.path.join(root, "artifact", "run_deepspeed.py"), "--pp", "2"],
                            capture_output=True, text=True, timeout=300)
        assert ds.returncode == 3 and "not installed" in ds.stderr

    spec = importlib.util.spec_from_file_location("artifact_site", os.path.join(root, "artifact", "sitecustomize.py"))
    hook = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(hook)
    g = torch.Generator().manual_seed(3)
    E, d, f = 4, 16, 8
    w1, w3, w2 = torch.randn(E, f, d, generator=g), torch.randn(E, f, d, generator=g), torch.randn(E, d, f, generator=g)
    counts, x = torch.tensor([3, 0, 5, 2]), torch.randn(10, d, generator=g)
    got = hook._padded_bmm_experts(w1, w2, w3, x, counts)
    want, s = torch.zeros_like(x), 0
    for e, n in enumerate(counts.tolist()):
        r = x[s:s + n]
        want[s:s + n] = (F.silu(r @ w1[e].t()) * (r @ w3[e].t())) @ w2[e].t()
        s += n
    assert torch.allclose(got, want, atol=1e-5)


def test_status_monitor_raises_for_the_previous_step_with_a_fake_status_word():
    """The step driver's status check, fed by a fake status tensor: 0 passes, 2 raises the comm timeout."""
    import pytest
    import torch

    from piper_b200.ops import native

    word = torch.zeros(1, dtype=torch.int32)
    mon = native.StatusMonitor(torch.device("cpu"), source=word)
    mon.post()
    mon.poll()                      # clean step: nothing raised
    word[0] = 2                     # a fused collective gave up waiting for a peer during this step
    mon.post()
    with pytest.raises(native.PiperCommTimeout):
        mon.poll()
    assert int(word[0]) == 0        # cleared, so that the caller can decide to continue
    word[0] = 3
    mon.post()
    with pytest.raises(native.PiperKernelError):
        mon.poll(wait=True)
    mon.poll()                      # nothing pending any more


def test_row_sharding_partitions_every_parameter_and_rebuilds_it():
    """Row sharding of a bucket (used by the fused data-parallel paths): the ranks' pieces tile every parameter
    exactly once, shard buffers hold the pieces, and decay follows torch.optim.Adam vs AdamW."""
    import torch

    from piper_b200.runtime.storage import AdamConfig, ParamSlot, ParamStorage, _adam_reference

    shapes = {"a.weight": (300, 16), "norm.weight": (130,), "b.weight": (64, 24)}
    dp = 3
    stores = []
    for r in range(dp):
        slots = [ParamSlot(pos=i, fqn=k, shape=v, dtype=torch.float32, requires_grad=True)
                 for i, (k, v) in enumerate(shapes.items())]
        st = ParamStorage("bucket", slots, torch.device("cpu"), torch.float32, "zero2", r, dp, None, AdamConfig())
        st.convert_to_rows(lambda name, n, dt: torch.zeros(n, dtype=dt))
        stores.append(st)
    full = stores[0].flat_params
    covered = torch.zeros(stores[0].numel, dtype=torch.int32)
    rebuilt = torch.zeros_like(full)
    for st in stores:
        assert st.shard_numel == stores[0].shard_numel
        for s, a, e, sh in st.owned_pieces():
            covered[a:e] += 1
            rebuilt[a:e] = st.shard_params[sh:sh + e - a]
            assert torch.equal(st.master[sh:sh + e - a], full[a:e].float())
            k = s.numel // s.shape[0]
            assert (a - s.offset) % k == 0                     # pieces start on a row boundary
    for s in stores[0].slots:
        assert torch.all(covered[s.offset:s.offset + s.numel] == 1)
        assert torch.equal(rebuilt[s.offset:s.offset + s.numel], full[s.offset:s.offset + s.numel])

    # decay semantics of the flat optimizer against torch.optim
    for cls, decoupled in ((torch.optim.Adam, False), (torch.optim.AdamW, True)):
        w = torch.nn.Parameter(torch.randn(50))
        opt = cls([w], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        master, m, v = w.detach().clone(), torch.zeros(50), torch.zeros(50)
        cfg = AdamConfig(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, decoupled=decoupled)
        for step in range(1, 4):
            g = torch.randn(50)
            w.grad = g.clone()
            opt.step()
            _adam_reference(master, m, v, g, None, cfg, step, 1.0)
            assert torch.allclose(master, w.detach(), atol=1e-6), cls


def test_optimizer_mapping_rejects_what_the_kernels_cannot_do():
    import functools

    import pytest
    import torch

    from piper_b200.engine import _adam_config

    assert _adam_config(torch.optim.Adam, {"lr": 3e-4, "weight_decay": 0.1}).decoupled is False
    cfg = _adam_config(functools.partial(torch.optim.AdamW, lr=1e-3, fused=True), None)
    assert cfg.decoupled is True and cfg.weight_decay == 1e-2 and cfg.lr == 1e-3
    with pytest.raises(ValueError):
        _adam_config(torch.optim.SGD, {"lr": 0.1})
    with pytest.raises(ValueError):
        _adam_config(torch.optim.Adam, {"amsgrad": True})


def test_launch_plan_matches_the_dag_edges_and_the_native_module_validates_plans():
    """The static plan handed to the C++ executor: a node waits exactly for its earlier predecessors that run on
    another stream (order between pipeline messages excepted), and the extension module rejects a malformed plan."""
    import importlib.util

    import pytest
    import torch

    from piper_b200 import piper_setup
    from piper_b200.compiler.builders import build_1f1b_schedule
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.ops import native
    from piper_b200.runtime.actor import DagExecutor

    cfg = LLAMA_CONFIGS["tiny"]
    x = torch.randint(0, cfg.vocab_size, (4, 32))
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0], "stream": "pp_stream"},
             {"op": "replicate", "filter": {"PP": 0}, "devices": [0], "reduce_stream": "dp_stream",
              "gather_stream": "gather_stream", "shard_grads": True, "shard_params": True, "bucket_size": 1},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}] + build_1f1b_schedule(1, 2)
    actor = piper_setup(Transformer, (cfg, 32, 1), optim_fn=torch.optim.Adam, example_inputs=[x], example_outputs=x,
                        model_dtype=torch.float32, const_attrs=Transformer.const_attrs(cfg, 32),
                        schedule_directives=sched, device="cpu")
    ex = DagExecutor(actor)
    fake = {}
    ex._stream = lambda node: fake.setdefault(node.stream, object())      # one stand-in stream per logical stream
    streams, node_stream, waits = ex.static_waits(actor.order)
    assert len(streams) == len({actor.dag.nodes[u].stream for u in actor.order}) >= 2
    index = {u: i for i, u in enumerate(actor.order)}
    n_cross = 0
    for i, uid in enumerate(actor.order):
        want = set()
        for e in actor.dag.in_edges(uid):
            j = index[e.src_uid]
            assert j < i                                                   # the dispatch order respects every edge
            if actor.dag.nodes[e.src_uid].stream != actor.dag.nodes[uid].stream:
                want.add(j)
        assert set(waits[i]) == want, uid
        n_cross += len(want)
    assert n_cross > 0

    path = native.lib_path().with_name("piper_plan.so")
    if path.exists():
        spec = importlib.util.spec_from_file_location("piper_plan", str(path))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        with pytest.raises(ValueError):
            mod.PlanExecutor(0, [0], [0, 0], [[1], []], ["a", "b"], False)     # waits for a later node
        with pytest.raises(ValueError):
            mod.PlanExecutor(0, [0], [0, 3], [[], []], ["a", "b"], False)      # unknown stream


def test_node_outputs_are_released_after_their_last_reader(monkeypatch):
    """Gradient tuples, receive buffers and exchange results leave the executor's table as soon as the last node
    that reads them has been issued, not at the end of the step."""
    import torch

    from piper_b200 import piper_exec_dag, piper_setup
    from piper_b200.compiler.builders import build_1f1b_schedule
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.nn import cross_entropy_loss
    from piper_b200.runtime import actor as actor_mod

    cfg = LLAMA_CONFIGS["tiny"]
    tok = torch.randint(0, cfg.vocab_size, (8, 33), generator=torch.Generator().manual_seed(0))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]}, {"op": "place", "filter": {"PP": 1}, "devices": [0]},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 8}] + build_1f1b_schedule(1, 8)
    actor = piper_setup(Transformer, (cfg, 32, 2), optim_fn=torch.optim.Adam, example_inputs=[x], example_outputs=y,
                        model_dtype=torch.float32, const_attrs=Transformer.const_attrs(cfg, 32),
                        schedule_directives=sched, device="cpu")
    seen = []
    orig = actor_mod.DagExecutor._release_outputs

    def spy(self, i):
        orig(self, i)
        seen.append(len(self.outs))

    monkeypatch.setattr(actor_mod.DagExecutor, "_release_outputs", spy)
    losses = piper_exec_dag(cross_entropy_loss)
    assert len(losses) == 8 and len(seen) == len(actor.order)
    assert seen[-1] == 0                               # nothing outlives the step
    assert max(seen) <= 4 < len(actor.order) // 4      # a few entries at a time, not one per node


def test_first_linear_weight_of_a_segment_is_found_for_the_gather_gemm():
    """ZeRO-3 buckets leave the weight of their segment's first linear layer to the GEMM that gathers it: the
    lookup returns that weight's slot when the linear call is the weight's only use, and -1 for segments that
    start with something else (an embedding) or whose parameters are not used by a linear call first."""
    import torch

    from piper_b200 import piper_setup
    from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer
    from piper_b200.parallel.fused import first_linear_slot

    cfg = LLAMA_CONFIGS["tiny"]
    x = torch.randint(0, cfg.vocab_size, (4, 32))
    sched = [{"op": "place", "filter": {"PP": 0}, "devices": [0]}, {"op": "place", "filter": {"PP": 1}, "devices": [0]},
             {"op": "replicate", "filter": {"PP": 0}, "devices": [0], "bucket_size": 1},
             {"op": "replicate", "filter": {"PP": 1}, "devices": [0], "bucket_size": 1},
             {"op": "split", "filter": {}, "dim_name": "MB", "num_microbatches": 2}]
    actor = piper_setup(Transformer, (cfg, 32, 2), optim_fn=torch.optim.Adam, example_inputs=[x], example_outputs=x,
                        model_dtype=torch.float32, const_attrs=Transformer.const_attrs(cfg, 32),
                        schedule_directives=sched, device="cpu")
    found = {}
    for key, b in actor.buckets.items():
        if b.storage is None:
            continue
        i = first_linear_slot(b.gm, [s.pos for s in b.storage.slots])
        found[key] = b.storage.slots[i].fqn if i >= 0 else None
    assert len(found) > 2                                              # the stages were cut into buckets
    named = [v for v in found.values() if v]
    assert named and all(v.endswith("weight") and "norm" not in v and "embed" not in v for v in named)
    first = next(iter(found))                                          # the first bucket starts with the embedding
    assert found[first] is None or "tok_embeddings" not in found[first]


def test_clock_sampler_with_a_stand_in_nvidia_smi(tmp_path, monkeypatch):
    """The benchmark's clock record: median SM clock, largest maximum and the set of active event reasons, parsed
    from the stream of a stand-in ``nvidia-smi``; a machine without the tool yields an empty record."""
    from baseline.clocks import ClockSampler

    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/bash\n"
                    "echo '0, 1500, 1965, Not Active, Not Active, Not Active, Active'\n"
                    "echo '1, 1700, 1965, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo '0, 1600, 1965, Not Active, Active, Not Active, Active'\n"
                    "echo 'garbage line'\nsleep 30\n")
    fake.chmod(0o755)
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    s = ClockSampler([0, 1])
    s.start()
    deadline = time.time() + 10
    while len(s.rows) < 4 and time.time() < deadline:
        time.sleep(0.05)
    rec = s.stop()
    assert rec == {"sm_mhz": 1600.0, "sm_max_mhz": 1965.0, "reasons": ["hw_thermal_slowdown", "sw_power_cap"],
                   "samples": 3}
    monkeypatch.setenv("PATH", str(tmp_path / "nowhere"))
    s = ClockSampler(0)
    s.start()
    assert s.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
