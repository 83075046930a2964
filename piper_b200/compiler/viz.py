"""Text and Graphviz artefacts of schedules and per-device DAGs.

Three outputs, as in the reference (``src/visualization.py``): the DOT description of a per-device DAG (nodes
ranked by topological level, data edges solid, temporal edges dashed blue), a text dump of the dispatch
order ``training_dag_order_rank{r}``, and a schedule grid (one row per physical rank, one column per time
slot, overlapped forward/backward pairs stacked in one cell) written as an HTML table inside a DOT label.
The DOT *source* is always written; a PNG is rendered only when a ``dot`` executable is installed.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from typing import Optional

from .dag import TrainingDAG
from .ordering import serial_topological_order

_KIND_COLOR = {"COMPUTE": "lightblue", "UPD": "gold", "SEND_COMM": "palegreen", "RECV_COMM": "palegreen",
               "REDUCE_COMM": "salmon", "REDUCE_SCATTER_COMM": "salmon", "ALL_GATHER_COMM": "orange",
               "A2A_COMM": "plum", "ORDER_DUMMY": "gray90"}
_PASS_COLOR = {"F": "#9ecae1", "B": "#fdae6b", "BI": "#fdd0a2", "BW": "#c7e9c0"}


def node_label(node) -> str:
    tags = ",".join(f"{k}={v}" for k, v in sorted(node.tag.items()) if v is not None)
    kind = node.compute_subkind or node.node_kind
    return f"{kind}:{tags}:uid{node.uid}"


def _render(dot_source: str, output_path: str) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(output_path)) or ".", exist_ok=True)
    src = output_path + ".dot"
    with open(src, "w", encoding="utf-8") as f:
        f.write(dot_source)
    exe = shutil.which("dot")
    if exe:
        try:
            subprocess.run([exe, "-Tpng", src, "-o", output_path + ".png"], check=True, timeout=120)
            return output_path + ".png"
        except (subprocess.SubprocessError, OSError):
            pass   # graphviz failed: the caller still gets the .dot source
    return src


def training_dag_dot(dag: TrainingDAG) -> str:
    levels = dag.topological_levels()
    by_level: dict[int, list[str]] = {}
    for u, lv in levels.items():
        by_level.setdefault(lv, []).append(u)
    q = lambda s: '"' + s.replace('"', "'") + '"'
    lines = ["digraph training_dag {", "  rankdir=TB;", "  node [shape=box, style=filled, fontsize=10];"]
    for lv in sorted(by_level):
        lines.append("  { rank=same; " + " ".join(q(u) for u in sorted(by_level[lv])) + " }")
    for u, n in dag.nodes.items():
        lines.append(f"  {q(u)} [label={q(node_label(n) + chr(92) + 'n' + n.stream)}, "
                     f"fillcolor={q(_KIND_COLOR.get(n.node_kind, 'white'))}];")
    for e in dag.edges:
        style = "" if e.dep_kind == "data" else " [style=dashed, color=blue]"
        lines.append(f"  {q(e.src_uid)} -> {q(e.dst_uid)}{style};")
    lines.append("}")
    return "\n".join(lines) + "\n"


def render_training_dag(dag: TrainingDAG, output_path: str) -> str:
    return _render(training_dag_dot(dag), output_path)


def print_training_dag_order(dag: TrainingDAG, label: str = "", rank: int = 0, out_dir: Optional[str] = None) -> list[str]:
    order = serial_topological_order(dag)
    lines = [f"# dispatch order {label} ({len(order)} nodes)"]
    for i, u in enumerate(order):
        n = dag.nodes[u]
        lines.append(f"{i:5d}  {n.stream:16s}  {node_label(n)}")
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, f"training_dag_order_rank{rank}"), "w", encoding="utf-8") as f:
            f.write("\n".join(lines) + "\n")
    return lines


def log_training_dag_dependencies(dag: TrainingDAG) -> list[str]:
    return [f"{e.src_uid} -[{e.dep_kind}]-> {e.dst_uid}" for e in dag.edges]


def _slot_text(slot: list[dict]) -> str:
    return "<BR/>".join(f"{f.get('PASS', '?')}{f.get('PP', '')}.{f.get('MB', '')}" for f in slot)


def compute_columns(rows: list[list[list[dict]]]) -> list[list[int]]:
    """Column of every slot: the longest dependency path, where a backward is two columns wide and a slot
    starts after its predecessor in the row and after the slot that produces its input on the neighbouring stage."""
    done: dict[tuple, int] = {}     # (pass class, PP, MB) -> end column
    cols = [[-1] * len(r) for r in rows]
    cursor = [0] * len(rows)
    progress = True
    pos = [0] * len(rows)
    n_stages = 1 + max((int(f.get("PP", 0)) for r in rows for s in r for f in s), default=0)
    while progress:
        progress = False
        for ri, row in enumerate(rows):
            while pos[ri] < len(row):
                slot = row[pos[ri]]
                start = cursor[ri]
                ready = True
                for f in slot:
                    pp, mb, p = int(f.get("PP", 0)), f.get("MB"), f.get("PASS")
                    if p == "F" and pp > 0:
                        dep = ("F", pp - 1, mb)
                    elif p in ("B", "BI") and pp < n_stages - 1:
                        dep = ("B", pp + 1, mb)
                    elif p in ("B", "BI"):
                        dep = ("F", pp, mb)
                    elif p == "BW":
                        dep = ("B", pp, mb)
                    else:
                        dep = None
                    if dep is not None:
                        if dep not in done:
                            ready = False
                            break
                        start = max(start, done[dep])
                if not ready:
                    break
                width = 2 if any(f.get("PASS") == "B" for f in slot) else 1
                cols[ri][pos[ri]] = start
                for f in slot:
                    cls = "F" if f.get("PASS") == "F" else ("W" if f.get("PASS") == "BW" else "B")
                    done[(cls, int(f.get("PP", 0)), f.get("MB"))] = start + width
                cursor[ri] = start + width
                pos[ri] += 1
                progress = True
    for ri, row in enumerate(rows):       # slots whose dependency never resolved: append in order
        for si in range(len(row)):
            if cols[ri][si] < 0:
                cols[ri][si] = cursor[ri]
                cursor[ri] += 1
    return cols


def schedule_grid_dot(order_directives: list[dict]) -> str:
    rows = [d["filters"] for d in order_directives if d.get("op") == "order"]
    cols = compute_columns(rows)
    width = 1 + max((c for r in cols for c in r), default=0) + 1
    html = ['<TABLE BORDER="0" CELLBORDER="1" CELLSPACING="0">']
    for ri, row in enumerate(rows):
        cells = [""] * (width + 1)
        colors = [None] * (width + 1)
        for slot, c in zip(row, cols[ri]):
            cells[c] = _slot_text(slot)
            colors[c] = _PASS_COLOR.get(slot[0].get("PASS"), "white")
        tds = "".join(f'<TD BGCOLOR="{colors[i] or "white"}">{cells[i] or " "}</TD>' for i in range(width))
        html.append(f"<TR><TD>rank {ri}</TD>{tds}</TR>")
    html.append("</TABLE>")
    return "digraph schedule {\n  node [shape=plaintext];\n  grid [label=<" + "".join(html) + ">];\n}\n"


def visualize_order_directives(order_directives: list[dict], output_path) -> str:
    base = str(output_path)
    if base.endswith(".png"):
        base = base[:-4]
    return _render(schedule_grid_dot(order_directives), base)
