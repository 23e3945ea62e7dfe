"""Computational-graph capture, analysis and serialisation.

Reference: src/MLFramework.Visualization/Graphs/{ComputationalGraph.cs:65-238 (nodes, edges, inputs / outputs,
topological order, cycles, components), GraphNode.cs, NodeType.cs, GraphAnalysis.cs:82-285 (parameter / operation
counts, depth, fan-in / fan-out, warnings, recommendations), GraphLogger.cs:46-197 (log, capture, analyse),
Serialization/GraphSerializer.cs}. Capture sources here: a module tree, the autograd graph behind a tensor (the real
operation graph of a step: every ``grad_fn`` is a node), or this package's high-level IR graph.
"""
from __future__ import annotations

import enum
import json
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch


class NodeType(enum.Enum):
    INPUT = "input"
    PARAMETER = "parameter"
    OPERATION = "operation"
    CONSTANT = "constant"
    OUTPUT = "output"
    MODULE = "module"


@dataclass
class GraphNode:
    id: str
    name: str
    type: NodeType
    op_type: Optional[str] = None
    shape: Optional[Tuple[int, ...]] = None
    dtype: Optional[str] = None
    attributes: Dict[str, Any] = field(default_factory=dict)
    input_ids: List[str] = field(default_factory=list)
    output_ids: List[str] = field(default_factory=list)

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape or ():
            n *= d
        return n if self.shape is not None else 0


class ComputationalGraph:
    def __init__(self, name: str, step: int = 0):
        if not name:
            raise ValueError("name must not be empty")
        self.name, self.step = name, step
        self.nodes: Dict[str, GraphNode] = {}
        self.edges: List[Tuple[str, str]] = []

    def add_node(self, node: GraphNode) -> GraphNode:
        if node.id in self.nodes:
            raise KeyError(f"node {node.id!r} already in the graph")
        self.nodes[node.id] = node
        return node

    def add_edge(self, src: str, dst: str):
        if src not in self.nodes or dst not in self.nodes:
            raise KeyError(f"edge {src!r} -> {dst!r} names an unknown node")
        if (src, dst) in self.edges:
            return
        self.edges.append((src, dst))
        self.nodes[src].output_ids.append(dst)
        self.nodes[dst].input_ids.append(src)

    def inputs(self) -> List[GraphNode]:
        return [n for n in self.nodes.values() if not n.input_ids]

    def outputs(self) -> List[GraphNode]:
        return [n for n in self.nodes.values() if not n.output_ids]

    def topological_order(self) -> List[GraphNode]:
        indeg = {k: len(n.input_ids) for k, n in self.nodes.items()}
        q = deque(k for k, d in indeg.items() if d == 0)
        out = []
        while q:
            k = q.popleft()
            out.append(self.nodes[k])
            for d in self.nodes[k].output_ids:
                indeg[d] -= 1
                if indeg[d] == 0:
                    q.append(d)
        if len(out) != len(self.nodes):
            raise ValueError("graph has a cycle")
        return out

    def has_cycle(self) -> bool:
        try:
            self.topological_order()
            return False
        except ValueError:
            return True

    @property
    def depth(self) -> int:
        """Nodes on the longest path."""
        if self.has_cycle():
            return -1
        d: Dict[str, int] = {}
        for n in self.topological_order():
            d[n.id] = 1 + max((d[i] for i in n.input_ids), default=0)
        return max(d.values(), default=0)

    def disconnected_components(self) -> List[List[GraphNode]]:
        seen, comps = set(), []
        for k in self.nodes:
            if k in seen:
                continue
            comp, q = [], deque([k])
            seen.add(k)
            while q:
                c = q.popleft()
                comp.append(self.nodes[c])
                for nb in self.nodes[c].input_ids + self.nodes[c].output_ids:
                    if nb not in seen:
                        seen.add(nb)
                        q.append(nb)
            comps.append(comp)
        return comps


@dataclass
class GraphAnalysis:
    total_parameters: int
    parameter_elements: int
    total_operations: int
    operation_counts: Dict[str, int]
    graph_depth: int
    max_fan_in: int
    max_fan_out: int
    skip_connections: int
    warnings: List[str] = field(default_factory=list)
    recommendations: List[str] = field(default_factory=list)


class GraphAnalyzer:
    DEEP, WIDE = 100, 10

    def analyze(self, g: ComputationalGraph) -> GraphAnalysis:
        counts: Dict[str, int] = {}
        n_par = n_el = n_op = fan_in = fan_out = 0
        for n in g.nodes.values():
            if n.type == NodeType.PARAMETER:
                n_par += 1
                n_el += n.numel
            elif n.type in (NodeType.OPERATION, NodeType.MODULE):
                n_op += 1
                counts[n.op_type or "Unknown"] = counts.get(n.op_type or "Unknown", 0) + 1
            fan_in, fan_out = max(fan_in, len(n.input_ids)), max(fan_out, len(n.output_ids))
        warn, rec = [], []
        cyc = g.has_cycle()
        depth = g.depth
        if cyc:
            warn.append("graph contains cycles: no topological order exists")
            rec.append("remove the cycle or unroll the recurrence")
        if depth > self.DEEP:
            warn.append(f"graph is very deep ({depth} nodes on the longest path): gradients may vanish or explode")
            rec.append("use skip connections or normalisation layers")
        if fan_in > self.WIDE:
            warn.append(f"high fan-in (max {fan_in}): a possible bottleneck")
            rec.append("restructure to reduce fan-in, or confirm that it is intended")
        if fan_out > self.WIDE:
            warn.append(f"high fan-out (max {fan_out}): a strongly branching structure")
            rec.append("check whether all branches are needed")
        skips = 0 if cyc else self._skip_connections(g)
        if skips:
            rec.append(f"{skips} skip connections found (good for gradient flow)")
        comps = g.disconnected_components()
        if len(comps) > 1:
            warn.append(f"graph has {len(comps)} disconnected components")
            rec.append("check for missing connections")
        lin = sum(v for k, v in counts.items() if k.lower() in ("linear", "matmul", "mm", "addmm", "mmbackward0", "addmmbackward0", "_linearfnbackward"))
        norm = sum(v for k, v in counts.items() if "norm" in k.lower())
        if lin >= 8 and norm == 0:
            rec.append(f"{lin} matrix products and no normalisation layer: consider LayerNorm / RMSNorm between blocks")
        return GraphAnalysis(n_par, n_el, n_op, counts, depth, fan_in, fan_out, skips, warn, rec)

    @staticmethod
    def _skip_connections(g: ComputationalGraph) -> int:
        """Edges that bypass at least one node: ``u -> v`` where ``v`` is also reachable from ``u`` through a longer path."""
        level: Dict[str, int] = {}
        for n in g.topological_order():
            level[n.id] = 1 + max((level[i] for i in n.input_ids), default=0)
        return sum(1 for u, v in g.edges if level[v] - level[u] > 1 and g.nodes[u].type != NodeType.PARAMETER
                   and g.nodes[u].type != NodeType.CONSTANT)


# ------------------------------------------------------------------ capture
def graph_from_module(model: torch.nn.Module, name: str = "model") -> ComputationalGraph:
    """The module tree: one node per sub-module (edges parent -> child) and one per parameter (parameter -> owner)."""
    g = ComputationalGraph(name)
    for n, m in model.named_modules():
        g.add_node(GraphNode(n or "<root>", n or "<root>", NodeType.MODULE, type(m).__name__))
    for n, _ in model.named_modules():
        if n:
            g.add_edge(n.rsplit(".", 1)[0] if "." in n else "<root>", n)
    for n, p in model.named_parameters():
        pid = "param:" + n
        g.add_node(GraphNode(pid, n, NodeType.PARAMETER, shape=tuple(p.shape), dtype=str(p.dtype).replace("torch.", "")))
        g.add_edge(pid, n.rsplit(".", 1)[0] if "." in n else "<root>")
    return g


def graph_from_autograd(output: torch.Tensor, params: Optional[Dict[str, torch.Tensor]] = None, name: str = "autograd",
                        max_nodes: int = 100_000) -> ComputationalGraph:
    """The operation graph recorded by autograd behind ``output`` (usually the loss): every backward function is an
    operation node named after the forward op it differentiates, leaves are parameters (named when ``params`` maps
    names to them) or inputs. Edges point in the FORWARD direction."""
    if output.grad_fn is None:
        raise ValueError("tensor has no autograd history")
    names = {id(p): n for n, p in (params or {}).items()}
    g = ComputationalGraph(name)
    ids: Dict[int, str] = {}

    def node_for(fn) -> str:
        k = id(fn)
        if k in ids:
            return ids[k]
        if hasattr(fn, "variable"):                       # AccumulateGrad: a leaf tensor
            v = fn.variable
            nid = f"leaf{len(ids)}"
            nm = names.get(id(v), nid)
            g.add_node(GraphNode(nid, nm, NodeType.PARAMETER if id(v) in names or isinstance(v, torch.nn.Parameter) else NodeType.INPUT,
                                 shape=tuple(v.shape), dtype=str(v.dtype).replace("torch.", "")))
        else:
            nid = f"op{len(ids)}"
            op = type(fn).__name__
            g.add_node(GraphNode(nid, op, NodeType.OPERATION, op[:-len("Backward0")] if op.endswith("Backward0") else op.replace("Backward", "")))
        ids[k] = nid
        return nid

    root_fn = output.grad_fn
    alive = [root_fn]                                     # wrappers stay alive so that their ids stay theirs
    root = node_for(root_fn)
    out_id = "output"
    g.add_node(GraphNode(out_id, "output", NodeType.OUTPUT, shape=tuple(output.shape), dtype=str(output.dtype).replace("torch.", "")))
    g.add_edge(root, out_id)
    stack, seen = [root_fn], {id(root_fn)}
    while stack:
        fn = stack.pop()
        for nxt, _ in getattr(fn, "next_functions", ()):
            if nxt is None:
                continue
            if len(g.nodes) >= max_nodes and id(nxt) not in ids:
                continue
            alive.append(nxt)
            g.add_edge(node_for(nxt), ids[id(fn)])
            if id(nxt) not in seen:
                seen.add(id(nxt))
                stack.append(nxt)
    return g


def graph_from_ir(hl) -> ComputationalGraph:
    """A high-level IR graph (:class:`ml_framework_b200.compiler.ir.HLGraph`) as a computational graph."""
    g = ComputationalGraph(hl.name)
    for n in hl.inputs:
        v = hl.values[n]
        g.add_node(GraphNode(n, n, NodeType.INPUT, shape=tuple(v.shape), dtype=str(v.dtype).replace("torch.", "")))
    for n, v in hl.values.items():
        if v.const is not None and n not in g.nodes:
            g.add_node(GraphNode(n, n, NodeType.CONSTANT, shape=tuple(v.shape), dtype=str(v.dtype).replace("torch.", "")))
    for o in hl.ops:
        v = hl.values[o.output]
        g.add_node(GraphNode(o.output, o.output, NodeType.OPERATION, o.kind, tuple(v.shape), str(v.dtype).replace("torch.", ""),
                             {k: a for k, a in o.attrs.items() if isinstance(a, (int, float, str, bool, tuple, list))}))
        for i in o.inputs:
            g.add_edge(i, o.output)
    return g


# ------------------------------------------------------------------ serialisation
class GraphSerializer:
    @staticmethod
    def to_dict(g: ComputationalGraph) -> Dict[str, Any]:
        return {"name": g.name, "step": g.step,
                "nodes": [{"id": n.id, "name": n.name, "type": n.type.value, "op_type": n.op_type, "shape": list(n.shape) if n.shape is not None else None,
                           "dtype": n.dtype, "attributes": n.attributes} for n in g.nodes.values()],
                "edges": [list(e) for e in g.edges]}

    @classmethod
    def to_json(cls, g: ComputationalGraph, indent: Optional[int] = None) -> str:
        return json.dumps(cls.to_dict(g), indent=indent, default=str)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> ComputationalGraph:
        g = ComputationalGraph(d["name"], d.get("step", 0))
        for n in d["nodes"]:
            g.add_node(GraphNode(n["id"], n["name"], NodeType(n["type"]), n.get("op_type"), tuple(n["shape"]) if n.get("shape") is not None else None,
                                 n.get("dtype"), n.get("attributes") or {}))
        for s, t in d["edges"]:
            g.add_edge(s, t)
        return g

    @classmethod
    def from_json(cls, text: str) -> ComputationalGraph:
        return cls.from_dict(json.loads(text))

    @staticmethod
    def to_dot(g: ComputationalGraph) -> str:
        shapes = {NodeType.PARAMETER: "box", NodeType.INPUT: "invhouse", NodeType.OUTPUT: "house", NodeType.CONSTANT: "note",
                  NodeType.OPERATION: "ellipse", NodeType.MODULE: "component"}
        esc = lambda s: str(s).replace('"', r'\"')      # noqa: E731
        lines = [f'digraph "{esc(g.name)}" {{', "  rankdir=TB;"]
        for n in g.nodes.values():
            label = n.op_type or n.name
            if n.shape is not None:
                label += f"\\n{list(n.shape)}"
            lines.append(f'  "{esc(n.id)}" [label="{esc(label)}", shape={shapes[n.type]}];')
        lines += [f'  "{esc(s)}" -> "{esc(t)}";' for s, t in g.edges]
        lines.append("}")
        return "\n".join(lines)


class GraphLogger:
    """Keeps logged graphs by name, writes each to the storage back-end as a graph event, analyses on request."""

    def __init__(self, storage=None):
        self.storage = storage
        self._graphs: Dict[str, ComputationalGraph] = {}
        self._capture: Optional[Tuple[str, torch.nn.Module, list, ComputationalGraph]] = None
        self._captured: Optional[ComputationalGraph] = None

    def log_graph(self, graph_or_model, name: Optional[str] = None) -> ComputationalGraph:
        g = graph_or_model if isinstance(graph_or_model, ComputationalGraph) else graph_from_module(graph_or_model, name or "model")
        self._graphs[g.name] = g
        if self.storage is not None:
            from .events import Event, EventType
            self.storage.write([Event(EventType.GRAPH, g.name, g.step, GraphSerializer.to_dict(g))])
        return g

    def start_graph_capture(self, name: str, model: torch.nn.Module):
        """Records the order in which ``model``'s leaf modules actually run (forward hooks) until ``stop_graph_capture``:
        nodes are module calls, edges follow the execution order inside each parent."""
        if self._capture is not None:
            raise RuntimeError("a capture is already running")
        g = ComputationalGraph(name)
        handles, last = [], {"id": None, "n": 0}
        names = {m: n for n, m in model.named_modules()}

        def hook(mod, inp, out):
            if any(True for _ in mod.children()):
                return
            nid = f"{names[mod]}#{last['n']}"
            last["n"] += 1
            shp = tuple(out.shape) if isinstance(out, torch.Tensor) else None
            g.add_node(GraphNode(nid, names[mod], NodeType.OPERATION, type(mod).__name__, shp))
            if last["id"] is not None:
                g.add_edge(last["id"], nid)
            last["id"] = nid
        for m in model.modules():
            handles.append(m.register_forward_hook(hook))
        self._capture = (name, model, handles, g)

    def stop_graph_capture(self) -> ComputationalGraph:
        if self._capture is None:
            raise RuntimeError("no capture is running")
        _, _, handles, g = self._capture
        for h in handles:
            h.remove()
        self._capture, self._captured = None, g
        self._graphs[g.name] = g
        return g

    def captured_graph(self) -> Optional[ComputationalGraph]:
        return self._captured

    def analyze_graph(self, name: str) -> GraphAnalysis:
        if name not in self._graphs:
            raise KeyError(f"no graph named {name!r}")
        return GraphAnalyzer().analyze(self._graphs[name])

    def analyze_all_graphs(self) -> Dict[str, GraphAnalysis]:
        return {k: GraphAnalyzer().analyze(g) for k, g in self._graphs.items()}

    def all_graphs(self) -> Dict[str, ComputationalGraph]:
        return dict(self._graphs)

    def clear_graphs(self):
        self._graphs.clear()
        self._captured = None
