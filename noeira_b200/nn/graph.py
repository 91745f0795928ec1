"""ComputeGraph: a named DAG of modules with explicit backward and fan-out gradient accumulation.

Declarations are a list of ``InputSlot(name)`` and ``Node(name, module, inputs=[...])`` in topological order
(checked at construction).  ``forward`` evaluates every node once; ``vjp`` takes ``{node name: gradient}`` for the
outputs that carry loss and walks the nodes in reverse, summing the gradients of values consumed more than once
(fan-out) before a node's own ``vjp`` runs.  Parameter paths are ``<node name>.<leaf path>``; a module shared by
several nodes is registered once under its first node name and accumulates parameter gradients over every use,
provided it is evaluated once per forward (modules cache one activation set).
Reference: ``ComputeGraph[*DECLS]`` (noeira/nn/combinators/compute_graph.mojo:74), declarations
``InputSlot / Node / ExternalNode`` (graph_decl.mojo:240,315,449), ``node_output``, ``grad_input``,
``set_node_attr``; ACT's loss graph is 4 input slots + 45 nodes (deep_agents/act/loss_graph.mojo:129-241).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from .module import Module


@dataclass
class InputSlot:
    name: str


@dataclass
class Node:
    name: str
    module: Optional[Module]
    inputs: Sequence[str] = field(default_factory=list)
    fn: Optional[Callable] = None        # ExternalNode: pure function of the inputs …
    fn_vjp: Optional[Callable] = None    # … with its backward ``(grad_out, *inputs) -> tuple of input grads``


def ExternalNode(name, fn, fn_vjp, inputs):
    return Node(name, None, inputs, fn, fn_vjp)


class ComputeGraph(Module):
    def __init__(self, decls: List):
        super().__init__()
        self.slots = [d.name for d in decls if isinstance(d, InputSlot)]
        self.nodes: List[Node] = [d for d in decls if isinstance(d, Node)]
        known = set(self.slots)
        seen_modules = {}
        for nd in self.nodes:
            if nd.name in known:
                raise ValueError(f"duplicate name {nd.name}")
            for i in nd.inputs:
                if i not in known:
                    raise ValueError(f"node {nd.name} reads {i} before it is defined")
            known.add(nd.name)
            if nd.module is not None and id(nd.module) not in seen_modules:
                seen_modules[id(nd.module)] = nd.name
                self.add_child(nd.name, nd.module)
        self._by_name = {nd.name: nd for nd in self.nodes}
        self.values: Dict[str, object] = {}
        self.grads: Dict[str, object] = {}

    # ------------------------------------------------------------------ forward / backward
    def set_input(self, name, value):
        assert name in self.slots, name
        self.values[name] = value

    def forward(self, *inputs, **named):
        for n, v in zip(self.slots, inputs):
            self.values[n] = v
        self.values.update(named)
        for nd in self.nodes:
            args = [self.values[i] for i in nd.inputs]
            self.values[nd.name] = nd.module.forward(*args) if nd.module is not None else nd.fn(*args)
        return self.values[self.nodes[-1].name]

    def node_output(self, name):
        return self.values[name]

    def vjp(self, grads):
        """``grads``: ``{name: grad}`` or a single gradient for the last node.  Returns ``{slot: grad}``."""
        if not isinstance(grads, dict):
            grads = {self.nodes[-1].name: grads}
        acc: Dict[str, object] = dict(grads)
        for nd in reversed(self.nodes):
            g = acc.pop(nd.name, None)
            if g is None:
                continue                       # nothing downstream of this node carries gradient
            if nd.module is not None:
                gi = nd.module.vjp(g)
            else:
                gi = nd.fn_vjp(g, *[self.values[i] for i in nd.inputs])
            if not isinstance(gi, (tuple, list)):
                gi = (gi,)
            for name, gin in zip(nd.inputs, gi):
                if gin is None:
                    continue
                acc[name] = gin if name not in acc else acc[name] + gin      # fan-out accumulation
        self.grads = acc
        return {s: acc.get(s) for s in self.slots}

    def grad_input(self, name):
        return self.grads.get(name)

    def set_node_attr(self, node, attr, value):
        self._by_name[node].module.set_attr(attr, value)

    def display_label(self):
        return f"ComputeGraph[{len(self.slots)} inputs, {len(self.nodes)} nodes]"

    # ------------------------------------------------------------------ exporters
    def describe(self, exporter: "GraphExporter", name: str = "graph") -> str:
        """Walk the declarations in order and let ``exporter`` render them
        (noeira/nn/combinators/graph_export.mojo:95,171,266: text, Mermaid and fusion-report visitors)."""
        exporter.begin(name, self)
        for s in self.slots:
            exporter.slot(s)
        consumers: Dict[str, List[str]] = {}
        for nd in self.nodes:
            for i in nd.inputs:
                consumers.setdefault(i, []).append(nd.name)
        for nd in self.nodes:
            label = nd.module.display_label() if nd.module is not None else f"external:{getattr(nd.fn, '__name__', 'fn')}"
            n_params = sum(p.numel for p in nd.module.params()) if nd.module is not None else 0
            exporter.node(nd.name, label, list(nd.inputs), n_params, consumers.get(nd.name, []))
        return exporter.end()


class GraphExporter:
    def begin(self, name, graph): ...
    def slot(self, name): ...
    def node(self, name, label, inputs, n_params, consumers): ...
    def end(self) -> str: return ""


class TextExporter(GraphExporter):
    """One line per declaration: ``name = Label(inputs)  [parameters]  -> consumers``."""

    def begin(self, name, graph):
        self.lines = [f"{name}: {graph.display_label()}"]

    def slot(self, name):
        self.lines.append(f"  input {name}")

    def node(self, name, label, inputs, n_params, consumers):
        tail = f"  [{n_params} params]" if n_params else ""
        fan = f"  -> {', '.join(consumers)}" if consumers else "  -> (output)"
        self.lines.append(f"  {name} = {label}({', '.join(inputs)}){tail}{fan}")

    def end(self):
        return "\n".join(self.lines)


class MermaidExporter(GraphExporter):
    """A ``flowchart TD`` document: rounded boxes for inputs, rectangles for nodes, one edge per use."""

    @staticmethod
    def _id(name):
        return "n_" + "".join(c if c.isalnum() else "_" for c in name)

    def begin(self, name, graph):
        self.lines = ["flowchart TD"]

    def slot(self, name):
        self.lines.append(f'  {self._id(name)}(["{name}"])')

    def node(self, name, label, inputs, n_params, consumers):
        self.lines.append(f'  {self._id(name)}["{name}<br/>{label}"]')
        for i in inputs:
            self.lines.append(f"  {self._id(i)} --> {self._id(name)}")

    def end(self):
        return "\n".join(self.lines)


class FusionReport(GraphExporter):
    """Lists what an epilogue-fusing backend can merge: a node with a single consumer whose consumer is an elementwise
    module (activation, bias add, scale, residual add) is a producer → epilogue pair; a value consumed more than once
    needs gradient accumulation in the backward (fan-out)."""

    ELEMENTWISE = ("Elementwise", "BiasAdd", "Scale", "Dropout", "external:add", "external:residual")

    def begin(self, name, graph):
        self.name, self.labels, self.inputs, self.consumers, self.order = name, {}, {}, {}, []

    def node(self, name, label, inputs, n_params, consumers):
        self.labels[name], self.inputs[name], self.consumers[name] = label, inputs, consumers
        self.order.append(name)

    def end(self):
        pairs, fanout = [], []
        for n in self.order:
            cons = self.consumers[n]
            if len(cons) == 1 and self.labels[cons[0]].startswith(self.ELEMENTWISE) and not self.labels[n].startswith(self.ELEMENTWISE):
                pairs.append((n, cons[0]))
            if len(cons) > 1:
                fanout.append((n, len(cons)))
        lines = [f"fusion report for {self.name}: {len(self.order)} nodes, {len(pairs)} producer/epilogue pairs, "
                 f"{len(fanout)} fan-out values"]
        lines += [f"  fuse {a} ({self.labels[a]}) + {b} ({self.labels[b]})" for a, b in pairs]
        lines += [f"  fan-out {n} x{k}: gradient accumulation in backward" for n, k in fanout]
        self.pairs, self.fanout = pairs, fanout
        return "\n".join(lines)
