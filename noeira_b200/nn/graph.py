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
