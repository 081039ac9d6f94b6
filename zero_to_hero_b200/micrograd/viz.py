"""Graphviz DOT text of a computation graph (nn/micrograd/viz.py:4-31 of the reference).
The DOT source is written directly, so neither the `graphviz` package nor the `dot` binary is
needed; nodes are records `label | data | grad`, every op gets its own small node."""
from __future__ import annotations


def to_dot(node) -> str:
    lines = ["digraph {", "\tgraph [rankdir=LR]"]
    visited = set()
    stack = [node]
    while stack:
        n = stack.pop()
        if id(n) in visited:
            continue
        visited.add(id(n))
        nid = str(id(n))
        lines.append(f'\t{nid} [label="{n.label} | data={n.data:.4f} | grad={n.grad:.4f}" shape=record]')
        if n._op:
            op_id = f'"{nid}_{n._op}"'
            lines.append(f'\t{op_id} [label="{n._op}"]')
            lines.append(f"\t{op_id} -> {nid}")
            for c in n._children:
                lines.append(f"\t{id(c)} -> {op_id}")
                stack.append(c)
    lines.append("}")
    return "\n" + "\n".join(lines) + "\n"
