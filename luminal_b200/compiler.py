"""Host-side mirror of the graph rewrite that inserts the quantized operators.

In luminal a `Compiler` pass walks the graph and replaces nodes; `CudaQuantizedCompiler<T>`
(crates/luminal_cuda/src/quantized.rs:235-272) is the pass of this path: every op directly downstream of a listed
Q8_0 weight node is replaced - a `Matmul` by `QuantizedMatmul`, a `CudaGather` by `QuantizedGather` - the weight has to
be input #1 of that op, and anything else panics.  "Downstream" follows a weight through chains of single-consumer ops
whose inputs all come from the weight set (src/module.rs:85-116), which is how a weight that first passes through a
copy-to-device node is still found.

This module is that pass over a small graph structure of its own (node id -> op, edges carrying the input index), so
that the rewrite rule can be exercised here, where the Rust crate (luminal_b200/rust) cannot be compiled.  The ops it
inserts are the operator mirrors of luminal_b200/ops.py.
"""
from dataclasses import dataclass, field

from . import ops


class CompileError(Exception):
    """What the reference reports with a panic."""


@dataclass
class Matmul:
    """Placeholder for crates/luminal_cuda/src/matmul.rs::Matmul<T> before the rewrite."""


@dataclass
class CudaGatherNode:
    """Placeholder for crates/luminal_cuda/src/binary.rs::CudaGather<T> before the rewrite."""
    embed_dim: int


@dataclass
class Function:
    """A weight / input node (luminal's `Function` op)."""
    name: str


@dataclass
class Graph:
    ops: dict = field(default_factory=dict)          # node id -> op object
    edges: list = field(default_factory=list)        # (source id, target id, input index of the target)
    _next: int = 0

    def add_op(self, op, inputs=()):
        """inputs: source node ids in input order (index 0, 1, ...), as `graph.add_op(op).input(src, ..)` lists them."""
        nid = self._next
        self._next += 1
        self.ops[nid] = op
        for i, src in enumerate(inputs):
            self.edges.append((src, nid, i))
        return nid

    def outgoing(self, nid):
        return [(dst, idx) for src, dst, idx in self.edges if src == nid]

    def incoming(self, nid):
        return [src for src, dst, _ in self.edges if dst == nid]


def _is_from_set(node, graph, orig):
    """All of `node`'s ancestors lead back to the original set (src/module.rs:118-133)."""
    if node in orig:
        return True
    srcs = graph.incoming(node)
    return bool(srcs) and all(_is_from_set(s, graph, orig) for s in srcs)


def downstream(nodes, graph):
    """Follows every node down single-consumer chains that are fed only from the set (src/module.rs:85-116)."""
    orig, out, seen = set(nodes), [], set()
    for node in nodes:
        while len(graph.outgoing(node)) == 1:
            nxt = graph.outgoing(node)[0][0]
            if not _is_from_set(nxt, graph, orig):
                break
            node = nxt
        if node not in seen:
            seen.add(node)
            out.append(node)
    return out


class BlumQuantizedCompiler:
    """The rewrite of CudaQuantizedCompiler<T>::compile with libblum's operators as the replacements."""

    def __init__(self, ctx, weights, dtype):
        self.ctx, self.weights, self.dtype = ctx, list(weights), dtype

    def compile(self, graph: Graph):
        replaced = []
        for weight in downstream(self.weights, graph):
            for target, inp_ind in graph.outgoing(weight):
                if inp_ind != 1:
                    raise CompileError("Quantized weight %r is the wrong input!" % (target,))
                op = graph.ops[target]
                if isinstance(op, CudaGatherNode):
                    graph.ops[target] = ops.QuantizedGather(self.ctx, op.embed_dim, self.dtype)
                elif isinstance(op, Matmul):
                    graph.ops[target] = ops.QuantizedMatmul(self.ctx, self.dtype)
                else:
                    raise CompileError("Quantized weight %r is an input to a node that isn't a matmul or gather (%r)" % (target, op))
                replaced.append(target)
        return replaced
