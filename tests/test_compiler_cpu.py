"""The graph rewrite that inserts the quantized operators (mirror of CudaQuantizedCompiler::compile,
crates/luminal_cuda/src/quantized.rs:244-271): which nodes are replaced, and what is refused."""
import pytest

from luminal_b200 import F32, ops
from luminal_b200.compiler import (BlumQuantizedCompiler, CompileError, CudaGatherNode, Function, Graph, Matmul,
                                   downstream)


def _llama_like():
    g = Graph()
    ids = g.add_op(Function("ids"))
    embed = g.add_op(Function("token_embd.weight"))
    x = g.add_op(CudaGatherNode(embed_dim=64), [ids, embed])
    wq = g.add_op(Function("blk.0.attn_q.weight"))
    q = g.add_op(Matmul(), [x, wq])
    wo = g.add_op(Function("blk.0.attn_output.weight"))
    copy = g.add_op(Function("copy_to_device"), [wo])          # a weight that first passes through a single-consumer node
    o = g.add_op(Matmul(), [q, copy])
    act = g.add_op(Function("activation"))
    other = g.add_op(Matmul(), [o, act])                       # an unquantized matmul stays as it is
    return g, dict(ids=ids, embed=embed, x=x, wq=wq, q=q, wo=wo, copy=copy, o=o, other=other)


def test_ops_downstream_of_the_listed_weights_are_replaced():
    g, n = _llama_like()
    done = BlumQuantizedCompiler(None, [n["embed"], n["wq"], n["wo"]], F32).compile(g)
    assert sorted(done) == sorted([n["x"], n["q"], n["o"]])
    assert isinstance(g.ops[n["x"]], ops.QuantizedGather) and g.ops[n["x"]].embed_dim == 64
    assert isinstance(g.ops[n["q"]], ops.QuantizedMatmul) and isinstance(g.ops[n["o"]], ops.QuantizedMatmul)
    assert isinstance(g.ops[n["other"]], Matmul)


def test_downstream_follows_single_consumer_chains_only():
    g, n = _llama_like()
    assert downstream([n["wo"]], g) == [n["copy"]]              # through the copy node, not into the matmul (x is not from the set)
    assert downstream([n["wq"]], g) == [n["wq"]]


def test_weight_as_input_zero_is_refused():
    g = Graph()
    w = g.add_op(Function("w"))
    x = g.add_op(Function("x"))
    g.add_op(Matmul(), [w, x])
    with pytest.raises(CompileError, match="wrong input"):
        BlumQuantizedCompiler(None, [w], F32).compile(g)


def test_weight_feeding_something_else_is_refused():
    g = Graph()
    w = g.add_op(Function("w"))
    x = g.add_op(Function("x"))
    g.add_op(Function("add"), [x, w])
    with pytest.raises(CompileError, match="isn't a matmul or gather"):
        BlumQuantizedCompiler(None, [w], F32).compile(g)
