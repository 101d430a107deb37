"""Per-intermediate accuracy check: which node of a compiled graph first disagrees with eager?

The reference debugs a wrong result by rewriting the files Inductor dumps
(``fx_graph_readable.py`` and ``output_code.py``) so that an md5 of every intermediate is
printed, or every tensor saved, on both sides, and diffing the two logs
(``test/npu_indexing/accuracy_check/fx_graph_gen.py:31-81``,
``test/npu_indexing/accuracy_check/gen_output_code.py:65-122,176-203``; the ``utils`` module
those scripts import is not part of the reference tree).  The same question is answered here
without text rewriting:

1. the graph Dynamo hands to the backend is captured together with its real inputs;
2. an FX interpreter runs it eagerly and records every tensor-valued node;
3. the graph is rebuilt so that it *returns* every such node and is compiled by the backend
   under test - the kernels stay fused, but each intermediate is also written out;
4. both sides are compared node by node (md5 of the float64 bytes, the reference's digest,
   plus maximum absolute / relative error) and the first node that is out of tolerance is named.

``check(fn, *args)`` does all four steps and returns a :class:`Report`.
"""
from __future__ import annotations

import dataclasses
import hashlib
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx

__all__ = ["md5_of", "trace_intermediates", "return_all_intermediates", "capture_graphs", "check",
           "NodeRecord", "Report"]


def md5_of(t: torch.Tensor) -> str:
    """Digest of a tensor as the reference prints it: md5 of its values widened to float64
    (``fx_graph_gen.py:62``)."""
    return hashlib.md5(t.detach().to(torch.float64).cpu().contiguous().numpy().tobytes()).hexdigest()


@dataclasses.dataclass
class NodeRecord:
    name: str
    op: str
    shape: Tuple[int, ...]
    dtype: torch.dtype
    eager_md5: str
    compiled_md5: Optional[str] = None
    max_abs: Optional[float] = None
    max_rel: Optional[float] = None
    ok: Optional[bool] = None


@dataclasses.dataclass
class Report:
    graphs: List[List[NodeRecord]]

    @property
    def records(self) -> List[NodeRecord]:
        return [r for g in self.graphs for r in g]

    @property
    def ok(self) -> bool:
        return all(r.ok is not False for r in self.records)

    def first_mismatch(self) -> Optional[NodeRecord]:
        """The first node, in execution order, that is out of tolerance: everything before
        it agreed, so the kernel that produces it is where to look."""
        for r in self.records:
            if r.ok is False:
                return r
        return None

    def format(self, side: str = "both") -> str:
        """One ``<side>:<node>:<md5>`` line per node, the shape of the reference's logs
        (``fx_graph_gen.py:63,80``), followed by the overall result."""
        lines = []
        for r in self.records:
            if side in ("eager", "both"):
                lines.append(f"eager:{r.name}:{r.eager_md5}")
            if side in ("compiled", "both") and r.compiled_md5 is not None:
                mark = "" if r.ok else f"   <-- max_abs {r.max_abs:.3e} max_rel {r.max_rel:.3e}"
                lines.append(f"compiled:{r.name}:{r.compiled_md5}{mark}")
        bad = self.first_mismatch()
        lines.append("all nodes within tolerance" if bad is None
                     else f"first mismatch: {bad.name} ({bad.op}, {tuple(bad.shape)}, {bad.dtype})")
        return "\n".join(lines)


def _tensor_nodes(gm: fx.GraphModule, values: Dict[str, Any]) -> List[fx.Node]:
    return [n for n in gm.graph.nodes
            if n.op not in ("placeholder", "output") and isinstance(values.get(n.name), torch.Tensor)]


class _Recorder(fx.Interpreter):
    def __init__(self, gm: fx.GraphModule):
        super().__init__(gm)
        self.values: Dict[str, Any] = {}

    def run_node(self, n: fx.Node) -> Any:
        out = super().run_node(n)
        self.values[n.name] = out
        return out


def trace_intermediates(gm: fx.GraphModule, *args) -> Tuple[List[NodeRecord], Dict[str, torch.Tensor]]:
    """Run ``gm`` node by node in eager mode.  Returns one record per tensor-valued node
    (tuple-valued ops such as ``var_mean`` are recorded through their ``getitem`` users, as
    the reference skips them, ``fx_graph_gen.py:5-16``) and the tensors themselves."""
    rec = _Recorder(gm)
    with torch.no_grad():
        rec.run(*args)
    nodes = _tensor_nodes(gm, rec.values)
    records = [NodeRecord(n.name, str(n.target) if n.op != "call_method" else f"method {n.target}",
                          tuple(rec.values[n.name].shape), rec.values[n.name].dtype,
                          md5_of(rec.values[n.name])) for n in nodes]
    return records, {n.name: rec.values[n.name] for n in nodes}


def return_all_intermediates(gm: fx.GraphModule, names: Sequence[str]) -> fx.GraphModule:
    """A copy of ``gm`` whose output is the tuple of the nodes called ``names``."""
    import copy

    g = copy.deepcopy(gm.graph)
    by_name = {n.name: n for n in g.nodes}
    out = next(n for n in g.nodes if n.op == "output")
    with g.inserting_before(out):
        g.output(tuple(by_name[k] for k in names))
    g.erase_node(out)
    g.lint()
    return fx.GraphModule(gm, g)


def capture_graphs(fn: Callable, *args, **kwargs) -> List[Tuple[fx.GraphModule, List[torch.Tensor]]]:
    """The graphs (one per graph break) and real inputs Dynamo would hand to a backend."""
    captured: List[Tuple[fx.GraphModule, List[torch.Tensor]]] = []

    def backend(gm: fx.GraphModule, example_inputs):
        captured.append((gm, [t.detach().clone() if isinstance(t, torch.Tensor) else t for t in example_inputs]))
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(fn, backend=backend)(*args, **kwargs)
    torch._dynamo.reset()
    return captured


def _inductor_compile(gm: fx.GraphModule, example_inputs):
    from torch._inductor.compile_fx import compile_fx

    return compile_fx(gm, example_inputs)


def _errors(actual: torch.Tensor, expected: torch.Tensor) -> Tuple[float, float]:
    a, e = actual.detach().to(torch.float64).cpu(), expected.detach().to(torch.float64).cpu()
    both_nan = torch.isnan(a) & torch.isnan(e)
    same_inf = torch.isinf(a) & torch.isinf(e) & (a == e)
    diff = torch.where(both_nan | same_inf, torch.zeros_like(a), (a - e).abs())
    diff = torch.nan_to_num(diff, nan=float("inf"))
    if diff.numel() == 0:
        return 0.0, 0.0
    scale = torch.maximum(e.abs(), e[torch.isfinite(e)].pow(2).mean().sqrt() if torch.isfinite(e).any()
                          else torch.ones(()))
    rel = diff / torch.clamp(scale, min=1e-30)
    return float(diff.max()), float(rel.max())


def check(fn: Callable, *args, rtol: Optional[float] = None, atol: float = 0.0,
          compile_fn: Optional[Callable] = None, **kwargs) -> Report:
    """Compare every intermediate of ``fn(*args)`` between eager execution and the compiled
    graph.  ``rtol`` defaults per dtype (1e-5 for fp32 and wider, 2e-2 for 16-bit floats,
    exact for integers and booleans), relative to ``max(|expected|, rms(expected))``.
    ``compile_fn(gm, example_inputs) -> callable`` defaults to Inductor with whatever backend
    is registered for the tensors' device."""
    compile_fn = compile_fn or _inductor_compile
    graphs: List[List[NodeRecord]] = []
    for gm, inputs in capture_graphs(fn, *args, **kwargs):
        records, eager = trace_intermediates(gm, *inputs)
        if not records:
            graphs.append(records)
            continue
        names = [r.name for r in records]
        gm_all = return_all_intermediates(gm, names)
        with torch.no_grad():
            compiled = compile_fn(gm_all, [t.clone() if isinstance(t, torch.Tensor) else t for t in inputs])
            outs = compiled(*[t.clone() if isinstance(t, torch.Tensor) else t for t in inputs])
        for r, got in zip(records, outs):
            want = eager[r.name]
            r.compiled_md5 = md5_of(got)
            r.max_abs, r.max_rel = _errors(got, want)
            if tuple(got.shape) != tuple(want.shape) or got.dtype != want.dtype:
                r.ok = False
            elif not want.dtype.is_floating_point:
                r.ok = r.max_abs == 0.0
            else:
                tol = rtol if rtol is not None else (2e-2 if want.element_size() <= 2 else 1e-5)
                r.ok = r.max_rel <= tol or r.max_abs <= atol
        graphs.append(records)
    return Report(graphs)
