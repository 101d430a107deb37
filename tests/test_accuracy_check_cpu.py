"""Host logic of the per-intermediate accuracy check (no GPU): graph capture, the all-
intermediates rewrite, digests in the reference's form, and that a deliberately wrong
"compiled" graph is pinned to the node that went wrong."""
import hashlib

import torch
import torch.fx as fx
import torch.nn.functional as F

from inductor_x_b200 import accuracy_check as ac


def fn(x, w, b):
    y = F.gelu(x * w + b)
    var, mean = torch.var_mean(y, -1, keepdim=True)
    return ((y - mean) * torch.rsqrt(var + 1e-5)).sum(-1)


def args():
    g = torch.Generator().manual_seed(0)
    return torch.randn(8, 64, generator=g), torch.randn(64, generator=g), torch.randn(64, generator=g)


def test_md5_is_the_reference_digest():
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    assert ac.md5_of(t) == hashlib.md5(t.to(torch.float64).numpy().tobytes()).hexdigest()
    assert ac.md5_of(t) == ac.md5_of(t.to(torch.bfloat16))      # values, not storage, are hashed


def test_identity_compile_agrees_everywhere():
    rep = ac.check(fn, *args(), compile_fn=lambda gm, inputs: gm.forward)
    assert rep.ok and rep.first_mismatch() is None
    names = [r.name for r in rep.records]
    assert len(names) >= 8 and all(r.compiled_md5 == r.eager_md5 for r in rep.records)
    # tuple-valued var_mean is recorded through its getitem users only
    assert not any(r.op.endswith("var_mean") for r in rep.records)
    text = rep.format()
    assert text.count("eager:") == len(names) and text.endswith("all nodes within tolerance")


def test_first_wrong_node_is_named():
    def faulty(gm: fx.GraphModule, inputs):
        # a backend whose gelu is off by 1e-3: everything downstream differs too, the report
        # must point at gelu itself
        g = gm.graph
        for n in list(g.nodes):
            if n.op == "call_function" and "gelu" in str(n.target):
                with g.inserting_after(n):
                    bumped = g.call_function(torch.add, (n, 1e-3))
                n.replace_all_uses_with(bumped, delete_user_cb=lambda u: u is not bumped)
        g.lint()
        gm.recompile()
        return gm.forward

    rep = ac.check(fn, *args(), compile_fn=faulty)
    bad = rep.first_mismatch()
    assert not rep.ok and bad is not None and "gelu" in bad.op
    assert bad.max_abs > 5e-4 and "first mismatch: " + bad.name in rep.format()
    before = rep.records[:[r.name for r in rep.records].index(bad.name)]
    assert before and all(r.ok for r in before)


def test_integer_nodes_compare_exactly():
    f = lambda x: (x.argmax(-1) + 1) * 2
    rep = ac.check(f, torch.randn(4, 9), compile_fn=lambda gm, inputs: gm.forward)
    assert rep.ok and any(not r.dtype.is_floating_point for r in rep.records)
