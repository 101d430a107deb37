"""CPU tests of the fused-attention FX patterns: the joint-graph pass is run by Inductor on CPU
tensors and the graph is inspected before code generation (the op itself has a device
implementation only, so nothing is executed)."""
import math

import pytest
import torch


class _Stop(Exception):
    pass


def _targets_after_joint_passes(fn, *args):
    """Call targets of the graph after Inductor's joint-graph patterns ran."""
    import inductor_x_b200  # noqa: F401  (registers the patterns)

    seen = {}

    def grab(graph):
        seen["targets"] = [str(n.target) for n in graph.nodes if n.op == "call_function"]
        raise _Stop()

    old = (torch._inductor.config.post_grad_custom_pre_pass, torch._inductor.config.fx_graph_cache)
    torch._inductor.config.post_grad_custom_pre_pass = grab
    torch._inductor.config.fx_graph_cache = False
    torch._dynamo.reset()
    try:
        torch.compile(fn)(*args)
    except Exception:
        pass
    finally:
        torch._inductor.config.post_grad_custom_pre_pass, torch._inductor.config.fx_graph_cache = old
        torch._dynamo.reset()
    return seen.get("targets", [])


def _literal_attention(tri: str, form: str, scale: float):
    def attention(q, k, v):
        s_len = q.shape[-2]
        keep = getattr(torch.ones(s_len, s_len, dtype=torch.bool, device=q.device), tri)()
        s = torch.matmul(q, k.transpose(-2, -1))
        s = s * scale if form == "mul" else s / (1.0 / scale)
        s = s.masked_fill(~keep, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), v)

    return attention


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("form", ["mul", "div"])
def test_literal_causal_attention_is_matched(dtype, form):
    """matmul -> scale -> masked_fill(causal) -> softmax -> matmul, the way benchmark
    configuration 4 writes it, becomes one b200_fa call and both batched matmuls disappear."""
    q, k, v = (torch.randn(2, 4, 64, 128).to(dtype) for _ in range(3))
    targets = _targets_after_joint_passes(_literal_attention("tril", form, 1 / math.sqrt(128)), q, k, v)
    assert "b200_graph.b200_sdpa.default" in targets
    assert "aten.bmm.default" not in targets


def test_masks_that_are_not_provably_causal_are_left_alone():
    q, k, v = (torch.randn(2, 4, 64, 128).bfloat16() for _ in range(3))
    # upper-triangular mask built in the graph
    targets = _targets_after_joint_passes(_literal_attention("triu", "mul", 0.1), q, k, v)
    assert "b200_graph.b200_sdpa.default" not in targets and targets.count("aten.bmm.default") == 2
    # a mask that is a graph input: nothing can be proven about it
    keep = torch.ones(64, 64, dtype=torch.bool).tril()

    def with_input_mask(q, k, v, keep):
        s = (torch.matmul(q, k.transpose(-2, -1)) * 0.1).masked_fill(~keep, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), v)

    targets = _targets_after_joint_passes(with_input_mask, q, k, v, keep)
    assert "b200_graph.b200_sdpa.default" not in targets
    # longer key sequence: top-left and bottom-right causal masks differ

    def longer_keys(q, k, v):
        keep = torch.ones(64, 128, dtype=torch.bool).tril()
        s = (torch.matmul(q, k.transpose(-2, -1)) * 0.1).masked_fill(~keep, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), v)

    k2, v2 = (torch.randn(2, 4, 128, 128).bfloat16() for _ in range(2))
    targets = _targets_after_joint_passes(longer_keys, q, k2, v2)
    assert "b200_graph.b200_sdpa.default" not in targets


def test_float32_attention_needs_the_opt_in():
    from inductor_x_b200 import config

    q, k, v = (torch.randn(2, 4, 64, 128) for _ in range(3))
    fn = _literal_attention("tril", "mul", 0.1)
    assert "b200_graph.b200_sdpa.default" not in _targets_after_joint_passes(fn, q, k, v)
    config.attention_fp32_as_fp16 = True
    try:
        assert "b200_graph.b200_sdpa.default" in _targets_after_joint_passes(fn, q, k, v)
    finally:
        config.attention_fp32_as_fp16 = False


def test_lower_triangular_proof():
    """The walker accepts only the forms tril() decomposes to."""
    from torch.fx.experimental.proxy_tensor import make_fx
    from torch._inductor.decomposition import select_decomp_table

    from inductor_x_b200.fusion_attention_graph import _is_lower_triangular

    def last(fn):
        gm = make_fx(fn, decomposition_table=select_decomp_table(), tracing_mode="fake")()
        return [n for n in gm.graph.nodes if n.op == "output"][0].args[0]

    assert _is_lower_triangular(last(lambda: torch.ones(8, 8, dtype=torch.bool).tril()))
    assert not _is_lower_triangular(last(lambda: torch.ones(8, 8, dtype=torch.bool).triu()))
    assert not _is_lower_triangular(last(lambda: torch.ones(8, 8, dtype=torch.bool).tril(1)))
    assert not _is_lower_triangular(last(lambda: torch.ones(8, 8, dtype=torch.bool).tril(-1)))
    assert not _is_lower_triangular(last(lambda: torch.rand(8, 8) > 0.5))


def _joint_targets(fn, *args):
    """Call targets of the joint (forward + backward) graph after the joint-graph patterns."""
    import inductor_x_b200  # noqa: F401

    seen = {}

    def grab(graph):
        seen["targets"] = [str(n.target) for n in graph.nodes if n.op == "call_function"]
        raise _Stop()

    old = (torch._inductor.config.joint_custom_post_pass, torch._inductor.config.fx_graph_cache)
    torch._inductor.config.joint_custom_post_pass = grab
    torch._inductor.config.fx_graph_cache = False
    torch._dynamo.reset()
    try:
        torch.compile(fn)(*args)
    except Exception:
        pass
    finally:
        torch._inductor.config.joint_custom_post_pass, torch._inductor.config.fx_graph_cache = old
        torch._dynamo.reset()
    return seen.get("targets", [])


@pytest.mark.parametrize("form", ["mul", "div"])
def test_training_graph_of_literal_causal_attention_is_matched(form):
    """With gradients required, forward AND backward of the pattern are replaced in the joint
    graph: the compact op and its registered gradient, no batched matmul left."""
    q, k, v = (torch.randn(2, 4, 64, 128).bfloat16().requires_grad_() for _ in range(3))
    targets = _joint_targets(_literal_attention("tril", form, 1 / math.sqrt(128)), q, k, v)
    assert "b200_graph.b200_sdpa.default" in targets
    assert "b200_graph.b200_sdpa_backward.default" in targets
    assert "aten.bmm.default" not in targets
    # an upper-triangular mask is left alone in training as well
    targets = _joint_targets(_literal_attention("triu", form, 0.1), q, k, v)
    assert "b200_graph.b200_sdpa.default" not in targets and targets.count("aten.bmm.default") == 6


def test_training_graph_of_the_reference_pattern_is_matched():
    """The reference's pattern 1 without dropout (permute x3, matmul, div, softmax, matmul)
    in a training graph: b200_fa forward, b200_fa_backward for the gradients."""
    def attention(q, k, v):
        q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        return torch.matmul(q, k.transpose(-2, -1)).div(11.3).softmax(dim=-1).matmul(v)

    q, k, v = (torch.randn(2, 64, 4, 128).half().requires_grad_() for _ in range(3))
    targets = _joint_targets(attention, q, k, v)
    assert "b200_graph.b200_fa.default" in targets
    assert "b200_graph.b200_fa_backward.default" in targets
    assert "aten.bmm.default" not in targets
