"""GPU parity tests of the fused-attention kernel (tcgen05 / TMEM / TMA) through the C ABI.

Tolerance: 2e-2 relative to max(|expected|, rms of the expected row) for fp16 / bf16
outputs (rows of a causal output differ in scale, so each is judged on its own);
log-sum-exp within 2e-3 absolute (it is accumulated in fp32)."""
import math

import pytest
import torch

from inductor_x_b200 import ops
from inductor_x_b200 import runtime as rt
from oracle import c_oracle, graphs, inputs

pytestmark = pytest.mark.gpu
TOL = 2e-2


def run(d, cuda, causal, **kw):
    q, k, v = (d[n].to(cuda) for n in "qkv")
    return ops.fused_attention(q, k, v, d["scale"], causal=causal, return_lse=True, check=True, **kw)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 384), (1, 1, 1000), (1, 2, 77),
                                   (2, 2, 1536)])
def test_attention_vs_oracle(cuda, dtype, causal, B, H, S):
    d = inputs.c4(B, H, S, 128, seed=B * 100 + S, dtype=dtype)
    out, lse = run(d, cuda, causal)
    exp, elog = graphs.attention(d["q"], d["k"], d["v"], d["scale"], causal=causal)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL
    assert float((lse.cpu() - elog).abs().max()) <= 2e-3


def test_attention_vs_c_oracle_small(cuda):
    d = inputs.c4(1, 2, 160, 128, seed=9)
    out, lse = run(d, cuda, True)
    exp, elog = c_oracle.attention(d["q"], d["k"], d["v"], d["scale"], causal=True)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL
    assert float((lse.cpu().double() - elog).abs().max()) <= 2e-3


def test_attention_cross_lengths(cuda):
    # Sk > Sq: non-causal and bottom-right aligned causal
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 2, 130, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 450, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 450, 128, generator=g).bfloat16()
    sc = 1 / math.sqrt(128)
    for causal in (False, True):
        out = ops.fused_attention(q.to(cuda), k.to(cuda), v.to(cuda), sc, causal=causal, check=True)
        exp, _ = graphs.attention(q, k, v, sc, causal=causal)
        assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL


def test_attention_transposed_layout_no_copy(cuda):
    # [B, S, N, D] storage viewed as [B, N, S, D], as the reference's replacement produces
    # with query.transpose(1, 2) (inductor_x/npu_fusion_attention_graph.py:150-164)
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, 300, 4, 128, generator=g).bfloat16() for _ in range(3))
    qd, kd, vd = (t.to(cuda).transpose(1, 2) for t in (q, k, v))
    assert not qd.is_contiguous()
    out = ops.fused_attention(qd, kd, vd, 0.1, causal=False, check=True)
    exp = graphs.attention_pattern(q.float(), k.float(), v.float(), 10.0)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL


def test_attention_reference_pattern_golden(cuda, golden):
    # the reference's own search pattern (fp32 eager) on its [B, S, N, D] inputs
    p = inputs.c4_pattern(2, 96, 3, 128, seed=4)
    exp = graphs.attention_pattern(p["query"], p["key"], p["value"], p["inv_scale_factor"])
    q, k, v = (p[n].bfloat16().to(cuda).transpose(1, 2) for n in ("query", "key", "value"))
    out = ops.fused_attention(q, k, v, 1.0 / p["inv_scale_factor"], causal=False, check=True)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL


def test_attention_large_scores_rescale_path(cuda):
    # scores that keep growing along the key axis force the lazy O rescale to trigger
    B, H, S = 1, 1, 1024
    q = torch.ones(B, H, S, 128)
    k = (torch.arange(S).float() / S * 3).view(1, 1, S, 1).expand(B, H, S, 128).contiguous()
    v = torch.randn(B, H, S, 128, generator=torch.Generator().manual_seed(1))
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out, lse = ops.fused_attention(q.to(cuda), k.to(cuda), v.to(cuda), 1.0, causal=False,
                                   return_lse=True, check=True)
    exp, elog = graphs.attention(q, k, v, 1.0, causal=False)
    assert graphs.max_rel_err(out.cpu(), exp, dim=-1) <= TOL
    assert float((lse.cpu() - elog).abs().max()) <= 5e-3 * float(elog.abs().max())


def test_attention_full_size_rows_vs_golden(cuda, golden):
    d = inputs.c4()
    out, lse = run(d, cuda, True)
    rows = golden["c4_rows"].tolist()
    for i, (b, h) in enumerate(golden["c4_heads"].tolist()):
        got = out[b, h][rows].cpu()
        assert graphs.max_rel_err(got, golden["c4_out_rows"][i], dim=-1) <= TOL
        assert float((lse[b, h][rows].cpu() - golden["c4_lse_rows"][i]).abs().max()) <= 2e-3
    # size-independent property: causal row 0 attends to key 0 only -> out[0] == v[0]
    assert torch.equal(out[:, :, 0].cpu(), d["v"][:, :, 0])
    # and every output row is a convex combination of V rows
    assert float(out.float().abs().max()) <= float(d["v"].float().abs().max()) + 1e-3


def test_attention_argument_errors(cuda):
    q = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(rt.IxbError) as e:
        ops.fused_attention(q, q, q, 1.0)
    assert e.value.status == rt.IXB_ERR_SHAPE  # head dim != 128
    q = torch.zeros(1, 1, 8, 128, dtype=torch.float32, device=cuda)
    with pytest.raises(ValueError):
        ops.fused_attention(q, q, q, 1.0)
    q = torch.zeros(1, 1, 300, 128, dtype=torch.bfloat16, device=cuda)
    k = torch.zeros(1, 1, 100, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(rt.IxbError):
        ops.fused_attention(q, k, k, 1.0, causal=True)  # causal with Sk < Sq
    empty = ops.fused_attention(q[:, :, :0], k, k, 1.0)
    assert empty.shape == (1, 1, 0, 128)


@pytest.mark.parametrize("layout", ["BNSD", "BSND", "BSH"])
@pytest.mark.parametrize("causal", [False, True])
def test_autograd_through_the_attention_op(layout, causal):
    """Gradients through `b200_fusion_attention_graph` (forward on the tcgen05 kernel,
    backward through `b200_fa_backward`) against autograd through eager fp32 attention on
    the same inputs.  Tolerance per tensor relative to max(|expected|, rms): 2e-2 for the
    output, 4e-2 for the bf16 gradients (probabilities and dS are rounded to bf16 before
    their products, as in every tensor-core attention backward)."""
    from inductor_x_b200.fusion_attention_graph import b200_fusion_attention_graph

    B, N, S, D = 2, 3, 192, 128
    g = torch.Generator().manual_seed(17)
    q, k, v, dy = (torch.randn(B, N, S, D, generator=g).to(torch.bfloat16).cuda() for _ in range(4))
    scale = 1.0 / math.sqrt(D)

    def to_layout(t):
        if layout == "BNSD":
            return t.clone()
        if layout == "BSND":
            return t.transpose(1, 2).contiguous()
        return t.transpose(1, 2).reshape(B, S, N * D).contiguous()

    ql, kl, vl = (to_layout(t).requires_grad_(True) for t in (q, k, v))
    out = b200_fusion_attention_graph(ql, kl, vl, N, layout, scale=1.0 / scale,
                                      sparse_mode=3 if causal else 0)[0]
    out.backward(to_layout(dy))

    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    s = torch.matmul(qr, kr.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=s.device).tril(), float("-inf"))
    ref = torch.matmul(torch.softmax(s, -1), vr)
    ref.backward(dy.float())
    assert graphs.max_rel_err(out.detach().float().cpu(), to_layout(ref.detach()).cpu()) <= 2e-2
    for got, want in ((ql.grad, qr.grad), (kl.grad, kr.grad), (vl.grad, vr.grad)):
        assert got is not None and got.dtype == torch.bfloat16
        assert graphs.max_rel_err(got.float().cpu(), to_layout(want).cpu()) <= 4e-2


# ---- backward (ixb_fa_bwd) ---------------------------------------------------------------
# Tolerance relative to max(|expected|, rms of the expected tensor): 4e-2 for bf16, 8e-3 for
# fp16.  P and dS are rounded to 16 bits before their products (8 / 11 significant bits) and
# delta uses the 16-bit forward output; the fp16 bound is the one that would expose a wrong
# mask edge or a misplaced tile.
GRAD_TOL = {torch.bfloat16: 4e-2, torch.float16: 8e-3}


def _backward_case(cuda, dtype, causal, B, H, Sq, Sk, seed):
    g = torch.Generator().manual_seed(seed)
    q, dy = (torch.randn(B, H, Sq, 128, generator=g).to(dtype) for _ in range(2))
    k, v = (torch.randn(B, H, Sk, 128, generator=g).to(dtype) for _ in range(2))
    scale = 1 / math.sqrt(128)
    qd, kd, vd, dyd = (t.to(cuda) for t in (q, k, v, dy))
    out, lse = ops.fused_attention(qd, kd, vd, scale, causal=causal, return_lse=True, check=True)
    got = ops.fused_attention_backward(qd, kd, vd, out, lse, dyd, scale, causal=causal, check=True)
    want = graphs.attention_backward(q, k, v, dy, scale, causal=causal)
    return got, want


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 384), (1, 2, 77), (1, 1, 1000)])
def test_attention_backward_vs_oracle(cuda, dtype, causal, B, H, S):
    got, want = _backward_case(cuda, dtype, causal, B, H, S, S, seed=B * 10 + S)
    for name, a, e in zip(("dq", "dk", "dv"), got, want):
        assert a.dtype == dtype and a.shape == e.shape
        assert graphs.max_rel_err(a.float().cpu(), e) <= GRAD_TOL[dtype], name


@pytest.mark.parametrize("causal", [False, True])
def test_attention_backward_cross_lengths(cuda, causal):
    # Sk > Sq, ragged in both: bottom-right aligned causal mask
    got, want = _backward_case(cuda, torch.float16, causal, 1, 2, 130, 450, seed=3)
    for name, a, e in zip(("dq", "dk", "dv"), got, want):
        assert graphs.max_rel_err(a.float().cpu(), e) <= GRAD_TOL[torch.float16], name


def test_attention_backward_transposed_layout_and_determinism(cuda):
    # [B, S, N, D] storage viewed as [B, N, S, D]: taken through strides, no copy; two runs
    # give the same bits (single owner per output tile, no atomics)
    g = torch.Generator().manual_seed(11)
    q, k, v, dy = (torch.randn(2, 300, 4, 128, generator=g).bfloat16() for _ in range(4))
    qd, kd, vd, dyd = (t.to(cuda).transpose(1, 2) for t in (q, k, v, dy))
    out, lse = ops.fused_attention(qd, kd, vd, 0.1, causal=True, return_lse=True, check=True)
    got = ops.fused_attention_backward(qd, kd, vd, out, lse, dyd, 0.1, causal=True, check=True)
    again = ops.fused_attention_backward(qd, kd, vd, out, lse, dyd, 0.1, causal=True, check=True)
    want = graphs.attention_backward(*(t.transpose(1, 2) for t in (q, k, v, dy)), 0.1, causal=True)
    for name, a, b2, e in zip(("dq", "dk", "dv"), got, again, want):
        assert torch.equal(a, b2), name
        assert graphs.max_rel_err(a.float().cpu(), e) <= GRAD_TOL[torch.bfloat16], name


def test_attention_backward_long_sequence_properties(cuda):
    # full-length rows (S = 4096): properties that need no CPU reference.  Causal row 0 sees
    # key 0 only, so its probability is 1 and dS is 0: dq[0] == 0; dv of the last key receives
    # only the last query: dv[-1] = P[-1, -1] * dy[-1]; and the gradients are linear in dy.
    B, H, S = 1, 2, 4096
    d = inputs.c4(B, H, S, 128, seed=21)
    q, k, v = (d[n].to(cuda) for n in "qkv")
    g = torch.Generator().manual_seed(22)
    dy = torch.randn(B, H, S, 128, generator=g).bfloat16().to(cuda)
    out, lse = ops.fused_attention(q, k, v, d["scale"], causal=True, return_lse=True, check=True)
    dq, dk, dv = ops.fused_attention_backward(q, k, v, out, lse, dy, d["scale"], causal=True, check=True)
    assert float(dq[:, :, 0].float().abs().max()) <= 1e-3 * float(dq.float().abs().max())
    s_last = (q[:, :, -1].float() * k[:, :, -1].float()).sum(-1) * d["scale"]
    p_last = torch.exp(s_last - lse[:, :, -1])
    want = p_last.unsqueeze(-1) * dy[:, :, -1].float()
    assert graphs.max_rel_err(dv[:, :, -1].float().cpu(), want.cpu()) <= GRAD_TOL[torch.bfloat16]
    dq2, dk2, dv2 = ops.fused_attention_backward(q, k, v, out, lse, dy * 2, d["scale"], causal=True, check=True)
    for a, b2 in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert graphs.max_rel_err(b2.float().cpu(), 2 * a.float().cpu()) <= GRAD_TOL[torch.bfloat16]


def test_attention_backward_argument_errors(cuda):
    q = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16, device=cuda)
    lse = torch.zeros(1, 1, 8, dtype=torch.float32, device=cuda)
    with pytest.raises(ValueError):
        ops.fused_attention_backward(q, q, q, q, lse[:, :, :4], q, 1.0)
    with pytest.raises(rt.IxbError):
        ops.fused_attention_backward(q, q, q, q, lse, q, -1.0)  # scale must be positive
    q64 = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(rt.IxbError) as e:
        ops.fused_attention_backward(q64, q64, q64, q64, lse, q64, 1.0)
    assert e.value.status == rt.IXB_ERR_SHAPE


def test_compiled_training_step_of_the_literal_causal_graph(cuda):
    """torch.compile of the literal causal attention with gradients required: the joint-graph
    pattern puts b200_sdpa and b200_sdpa_backward in the graph; loss gradients match autograd
    through the eager graph."""
    import inductor_x_b200  # noqa: F401
    from torch._dynamo.utils import counters

    S = 256
    scale = 1 / math.sqrt(128)

    def attention(q, k, v):
        keep = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = (torch.matmul(q, k.transpose(-2, -1)) * scale).masked_fill(~keep, float("-inf"))
        return torch.matmul(torch.softmax(s, dim=-1), v)

    g = torch.Generator().manual_seed(5)
    base = [torch.randn(2, 4, S, 128, generator=g).bfloat16().to(cuda) for _ in range(4)]
    dy = base[3]
    a = [t.clone().requires_grad_(True) for t in base[:3]]
    b = [t.float().clone().requires_grad_(True) for t in base[:3]]
    torch._dynamo.reset()
    counters.clear()
    rt.native_calls = 0
    out = torch.compile(attention)(*a)
    out.backward(dy)
    assert counters["inductor"]["fuse_attention"] >= 1
    assert rt.native_calls >= 2  # forward and backward entry points of the library
    ref = attention(*b)
    ref.backward(dy.float())
    assert graphs.max_rel_err(out.detach().float().cpu(), ref.detach().cpu(), dim=-1) <= TOL
    for x, y in zip(a, b):
        assert x.grad is not None and graphs.max_rel_err(x.grad.float().cpu(), y.grad.cpu()) <= GRAD_TOL[torch.bfloat16]
