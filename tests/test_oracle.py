"""CPU tests of the oracle: the eager-PyTorch restatement against the committed golden
vectors, and the independent C restatement against both."""
import torch

from oracle import c_oracle, graphs, inputs

C2_ROWS = [0, 1, 2, 4095, 4096, 8191, 12345, 16383]


def test_golden_header(golden):
    assert "torch_version" in golden


def test_c1_full_matches_golden(golden):
    d = inputs.c1()
    out = graphs.affine_gelu_rowsum(**d)
    # same graph, same library: only summation-order noise between runs / thread counts
    assert graphs.max_rel_err(out, golden["c1_out_eager"]) <= 1e-5
    assert graphs.max_rel_err(out, golden["c1_out_f64"]) <= 1e-5


def test_c1_c_oracle_matches_golden(golden):
    d = inputs.c1()
    sub = {"x": d["x"][:256], "w": d["w"], "b": d["b"]}
    out = c_oracle.affine_gelu_rowsum(**sub)
    assert graphs.max_rel_err(out, golden["c1_out_f64"][:256]) <= 1e-6


def test_c2_rows_match_golden(golden):
    d = inputs.c2()
    assert golden["c2_rows"].tolist() == C2_ROWS
    sub = {"x": d["x"][C2_ROWS], "g": d["g"], "gamma": d["gamma"], "beta": d["beta"]}
    y = graphs.softmax_layernorm(**sub)
    assert torch.equal(y, golden["c2_y_fused_f32"])
    # fused fp32 graph vs fp64 truth vs op-by-op eager bf16: all inside the half tolerance
    assert graphs.max_rel_err(y, golden["c2_y_f64"]) <= 2e-2
    assert graphs.max_rel_err(golden["c2_y_eager"], golden["c2_y_f64"]) <= 2e-2
    yc = c_oracle.softmax_layernorm(**sub)
    assert graphs.max_rel_err(yc, golden["c2_y_f64"]) <= 1e-5


def test_c3a_small_matches_golden_and_c(golden):
    d = inputs.c3a((3, 8, 16, 64), seed=13)
    x = d["x"]
    amax = graphs.permuted_amax(x)
    ssum = graphs.permuted_sum(x)
    assert torch.equal(amax, golden["c3a_small_amax"])
    assert torch.equal(ssum, golden["c3a_small_sum"])
    # independent C restatement: amax over c of x[a,b,c,d]; sum over d transposed to [a,c,b]
    a, b, c, dd = x.shape
    cmax = c_oracle.reduce_mid(x.reshape(a * b, c, dd), "amax").reshape(a, b, dd)
    assert torch.equal(cmax.to(x.dtype), amax)
    csum = c_oracle.reduce_mid(x.reshape(a * b * c, dd, 1), "sum").reshape(a, b, c).permute(0, 2, 1)
    assert torch.equal(csum.to(x.dtype), ssum)


def test_c3b_digest(golden):
    import hashlib

    d = inputs.c3b()
    out = graphs.index_select_rows(**d)
    assert hashlib.sha256(out.view(torch.uint8).numpy().tobytes()).hexdigest() == golden["c3b_sha256"]
    assert torch.equal(out[:8], golden["c3b_head"])
    sub, bad = c_oracle.index_select_rows(d["table"], d["idx"][:4096])
    assert bad == 0 and torch.equal(sub, out[:4096])


def test_index_select_contract():
    table = torch.arange(40, dtype=torch.float32).reshape(10, 4)
    idx = torch.tensor([0, -1, 9, 10, 3])
    out, bad = c_oracle.index_select_rows(table, idx, wrap_negative=True)
    assert bad == 4  # position 3 (+1) is out of range
    assert torch.equal(out[1], table[9]) and torch.equal(out[3], torch.zeros(4))
    out, bad = c_oracle.index_select_rows(table, idx, wrap_negative=False)
    assert bad == 2


def test_attention_pattern_matches_golden(golden):
    p = inputs.c4_pattern()
    out = graphs.attention_pattern(p["query"], p["key"], p["value"], p["inv_scale_factor"])
    assert graphs.max_rel_err(out, golden["c4_pattern_out"]) <= 1e-5
    # the oracle's BNSD attention equals the reference pattern on permuted inputs
    q, k, v = (p[n].permute(0, 2, 1, 3).contiguous() for n in ("query", "key", "value"))
    o2, _ = graphs.attention(q, k, v, 1.0 / p["inv_scale_factor"], causal=False)
    assert graphs.max_rel_err(o2, golden["c4_pattern_out"]) <= 1e-5
    o3, _ = c_oracle.attention(q, k, v, 1.0 / p["inv_scale_factor"], causal=False)
    assert graphs.max_rel_err(o3, golden["c4_pattern_out"]) <= 1e-5


def test_causal_attention_small_c_vs_torch():
    d = inputs.c4(1, 2, 80, 32, seed=5)
    o, l = graphs.attention(d["q"], d["k"], d["v"], d["scale"], causal=True)
    oc, lc = c_oracle.attention(d["q"], d["k"], d["v"], d["scale"], causal=True)
    assert graphs.max_rel_err(o, oc) <= 2e-2
    assert float((l.double() - lc).abs().max()) <= 1e-4


def test_llama_layer_runs_small():
    w = inputs.c5_weights(hidden=64, heads=4, ffn=176, seed=0)
    x = inputs.c5_input(2, 16, 64, seed=1)
    y = graphs.llama_layer(x, w, heads=4)
    assert y.shape == x.shape and torch.isfinite(y.float()).all()


# ---- context-parallel merge -----------------------------------------------------------------
def _cp_golden():
    import os
    return torch.load(os.path.join(os.path.dirname(__file__), "golden", "golden_cp.pt"), weights_only=True)


def test_cp_forward_update_matches_golden_and_scalar_restatement():
    """Eager merge against the committed fixture and against a scalar loop that follows the
    hand-written kernel's index arithmetic (attn_cp_triton_kernel_3d.py:36-82)."""
    import math
    g = _cp_golden()
    d = inputs.cp_merge(S=48, B=2, H=256, N=2, seed=21)
    out, mx, sm = graphs.cp_forward_update(**d)
    assert torch.equal(out, g["cp_small"][0]) and torch.equal(mx, g["cp_small"][1])
    assert torch.allclose(sm, g["cp_small"][2], rtol=1e-6, atol=0)
    S, B, H = d["cur_attn_out"].shape
    N = 2
    D = H // N
    for (s, b, h) in [(0, 0, 0), (47, 1, 255), (13, 0, 128), (30, 1, 127)]:
        n = h // D
        pm, cm = float(d["prev_softmax_max"][b, n, s, 0]), float(d["cur_softmax_max"][b, n, s, 0])
        m = max(pm, cm)
        ps = float(d["prev_softmax_sum"][b, n, s, 0]) * math.exp(pm - m)
        cs = float(d["cur_softmax_sum"][b, n, s, 0]) * math.exp(cm - m)
        want = float(d["prev_attn_out"][s, b, h]) * ps / (ps + cs) + float(d["cur_attn_out"][s, b, h]) * cs / (ps + cs)
        assert abs(float(out[s, b, h]) - want) <= 2e-2 * max(1.0, abs(want))
        assert abs(float(sm[b, n, s, 3]) - (ps + cs)) <= 1e-5


def test_cp_lse_form_agrees_with_max_sum_form():
    """lse = max + log(sum): merging in the log-sum-exp form must give the same attention
    output as merging (max, sum) pairs."""
    g = _cp_golden()
    pa, pl, ca, cl = g["cp_la_inputs"]
    attn, lse = graphs.cp_forward_update_la(pa, pl, ca, cl)
    assert torch.allclose(attn, g["cp_la_small"][0], rtol=1e-6, atol=1e-6)
    assert torch.allclose(lse, g["cp_la_small"][1], rtol=1e-6, atol=1e-6)
    # the same step written with (max, sum): choose max = lse, sum = 1
    B, N, S, D = pa.shape
    rep = lambda t: t.unsqueeze(3).repeat(1, 1, 1, 8)
    sbh = lambda t: t.permute(2, 0, 1, 3).reshape(S, B, N * D)
    out, mx, sm = graphs.cp_forward_update(sbh(pa), rep(pl), rep(torch.ones_like(pl)), sbh(ca), rep(cl),
                                           rep(torch.ones_like(cl)))
    assert torch.allclose(out, sbh(attn), rtol=1e-5, atol=1e-5)
    assert torch.allclose(mx[..., 0] + torch.log(sm[..., 0]), lse, rtol=1e-5, atol=1e-5)
