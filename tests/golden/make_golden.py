"""Generates tests/golden/golden.pt: expected outputs of the benchmark graphs computed by
eager PyTorch on CPU - the ground truth the reference's own tests compare against
(test/npu_indexing/reduction_test.py:28-30 asserts compiled == eager).

Run from the repository root:  python tests/golden/make_golden.py
Inputs are not stored; they are regenerated from their seeds by oracle/inputs.py.  Full
size outputs are kept as samples (rows / slabs) plus a digest so the file stays small.
"""
import hashlib
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import graphs, inputs  # noqa: E402

C2_ROWS = [0, 1, 2, 4095, 4096, 8191, 12345, 16383]
C3A_SLABS = [0, 31, 63]
C4_HEADS = [(0, 0), (7, 31)]
C4_ROWS = [0, 1, 127, 128, 2047, 2048, 4095]


def digest(t: torch.Tensor) -> str:
    raw = t.contiguous().view(torch.uint8) if t.dtype != torch.bfloat16 else t.contiguous().view(torch.int16).view(torch.uint8)
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def main():
    torch.manual_seed(0)
    torch.set_num_threads(os.cpu_count() or 1)
    g = {"torch_version": str(torch.__version__)}

    # ---- config 1, full size: whole output (32 KiB), eager fp32 and fp64 truth
    d = inputs.c1()
    g["c1_out_eager"] = F.gelu(d["x"] * d["w"] + d["b"]).sum(-1)
    g["c1_out_f64"] = graphs.affine_gelu_rowsum(d["x"].double(), d["w"].double(), d["b"].double())

    # ---- config 2, full size: sampled rows, fp32-compute oracle, fp64 truth and op-by-op eager
    d = inputs.c2()
    sub = {"x": d["x"][C2_ROWS], "g": d["g"], "gamma": d["gamma"], "beta": d["beta"]}
    g["c2_rows"] = torch.tensor(C2_ROWS)
    g["c2_y_fused_f32"] = graphs.softmax_layernorm(**sub)
    g["c2_y_f64"] = graphs.softmax_layernorm(**sub, compute=torch.float64, round_output=False).float()
    g["c2_y_eager"] = graphs.eager_softmax_layernorm(**sub)

    # ---- config 3a, full size: sampled `a` slabs
    d = inputs.c3a()
    xs = d["x"][C3A_SLABS]
    g["c3a_slabs"] = torch.tensor(C3A_SLABS)
    g["c3a_amax"] = xs.permute(0, 2, 1, 3).amax(1)             # eager, fp16: exact
    g["c3a_sum_f32acc"] = graphs.permuted_sum(xs)                  # fp32 accumulate, round once
    g["c3a_sum_eager"] = xs.permute(0, 2, 1, 3).sum(3)             # eager fp16 sum

    # ---- config 3b, full size: digest + head of the gathered rows
    d = inputs.c3b()
    out = graphs.index_select_rows(**d)
    g["c3b_sha256"] = digest(out)
    g["c3b_head"] = out[:8].clone()
    g["c3b_idx_head"] = d["idx"][:8].clone()

    # ---- config 4: (i) the reference's search pattern on a small [B,S,N,D] problem,
    # (ii) sampled rows of two heads of the full-size causal problem
    p = inputs.c4_pattern()
    g["c4_pattern_out"] = graphs.attention_pattern(p["query"], p["key"], p["value"], p["inv_scale_factor"])
    d = inputs.c4()
    rows = torch.tensor(C4_ROWS)
    outs, lses = [], []
    for (b, h) in C4_HEADS:
        o, l = graphs.attention(d["q"][b:b + 1, h:h + 1], d["k"][b:b + 1, h:h + 1],
                                d["v"][b:b + 1, h:h + 1], d["scale"], causal=True)
        outs.append(o[0, 0][rows])
        lses.append(l[0, 0][rows])
    g["c4_heads"] = torch.tensor(C4_HEADS)
    g["c4_rows"] = rows
    g["c4_out_rows"] = torch.stack(outs)
    g["c4_lse_rows"] = torch.stack(lses)

    # ---- small cases, complete outputs (the shapes the CPU tests and smoke() use)
    d = inputs.c1(64, 1024, seed=11)
    g["c1_small_out"] = graphs.affine_gelu_rowsum(**d)
    d = inputs.c2(16, 4096, seed=12)
    g["c2_small_y"] = graphs.softmax_layernorm(**d)
    d = inputs.c3a((3, 8, 16, 64), seed=13)
    g["c3a_small_amax"] = graphs.permuted_amax(d["x"])
    g["c3a_small_sum"] = graphs.permuted_sum(d["x"])

    path = os.path.join(ROOT, "tests", "golden", "golden.pt")
    torch.save(g, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_cp():
    """Fixtures of the context-parallel merge kernels (a file of their own so that adding
    them did not rewrite the fixtures above): complete outputs of a small (max, sum) merge
    with statistics sliced out of a longer buffer, and of a small log-sum-exp merge."""
    g = {"torch_version": str(torch.__version__)}
    d = inputs.cp_merge(S=48, B=2, H=256, N=2, seed=21)
    g["cp_small"] = [t.clone() for t in graphs.cp_forward_update(**d)]
    gen = torch.Generator().manual_seed(22)
    pa, ca = torch.randn((2, 3, 40, 64), generator=gen), torch.randn((2, 3, 40, 64), generator=gen)
    pl, cl = torch.randn((2, 3, 40), generator=gen) * 3, torch.randn((2, 3, 40), generator=gen) * 3
    g["cp_la_inputs"] = [pa, pl, ca, cl]
    g["cp_la_small"] = list(graphs.cp_forward_update_la(pa, pl, ca, cl))
    path = os.path.join(ROOT, "tests", "golden", "golden_cp.pt")
    torch.save(g, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "cp":
        main_cp()
        sys.exit(0)
    main()
