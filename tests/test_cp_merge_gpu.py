"""Parity of the context-parallel attention merge kernels with the eager forms the reference
states them in (test/npu_indexing/attn_cp_test.py:36-59 and the data_validation routine
there), through the C ABI.  Tolerances: statistics are fp32 (rel 1e-5), merged attention
outputs follow the storage type (2e-2 for 16-bit, 1e-5 for fp32)."""
import os

import pytest
import torch

from oracle import graphs, inputs

pytestmark = pytest.mark.gpu


def _golden():
    return torch.load(os.path.join(os.path.dirname(__file__), "golden", "golden_cp.pt"), weights_only=True)


@pytest.fixture(scope="module")
def ops():
    from inductor_x_b200 import ops as o
    return o


def _check(got, want, dtype):
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert graphs.max_rel_err(got[0], want[0]) <= tol
    assert graphs.max_rel_err(got[1], want[1]) <= 1e-6      # a maximum: no rounding at all
    assert torch.equal(got[1].cpu(), want[1])
    assert graphs.max_rel_err(got[2], want[2]) <= 1e-5


def test_forward_update_matches_golden(ops):
    d = inputs.cp_merge(S=48, B=2, H=256, N=2, seed=21)
    got = ops.forward_update(*(d[k].cuda() for k in ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum",
                                                      "cur_attn_out", "cur_softmax_max", "cur_softmax_sum")))
    _check([t.cpu() for t in got], _golden()["cp_small"], torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("S,B,H,N", [(64, 1, 1536, 12), (33, 3, 512, 4), (1, 1, 128, 1), (256, 2, 6144, 48)])
def test_forward_update_vs_oracle(ops, dtype, S, B, H, N):
    d = inputs.cp_merge(S=S, B=B, H=H, N=N, seed=S + H, dtype=dtype)
    want = graphs.cp_forward_update(**d)
    got = ops.forward_update(*(d[k].cuda() for k in ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum",
                                                      "cur_attn_out", "cur_softmax_max", "cur_softmax_sum")))
    _check([t.cpu() for t in got], want, dtype)


def test_forward_update_on_a_sequence_slice(ops):
    """The reference's "_s" case: the running result is the second half of buffers that hold a
    doubled sequence (test/npu_indexing/written/test_attn_cp.py:254-262)."""
    S, B, H, N = 128, 1, 1024, 8
    big = inputs.cp_merge(S=2 * S, B=B, H=H, N=N, seed=5)
    cur = inputs.cp_merge(S=S, B=B, H=H, N=N, seed=6)
    prev_attn = big["prev_attn_out"].cuda().view(2, S, B, H)[1]
    prev_max = big["prev_softmax_max"].cuda().view(B, N, 2, S, 8)[:, :, 1]
    prev_sum = big["prev_softmax_sum"].cuda().view(B, N, 2, S, 8)[:, :, 1]
    assert not prev_max.is_contiguous()
    got = ops.forward_update(prev_attn, prev_max, prev_sum, cur["cur_attn_out"].cuda(),
                             cur["cur_softmax_max"].cuda(), cur["cur_softmax_sum"].cuda())
    want = graphs.cp_forward_update(prev_attn.cpu(), prev_max.cpu(), prev_sum.cpu(), cur["cur_attn_out"],
                                    cur["cur_softmax_max"], cur["cur_softmax_sum"])
    _check([t.cpu() for t in got], want, torch.bfloat16)


def test_forward_update_statistics_entry_by_entry(ops):
    """Entries 1..7 of a statistics row are merged on their own values, entry 0 scales the
    attention output (attn_cp_test.py:24-33)."""
    d = inputs.cp_merge(S=16, B=1, H=256, N=2, seed=9)
    d["prev_softmax_max"] = d["prev_softmax_max"] + torch.arange(8.0) * 0.125
    d["cur_softmax_sum"] = d["cur_softmax_sum"] * (1 + torch.arange(8.0))
    want = graphs.cp_forward_update(**d)
    got = ops.forward_update(*(d[k].cuda() for k in ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum",
                                                      "cur_attn_out", "cur_softmax_max", "cur_softmax_sum")))
    _check([t.cpu() for t in got], want, torch.bfloat16)


def test_forward_update_la_in_place(ops):
    g = _golden()
    pa, pl, ca, cl = (t.cuda() for t in g["cp_la_inputs"])
    ops.forward_update_la(pa, pl, ca, cl)
    assert graphs.max_rel_err(pa.cpu(), g["cp_la_small"][0]) <= 1e-5
    assert graphs.max_rel_err(pl.cpu(), g["cp_la_small"][1]) <= 1e-5


@pytest.mark.parametrize("B,N,S,D", [(1, 48, 512, 128), (2, 3, 77, 64), (1, 1, 5, 4), (1, 2, 64, 320)])
def test_forward_update_la_vs_oracle(ops, B, N, S, D):
    gen = torch.Generator().manual_seed(B * 1000 + S)
    # the running result is a slice along S of a longer buffer, as in a ring step
    pa_big = torch.randn((B, N, 2 * S, D), generator=gen).cuda()
    pl_big = (torch.randn((B, N, 2 * S), generator=gen) * 4).cuda()
    pa, pl = pa_big[:, :, S:], pl_big[:, :, S:]
    ca, cl = torch.randn((B, N, S, D), generator=gen), torch.randn((B, N, S), generator=gen) * 4
    cl[..., 0] = -float("inf")                       # a step that contributed nothing to a row
    want = graphs.cp_forward_update_la(pa.cpu(), pl.cpu(), ca, cl)
    untouched = pa_big[:, :, :S].clone()
    ops.forward_update_la(pa, pl, ca.cuda(), cl.cuda())
    assert graphs.max_rel_err(pa.cpu(), want[0]) <= 1e-5
    assert graphs.max_rel_err(pl.cpu(), want[1]) <= 1e-5
    assert torch.equal(pa_big[:, :, :S], untouched)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_grad_accumulate_is_torch_add(ops, dtype):
    """dq.add_(cur_dq.view(dq.shape)) and friends (test_attn_cp.py:267-287): bit-exact with
    torch's own in-place add."""
    gen = torch.Generator().manual_seed(3)
    acc = torch.randn((2, 96, 1, 1536), generator=gen).to(dtype)
    cur = torch.randn((192, 1, 1536), generator=gen).to(dtype)
    want = acc.clone().add_(cur.view(acc.shape))
    got = ops.grad_accumulate(acc.cuda(), cur.cuda())
    assert torch.equal(got.cpu(), want)
    # accumulate into one half only: dk[0].add_(cur_dk)
    acc2 = acc.cuda()
    ops.grad_accumulate(acc2[0], cur.cuda()[:96].contiguous())
    want2 = acc.clone()
    want2[0].add_(cur[:96])
    assert torch.equal(acc2.cpu(), want2)


def test_rejects_what_it_cannot_do(ops):
    d = inputs.cp_merge(S=8, B=1, H=256, N=2, seed=1)
    with pytest.raises(ValueError):
        ops.forward_update(*(d[k] for k in ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum",
                                            "cur_attn_out", "cur_softmax_max", "cur_softmax_sum")))   # CPU tensors
    bad = {k: v.cuda() for k, v in d.items()}
    bad["prev_softmax_sum"] = bad["prev_softmax_sum"].double()
    with pytest.raises(ValueError):
        ops.forward_update(*(bad[k] for k in ("prev_attn_out", "prev_softmax_max", "prev_softmax_sum",
                                              "cur_attn_out", "cur_softmax_max", "cur_softmax_sum")))
