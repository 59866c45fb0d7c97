"""The oracle against the golden vectors produced by the reference itself."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(glob.glob(os.path.join(GOLD, "nsa_g*.npz")))


def _load(path):
    z = np.load(path)
    d = {k: torch.from_numpy(z[k]) for k in z.files}
    B, Hq, Hkv, D, T, bs, S, W = (int(x) for x in d.pop("meta"))
    return d, dict(B=B, Hq=Hq, Hkv=Hkv, D=D, T=T, bs=bs, S=S, W=W)


def _close(a, b, tol=2e-5):
    a, b = a.float(), b.float()
    assert a.shape == b.shape
    assert (a - b).abs().max().item() <= tol, (a - b).abs().max().item()


def test_golden_files_present():
    assert len(CASES) == 3


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_ref_family_matches_reference(path):
    d, c = _load(path)
    bs, W = c["bs"], c["W"]
    for branch, fn in (
        ("sel", lambda q, k, v: O.ref_selection_forward(q, k, v, d["block_idx"], bs)),
        ("win", lambda q, k, v: O.ref_range_attn(q, k, v, O.MODE_WINDOW, W, 0)),
        ("cmp", lambda q, k, v: O.ref_range_attn(q, k, v, O.MODE_COMPRESS, 0, bs)),
    ):
        kk, vv = {"sel": ("ks", "vs"), "win": ("kw", "vw"), "cmp": ("k_pool", "v_pool")}[branch]
        q, k, v = (d[n].clone().requires_grad_(True) for n in ("q", kk, vv))
        o = fn(q, k, v)
        o.backward(d["do"])
        _close(o, d[branch + "_o"])
        _close(q.grad, d[branch + "_dq"])
        _close(k.grad, d[branch + "_dk"])
        _close(v.grad, d[branch + "_dv"])
    _close(O.ref_block_mean_pool(d["kc"], bs), d["k_pool"], 1e-6)
    names = ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]
    ins = [d[n].clone().requires_grad_(True) for n in names]
    o = O.ref_nsa_fused(*ins, d["block_idx"], bs, W)
    o.backward(d["do"])
    _close(o, d["fused_o"])
    for n, t in zip(names, ins):
        _close(t.grad, d["fused_d" + n])


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_stream_family_matches_reference(path):
    d, c = _load(path)
    bs, W, T = c["bs"], c["W"], c["T"]
    n_blk = T // bs
    for branch, keep_fn, kk, vv in (
        ("sel", O.selection_keep_fn(d["block_idx"], T, bs), "ks", "vs"),
        ("win", O.window_keep_fn(T, W), "kw", "vw"),
        ("cmp", O.compress_keep_fn(n_blk, bs), "k_pool", "v_pool"),
    ):
        for chunk in (32, 4096):
            o, lse = O.stream_attn_forward(d["q"], d[kk], d[vv], keep_fn, chunk)
            _close(o, d[branch + "_o"])
            dq, dk, dv = O.stream_attn_backward(d["q"], d[kk], d[vv], o, lse, d["do"], keep_fn, chunk)
            _close(dq, d[branch + "_dq"])
            _close(dk, d[branch + "_dk"])
            _close(dv, d[branch + "_dv"])
        # empty rows: output 0 and the finite LSE sentinel
        empty = ~keep_fn(0, T).reshape(-1, T, keep_fn(0, T).shape[-1]).any(-1).all(0)
        if empty.any():
            assert (o[:, :, empty] == 0).all()
            assert (lse[:, :, empty] == O.LSE_EMPTY).all()
    fwd = O.stream_nsa_forward(d["q"], d["kc"], d["vc"], d["ks"], d["vs"], d["kw"], d["vw"],
                               d["gate"], bs, c["S"], W, block_idx=d["block_idx"], chunk=64)
    _close(fwd["out"], d["fused_o"])
    g = O.stream_nsa_backward(d["q"], d["kc"], d["vc"], d["ks"], d["vs"], d["kw"], d["vw"],
                              d["gate"], bs, W, fwd, d["do"], chunk=64)
    for n in ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]:
        _close(g[n], d["fused_d" + n])


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p) for p in CASES])
def test_compressor_scoring_csr(path):
    d, c = _load(path)
    bs = c["bs"]
    y = O.ref_block_compressor(d["kc"], d["comp_intra"], d["comp_logits"], d["comp_proj"], bs)
    _close(y, d["comp_y"])
    dx, di, dl, dp = O.compressor_backward(d["kc"], d["comp_intra"], d["comp_logits"],
                                           d["comp_proj"], bs, d["comp_dy"])
    _close(dx, d["comp_dx"])
    _close(di, d["comp_dintra"], 1e-4)
    _close(dl, d["comp_dlogits"], 1e-4)
    _close(dp, d["comp_dproj"], 1e-4)
    # scoring: importance and the reference's own topk call
    imp, valid = O.ref_importance(d["q"], d["comp_y"], bs)
    _close(imp, d["score_imp"], 1e-6)
    imp2, _ = O.stream_importance(d["q"], d["comp_y"], bs, chunk=48)
    _close(imp2, d["score_imp"], 1e-6)
    ref_topk = d["score_topk"].long()
    mine = O.canonical_topn(imp, valid, c["S"])
    k_top = ref_topk.shape[-1]
    n_valid = valid.sum(-1)                                   # [T]
    for t in range(c["T"]):
        nv = int(n_valid[t])
        got = mine[:, :, t, :k_top].long()
        if nv >= k_top:   # the set torch.topk picked == the canonical set (no exact ties here)
            assert (got.sort(-1).values == ref_topk[:, :, t].sort(-1).values).all()
        else:             # all valid blocks, then -1 padding
            assert (got[..., :nv].sort(-1).values == torch.arange(nv)).all()
            assert (got[..., nv:] == -1).all()
        # canonical order: importance descending, index ascending among ties
        vals = torch.gather(imp[:, :, t], -1, got.clamp(min=0))[..., :min(nv, k_top)]
        assert (vals[..., :-1] >= vals[..., 1:]).all()
    assert (mine[..., k_top:] == -1).all()
    qob, off, pbh = O.build_block_to_query_csr(d["block_idx"], bs)
    assert (qob == d["csr_q"].numpy()).all()
    assert (off == d["csr_off"].numpy()).all()
    assert (pbh == d["csr_bh"].numpy()).all()


def test_whole_module_matches_reference():
    """nsa_model.py:196-304 restated from oracle pieces: projections, learned
    pooling, reference top-k, three branches, gate, out_proj."""
    z = np.load(os.path.join(GOLD, "nsa_module.npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files}
    x = d["x"]
    B, T, _ = x.shape
    Hq, Hkv, bs, n_sel, W = 4, 2, 16, 3, 24
    D = 64 // Hq
    P = lambda n: d["p." + n]
    split = lambda y, h: y.view(B, T, h, D).transpose(1, 2)
    q = split(x @ P("q_proj.weight").t(), Hq)
    kv = {n: split(x @ P(n + ".weight").t(), Hkv) for n in
          ("k_cmp", "v_cmp", "k_slc", "v_slc", "k_win", "v_win")}
    comp = dict(k_intra=P("comp_k.intra_pos"), k_logits=P("comp_k.pool_logits"),
                k_proj=P("comp_k.proj.weight"), v_intra=P("comp_v.intra_pos"),
                v_logits=P("comp_v.pool_logits"), v_proj=P("comp_v.proj.weight"))
    gate = (x @ P("gate.weight").t() + P("gate.bias")).view(B, T, Hq, 3).permute(0, 2, 1, 3)
    k_cmp = O.ref_block_compressor(kv["k_cmp"], comp["k_intra"], comp["k_logits"], comp["k_proj"], bs)
    idx = O.ref_topk_blocks(q, k_cmp, bs, n_sel)
    fwd = O.stream_nsa_forward(q, kv["k_cmp"], kv["v_cmp"], kv["k_slc"], kv["v_slc"],
                               kv["k_win"], kv["v_win"], gate, bs, n_sel, W,
                               block_idx=idx, compressor=comp, chunk=40)
    out = fwd["out"].transpose(1, 2).reshape(B, T, Hq * D)
    y = out @ P("out_proj.weight").t()
    _close(y, d["y"], 5e-5)
    # gradients of the op inputs, pushed back to x through the projections
    d_out = (d["dy"] @ P("out_proj.weight")).view(B, T, Hq, D).transpose(1, 2)
    g = O.stream_nsa_backward(q, kv["k_cmp"], kv["v_cmp"], kv["k_slc"], kv["v_slc"],
                              kv["k_win"], kv["v_win"], gate, bs, W, fwd, d_out,
                              compressor=comp, chunk=40)
    merge = lambda t: t.transpose(1, 2).reshape(B, T, -1)
    dx = merge(g["q"]) @ P("q_proj.weight")
    for nm, key in (("k_cmp", "kc"), ("v_cmp", "vc"), ("k_slc", "ks"), ("v_slc", "vs"),
                    ("k_win", "kw"), ("v_win", "vw")):
        dx = dx + merge(g[key]) @ P(nm + ".weight")
        _close(merge(g[key]).reshape(B * T, -1).t() @ x.reshape(B * T, -1),
               d["g." + nm + ".weight"], 2e-4)
    dgate = g["gate"].permute(0, 2, 1, 3).reshape(B, T, Hq * 3)
    dx = dx + dgate @ P("gate.weight")
    _close(dx, d["dx"], 2e-4)
    _close(dgate.sum((0, 1)), d["g.gate.bias"], 2e-4)
    for nm, key in (("comp_k.intra_pos", "k_intra"), ("comp_k.pool_logits", "k_logits"),
                    ("comp_k.proj.weight", "k_proj"), ("comp_v.intra_pos", "v_intra"),
                    ("comp_v.pool_logits", "v_logits"), ("comp_v.proj.weight", "v_proj")):
        _close(g[key], d["g." + nm], 2e-4)


def test_generators_and_counts():
    idx = O.make_block_idx_recent(1, 2, 256, 32, 4)
    assert idx.shape == (1, 2, 256, 4) and idx[0, 0, 31, 0] == 0 and idx[0, 0, 30, 0] == -1
    idx2 = O.make_block_idx(2, 2, 128, 16, 5, seed=0)
    t = torch.arange(128).view(1, 1, 128, 1)
    assert ((idx2 < 0) | ((idx2 + 1) * 16 <= t + 1)).all()
    n = O.attended_keys(idx, 256, 32, 50)
    keep = O.selection_keep(idx, 0, 256, 256, 32)
    assert n["slc"] == int(keep.sum())
    assert n["win"] == 2 * int(O.window_keep(0, 256, 256, 50).sum())
    assert n["cmp"] == 2 * int(O.compress_keep(0, 256, 8, 32).sum())


# ---------------------------------------------------------------------------------------------
# The generalised geometry (summaries of len tokens every stride, forced blocks) has no reference
# code: what can be checked on the CPU is that each restatement collapses to its pinned form on
# the reference's grid, that the analytic backward agrees with autograd, and the rule's invariants.
# ---------------------------------------------------------------------------------------------
def test_generalised_forms_collapse_to_the_pinned_ones():
    g = torch.Generator().manual_seed(0)
    B, H, T, D, bs = 2, 2, 200, 16, 32
    x = torch.randn(B, H, T, D, generator=g)
    ip, pl, W = 0.1 * torch.randn(bs, D, generator=g), torch.randn(bs, generator=g), torch.randn(D, D, generator=g)
    assert O.n_summaries(T, bs, bs) == T // bs and O.n_summaries(10, bs, 8) == 0
    assert torch.equal(O.ref_block_compressor(x, ip, pl, W, bs), O.ref_block_compressor(x, ip, pl, W, bs, bs))
    assert torch.equal(O.compress_keep(0, T, T // bs, bs), O.compress_keep(0, T, T // bs, bs, bs))
    imp = torch.rand(B, H, T, T // bs, generator=g) * O.compress_keep(0, T, T // bs, bs)[None, None]
    valid = O.compress_keep(0, T, T // bs, bs)
    ib, vb = O.block_importance(imp, T, bs, bs, bs)
    assert torch.equal(ib[..., :T // bs], imp) and torch.equal(vb[:, :T // bs], valid) and not vb[:, T // bs:].any()
    assert torch.equal(O.forced_topn(ib, vb, 3, T, bs, 0, 0), O.canonical_topn(imp, valid, 3))


@pytest.mark.parametrize("stride", [32, 16, 8])
def test_strided_compressor_backward_is_autograd(stride):
    g = torch.Generator().manual_seed(1)
    B, H, T, D, bs = 1, 2, 150, 8, 32
    x = torch.randn(B, H, T, D, generator=g, requires_grad=True)
    ps = [(0.1 * torch.randn(bs, D, generator=g)).requires_grad_(True), torch.randn(bs, generator=g).requires_grad_(True),
          torch.randn(D, D, generator=g).requires_grad_(True)]
    y = O.ref_block_compressor(x, *ps, bs, stride)
    assert y.shape[2] == O.n_summaries(T, bs, stride)
    do = torch.randn(y.shape, generator=g)
    want = torch.autograd.grad(y, [x] + ps, do)
    got = O.compressor_backward(x.detach(), *(p.detach() for p in ps), bs, do, stride)
    for a, b in zip(got, want):
        assert (a - b).abs().max().item() <= 1e-5


def test_block_importance_and_forced_lists():
    g = torch.Generator().manual_seed(2)
    T, l, d, lsel, S = 400, 32, 16, 64, 6
    n_cmp = O.n_summaries(T, l, d)
    keep = O.compress_keep(0, T, n_cmp, l, d)
    imp = torch.rand(1, 1, T, n_cmp, generator=g) * keep[None, None]
    ib, vb = O.block_importance(imp, T, l, d, lsel)
    r, o = lsel // d, l // d
    for b in range(ib.shape[-1]):
        j0, j1 = max(0, r * b - o + 1), min(n_cmp - 1, r * b + r - 1)
        assert torch.allclose(ib[..., b], imp[..., j0:j1 + 1].sum(-1))
        # a block is a candidate exactly when its first overlapping summary is visible
        assert torch.equal(vb[:, b], keep[:, j0] if j0 < n_cmp else torch.zeros(T, dtype=torch.bool))
    idx = O.forced_topn(ib, vb, S, T, lsel, 1, 2)
    t = torch.arange(T)
    cur = (t // lsel).view(1, 1, T, 1)
    assert (idx[..., 0] == 0).all()                                  # block 0 first, always
    assert (idx == cur).any(-1).all()                                # the block holding t is listed
    assert ((idx == cur - 1).any(-1) | (cur[..., 0] == 0)).all()     # and the one before it
    assert (idx <= cur).all()                                        # nothing from the future
    for row in idx.view(-1, S)[::37]:                                # no block twice
        kept = row[row >= 0]
        assert kept.unique().numel() == kept.numel()


def test_sampled_unit_check_agrees_with_the_whole_oracle():
    """The sampled checks the GPU tests use at the benchmark sizes (tests/util.check_unit_sampled:
    some query rows, some window key tiles, some selection blocks, the compression branch of one
    unit) reproduce the whole-op oracle when fed the oracle's own results."""
    from tests.util import check_unit_sampled, unit_slices
    B, Hq, Hkv, T, D, bs, S, W = 2, 8, 2, 640, 32, 64, 3, 100
    G = Hq // Hkv
    g = torch.Generator().manual_seed(3)
    t = {"q": torch.randn(B, Hq, T, D, generator=g) * D ** -0.5}
    for n in ("kc", "vc", "ks", "vs", "kw", "vw"):
        t[n] = torch.randn(B, Hkv, T, D, generator=g) * D ** -0.5
    t["gate"] = torch.randn(B, Hq, T, 3, generator=g)
    t["do"] = torch.randn(B, Hq, T, D, generator=g)
    names = ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]
    fwd = O.stream_nsa_forward(*(t[n] for n in names), bs, S, W)
    grads = O.stream_nsa_backward(*(t[n] for n in names), bs, W, fwd, t["do"])
    t["block_idx"] = fwd["block_idx"]
    for b, h in ((0, 1), (1, 0)):
        u = unit_slices(t, b, h, G)
        got = unit_slices({"q": grads["q"], "gate": grads["gate"], "ks": grads["ks"], "vs": grads["vs"],
                           "kw": grads["kw"], "vw": grads["vw"]}, b, h, G)
        got["out"] = fwd["out"][b:b + 1, h * G:(h + 1) * G]
        k_cmp, v_cmp = fwd["k_cmp"][b:b + 1, h:h + 1], fwd["v_cmp"][b:b + 1, h:h + 1]
        dk_cmp, dv_cmp = check_unit_sampled(u, k_cmp, v_cmp, got, T, bs, W, torch.float32, "self",
                                            [(0, 70), (300, 420), (600, 640)], [0, 4, 9], [0, 3, 8])
        dkc = O.mean_pool_backward(dk_cmp, T, bs)
        assert (dkc - grads["kc"][b:b + 1, h:h + 1]).abs().max().item() <= 1e-5
