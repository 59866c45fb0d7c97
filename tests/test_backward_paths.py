"""The two ways dq leaves the whole-op backward (fp32 accumulator by TMA reduce-add, or bf16
partial slots added in a fixed order), run-to-run reproducibility, and the give-up path of the
bounded device waits, exercised from the host."""
import ctypes
import importlib

import pytest
import torch

from oracle import nsa_oracle as O
from tests.util import TC_CONFIGS, cfg_id, check, dev, make_inputs, pkg, window_for

pytestmark = pytest.mark.gpu

NAMES = ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]


@pytest.fixture(autouse=True)
def _reset():
    yield
    pkg().set_dq_accumulator(False)
    pkg().set_impl("auto")
    pkg().set_option("sel_fwd_variant", 0)
    pkg().set_option("debug_starve_load", 0)


def _op(nsa, t, c, dtype, comp=None, idx=None):
    ins = [dev(t[n], dtype).requires_grad_(True) for n in NAMES]
    comp_d = {k: v.cuda().requires_grad_(True) for k, v in comp.items()} if comp else None
    out, idx = nsa.nsa_attention(*ins, c["block_size"], c["S"], window_for(c), compressor=comp_d,
                                 block_idx=idx, return_block_idx=True)
    out.backward(dev(t["do"], dtype))
    g = {n: x.grad for n, x in zip(NAMES, ins)}
    if comp_d:
        g.update({k: v.grad for k, v in comp_d.items()})
    return out, idx, g


def _compressor(c, seed=7):
    g = torch.Generator().manual_seed(seed)
    D, bs = c["D"], c["block_size"]
    comp = {}
    for p in ("k", "v"):
        comp[p + "_intra"] = 0.02 * torch.randn(bs, D, generator=g)
        comp[p + "_logits"] = 0.3 * torch.randn(bs, generator=g)
        comp[p + "_proj"] = torch.randn(D, D, generator=g) * D ** -0.5
    return comp


@pytest.mark.parametrize("c", TC_CONFIGS[:6] + [TC_CONFIGS[7]], ids=cfg_id)
def test_accumulator_and_slot_backward_agree_with_the_oracle(c):
    """Whole op on tcgen05 shapes, both dq paths: each against the oracle, and against each other
    (the forward is bit-identical; the gradients agree within one bf16 rounding step of their
    largest entry: the paths differ in how dq is added up, and dk / dv of a key tile collect their
    row tiles in the order the kernel's two compute groups happen to issue them)."""
    nsa = pkg()
    dtype = torch.bfloat16
    if not nsa.tc_supported(c["B"], c["Hq"], c["Hkv"], c["T"], c["D"], dtype, c["block_size"]):
        pytest.skip("no tcgen05 path for this shape")
    t = make_inputs(c, dtype, seed=11, scale_qkv=True)
    comp = _compressor(c)
    res = {}
    for acc in (False, True):
        nsa.set_dq_accumulator(acc)
        out, idx, g = _op(nsa, t, c, dtype, comp)
        fwd = O.stream_nsa_forward(*(t[n] for n in NAMES), c["block_size"], c["S"], window_for(c),
                                   block_idx=idx.cpu(), compressor=comp)
        g_ref = O.stream_nsa_backward(*(t[n] for n in NAMES), c["block_size"], window_for(c), fwd, t["do"],
                                      compressor=comp)
        tag = "accumulator" if acc else "slots"
        check(out, fwd["out"], dtype, f"{tag} out", scale_abs=False)
        for n in NAMES:
            check(g[n], g_ref[n], dtype, f"{tag} d{n}", scale_abs=False)
        res[acc] = (out, idx, g)
    assert torch.equal(res[False][0], res[True][0]) and torch.equal(res[False][1], res[True][1])
    for n in NAMES:
        a, b = res[True][2][n].float(), res[False][2][n].float()
        assert (a - b).abs().max().item() <= 2.0 ** -7 * max(b.abs().max().item(), 1e-6), n
    assert nsa.lib().nsa_device_status(None) == 0


def test_run_to_run_reproducibility():
    """The same inputs twice.  Forward (out, block lists): bit-identical, nothing in it is added in
    a timing-dependent order.  Backward, default path: dq and d_gate bit-identical (every
    (row tile, key tile) dQ partial is computed on its own and the partials of a query are added in
    a fixed order).  dk / dv of a key tile are accumulated in TMEM over its row tiles in the order
    the kernel's two compute groups issue them, split key tiles and the compressor parameter
    gradients meet in fp32 atomics: reproducible up to the order of fp32 adds, bounded here at 2^-7
    of the largest entry (one bf16 rounding step).  Accumulator path: dq within the same bound."""
    nsa = pkg()
    dtype = torch.bfloat16
    c = dict(B=2, Hq=16, Hkv=2, D=128, T=2048, block_size=64, S=16, window=512)
    t = make_inputs(c, dtype, seed=5, scale_qkv=True)
    comp = _compressor(c)
    for acc in (False, True):
        nsa.set_dq_accumulator(acc)
        (o1, i1, g1), (o2, i2, g2) = [_op(nsa, t, c, dtype, comp) for _ in range(2)]
        assert torch.equal(o1, o2) and torch.equal(i1, i2)
        exact = ["gate"] + ([] if acc else ["q"])
        for n in exact:
            assert torch.equal(g1[n], g2[n]), (acc, n)
        for n in [k for k in g1 if k not in exact]:
            a, b = g1[n].float(), g2[n].float()
            # (floor 1e-4: d k_intra is analytically zero, what is left of it is rounding noise)
            assert (a - b).abs().max().item() <= 2.0 ** -7 * max(b.abs().max().item(), 1e-4), (acc, n)
    assert nsa.lib().nsa_device_status(None) == 0


def test_range_backward_accumulator_entry_point():
    """nsa_range_attn_bwd_acc + nsa_dq_finish through the C ABI against nsa_range_attn_bwd on the
    same gated branch: dq, dk, dv within one bf16 rounding step of the slot path."""
    nsa = pkg()
    L = importlib.import_module("openbox-llm_b200._lib")
    dtype = torch.bfloat16
    for c, mode in ((TC_CONFIGS[1], nsa.MODE_WINDOW), (TC_CONFIGS[2], nsa.MODE_WINDOW), (TC_CONFIGS[1], nsa.MODE_COMPRESS)):
        t = make_inputs(c, dtype, seed=3, scale_qkv=True)
        B, Hq, Hkv, T, D, bs = c["B"], c["Hq"], c["Hkv"], c["T"], c["D"], c["block_size"]
        W = window_for(c)
        q, do = dev(t["q"], dtype), dev(t["do"], dtype)
        if mode == nsa.MODE_WINDOW:
            k, v = dev(t["kw"], dtype), dev(t["vw"], dtype)
        else:
            k = dev(O.ref_block_mean_pool(t["kc"], bs), dtype)
            v = dev(O.ref_block_mean_pool(t["vc"], bs), dtype)
        o, lse = nsa.range_attn_forward(q, k, v, mode, W, bs)
        rs = torch.rand(B, Hq, T, device="cuda") * 0.9 + 0.05              # a gate value per row
        rd = (do.float() * o.float()).sum(-1)
        dq_ref, dk_ref, dv_ref = nsa.range_attn_backward(q, k, v, o, lse, do, mode, W, bs, rs, rd)
        acc = torch.zeros(B * Hkv, T, Hq // Hkv, D, device="cuda")
        dk, dv = nsa.ops.range_attn_backward_acc(q, k, v, o, lse, do, mode, W, bs, rs, rd, acc)
        dq = torch.empty_like(q)
        L.check(L.lib().nsa_dq_finish(L.dims(B, Hq, Hkv, T, D, L.DTYPE_BF16), 0, 64, L.ptr(acc), None,
                                      L.ptr(dq), L.stream()))
        for got, ref, nm in ((dq, dq_ref, "dq"), (dk, dk_ref, "dk"), (dv, dv_ref, "dv")):
            d = (got.float() - ref.float()).abs().max().item()
            assert d <= 2.0 ** -7 * ref.float().abs().max().item() + 1e-6, (cfg_id(c), mode, nm, d)
    assert nsa.lib().nsa_device_status(None) == 0


def test_status_word_give_up_path_from_the_host():
    """With the device status word set (from the host: no kernel waits for anything), a tcgen05
    launch returns at entry and leaves its outputs untouched; nsa_device_status reports the word and
    clears it; the next launch is correct.  Nothing here faults, traps or hangs."""
    nsa = pkg()
    L = importlib.import_module("openbox-llm_b200._lib")
    lib = L.lib()
    dtype = torch.bfloat16
    c = TC_CONFIGS[1]
    t = make_inputs(c, dtype, seed=9, scale_qkv=True)
    B, Hq, Hkv, T, D = c["B"], c["Hq"], c["Hkv"], c["T"], c["D"]
    q, k, v = dev(t["q"], dtype), dev(t["kw"], dtype), dev(t["vw"], dtype)
    d = L.dims(B, Hq, Hkv, T, D, L.DTYPE_BF16)

    def launch(o, lse):
        return lib.nsa_range_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse), d, T,
                                      L.MODE_WINDOW, 512, 0, L.IMPL["tc"], L.stream())

    o_ok = torch.empty_like(q)
    lse_ok = torch.empty(B, Hq, T, device="cuda")
    assert launch(o_ok, lse_ok) == 0 and lib.nsa_device_status(None) == 0
    assert lib.nsa_debug_set_device_status(0x400, None) == 0
    canary = 1.5
    o = torch.full_like(q, canary)
    lse = torch.full((B, Hq, T), canary, device="cuda")
    assert launch(o, lse) == 0                                 # the launch itself succeeds
    torch.cuda.synchronize()
    assert (o.float() == canary).all() and (lse == canary).all(), "an aborted launch must not write"
    with pytest.raises(L.NsaError, match="bounded wait"):
        L.check_device_status()                                 # reports ...
    assert lib.nsa_device_status(None) == 0                     # ... and clears
    assert launch(o, lse) == 0
    torch.cuda.synchronize()
    assert torch.equal(o, o_ok) and torch.equal(lse, lse_ok)
    # the polling point of the training step raises on a raised word and leaves it cleared
    assert lib.nsa_debug_set_device_status(1, None) == 0
    DP = importlib.import_module("openbox-llm_b200.dp_step")
    lin = torch.nn.Linear(4, 4).cuda()
    step = DP.DataParallelStep.__new__(DP.DataParallelStep)
    step.flat = DP.FlatParams(lin)
    with pytest.raises(L.NsaError):
        step.check_status()
    assert lib.nsa_device_status(None) == 0


def test_wait_that_runs_out_gives_up_and_leaves_the_context_usable():
    """A bounded device wait made to run out, in the one form that faults and hangs nothing: with the
    test-only option the forward kernel never sends one of its loads, so the CTAs that need it spin
    for their limit (about a second, all at the same time), raise the status word, wait for what
    they have in flight, give their tensor memory back and return without writing.  The launch and
    the synchronisation succeed, the status word names the wait, rows of CTAs that never needed the
    missing load are correct, all others are untouched, and the next call is correct."""
    nsa = pkg()
    L = importlib.import_module("openbox-llm_b200._lib")
    lib = L.lib()
    dtype = torch.bfloat16
    B, Hq, Hkv, T, D, W = 1, 16, 1, 256, 128, 128
    g = torch.Generator().manual_seed(21)
    q = (torch.randn(B, Hq, T, D, generator=g) * D ** -0.5).to(dtype).cuda()
    k = (torch.randn(B, Hkv, T, D, generator=g) * D ** -0.5).to(dtype).cuda()
    v = torch.randn(B, Hkv, T, D, generator=g).to(dtype).cuda()
    d = L.dims(B, Hq, Hkv, T, D, L.DTYPE_BF16)

    def launch(o, lse):
        return lib.nsa_range_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse), d, T,
                                      L.MODE_WINDOW, W, 0, L.IMPL["tc"], L.stream())

    o_ok, lse_ok = torch.empty_like(q), torch.empty(B, Hq, T, device="cuda")
    assert launch(o_ok, lse_ok) == 0 and lib.nsa_device_status(None) == 0
    canary = 1.5
    o = torch.full_like(q, canary)
    lse = torch.full((B, Hq, T), canary, device="cuda")
    nsa.set_option("debug_starve_load", 1)
    try:
        assert launch(o, lse) == 0
        torch.cuda.synchronize()                       # returns: the waits are bounded
    finally:
        nsa.set_option("debug_starve_load", 0)
    assert lib.nsa_device_status(None) == -5           # NSA_ERR_DEVICE_WAIT; reads and clears
    msg = lib.nsa_last_error().decode()
    status = int(msg[msg.index("0x"):].rstrip(")"), 16)
    # the V-tile wait (16) starves; the waits behind it (S ready 4, O ready 8) start at the same
    # moment in other threads and may be the first to reach the limit
    assert status != 0 and (status & ~(4 | 8 | 16)) == 0, msg
    assert lib.nsa_device_status(None) == 0
    # queries 0..63 see one key tile only: their CTAs finished before anything ran out
    assert torch.equal(o[:, :, :64], o_ok[:, :, :64]) and torch.equal(lse[:, :, :64], lse_ok[:, :, :64])
    # every CTA that needed the second tile gave up and wrote nothing
    assert (o[:, :, 64:].float() == canary).all() and (lse[:, :, 64:] == canary).all()
    assert launch(o, lse) == 0
    torch.cuda.synchronize()
    assert lib.nsa_device_status(None) == 0
    assert torch.equal(o, o_ok) and torch.equal(lse, lse_ok)


def test_selection_plan_gives_the_same_results():
    """The index structures of a block list built once (nsa_selection_plan_build) and handed to
    nsa_selection_fwd_planned / nsa_selection_bwd_planned, against the calls that build them inside
    their workspace: o, lse and dq bit for bit (integer structures, same kernels), dk / dv within
    the accumulation-order bound."""
    nsa = pkg()
    dtype = torch.bfloat16
    for c in (TC_CONFIGS[1], TC_CONFIGS[3]):
        if not nsa.tc_supported(c["B"], c["Hq"], c["Hkv"], c["T"], c["D"], dtype, c["block_size"]):
            continue
        t = make_inputs(c, dtype, seed=13, scale_qkv=True)
        q, k, v, do = (dev(t[n], dtype) for n in ("q", "ks", "vs", "do"))
        idx = t["block_idx"].cuda() if "block_idx" in t else O.make_block_idx(
            c["B"], c["Hkv"], c["T"], c["block_size"], c["S"], seed=3).cuda()
        plan = nsa.ops.selection_plan(q, k, idx, c["block_size"])
        assert plan is not None
        o0, l0 = nsa.selection_forward_triton(q, k, v, idx, c["block_size"], return_lse=True)
        o1, l1 = nsa.selection_forward_triton(q, k, v, idx, c["block_size"], return_lse=True, plan=plan)
        assert torch.equal(o0, o1) and torch.equal(l0, l1), cfg_id(c)
        g0 = nsa.ops._selection_backward(q, k, v, idx, c["block_size"], do, o0, l0)
        g1 = nsa.ops._selection_backward(q, k, v, idx, c["block_size"], do, o0, l0, plan=plan)
        assert torch.equal(g0[0], g1[0]), cfg_id(c)
        for a, b in zip(g0[1:], g1[1:]):
            assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -7 * max(b.float().abs().max().item(), 1e-6)
    assert nsa.lib().nsa_device_status(None) == 0
