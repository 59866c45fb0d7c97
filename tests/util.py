"""Shared helpers of the parity tests."""
import importlib
import os

import numpy as np
import torch

from oracle import nsa_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# the reference's own gate matrix (test_kernel.py:25-33)
REF_CONFIGS = [
    dict(B=2, Hq=4, Hkv=2, D=32, T=256, block_size=16, S=4),
    dict(B=1, Hq=8, Hkv=2, D=64, T=512, block_size=32, S=8),
    dict(B=2, Hq=12, Hkv=4, D=64, T=512, block_size=16, S=8),
    dict(B=1, Hq=16, Hkv=4, D=128, T=1024, block_size=64, S=16),
    dict(B=1, Hq=4, Hkv=4, D=64, T=384, block_size=16, S=6),
    dict(B=2, Hq=6, Hkv=3, D=32, T=256, block_size=32, S=3),
    dict(B=1, Hq=8, Hkv=2, D=64, T=512, block_size=16, S=32),
]

# shapes the tcgen05 kernels serve (bf16, D in {64,128}, 64-token blocks)
TC_CONFIGS = [
    dict(B=1, Hq=16, Hkv=1, D=128, T=512, block_size=64, S=4, window=200),
    dict(B=2, Hq=16, Hkv=2, D=128, T=1024, block_size=64, S=16, window=512),
    dict(B=1, Hq=8, Hkv=2, D=64, T=768, block_size=64, S=5, window=133),
    dict(B=1, Hq=4, Hkv=1, D=128, T=448, block_size=64, S=3, window=64),
    dict(B=1, Hq=16, Hkv=4, D=64, T=1000, block_size=64, S=16, window=77),   # ragged T
    dict(B=1, Hq=2, Hkv=1, D=128, T=320, block_size=64, S=2, window=3),
    dict(B=1, Hq=1, Hkv=1, D=64, T=256, block_size=64, S=4, window=300),
    dict(B=2, Hq=6, Hkv=2, D=64, T=576, block_size=64, S=6, window=150),     # 3 heads per kv head (the model config)
]


def pkg():
    return importlib.import_module("openbox-llm_b200")


def cfg_id(c):
    return "B{B}_Hq{Hq}_Hkv{Hkv}_D{D}_T{T}_bs{block_size}_S{S}".format(**c)


def window_for(c):
    """test_kernel_fused.py:29-31: deliberately not a multiple of any tile."""
    return c.get("window", min(c["T"], 2 * c["block_size"] + 5))


def make_inputs(c, dtype, seed=0, scale_qkv=False):
    """CPU tensors in the order of test_kernel_fused.py:34-42, rounded to `dtype`.
    Returns a dict of fp32 CPU tensors holding exactly the values the device will see."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    B, Hq, Hkv, D, T = c["B"], c["Hq"], c["Hkv"], c["D"], c["T"]
    mk = lambda h: torch.randn(B, h, T, D, generator=g)
    names = ["q", "kc", "vc", "ks", "vs", "kw", "vw"]
    t = {"q": mk(Hq)}
    for n in names[1:]:
        t[n] = mk(Hkv)
    if scale_qkv:
        for n in names:
            t[n] = t[n] * D ** -0.5
    t["gate"] = torch.randn(B, Hq, T, 3, generator=g)
    t["do"] = torch.randn(B, Hq, T, D, generator=g)
    for n in list(t):
        t[n] = t[n].to(dtype).float()
    t["block_idx"] = O.make_block_idx(B, Hkv, T, c["block_size"], c["S"], seed=seed)
    return t


def dev(t, dtype):
    if t.dtype in (torch.int32, torch.int64):
        return t.cuda()
    return t.to(dtype).cuda()


def err(a, b):
    """(max-abs, relative L2) of a against b."""
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    d = (a - b)
    return d.abs().max().item() if d.numel() else 0.0, \
        (d.norm() / (b.norm() + 1e-12)).item() if d.numel() else 0.0


# worst measured error per kind of tensor, printed at the end of the session (tests/conftest.py)
WORST = {}


def _record(what, dtype, ma, rl, bound):
    key = ("f32 " if dtype == torch.float32 else "bf16 ") + what.split(" ")[-1]
    w = WORST.get(key, (0.0, 0.0, 0.0, ""))
    if ma / bound >= w[2]:
        WORST[key] = (ma, rl, ma / bound, what)


def check(a, b, dtype, what, abs32=2e-3, abs16=2e-2, rel16=1e-2, scale_abs=True):
    """fp32: max-abs <= abs32 (the reference's fp32 gates are 2e-3..4e-3).
    bf16, inputs scaled as the benchmark configurations scale them (q, k, v times D^-1/2; call with
    scale_abs=False): max-abs <= abs16 = 2e-2 and relative L2 <= rel16 = 1e-2 against the fp32
    oracle on the bf16-rounded inputs.  A bf16 result cannot be closer to a reference entry x than
    |x| * 2^-9 (round to nearest, 8 significant bits), so where the reference holds entries above
    5.12 (dV with dO ~ N(0,1) does) the absolute bound is max(2e-2, 2^-8 * max|b|): the rounding
    of the largest entry plus as much again.  bf16 with unscaled N(0,1) inputs (the reference's
    own gate inputs, where gradients reach tens): the absolute bound is taken relative to the
    largest reference entry, max-abs <= abs16 * max(1, max|b|); the relative-L2 bound is the same."""
    ma, rl = err(a, b)
    assert not torch.isnan(a.float()).any(), what + ": NaN"
    if dtype == torch.float32:
        _record(what, dtype, ma, rl, abs32)
        assert ma <= abs32, f"{what}: max-abs {ma:.3e} > {abs32} (rel-L2 {rl:.3e})"
    else:
        bmax = b.abs().max().item() if b.numel() else 0.0
        bound = abs16 * max(1.0, bmax) if scale_abs else max(abs16, 2.0 ** -8 * bmax)
        _record(what, dtype, ma, rl, bound)
        assert ma <= bound, f"{what}: max-abs {ma:.3e} > {bound:.3e} (rel-L2 {rl:.3e}, max|ref| {bmax:.3g})"
        assert rl <= rel16, f"{what}: rel-L2 {rl:.3e} > {rel16} (max-abs {ma:.3e})"


# ---------------------------------------------------------------------------------------------
# sampled oracle checks at sizes where the whole oracle would take minutes: one (batch, kv head)
# unit, some query rows, some key tiles.  Everything below calls the oracle's own functions.
# ---------------------------------------------------------------------------------------------
def unit_slices(t, b, h, G):
    """fp32 CPU views of one (batch, kv head) unit of a dict of [B,H,T,X] tensors."""
    out = {}
    for n, x in t.items():
        if n in ("q", "gate", "do"):
            out[n] = x[b:b + 1, h * G:(h + 1) * G].float().cpu()
        elif n == "block_idx":
            out[n] = x[b:b + 1, h:h + 1].cpu()
        else:
            out[n] = x[b:b + 1, h:h + 1].float().cpu()
    return out


def selection_keep_rows(idx_unit, rows, T, block_size):
    """Keep mask [1,1,R,T] of the selection branch for arbitrary query positions `rows` of one
    unit (the rule of oracle.selection_keep, nsa_selection_kernel.py:73-84,142-144)."""
    rows = torch.as_tensor(rows)
    sub = idx_unit[:, :, rows]                                    # [1,1,R,S]
    n_blk = -(-T // block_size)
    valid = (sub >= 0) & (sub < n_blk)
    oh = torch.zeros(1, 1, len(rows), sub.shape[-1], n_blk, dtype=torch.bool)
    oh.scatter_(-1, sub.long().clamp(min=0).unsqueeze(-1), valid.unsqueeze(-1))
    chosen = oh.any(dim=3)
    keep = chosen[..., torch.arange(T) // block_size]
    return keep & (torch.arange(T)[None, :] <= rows[:, None])[None, None]


def rows_forward_backward(q_rows, k, v, keep, gate_rows, do_rows, chunk=256):
    """One branch on a set of query rows of one unit: q_rows, do_rows [1,G,R,D]; k, v [1,1,Lk,D];
    keep [R,Lk] or [1,1,R,Lk]; gate_rows [1,G,R] = the branch's sigmoid gate (the branch's own
    upstream gradient is gate * dO).  Returns o, lse, dq, dk, dv (dk, dv: these rows' share)."""
    keep_fn = (lambda a, b: keep[..., a:b, :]) if keep.dim() == 4 else (lambda a, b: keep[a:b])
    o, lse = O.stream_attn_forward(q_rows, k, v, keep_fn, chunk=chunk)
    do_b = do_rows * gate_rows[..., None]
    dq, dk, dv = O.stream_attn_backward(q_rows, k, v, o, lse, do_b, keep_fn, chunk=chunk)
    return o, lse, dq, dk, dv


def check_unit_sampled(u, k_cmp, v_cmp, got, T, block_size, window, dtype, tag, row_windows,
                       win_tiles, sel_blocks, cmp_len=None, cmp_stride=None):
    """Oracle comparison of one unit `u` (unit_slices of the inputs, block_idx and dO) against
    `got` (unit_slices of out and the gradients q, ks, vs, kw, vw, gate; optional dk_cmp,
    dv_cmp [1,1,n_cmp,D] when the caller can isolate them):
      * out, dq, d_gate on the query-row windows `row_windows`;
      * dk, dv of the window branch on the 64-key tiles `win_tiles` (from every query that sees them);
      * dk, dv of the selection branch on the blocks `sel_blocks` (from every query that lists them);
      * dk, dv of the compression branch on all summaries (returned, for the caller to push through
        the pooling backward)."""
    cl = block_size if cmp_len is None else cmp_len
    cs = cl if cmp_stride is None else cmp_stride
    G = u["q"].shape[1]
    sg = torch.sigmoid(u["gate"])                                    # [1,G,T,3]
    n_cmp = k_cmp.shape[2]
    for t0, t1 in row_windows:
        qs, dos = u["q"][:, :, t0:t1], u["do"][:, :, t0:t1]
        keeps = (O.compress_keep(t0, t1, n_cmp, cl, cs),
                 O.selection_keep(u["block_idx"], t0, t1, T, block_size),
                 O.window_keep(t0, t1, T, window))
        kvs = ((k_cmp, v_cmp), (u["ks"], u["vs"]), (u["kw"], u["vw"]))
        outs, dq = [], 0
        for bi, ((k, v), keep) in enumerate(zip(kvs, keeps)):
            o, _, dq_b, _, _ = rows_forward_backward(qs, k, v, keep, sg[:, :, t0:t1, bi], dos)
            outs.append(o)
            dq = dq + dq_b
        ref_out = O.ref_gate_combine(*outs, u["gate"][:, :, t0:t1])
        d_gate = O.gate_combine_backward(*outs, u["gate"][:, :, t0:t1], dos)[3]
        check(got["out"][:, :, t0:t1], ref_out, dtype, f"{tag} rows {t0}:{t1} out", scale_abs=False)
        check(got["q"][:, :, t0:t1], dq, dtype, f"{tag} rows {t0}:{t1} dq", scale_abs=False)
        check(got["gate"][:, :, t0:t1], d_gate, dtype, f"{tag} rows {t0}:{t1} dgate", scale_abs=False)
    for j in win_tiles:                                              # window: keys [64 j, 64 j + 64)
        k0, k1 = j * 64, min(T, j * 64 + 64)
        r0, r1 = k0, min(T, k1 - 1 + window)                         # every query that sees one of them
        c0 = max(0, r0 - window + 1)                                 # ... and every key those queries see
        keep = O.window_keep(r0, r1, T, window)[:, c0:r1]
        _, _, _, dk, dv = rows_forward_backward(u["q"][:, :, r0:r1], u["kw"][:, :, c0:r1], u["vw"][:, :, c0:r1],
                                                keep, sg[:, :, r0:r1, 2], u["do"][:, :, r0:r1])
        check(got["kw"][:, :, k0:k1], dk[:, :, k0 - c0:k1 - c0], dtype, f"{tag} window tile {j} dk", scale_abs=False)
        check(got["vw"][:, :, k0:k1], dv[:, :, k0 - c0:k1 - c0], dtype, f"{tag} window tile {j} dv", scale_abs=False)
    idx = u["block_idx"]
    tt = torch.arange(T)
    for j in sel_blocks:                                             # selection: every query listing block j
        lists = ((idx[0, 0] == j).any(-1)) & (tt >= j * block_size)
        rows = torch.nonzero(lists).flatten()
        if rows.numel() == 0:
            continue
        keep = selection_keep_rows(idx, rows, T, block_size)
        _, _, _, dk, dv = rows_forward_backward(u["q"][:, :, rows], u["ks"], u["vs"], keep,
                                                sg[:, :, rows, 1], u["do"][:, :, rows])
        k0, k1 = j * block_size, min(T, (j + 1) * block_size)
        check(got["ks"][:, :, k0:k1], dk[:, :, k0:k1], dtype, f"{tag} selection block {j} ({rows.numel()} queries) dk", scale_abs=False)
        check(got["vs"][:, :, k0:k1], dv[:, :, k0:k1], dtype, f"{tag} selection block {j} ({rows.numel()} queries) dv", scale_abs=False)
    # compression: all rows of the unit (few keys, so this is cheap)
    keep_fn = O.compress_keep_fn(n_cmp, cl, cs)
    o, lse = O.stream_attn_forward(u["q"], k_cmp, v_cmp, keep_fn)
    _, dk_cmp, dv_cmp = O.stream_attn_backward(u["q"], k_cmp, v_cmp, o, lse, u["do"] * sg[..., 0:1], keep_fn)
    return dk_cmp, dv_cmp


def load_golden(name):
    z = np.load(os.path.join(GOLD, name))
    return {k: torch.from_numpy(z[k]) for k in z.files}
