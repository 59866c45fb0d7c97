"""Generate the golden vectors in this directory from the reference itself.

Run once, in a container that has the reference checkout (it is not needed to
run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The script imports the reference's pure-torch functions, runs them on small
seeded inputs in fp32 on the CPU and stores inputs and outputs (and autograd
gradients) as .npz files.  The test-suite checks the oracle against these
files; the CUDA kernels are then checked against the oracle.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().numpy()


def main(ref_dir):
    sys.path.insert(0, ref_dir)
    sys.dont_write_bytecode = True
    import nsa_fsa
    import nsa_fused_kernel as fk
    import nsa_model
    import nsa_selection_kernel as sk

    # test_kernel.py needs CUDA at import time, so its generator is restated here
    # exactly (test_kernel.py:39-58) and checked against bench-style generators below.
    def make_block_idx(B, Hkv, T, block_size, S, seed=0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        n_blk = T // block_size
        valid = (torch.arange(n_blk)[None, :] + 1) * block_size <= (torch.arange(T)[:, None] + 1)
        score = torch.rand(B, Hkv, T, n_blk, generator=g).masked_fill(~valid[None, None], -1.0)
        k = min(S, n_blk)
        topv, topi = score.topk(k, dim=-1)
        sel = torch.where(topv >= 0, topi.to(torch.int32),
                          torch.full_like(topi, -1, dtype=torch.int32))
        idx = torch.full((B, Hkv, T, S), -1, dtype=torch.int32)
        idx[..., :k] = sel
        return idx

    cases = [
        dict(name="g2_d16", B=2, Hq=4, Hkv=2, D=16, T=96, bs=16, S=3, window=37),
        dict(name="g3_d32", B=1, Hq=6, Hkv=2, D=32, T=128, bs=16, S=8, window=21),
        dict(name="g4_d32", B=1, Hq=4, Hkv=1, D=32, T=160, bs=32, S=4, window=69),
    ]
    for c in cases:
        torch.manual_seed(7)
        B, Hq, Hkv, D, T, bs, S, W = (c[k] for k in ("B", "Hq", "Hkv", "D", "T", "bs", "S", "window"))
        mk = lambda h: torch.randn(B, h, T, D)
        q = mk(Hq)
        kc, vc, ks, vs, kw, vw = (mk(Hkv) for _ in range(6))
        gate = torch.randn(B, Hq, T, 3)
        do = torch.randn(B, Hq, T, D)
        idx = make_block_idx(B, Hkv, T, bs, S, seed=3)
        # a partially-future block in one row: the kernels attend its causal part
        idx[0, 0, T // 2, 0] = (T // 2) // bs
        out = {"q": q, "kc": kc, "vc": vc, "ks": ks, "vs": vs, "kw": kw, "vw": vw,
               "gate": gate, "do": do, "block_idx": idx,
               "meta": np.array([B, Hq, Hkv, D, T, bs, S, W], dtype=np.int64)}

        # selection branch forward + autograd backward
        qs, kk, vv = (t.clone().requires_grad_(True) for t in (q, ks, vs))
        o = sk.selection_forward_reference(qs, kk, vv, idx, bs)
        o.backward(do)
        out.update(sel_o=o, sel_dq=qs.grad, sel_dk=kk.grad, sel_dv=vv.grad)

        # window branch
        qs, kk, vv = (t.clone().requires_grad_(True) for t in (q, kw, vw))
        o = fk._range_attn_reference(qs, kk, vv, fk.MODE_WINDOW, W, 0)
        o.backward(do)
        out.update(win_o=o, win_dq=qs.grad, win_dk=kk.grad, win_dv=vv.grad)

        # compression branch on mean-pooled keys
        kcp = fk.block_mean_pool(kc, bs)
        vcp = fk.block_mean_pool(vc, bs)
        qs, kk, vv = (t.clone().requires_grad_(True) for t in (q, kcp, vcp))
        o = fk._range_attn_reference(qs, kk, vv, fk.MODE_COMPRESS, 0, bs)
        o.backward(do)
        out.update(k_pool=kcp, v_pool=vcp, cmp_o=o, cmp_dq=qs.grad, cmp_dk=kk.grad, cmp_dv=vv.grad)

        # fused three-branch op, all gradients
        ins = [t.clone().requires_grad_(True) for t in (q, kc, vc, ks, vs, kw, vw, gate)]
        o = fk.nsa_fused_reference(*ins, idx, bs, W)
        o.backward(do)
        out["fused_o"] = o
        for nm, t in zip(["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"], ins):
            out["fused_d" + nm] = t.grad

        # learned compressor (nsa_model.py:100-123) with non-trivial parameters
        comp = nsa_model.BlockCompressor(bs, D)
        with torch.no_grad():
            comp.intra_pos.normal_(0, 0.5)
            comp.pool_logits.normal_(0, 0.5)
        x = kc.clone().requires_grad_(True)
        n_blk = T // bs
        y = comp(x[:, :, :n_blk * bs].view(B, Hkv, n_blk, bs, D))
        dy = torch.randn_like(y)
        y.backward(dy)
        out.update(comp_intra=comp.intra_pos, comp_logits=comp.pool_logits,
                   comp_proj=comp.proj.weight, comp_y=y, comp_dy=dy, comp_dx=x.grad,
                   comp_dintra=comp.intra_pos.grad, comp_dlogits=comp.pool_logits.grad,
                   comp_dproj=comp.proj.weight.grad)

        # block scoring + top-k exactly as nsa_model.py:343-355
        s_cmp = torch.matmul(q, nsa_model.expand_kv(y.detach(), Hq // Hkv).transpose(-1, -2)) * D ** -0.5
        t_idx = torch.arange(T)[:, None]
        blk_end = (torch.arange(n_blk) + 1) * bs - 1
        keep = (blk_end[None, :] <= t_idx)
        p_cmp = nsa_model.masked_softmax(s_cmp, keep[None, None].expand(B, Hq, T, n_blk))
        imp = p_cmp.view(B, Hkv, Hq // Hkv, T, n_blk).sum(dim=2)
        impm = imp.masked_fill(~keep[None, None], torch.finfo(imp.dtype).min)
        topk = torch.topk(impm, min(S, n_blk), dim=-1).indices.to(torch.int32)
        out.update(score_imp=imp, score_topk=topk)

        # CSR inversion
        qob, off, pbh = nsa_fsa.build_block_to_query_csr(idx, bs)
        out.update(csr_q=qob, csr_off=off, csr_bh=pbh)

        np.savez_compressed(os.path.join(HERE, f"nsa_{c['name']}.npz"),
                            **{k: (_np(v) if isinstance(v, torch.Tensor) else v) for k, v in out.items()})
        print("wrote", c["name"])

    # whole attention module (nsa_model.py:196-304): ref path output + grads wrt x
    torch.manual_seed(11)
    attn = nsa_model.NSAAttention(d_model=64, n_q_heads=4, n_kv_heads=2, block_size=16,
                                  n_selected_blocks=3, window=24, attn_impl="ref")
    with torch.no_grad():
        for comp in (attn.comp_k, attn.comp_v):
            comp.intra_pos.normal_(0, 0.1)
            comp.pool_logits.normal_(0, 0.3)
    x = torch.randn(2, 96, 64, requires_grad=True)
    y = attn(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    mod = {"x": x, "y": y, "dy": dy, "dx": x.grad}
    for n, p in attn.named_parameters():
        mod["p." + n] = p
        mod["g." + n] = p.grad
    np.savez_compressed(os.path.join(HERE, "nsa_module.npz"), **{k: _np(v) for k, v in mod.items()})
    print("wrote module")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of an openbox-llm checkout>")
    main(sys.argv[1])
