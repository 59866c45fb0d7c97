"""Multi-GPU path on CPU: two gloo ranks each take their (batch, kv-head) units, run the op
(here: the oracle, there is no GPU) on their slice only, and the merged result equals the
unsharded one.  No data-path collective is involved; all_gather is only the test's way of
collecting the parts."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nsa_oracle as O

S = importlib.import_module("openbox-llm_b200.shard")


def test_unit_ranges_cover_everything_once():
    for n in (1, 3, 4, 16, 17):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                a, b = S.unit_range(n, world, r)
                assert 0 <= a <= b <= n and b - a in (n // world, n // world + 1)
                seen += list(range(a, b))
            assert seen == list(range(n))


def _inputs():
    g = torch.Generator().manual_seed(0)
    B, Hq, Hkv, T, D = 2, 4, 2, 96, 16
    mk = lambda h: torch.randn(B, h, T, D, generator=g)
    t = {"q": mk(Hq)}
    for n in ("kc", "vc", "ks", "vs", "kw", "vw"):
        t[n] = mk(Hkv)
    t["gate"] = torch.randn(B, Hq, T, 3, generator=g)
    return t, (B, Hq, Hkv, T, D)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    t, (B, Hq, Hkv, T, D) = _inputs()
    a, b = S.unit_range(B * Hkv, world, rank)
    loc = {n: S.slice_units(x, Hkv, a, b) for n, x in t.items()}      # [units, G or 1, T, *]
    res = O.stream_nsa_forward(loc["q"], loc["kc"], loc["vc"], loc["ks"], loc["vs"], loc["kw"],
                               loc["vw"], loc["gate"], 16, 3, 24)
    parts = [None] * world
    dist.all_gather_object(parts, res["out"])
    idx_parts = [None] * world
    dist.all_gather_object(idx_parts, res["block_idx"])
    if rank == 0:
        out.put((S.merge_units(parts, B, Hkv), torch.cat(idx_parts, 0).reshape(B, Hkv, T, 3)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_op():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    merged, idx = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    t, (B, Hq, Hkv, T, D) = _inputs()
    full = O.stream_nsa_forward(t["q"], t["kc"], t["vc"], t["ks"], t["vs"], t["kw"], t["vw"],
                                t["gate"], 16, 3, 24)
    assert torch.equal(idx, full["block_idx"])
    assert (merged - full["out"]).abs().max().item() <= 1e-6


@pytest.mark.gpu
def test_unit_shards_on_the_gpu_reproduce_the_unsharded_call_bit_for_bit():
    """What bench.py does under torchrun, on one GPU: the 4 (batch, kv-head) units of a call are
    run as two shards of two units, back to back, through the CUDA kernels; the merged out, block
    lists, dq and d_gate equal the unsharded call bit for bit, dk / dv up to the order of their fp32
    accumulation, and the shards' compressor parameter gradients add up to the unsharded ones."""
    nsa = importlib.import_module("openbox-llm_b200")
    dtype = torch.bfloat16
    B, Hq, Hkv, T, D, bs, n_sel, W = 2, 16, 2, 1024, 128, 64, 8, 200
    G = Hq // Hkv
    g = torch.Generator().manual_seed(12)
    mk = lambda h: (torch.randn(B, h, T, D, generator=g) * D ** -0.5).to(dtype).cuda()
    t = {"q": mk(Hq)}
    for n in ("kc", "vc", "ks", "vs", "kw", "vw"):
        t[n] = mk(Hkv)
    t["gate"] = torch.randn(B, Hq, T, 3, generator=g).to(dtype).cuda()
    do = torch.randn(B, Hq, T, D, generator=g).to(dtype).cuda()
    comp = {}
    for p in ("k", "v"):
        comp[p + "_intra"] = (0.02 * torch.randn(bs, D, generator=g)).cuda()
        comp[p + "_logits"] = (0.3 * torch.randn(bs, generator=g)).cuda()
        comp[p + "_proj"] = (torch.randn(D, D, generator=g) * D ** -0.5).cuda()
    names = ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]

    def run(tensors, d_out):
        ins = [tensors[n].clone().requires_grad_(True) for n in names]
        cps = {k: v.clone().requires_grad_(True) for k, v in comp.items()}
        out, idx = nsa.nsa_attention(*ins, bs, n_sel, W, compressor=cps, return_block_idx=True)
        out.backward(d_out)
        return out.detach(), idx, [x.grad for x in ins], {k: v.grad for k, v in cps.items()}

    try:
        full_out, full_idx, full_g, full_p = run(t, do)
        parts = []
        for rank in range(2):
            a, b = S.unit_range(B * Hkv, 2, rank)
            loc = {n: S.slice_units(x, Hkv, a, b).contiguous() for n, x in t.items()}
            parts.append(run(loc, S.slice_units(do, Hkv, a, b).contiguous()))
    finally:
        pass
    assert torch.equal(S.merge_units([p[0] for p in parts], B, Hkv), full_out)
    assert torch.equal(torch.cat([p[1] for p in parts], 0).reshape(B, Hkv, T, n_sel), full_idx)
    for i, n in enumerate(names):
        merged = S.merge_units([p[2][i] for p in parts], B, Hkv)
        if n in ("q", "gate"):          # added up in a fixed order: bit for bit
            assert torch.equal(merged, full_g[i]), n
        else:                           # dk / dv of a key tile collect their row tiles in TMEM in the order
            a, b = merged.float(), full_g[i].float()      # the two compute groups happen to issue them
            assert (a - b).abs().max().item() <= 2.0 ** -7 * b.abs().max().item(), n
    for k in comp:
        s = parts[0][3][k] + parts[1][3][k]
        ref = full_p[k]
        assert (s - ref).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item()), k
    assert nsa.lib().nsa_device_status(None) == 0


@pytest.mark.gpu
def test_query_heads_of_a_group_dealt_out_over_two_parts():
    """Forward with fewer (batch, kv-head) units than devices, as bench.py runs the long-context
    sweep on eight ranks: each part takes half of a group's query heads, the block lists come from
    the whole group (select_blocks), K / V are the unit's.  The lists equal the unsplit op's bit
    for bit; the outputs agree within bf16 rounding (a part has other row tiles than the whole
    group, so its key tiles, hence the order of its sums, differ)."""
    nsa = importlib.import_module("openbox-llm_b200")
    dtype = torch.bfloat16
    B, Hq, Hkv, T, D, bs, n_sel, W = 1, 16, 1, 2048, 128, 64, 8, 512
    g = torch.Generator().manual_seed(31)
    mk = lambda h: (torch.randn(B, h, T, D, generator=g) * D ** -0.5).to(dtype).cuda()
    q = mk(Hq)
    kv = [mk(Hkv) for _ in range(6)]
    gate = torch.randn(B, Hq, T, 3, generator=g).to(dtype).cuda()
    comp = {}
    for p in ("k", "v"):
        comp[p + "_intra"] = (0.02 * torch.randn(bs, D, generator=g)).cuda()
        comp[p + "_logits"] = (0.3 * torch.randn(bs, generator=g)).cuda()
        comp[p + "_proj"] = (torch.randn(D, D, generator=g) * D ** -0.5).cuda()
    with torch.no_grad():
        full, full_idx = nsa.nsa_attention(q, *kv, gate, bs, n_sel, W, compressor=comp, return_block_idx=True)
        idx = nsa.select_blocks(q, kv[0], kv[1], bs, n_sel, compressor=comp)
        assert torch.equal(idx, full_idx)
        outs = []
        for part in range(2):
            hs = slice(part * 8, part * 8 + 8)
            outs.append(nsa.nsa_attention(q[:, hs].contiguous(), *kv, gate[:, hs].contiguous(), bs, n_sel, W,
                                          compressor=comp, block_idx=idx))
    merged = torch.cat(outs, 1)
    d = (merged.float() - full.float()).abs().max().item()
    assert d <= 2.0 ** -7 * max(full.float().abs().max().item(), 1e-3), d
    assert nsa.lib().nsa_device_status(None) == 0
