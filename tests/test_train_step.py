"""Data-parallel training step: the bucketed gradient all-reduce on two gloo ranks (CPU), and on a
GPU the clip + AdamW kernels against torch and the whole step against the reference's recipe
(autocast forward, backward, clip_grad_norm_, torch.optim.AdamW: train.py:148-149, :256-264)."""
import copy
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

DP = importlib.import_module("openbox-llm_b200.dp_step")


def _mlp(seed):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.Tanh(), torch.nn.Linear(32, 32),
                               torch.nn.Tanh(), torch.nn.Linear(32, 3))


def test_flat_views_and_bucket_layout():
    m = _mlp(0)
    before = [p.detach().clone() for p in m.parameters()]
    flat = DP.FlatParams(m)
    b = DP.GradBuckets(flat, bucket_bytes=1024)
    assert all(torch.equal(p.detach(), q) for p, q in zip(m.parameters(), before))
    # the ranges tile the buffer from the end backwards, every parameter in exactly one bucket
    assert b.ranges[0][1] == flat.numel and b.ranges[-1][0] == 0
    assert all(b.ranges[i][0] == b.ranges[i + 1][1] for i in range(len(b.ranges) - 1))
    assert sum(b.pending0) == len(flat.params)
    flat.zero_grad(); b.start()
    m(torch.randn(4, 12)).square().sum().backward()
    b.finish()
    assert b.pending == [0] * len(b.ranges)
    ref = copy.deepcopy(m)
    for p in ref.parameters():
        p.grad = None
    # the flat gradient is what autograd wrote through the views
    for p, off in zip(flat.params, flat.offsets):
        assert torch.equal(flat.grad[off:off + p.numel()].view(p.shape), p.grad)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m = _mlp(0)                                   # identical replicas
    flat = DP.FlatParams(m)
    b = DP.GradBuckets(flat, bucket_bytes=512)    # several buckets
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(6, 12, generator=g)           # each rank its own micro-batch
    flat.zero_grad(); b.start()
    m(x).square().mean().backward()
    b.finish()
    out.put((rank, x, flat.grad.clone() / world))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_average_their_gradients():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([out.get(timeout=120) for _ in range(2)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # both ranks hold the same averaged gradient = gradient of the mean loss over both micro-batches
    assert torch.equal(got[0][2], got[1][2])
    m = _mlp(0)
    loss = sum(m(x).square().mean() for _, x, _ in got) / 2
    loss.backward()
    want = torch.cat([torch.nn.functional.pad(p.grad.reshape(-1), (0, (-p.numel()) % 4)) for p in m.parameters()])
    assert (got[0][2] - want).abs().max().item() <= 1e-6


def _same_training(a, b, lr, steps):
    """Two replicas trained on the same batches by two implementations of one step.  Kernels that
    accumulate with fp32 atomics make the gradients differ in the last bits from run to run, and
    Adam turns a gradient whose sign is noise into a step of +-lr either way: single entries may
    drift by up to 2 * lr per step (no bound on the maximum can fail, so none is asserted), the
    bulk may not."""
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert (p - q).abs().mean().item() <= 0.05 * lr * steps, n


@pytest.mark.gpu
def test_fused_clip_adamw_matches_torch():
    m = _mlp(1).cuda()
    ref = copy.deepcopy(m)
    flat = DP.FlatParams(m)
    opt = DP.FusedAdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_clip=0.5)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    g = torch.Generator(device="cuda").manual_seed(0)
    for step in range(6):
        x = torch.randn(16, 12, generator=g, device="cuda") * (3.0 if step % 2 else 0.1)   # clipped and unclipped steps
        flat.zero_grad()
        m(x).square().sum().backward()
        opt.step()
        ropt.zero_grad(set_to_none=True)
        ref(x).square().sum().backward()
        norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        ropt.step()
        assert abs(opt.grad_norm() - float(norm)) <= 1e-4 * max(1.0, float(norm))
        for p, q in zip(m.parameters(), ref.parameters()):
            assert (p - q).abs().max().item() <= 2e-6, step


@pytest.mark.gpu
def test_training_step_matches_the_reference_recipe():
    M = importlib.import_module("openbox-llm_b200.model")
    torch.manual_seed(0)
    kw = dict(vocab_size=512, d_model=128, n_layers=2, n_q_heads=4, n_kv_heads=2, max_seq_len=256,
              block_size=64, n_selected_blocks=2, window=64)
    a = M.NSATransformerB200(**kw).cuda()
    b = copy.deepcopy(a)
    assert a.lm_head.weight is a.tok_emb.weight and b.lm_head.weight is b.tok_emb.weight
    step = DP.DataParallelStep(a, lr=1e-3, weight_decay=0.1, grad_clip=1.0)
    ropt = torch.optim.AdamW(b.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    losses = []
    for _ in range(3):
        idx = torch.randint(0, 512, (2, 256), generator=g).cuda()
        tgt = torch.randint(0, 512, (2, 256), generator=g).cuda()
        la = step.step(idx, tgt)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, lb = b(idx, tgt)
        ropt.zero_grad(set_to_none=True)
        lb.backward()
        torch.nn.utils.clip_grad_norm_(b.parameters(), 1.0)
        ropt.step()
        losses.append((float(la), float(lb.detach())))
    for la, lb in losses:
        assert abs(la - lb) <= 2e-3 * max(1.0, abs(lb)), losses
    _same_training(a, b, 1e-3, 3)
    # a snapshot with the reference's key names loads (nsa_model.py:455-478 module tree)
    keys = set(a.state_dict())
    assert {"tok_emb.weight", "pos_emb.weight", "blocks.0.ln1.weight", "blocks.0.attn.q_proj.weight",
            "blocks.0.attn.comp_k.intra_pos", "blocks.0.attn.gate.bias", "blocks.1.ffn.2.weight",
            "ln_f.bias", "lm_head.weight"} <= keys


@pytest.mark.gpu
def test_graph_replay_gives_the_eager_step():
    """Forward + backward replayed from a CUDA graph against the eager step on the same batches
    (the attention kernels, their work lists and device-side choices all run inside the capture).
    With lr = 0 the two replicas keep identical parameters, so every step compares the loss and the
    flat gradient of one and the same function: what may differ is the order of fp32 atomic adds
    and of the dK / dV accumulation, nothing else."""
    M = importlib.import_module("openbox-llm_b200.model")
    torch.manual_seed(0)
    kw = dict(vocab_size=512, d_model=128, n_layers=2, n_q_heads=4, n_kv_heads=2, max_seq_len=256,
              block_size=64, n_selected_blocks=2, window=64)
    a = M.NSATransformerB200(**kw).cuda()
    b = copy.deepcopy(a)
    sa = DP.DataParallelStep(a, lr=0.0, use_graph=True, graph_warmup=2)
    sb = DP.DataParallelStep(b, lr=0.0)
    g = torch.Generator().manual_seed(2)
    worst = 0.0
    for i in range(6):
        idx = torch.randint(0, 512, (2, 256), generator=g).cuda()
        tgt = torch.randint(0, 512, (2, 256), generator=g).cuda()
        la, lb = float(sa.step(idx, tgt)), float(sb.step(idx, tgt))
        assert abs(la - lb) <= 1e-5 * max(1.0, abs(lb)), (i, la, lb)
        ga, gb = sa.flat.grad.float(), sb.flat.grad.float()
        rel = ((ga - gb).norm() / gb.norm().clamp_min(1e-12)).item()
        worst = max(worst, rel)
        assert rel <= 1e-3, (i, rel)
        assert (ga - gb).abs().max().item() <= 1e-3 * gb.abs().max().item(), i
    assert sa.graph is not None
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.equal(p, q)
    print(f"graph vs eager: worst relative L2 of the flat gradient {worst:.2e}")
    lib = importlib.import_module("openbox-llm_b200._lib").lib()
    assert lib.nsa_device_status(None) == 0


@pytest.mark.gpu
def test_graph_replay_trains_like_the_eager_step():
    """Six optimizer steps, graph against eager: the losses stay together (parameters are not
    compared entry by entry: Adam turns a gradient entry whose sign is rounding noise into a step of
    +-lr either way, so single entries may part while the function does not)."""
    M = importlib.import_module("openbox-llm_b200.model")
    torch.manual_seed(0)
    kw = dict(vocab_size=512, d_model=128, n_layers=2, n_q_heads=4, n_kv_heads=2, max_seq_len=256,
              block_size=64, n_selected_blocks=2, window=64)
    a = M.NSATransformerB200(**kw).cuda()
    b = copy.deepcopy(a)
    sa = DP.DataParallelStep(a, lr=1e-3, use_graph=True, graph_warmup=2)
    sb = DP.DataParallelStep(b, lr=1e-3)
    g = torch.Generator().manual_seed(2)
    for i in range(6):
        idx = torch.randint(0, 512, (2, 256), generator=g).cuda()
        tgt = torch.randint(0, 512, (2, 256), generator=g).cuda()
        la, lb = float(sa.step(idx, tgt)), float(sb.step(idx, tgt))
        assert abs(la - lb) <= 2e-3 * max(1.0, abs(lb)), (i, la, lb)
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert (p - q).abs().mean().item() <= 0.05 * 1e-3 * 6, n


@pytest.mark.gpu
def test_model_against_the_reference_transformer():
    """NSATransformerB200 against the reference's own NSATransformer(attn_impl="ref") (pure torch,
    nsa_model.py:455-506) holding the same state_dict: one forward + backward under bf16 autocast on
    one batch, loss and every parameter gradient.  Bounds: the reference's own model-level gate
    (test_integration.py: loss 5e-2, gradients 8e-2 max-abs in bf16)."""
    MR = importlib.import_module("oracle.make_ref")
    if not MR.available():
        pytest.skip("oracle/_ref holds no copy of the reference modules (python oracle/make_ref.py)")
    MR.import_path()
    ref_mod = importlib.import_module("nsa_model")
    M = importlib.import_module("openbox-llm_b200.model")
    torch.manual_seed(0)
    kw = dict(vocab_size=512, d_model=128, n_layers=2, n_q_heads=4, n_kv_heads=2, max_seq_len=256,
              block_size=64, n_selected_blocks=2, window=64)
    ref = ref_mod.NSATransformer(attn_type="nsa", attn_impl="ref", **kw).cuda()
    ours = M.NSATransformerB200(**kw).cuda()
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, 512, (2, 256), generator=g).cuda()
    tgt = torch.randint(0, 512, (2, 256), generator=g).cuda()
    grads = []
    for m in (ref, ours):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = m(idx, tgt)
        m.zero_grad(set_to_none=True)
        loss.backward()
        grads.append((float(loss.detach()), {n: p.grad.float() for n, p in m.named_parameters() if p.grad is not None}))
    (lr_, gr), (lo, go) = grads
    assert abs(lr_ - lo) <= 5e-2, (lr_, lo)
    assert set(gr) == set(go)
    worst = max(((gr[n] - go[n]).abs().max().item(), n) for n in gr)
    assert worst[0] <= 8e-2, worst
    # Relative L2 over all parameters, which the reference's gate does not ask for.  Loose on
    # purpose: under autocast the reference's pure-torch path rounds its scores to bf16 and picks
    # its blocks from those (nsa_model.py:226-258), this build scores in fp32, so near-tied rows
    # attend different blocks on the two sides; the kernel-level tests, where the lists are an
    # input, carry the tight bounds.
    num = sum(((gr[n] - go[n]) ** 2).sum().item() for n in gr) ** 0.5
    den = sum((gr[n] ** 2).sum().item() for n in gr) ** 0.5
    assert num <= 0.25 * den, (num, den, num / den)
    print(f"model vs reference: loss {lr_:.5f} / {lo:.5f}, worst gradient max-abs {worst[0]:.2e} ({worst[1]}), rel-L2 {num / den:.2e}")
