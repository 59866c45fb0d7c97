"""Benchmark of the NSA attention op, forward + backward, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one forward + backward pass of the whole op (learned block pooling, compression
attention, block scoring + top-n, selected-block attention, sliding-window attention, gate
combine and every input/parameter gradient) over one batch of synthetic input.  Workload
"c4_t32k" is the configuration the headline metric is quoted on (B=8, T=32768, 16 query heads /
2 kv heads, D=128, 64-token blocks, top-16, window 512, bf16).  Under torchrun the workload's
B x Hkv = 16 (batch, kv-head) units are dealt out over the ranks (shard.unit_range): every rank
runs the op on its own units only, nothing is exchanged on the data path, and the six shared
compressor parameter gradients are summed over ranks by one small NCCL all-reduce inside the
timed step.  The reported value is the whole job's tokens (B x T per step, whatever N) divided
by the slowest rank's time: "strong" scaling.  `also` holds further legs on the driver's record:
the replica run of earlier builds (every rank the full workload, "weak"), the same shape on
"most recent blocks" lists (the reference's own bench lists, bench_kernel.py:43-53, where the
query-outer selection kernel serves the call), the forward-only long-context shapes and the
12-layer model step.

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's own pure-torch functions
(oracle/_ref, a copy of its modules made by oracle/make_ref.py) on the host cores instead, or the
oracle's restatement of them when that copy is absent.
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # the T=32K training shape the headline metric is quoted on
    "c4_t32k": dict(B=8, T=32768, Hq=16, Hkv=2, D=128, block_size=64, n_sel=16, window=512),
    # the same shape with the published NSA geometry (not expressible in the reference):
    # summaries of 32 tokens every 16, block 0 and the two local blocks in every list
    "c4_t32k_l32d16": dict(B=8, T=32768, Hq=16, Hkv=2, D=128, block_size=64, n_sel=16, window=512,
                           cmp_len=32, cmp_stride=16, n_init=1, n_local=2),
    # the single-kv-head 8K shape (16 query heads share one kv head)
    "c2_t8k": dict(B=4, T=8192, Hq=16, Hkv=1, D=128, block_size=64, n_sel=16, window=512),
    "tiny": dict(B=1, T=2048, Hq=16, Hkv=2, D=128, block_size=64, n_sel=16, window=512),
    # a quarter-length, quarter-batch cut of c4_t32k (same heads, so the same bytes per unit and token):
    # the case counter captures are taken on (inputs above the 126 MB L2, a few GB on the device)
    "c4_t16k_b2": dict(B=2, T=16384, Hq=16, Hkv=2, D=128, block_size=64, n_sel=16, window=512),
    # forward only at long context, 64 query / 4 kv heads (value = forward tokens/s)
    "c3_t16k_fwd": dict(B=1, T=16384, Hq=64, Hkv=4, D=128, block_size=64, n_sel=16, window=512, fwd_only=True),
    "c3_t32k_fwd": dict(B=1, T=32768, Hq=64, Hkv=4, D=128, block_size=64, n_sel=16, window=512, fwd_only=True),
    "c3_t64k_fwd": dict(B=1, T=65536, Hq=64, Hkv=4, D=128, block_size=64, n_sel=16, window=512, fwd_only=True),
    "c3_t128k_fwd": dict(B=1, T=131072, Hq=64, Hkv=4, D=128, block_size=64, n_sel=16, window=512, fwd_only=True),
}
METRIC = "NSA fwd+bwd tokens/s per B200 at T=32K bf16; % of tensor-pipe peak"

NAMES = ["q", "kc", "vc", "ks", "vs", "kw", "vw", "gate"]
COMP = ["k_intra", "k_logits", "k_proj", "v_intra", "v_logits", "v_proj"]


def load_traffic():
    """DRAM bytes per launch of the main kernels from the tracked ncu summary: measured on a small
    capture and scaled to a launch of this workload by the units it processes (the file says on
    which shape, by which command and with which rule)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    return json.load(open(path))


def config_of(name, w, world=1, sharding=None):
    cl = w.get("cmp_len") or w["block_size"]
    cs = w.get("cmp_stride") or cl
    cfg = dict(workload=name, **w,
               compression=f"learned pooling, summaries of {cl} tokens every {cs}" +
                           (" (the reference's grid)" if cl == cs == w["block_size"] else
                            " (not expressible in the reference)"),
               kv_tensors="six independent (kc,vc,ks,vs,kw,vw)",
               l2="inputs (2.9 GB per step at c4_t32k) exceed the 126 MB L2")
    if sharding:
        cfg["sharding"] = sharding
    return cfg


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops=float(p["bf16_tflops_sustained"]), tflops_burst=float(p["bf16_tflops"]),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1400.0, tflops_burst=1590.0, hbm=6650.0, source="fallback")


def unit_inputs(w, units, seed, device):
    """Synthetic inputs of the (batch, kv-head) units `units` of a workload, as the op sees a shard:
    q, gate, dO [n, G, T, *] and six K/V tensors [n, 1, T, D] (a unit is a batch entry with one kv
    head), all ~ N(0,1) in bf16, every unit from its own seed so that a unit's data does not depend
    on how many ranks share the job; compressor parameters as the reference initialises them
    (nsa_model.py:113-116) with 0.02-std noise on the two zero-initialised ones, the same on
    every rank."""
    T, D, bs, G = w["T"], w["D"], w["block_size"], w["Hq"] // w["Hkv"]
    n = len(units)
    t = {"q": torch.empty(n, G, T, D, device=device, dtype=torch.bfloat16),
         "gate": torch.empty(n, G, T, 3, device=device, dtype=torch.bfloat16),
         "do": torch.empty(n, G, T, D, device=device, dtype=torch.bfloat16)}
    for nm in NAMES[1:7]:
        t[nm] = torch.empty(n, 1, T, D, device=device, dtype=torch.bfloat16)
    for i, u in enumerate(units):
        g = torch.Generator(device=device).manual_seed(seed * 100003 + u)
        mk = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        t["q"][i] = mk(G, T, D)
        for nm in NAMES[1:7]:
            t[nm][i] = mk(1, T, D)
        t["gate"][i] = mk(G, T, 3)
        t["do"][i] = mk(G, T, D)
    g = torch.Generator(device=device).manual_seed(seed)
    comp = {}
    cl = w.get("cmp_len") or bs
    for p in ("k", "v"):
        comp[p + "_intra"] = 0.02 * torch.randn(cl, D, generator=g, device=device)
        comp[p + "_logits"] = 0.02 * torch.randn(cl, generator=g, device=device)
        bound = D ** -0.5                                   # nn.Linear default init range
        comp[p + "_proj"] = (torch.rand(D, D, generator=g, device=device) * 2 - 1) * bound
    return t, comp


def recent_block_idx(n_units, T, bs, S, device):
    """"S most recent complete blocks" lists (bench_kernel.py:43-53), built on the device."""
    tt = torch.arange(T, device=device)
    last = (tt + 1) // bs - 1                                       # newest complete block
    idx = last[:, None] - torch.arange(S, device=device)[None, :]
    idx = torch.where(idx >= 0, idx, torch.full_like(idx, -1)).to(torch.int32)
    return idx[None, None].expand(n_units, 1, T, S).contiguous()


def run_step(nsa, t, comp, w, block_idx=None, reduce_params=None):
    """One pass of the op over the tensors of a shard.  reduce_params(list of the six compressor
    parameter gradients) sums them over the ranks (the only cross-unit reduction of the op)."""
    kw = dict(n_init_blocks=w.get("n_init", 0), n_local_blocks=w.get("n_local", 0),
              cmp_len=w.get("cmp_len"), cmp_stride=w.get("cmp_stride"), block_idx=block_idx,
              return_block_idx=True)
    if w.get("fwd_only"):
        with torch.no_grad():
            out, idx = nsa.nsa_attention(*(t[n] for n in NAMES), w["block_size"], w["n_sel"], w["window"],
                                         compressor=comp, **kw)
        return out, idx, ()
    ins = [t[n].detach().requires_grad_(True) for n in NAMES]
    cps = {k: v.detach().requires_grad_(True) for k, v in comp.items()}
    out, idx = nsa.nsa_attention(*ins, w["block_size"], w["n_sel"], w["window"], compressor=cps, **kw)
    grads = torch.autograd.grad(out, ins + [cps[k] for k in COMP], t["do"])
    if reduce_params is not None:
        grads = list(grads[:len(ins)]) + reduce_params(list(grads[len(ins):]))
    return out, idx, grads


def attended(idx, w):
    """Exact (query, key) pairs attended per branch, summed over the units of idx; every one of
    them is visited by each of the G query heads of its group."""
    T, bs, W = w["T"], w["block_size"], w["window"]
    tt = torch.arange(T, device=idx.device)
    units = idx.shape[0] * idx.shape[1]
    cl = w.get("cmp_len") or bs
    cs = w.get("cmp_stride") or cl
    n_sum = (T - cl) // cs + 1 if T >= cl else 0
    n_cmp = int(torch.clamp((tt + 1 - cl) // cs + 1, min=0, max=n_sum).sum().item()) * units
    n_win = int(torch.clamp(tt + 1, max=W).sum().item()) * units
    n_slc, n_pairs = 0, 0
    for u in range(idx.shape[0]):                                  # unit by unit: int64 temporaries stay small
        i64 = idx[u].long()
        start = i64 * bs
        live = (i64 >= 0) & (start <= tt.view(1, T, 1))
        end = torch.minimum(start + bs - 1, tt.view(1, T, 1))
        n_slc += int(torch.where(live, end - start + 1, torch.zeros_like(i64)).sum().item())
        n_pairs += int(live.sum().item())
    return {"cmp": n_cmp, "slc": n_slc, "win": n_win, "sel_pairs": n_pairs}


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_port_pass(w, rows, threads, seed=0):
    """One forward+backward of the reference's pure-torch algorithm (dense masked scores over
    all T keys per query row, as nsa_model.py:196-304 computes them) restated by the oracle,
    on `rows` query rows of ONE (batch, kv-head) unit.  Returns seconds."""
    from oracle import nsa_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    T, D, bs, G = w["T"], w["D"], w["block_size"], w["Hq"] // w["Hkv"]
    r0 = T - rows
    q = torch.randn(1, G, rows, D, generator=g)
    kv = [torch.randn(1, 1, T, D, generator=g) for _ in range(6)]
    gate = torch.randn(1, G, rows, 3, generator=g)
    do = torch.randn(1, G, rows, D, generator=g)
    idx = O.make_block_idx_recent(1, 1, T, bs, w["n_sel"])
    t0 = time.perf_counter()
    cl = w.get("cmp_len") or bs
    cs = w.get("cmp_stride") or cl
    k_cmp = O._windows(kv[0], cl, cs).mean(dim=-2)        # uniform pooling over each summary window
    v_cmp = O._windows(kv[1], cl, cs).mean(dim=-2)
    n_blk = k_cmp.shape[2]
    fns = [(k_cmp, v_cmp, lambda a, b: O.compress_keep(r0 + a, r0 + b, n_blk, cl, cs)),
           (kv[2], kv[3], lambda a, b: O.selection_keep(idx, r0 + a, r0 + b, T, bs)),
           (kv[4], kv[5], lambda a, b: O.window_keep(r0 + a, r0 + b, T, w["window"]))]
    outs = [O.stream_attn_forward(q, k, v, fn, chunk=256) for k, v, fn in fns]
    out = O.ref_gate_combine(outs[0][0], outs[1][0], outs[2][0], gate)
    dos = O.gate_combine_backward(outs[0][0], outs[1][0], outs[2][0], gate, do)
    for (k, v, fn), (o, lse), d in zip(fns, outs, dos[:3]):
        O.stream_attn_backward(q, k, v, o, lse, d, fn, chunk=256)
    return time.perf_counter() - t0, float(out.abs().mean())


def reference_modules():
    """The reference's own modules from oracle/_ref, or None when that copy is absent."""
    try:
        from oracle import make_ref
        if not make_ref.available():
            return None
        make_ref.import_path()
        import nsa_fused_kernel
        import nsa_model
        import nsa_selection_kernel
        return nsa_model, nsa_fused_kernel, nsa_selection_kernel
    except Exception:
        return None


def cpu_reference_pass(mods, G, Ts, D, bs, S, W, threads, seed=0):
    """One forward+backward of the whole op by the reference's OWN pure-torch functions on the host
    cores, fp32: what NSAAttention._forward_fused does (nsa_model.py:325-368) with
    _range_attn_reference / selection_forward_reference in place of the Triton kernels: learned
    BlockCompressor pooling, compression attention, block scoring + torch.topk, selected-block
    attention, window attention, sigmoid gate blend, autograd backward to every input and
    compressor parameter.  One (batch, kv-head) unit: G query heads, one kv head, Ts tokens (the
    reference materialises [G, Ts, Ts] score tensors, so Ts is bounded by host memory).
    Returns seconds."""
    nsa_model, fused, selk = mods
    torch.set_num_threads(threads)
    torch.manual_seed(seed)
    req = lambda *s: torch.randn(*s).requires_grad_(True)
    q = req(1, G, Ts, D)
    kc, vc, ks, vs, kw, vw = (req(1, 1, Ts, D) for _ in range(6))
    gate, do = req(1, G, Ts, 3), torch.randn(1, G, Ts, D)
    comp_k, comp_v = nsa_model.BlockCompressor(bs, D), nsa_model.BlockCompressor(bs, D)
    with torch.no_grad():
        for c in (comp_k, comp_v):
            c.intra_pos.normal_(0, 0.02)
            c.pool_logits.normal_(0, 0.02)
    n_blk = Ts // bs
    t0 = time.perf_counter()
    k_cmp = comp_k(kc[:, :, :n_blk * bs].view(1, 1, n_blk, bs, D))
    v_cmp = comp_v(vc[:, :, :n_blk * bs].view(1, 1, n_blk, bs, D))
    o_cmp = fused._range_attn_reference(q, k_cmp, v_cmp, fused.MODE_COMPRESS, 0, bs)
    with torch.no_grad():                                         # nsa_model.py:343-355
        s_cmp = torch.matmul(q, nsa_model.expand_kv(k_cmp, G).transpose(-1, -2)) * D ** -0.5
        t_idx = torch.arange(Ts)[:, None]
        blk_end = (torch.arange(n_blk) + 1) * bs - 1
        keep = (blk_end[None, :] <= t_idx)[None, None].expand(1, G, Ts, n_blk)
        imp = nsa_model.masked_softmax(s_cmp, keep).view(1, 1, G, Ts, n_blk).sum(dim=2)
        imp = imp.masked_fill(~(blk_end[None, :] <= t_idx)[None, None], torch.finfo(imp.dtype).min)
        block_idx = torch.topk(imp, min(S, n_blk), dim=-1).indices.to(torch.int32)
    o_slc = selk.selection_forward_reference(q, ks, vs, block_idx, bs)
    o_win = fused._range_attn_reference(q, kw, vw, fused.MODE_WINDOW, W, 0)
    g = torch.sigmoid(gate)
    out = g[..., 0:1] * o_cmp + g[..., 1:2] * o_slc + g[..., 2:3] * o_win
    out.backward(do)
    return time.perf_counter() - t0, float(out.detach().abs().mean())


def _reference_sample(w, mods, threads, target_s):
    """Largest Ts (a multiple of the block size, at most 4096) whose pass stays near target_s."""
    G, D, bs, S, W = w["Hq"] // w["Hkv"], w["D"], w["block_size"], w["n_sel"], w["window"]
    Ts = min(1024, w["T"])
    cpu_reference_pass(mods, G, Ts, D, bs, S, W, threads)                # warm-up (thread pool, allocator)
    dt, _ = cpu_reference_pass(mods, G, Ts, D, bs, S, W, threads)        # calibration
    grow = (target_s / max(dt, 1e-3)) ** 0.5                            # dense cost grows with Ts^2
    Ts = int(max(bs, min(w["T"], 4096, Ts * grow) // bs * bs))
    return G, Ts, D, bs, S, W


def cpu_baseline(w, threads, budget_s=20.0):
    """CPU leg of the main line.  With oracle/_ref: the reference's own functions on the first Ts
    tokens of one (batch, kv-head) unit of the workload (a causal prefix is a sub-problem of the
    workload; the reference cannot hold [T, T] scores at T = 32768, and its cost per token grows
    with the prefix length, so this flatters it).  The oracle's restatement on the LAST rows of
    a unit against all T keys, the cost the dense algorithm would have at full length, is reported
    beside it, and alone when the copy of the reference is absent."""
    rows = 64
    dt, _ = cpu_port_pass(w, rows, threads)                # warm-up and calibration
    rows = int(max(64, min(w["T"], rows * (budget_s / 2) / max(dt, 1e-3) // 64 * 64)))
    dt, _ = cpu_port_pass(w, rows, threads)
    # a token is one (batch, position) over all Hq heads = Hkv units' rows
    port = {"value": rows / (dt * w["Hkv"]), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{rows} query rows (the last ones) of one (batch, kv-head) unit against all "
                      f"T={w['T']} keys, fp32 fwd+bwd of the three branches + gate by the oracle's "
                      f"restatement, {dt:.1f} s; scaled by the {w['Hkv']} units a token spans"}
    mods = reference_modules()
    if mods is None:
        return port
    G, Ts, D, bs, S, W = _reference_sample(w, mods, threads, budget_s / 4)
    dt, _ = cpu_reference_pass(mods, G, Ts, D, bs, S, W, threads, seed=1)
    return {"value": Ts / (dt * w["Hkv"]), "unit": "tokens/s", "cores": threads, "kind": "reference",
            "sample": f"the reference's own pure-torch functions (learned pooling, compression, scoring + "
                      f"topk, selection, window, gate; autograd backward), fp32, on the first {Ts} tokens of "
                      f"one (batch, kv-head) unit ({G} query heads), {dt:.1f} s; scaled by the {w['Hkv']} "
                      f"units a token spans; the reference cannot materialise [T,T] at T={w['T']}",
            "port_at_full_length": port}


def reference_arm(args, w, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    mods = reference_modules()
    times = []
    if mods is not None:
        G, Ts, D, bs, S, W = _reference_sample(w, mods, threads, 4.0)   # about 4 s a step
        for i in range(args.warmup + args.steps):
            dt, _ = cpu_reference_pass(mods, G, Ts, D, bs, S, W, threads, seed=i)
            if i >= args.warmup:
                times.append(dt)
        tok_s = Ts * len(times) / (sum(times) * w["Hkv"])
        kind = "reference"
        sample = (f"each step: the reference's own pure-torch functions (oracle/_ref), fp32 fwd+bwd of the "
                  f"whole op on the first {Ts} tokens of one (batch, kv-head) unit ({G} query heads) of the "
                  f"workload; the reference cannot materialise [T,T] at T={w['T']}, and its cost per token "
                  f"grows with the prefix length, so the prefix flatters it")
    else:
        rows = 64
        dt, _ = cpu_port_pass(w, rows, threads)
        rows = int(max(64, min(w["T"], rows * 6.0 / max(dt, 1e-3) // 64 * 64)))   # about 6 s a step
        for i in range(args.warmup + args.steps):
            dt, _ = cpu_port_pass(w, rows, threads, seed=i)
            if i >= args.warmup:
                times.append(dt)
        tok_s = rows * len(times) / (sum(times) * w["Hkv"])
        kind = "port"
        sample = (f"each step: {rows} query rows of one (batch, kv-head) unit against all T={w['T']} "
                  f"keys, fp32, oracle restatement of the reference's pure-torch path (oracle/_ref absent)")
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_of(args.workload, w),
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": kind,
                             "sample": sample},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


MODEL_C5 = dict(vocab_size=50304, d_model=768, n_layers=12, n_q_heads=12, n_kv_heads=4,
                max_seq_len=4096, ffn_mult=4, block_size=64, n_selected_blocks=16, window=512)


def model_workload(args, rank, world, dev, dist, steps=None):
    """The model-level workload: one optimizer step of the 12-layer model (d_model 768, 12 query / 4 kv
    heads, head dim 64, T=4096, micro-batch 8 per GPU; the reference's ~150 M configuration),
    replicas kept in step by the NCCL gradient all-reduce of dp_step.py.  Token ids and targets are
    uniform random (no corpus here), uploaded from pinned host memory every step; the loss is read
    back every step in the end-to-end leg.  Returns the JSON line (rank 0) or None."""
    steps = steps or args.steps
    L = importlib.import_module("openbox-llm_b200._lib")
    M = importlib.import_module("openbox-llm_b200.model")
    DP = importlib.import_module("openbox-llm_b200.dp_step")
    torch.manual_seed(0)                                     # identical replicas
    model = M.NSATransformerB200(**MODEL_C5).to(dev)
    # forward + backward replayed from a CUDA graph: the eager step is bound by the host issuing
    # ~3000 launches (112 ms to enqueue one step against ~90 ms of GPU work)
    step = DP.DataParallelStep(model, lr=3e-4, weight_decay=0.1, grad_clip=1.0,
                               use_graph=not args.no_graph, graph_warmup=2, status_every=0)
    mb, T = 8, MODEL_C5["max_seq_len"]
    g = torch.Generator().manual_seed(1234 + rank)           # every rank its own micro-batches
    host = [(torch.randint(0, MODEL_C5["vocab_size"], (mb, T), generator=g).pin_memory(),
             torch.randint(0, MODEL_C5["vocab_size"], (mb, T), generator=g).pin_memory()) for _ in range(4)]
    devb = [(a.to(dev), b.to(dev)) for a, b in host]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step.step(*devb[i % 4])
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(gpu_index(dev))
    L.lib().nsa_profile_enable(1)
    launches0 = L.lib().nsa_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(steps):
        loss = step.step(*devb[i % 4])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = L.lib().nsa_launch_count() - launches0
    prof = L.profile_summary()
    L.lib().nsa_profile_enable(0)
    clocks = sampler.stop()
    step.check_status()
    # end to end: ids and targets from pinned host memory, the loss back to the host, every step
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    last = 0.0
    for i in range(steps):
        a, b = host[i % 4]
        last = float(step.step(a.to(dev, non_blocking=True), b.to(dev, non_blocking=True)))
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    if dist is not None:
        tt = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = tt.tolist()
    line = None
    if rank == 0:
        tokens = world * mb * T * steps
        total_ms = sum(v[1] for v in prof.values()) or 1.0
        n_params = sum(p.numel() for p in step.flat.params)
        line = {"metric": "optimizer-step tokens/s of the 12-layer NSA model (d_model 768, T=4096, micro-batch 8 per GPU)",
                "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms / steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": dict(workload="c5_model", **MODEL_C5, micro_batch_per_gpu=mb, params=n_params,
                               optimizer="AdamW betas (0.9, 0.95) wd 0.1, clip 1.0, fp32 parameters, bf16 autocast",
                               parallelism=(f"dp{world}: bucketed NCCL all-reduce overlapping backward, eager"
                                            if args.no_graph else
                                            f"dp{world}: forward+backward as one CUDA graph, one NCCL all-reduce after it"),
                               l2="activations of a step exceed the 126 MB L2"),
                "clocks": clocks, "final_loss": last,
                "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": 2 * mb * T * 8, "d2h_bytes_per_step": 4},
                "gpu_launches": int(launches),
                # per-kernel events are not recorded inside a graph replay
                "nsa_kernel_share_of_step": total_ms / ms if args.no_graph else None,
                "kernels": {k: {"launches": v[0], "ms": round(v[1], 3)} for k, v in
                            sorted(prof.items(), key=lambda kv: -kv[1][1])[:12]},
                "roofline": None, "cpu_baseline": None,
                "peak_hbm_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    del step, model, devb
    torch.cuda.empty_cache()
    return line


def gpu_index(dev):
    if "CUDA_VISIBLE_DEVICES" in os.environ:
        return os.environ["CUDA_VISIBLE_DEVICES"].split(",")[dev.index]
    return dev.index


def timed(fn, steps, barrier):
    """ms of `steps` calls of fn between two CUDA events, a barrier + synchronize on both sides."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def main_leg(args, name, w, rank, world, dev, dist, nsa, L):
    """The sharded run of one workload: device-resident timing, the end-to-end leg, the roofline of
    the dominant kernel.  Returns the JSON line on rank 0."""
    shard = importlib.import_module("openbox-llm_b200.shard")
    n_units = w["B"] * w["Hkv"]
    first, last = shard.unit_range(n_units, world, rank)
    units = list(range(first, last))
    G = w["Hq"] // w["Hkv"]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if dist is None:
            return list(vals)
        tt = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt.tolist()

    def sum_over_ranks(*vals):
        if dist is None:
            return list(vals)
        tt = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        return tt.tolist()

    reduce_params = None
    if dist is not None and not w.get("fwd_only"):
        def reduce_params(gs):                                  # one small all-reduce for the six tensors
            flat = torch.cat([g.reshape(-1).float() for g in gs])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            out, off = [], 0
            for g in gs:
                out.append(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
            return out

    if not units:                                               # more ranks than units: this rank idles
        t = comp = None
        step = lambda: ((), None, ())
    else:
        t, comp = unit_inputs(w, units, seed=1234, device=dev)
        step = lambda: run_step(nsa, t, comp, w, reduce_params=reduce_params)
    if not units and reduce_params is not None:                 # still joins the parameter reduction
        zeros = [torch.zeros(s, device=dev) for s in
                 [(w.get("cmp_len") or w["block_size"], w["D"]), (w.get("cmp_len") or w["block_size"],), (w["D"], w["D"])] * 2]
        step = lambda: ((), None, reduce_params(list(zeros)))
    torch.cuda.reset_peak_memory_stats()
    for _ in range(args.warmup):
        out, idx, grads = step()
    torch.cuda.synchronize()
    counts = attended(idx, w) if units else {"cmp": 0, "slc": 0, "win": 0, "sel_pairs": 0}

    # ---- device-resident timing ------------------------------------------------------------
    sampler = ClockSampler(gpu_index(dev))
    L.lib().nsa_profile_enable(1)
    launches0 = L.lib().nsa_launch_count()
    ms = timed(step, args.steps, barrier)
    launches = L.lib().nsa_launch_count() - launches0
    prof = L.profile_summary()
    L.lib().nsa_profile_enable(0)
    clocks = sampler.stop()
    L.check_device_status()
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30

    # ---- end to end: pinned host buffers in, results out, every step ---------------------------
    ms_e2e, h2d, d2h = 0.0, 0, 0
    if units:
        in_names = NAMES if w.get("fwd_only") else NAMES + ["do"]
        host_in = {n: torch.empty(t[n].shape, dtype=t[n].dtype, pin_memory=True).copy_(t[n]) for n in in_names}
        host_out = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in [out] + list(grads)]
        h2d = sum(x.numel() * x.element_size() for x in host_in.values())
        d2h = sum(x.numel() * x.element_size() for x in host_out)
        # Two device input sets and three streams: the upload of step k+1 and the download of
        # step k-1 overlap the kernels of step k.  Every step still uploads all of its inputs from
        # pinned host memory and downloads all of its results.
        dbufs = [{n: torch.empty_like(t[n]) for n in host_in} for _ in range(2)]
        host_outs = [host_out, [torch.empty_like(x).pin_memory() for x in host_out]]
        s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
        main = torch.cuda.current_stream()

    def e2e_run(n_steps):
        if not units:
            for _ in range(n_steps):
                step()
            return
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [None, None]
        for k in range(n_steps):
            bi = k % 2
            with torch.cuda.stream(s_up):
                if in_free[bi] is not None:
                    s_up.wait_event(in_free[bi])
                for n in host_in:
                    dbufs[bi][n].copy_(host_in[n], non_blocking=True)
                in_ready[bi].record(s_up)
            main.wait_event(in_ready[bi])
            o, _, g = run_step(nsa, dbufs[bi], comp, w, reduce_params=reduce_params)
            done = torch.cuda.Event()
            done.record(main)
            in_free[bi] = done
            with torch.cuda.stream(s_down):
                s_down.wait_event(done)
                for dst, src in zip(host_outs[bi], [o] + list(g)):
                    src.record_stream(s_down)
                    dst.copy_(src, non_blocking=True)
        main.wait_stream(s_down)
        main.wait_stream(s_up)

    e2e_run(2)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    e2e_run(args.steps)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    ms, ms_e2e, peak_gb = max_over_ranks(ms, ms_e2e, peak_gb)
    tot = sum_over_ranks(counts["cmp"], counts["slc"], counts["win"], h2d, d2h, launches)
    if rank != 0:
        return None

    tokens = w["B"] * w["T"] * args.steps                  # the whole job, whatever the number of ranks
    pk = peaks()
    # ---- roofline of the dominant kernel (rank 0's launches over rank 0's units) -------------
    # Contractions (tc_* / simt_* attention kernels): bound = tensor pipe, achieved = algorithmic
    # FLOPs per launch / measured launch time.  Algorithmic FLOPs: 4*D per attended (query head,
    # key) pair forward (QK^T and PV), backward 2.5x that (recomputed S, dP, dV, dK, dQ); masked
    # or padded MMA work is not counted.  Streaming kernels: bound = HBM, achieved = the bytes
    # the kernel has to move once (its inputs and outputs) / launch time.
    pairs = {k: counts[k] * G for k in ("cmp", "slc", "win")}
    D = w["D"]
    flop_tab = {}
    for br in ("cmp", "slc", "win"):
        flop_tab["tc_fwd_" + br] = 4 * D * pairs[br]
        flop_tab["tc_bwd_" + br] = 10 * D * pairs[br]        # S, dP, dV, dK, dQ
        flop_tab["simt_fwd_" + br] = 4 * D * pairs[br]
        flop_tab["simt_bwd_" + br] = 10 * D * pairs[br]
    flop_tab["tc_fwd_slc_pairs"] = 4 * D * pairs["slc"]
    n_loc, T_, S_ = len(units), w["T"], w["n_sel"]
    n_pairs = counts["sel_pairs"]
    full = n_loc * G * T_ * D * 2                          # one [units,G,T,D] bf16 tensor
    row = G * D * 2                                        # the G head rows of one query
    t1 = torch.arange(T_)
    win_slots = int(((t1 >> 6) - (torch.clamp(t1 - w["window"] + 1, min=0) >> 6) + 1).sum().item())
    cl_ = w.get("cmp_len") or w["block_size"]
    cs_ = w.get("cmp_stride") or cl_
    n_sum_ = (T_ - cl_) // cs_ + 1 if T_ >= cl_ else 0
    cmp_slots = int(((torch.clamp((t1 + 1 - cl_) // cs_ + 1, min=0, max=n_sum_) + 63) // 64).sum().item())
    # the dQ reduction reads every partial row once (selection: one per pair; window / compression: one
    # per key tile a query attends, or the fp32 accumulator instead) and writes dq
    range_part = 2 * full if nsa.get_dq_accumulator() else n_loc * (win_slots + cmp_slots) * row
    bytes_tab = {
        "sel_combine_kernel": n_pairs * (row + G * 12) + n_loc * T_ * S_ * 4 + full + n_loc * G * T_ * 4,
        "dq_reduce3": n_pairs * row + n_loc * T_ * S_ * 4 + range_part + full,
        "gate_fwd_kernel": 4 * full, "gate_bwd_rows_kernel": 4 * full, "sum3_kernel": 4 * full,
    }
    traffic = load_traffic()
    total_ms = sum(v[1] for v in prof.values()) or 1.0
    top = max(prof.items(), key=lambda kv: kv[1][1]) if prof else (None, (0, 0.0))
    roof = None
    if top[0] is not None:
        kname, (cnt, tms) = top
        sec = tms / max(cnt, 1) * 1e-3
        if kname in flop_tab:
            ach = flop_tab[kname] / sec / 1e12
            roof = {"kernel": kname, "bound": "tensor", "achieved": ach, "peak": pk["tflops"],
                    "unit": "TFLOP/s", "frac": ach / pk["tflops"],
                    "frac_of_burst_peak": ach / pk["tflops_burst"],
                    "peak_source": pk["source"] + " (sustained bf16 GEMM)"}
        else:
            ach = bytes_tab[kname] / sec / 1e9 if kname in bytes_tab else None
            roof = {"kernel": kname, "bound": "hbm", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s",
                    "frac": ach / pk["hbm"] if ach is not None else None,
                    "peak_source": pk["source"] + " (copy bandwidth)"}
        # DRAM bytes of a launch: ncu figure of a small capture, per (batch, kv-head) unit and token,
        # times the units and tokens of this launch
        tr, src = None, None
        if traffic and kname in traffic.get("bytes_per_unit_token", {}):
            tr = traffic["bytes_per_unit_token"][kname] * n_loc * T_
            src = traffic.get("source")
        roof.update({"traffic": tr, "traffic_source": src,
                     "dram_gbs": tr / sec / 1e9 if tr else None,
                     "dram_frac_of_copy_peak": tr / sec / 1e9 / pk["hbm"] if tr else None,
                     "launch_ms": sec * 1e3, "share_of_kernel_time": tms / total_ms})
    total_flops = (4 if w.get("fwd_only") else 14) * D * G * (tot[0] + tot[1] + tot[2])
    sec_step = ms / args.steps * 1e-3
    return {
        "metric": METRIC if not w.get("fwd_only") else "NSA forward tokens/s per B200 at long context, bf16",
        "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": config_of(name, w, world,
                            sharding=f"{n_units} (batch, kv-head) units dealt out over {world} rank(s), "
                                     f"{len(units)} on rank 0; no data-path collective" +
                                     ("" if w.get("fwd_only") or world == 1 else
                                      "; one NCCL all-reduce of the six compressor parameter gradients per step")),
        "tflops_algorithmic": total_flops / sec_step / 1e12,
        "frac_of_tensor_peak": total_flops / sec_step / 1e12 / (pk["tflops"] * world),
        "clocks": clocks,
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(tot[3]),
                "d2h_bytes_per_step": int(tot[4])},
        "gpu_launches": int(tot[5]),
        "peak_hbm_gb": peak_gb,
        "roofline": roof,
        "kernels": {k: {"launches": v[0], "ms": round(v[1], 3), "share": round(v[1] / total_ms, 4)}
                    for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
        "impl": nsa.get_impl(),
        "backward": "dq of window + compression through an fp32 accumulator (TMA reduce-add)"
                    if nsa.get_dq_accumulator() else "bf16 dq partial slots added in a fixed order",
    }


def short_leg(args, name, w, rank, world, dev, dist, nsa, L, units, steps=5, block_idx_fn=None, kernels=()):
    """A few device-resident steps of another workload on `units` of this rank.  Returns
    (ms per step as the max over ranks, peak GB, {kernel: ms per launch} on this rank, counts)."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    counts = None
    if units:
        t, comp = unit_inputs(w, units, seed=4321, device=dev)
        bidx = block_idx_fn(len(units)) if block_idx_fn else None
        step = lambda: run_step(nsa, t, comp, w, block_idx=bidx)
    else:
        step = lambda: None
    for _ in range(3):
        r = step()
    torch.cuda.synchronize()
    if units:
        counts = attended(r[1], w)
    L.lib().nsa_profile_enable(1)
    ms = timed(step, steps, barrier) / steps
    prof = L.profile_summary()
    L.lib().nsa_profile_enable(0)
    L.check_device_status()
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    if dist is not None:
        tt = torch.tensor([ms, peak], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, peak = tt.tolist()
    per = {k: prof[k][1] / max(prof[k][0], 1) for k in kernels if k in prof}
    return ms, peak, per, counts


def head_split_leg(w, rank, used, parts, dev, dist, nsa, L, steps=5):
    """Forward of a workload whose (batch, kv-head) units are fewer than the ranks: rank r takes
    unit r // parts and the part r % parts of its query heads.  The block lists come from the
    whole group (select_blocks, the same on every rank of a unit), everything else is the rank's
    own heads against the unit's K / V.  Returns (ms per step as the max over ranks, peak GB)."""
    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    step = lambda: None
    if rank < used:
        u, part = rank // parts, rank % parts
        t, comp = unit_inputs(w, [u], seed=4321, device=dev)
        G = t["q"].shape[1]
        hs = slice(part * (G // parts), (part + 1) * (G // parts))
        kw = dict(n_init_blocks=w.get("n_init", 0), n_local_blocks=w.get("n_local", 0),
                  cmp_len=w.get("cmp_len"), cmp_stride=w.get("cmp_stride"))

        q_part, gate_part = t["q"][:, hs].contiguous(), t["gate"][:, hs].contiguous()

        def step():
            with torch.no_grad():
                idx = nsa.select_blocks(t["q"], t["kc"], t["vc"], w["block_size"], w["n_sel"], compressor=comp, **kw)
                return nsa.nsa_attention(q_part, *(t[n] for n in NAMES[1:7]), gate_part, w["block_size"],
                                         w["n_sel"], w["window"], compressor=comp, block_idx=idx, **kw)
    for _ in range(3):
        step()
    ms = timed(step, steps, barrier) / steps
    L.check_device_status()
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    if dist is not None:
        tt = torch.tensor([ms, peak], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, peak = tt.tolist()
    return ms, peak


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4_t32k", choices=sorted(WORKLOADS) + ["c5_model"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the extra legs reported under `also`")
    ap.add_argument("--no-graph", action="store_true", help="c5_model: eager step with overlapped bucketed all-reduce")
    ap.add_argument("--dq-accumulator", action="store_true",
                    help="dQ of window + compression through the fp32 accumulator (less memory, slower)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.workload == "c5_model":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the CPU arm times the attention op; the model workload has no CPU arm"}))
            return
        reference_arm(args, WORKLOADS[args.workload], rank)
        return

    assert args.warmup >= 3, "timing rules: at least 3 warm-up steps"
    nsa = importlib.import_module("openbox-llm_b200")
    L = importlib.import_module("openbox-llm_b200._lib")
    shard = importlib.import_module("openbox-llm_b200.shard")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    nsa.set_dq_accumulator(args.dq_accumulator)
    try:
        if args.workload == "c5_model":
            line = model_workload(args, rank, world, dev, dist)
            if rank == 0:
                print(json.dumps(line))
            return
        w = WORKLOADS[args.workload]
        line = main_leg(args, args.workload, w, rank, world, dev, dist, nsa, L)
        if rank == 0:
            line["cpu_baseline"] = (cpu_baseline(w, os.cpu_count() or 1)
                                    if world == 1 and not args.no_cpu_baseline else None)
            line["also"] = None
        if args.workload == "c4_t32k" and not args.no_also:
            also = {}
            pk = peaks()
            G = w["Hq"] // w["Hkv"]
            n_units = w["B"] * w["Hkv"]
            mine = list(range(*shard.unit_range(n_units, world, rank)))
            # (1) every rank the full workload: the replica run of earlier builds
            if world > 1:
                ms, peak, _, _ = short_leg(args, "c4_t32k", w, rank, world, dev, dist, nsa, L,
                                           list(range(n_units)), steps=3)
                also["weak"] = {"workload": "c4_t32k", "what": "every rank runs all 16 units (replicas)",
                                "scaling": "weak", "value": world * w["B"] * w["T"] / (ms * 1e-3),
                                "unit": "tokens/s", "ms_per_step": ms, "steps": 3, "warmup": 3}
            # (2) the same shape on "most recent blocks" lists: neighbouring queries share their
            # blocks, so the device-side rule picks the query-outer selection forward
            ks_ = ("tc_fwd_slc", "tc_bwd_slc", "tc_fwd_slc_pairs")
            ms, peak, per, counts = short_leg(
                args, "c4_t32k", w, rank, world, dev, dist, nsa, L, mine, steps=5, kernels=ks_,
                block_idx_fn=lambda n: recent_block_idx(n, w["T"], w["block_size"], w["n_sel"], dev))
            if rank == 0:
                fl = counts["slc"] * G * w["D"]
                also["recent_lists"] = {
                    "workload": "c4_t32k", "block_lists": "the S most recent complete blocks (bench_kernel.py:43-53)",
                    "value": w["B"] * w["T"] / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                    "steps": 5, "warmup": 3,
                    "selection_kernels": {k: {"launch_ms": v, "tflops": (4 if "fwd" in k else 10) * fl / (v * 1e-3) / 1e12,
                                              "frac_of_tensor_peak": (4 if "fwd" in k else 10) * fl / (v * 1e-3) / 1e12 / pk["tflops"]}
                                          for k, v in per.items() if v > 0.5}}
            # (3) the published geometry (summaries 32 / 16, forced blocks): parity unpinned.  Its 2047
            # summaries take 32 dQ slots per query in the compression backward (34 GB of partials on
            # one GPU); --dq-accumulator trades them for the slower fp32 accumulator
            w2 = WORKLOADS["c4_t32k_l32d16"]
            ms, peak, _, _ = short_leg(args, "c4_t32k_l32d16", w2, rank, world, dev, dist, nsa, L, mine, steps=3)
            also["c4_t32k_l32d16"] = {"config": config_of("c4_t32k_l32d16", w2), "value": w2["B"] * w2["T"] / (ms * 1e-3),
                                      "unit": "tokens/s", "ms_per_step": ms, "steps": 3, "warmup": 3,
                                      "peak_hbm_gb": peak, "parity": "unpinned",
                                      "backward": ("dq of window + compression through the fp32 accumulator"
                                                   if args.dq_accumulator else "bf16 dq partial slots")}
            # (4) forward only at long context: the 4 kv-head units over up to 4 ranks; with 8 ranks
            # every unit's 16 query heads are dealt out over two ranks (K / V of the unit on both, the
            # block lists computed from the whole group on both, no communication)
            sweep = {}
            for nm in ("c3_t16k_fwd", "c3_t32k_fwd", "c3_t64k_fwd", "c3_t128k_fwd"):
                w3 = WORKLOADS[nm]
                n3 = w3["B"] * w3["Hkv"]
                parts = 2 if world >= 2 * n3 else 1
                used = min(world, n3) * parts
                if parts == 1:
                    u3 = list(range(*shard.unit_range(n3, min(world, n3), rank))) if rank < n3 else []
                    ms, peak, _, _ = short_leg(args, nm, w3, rank, world, dev, dist, nsa, L, u3, steps=5)
                else:
                    ms, peak = head_split_leg(w3, rank, used, parts, dev, dist, nsa, L, steps=5)
                sweep[nm] = {"T": w3["T"], "value": w3["B"] * w3["T"] / (ms * 1e-3), "unit": "forward tokens/s",
                             "ms_per_step": ms, "peak_hbm_gb": peak, "ranks_used": used,
                             "split": "units" if parts == 1 else "units x halves of each unit's query heads",
                             "steps": 5, "warmup": 3}
            also["c3_forward_sweep"] = {"shape": "B=1, 64 query / 4 kv heads, D=128", "points": sweep}
            # (5) the 12-layer model step
            m = model_workload(args, rank, world, dev, dist, steps=8)
            if rank == 0:
                also["c5_model"] = {k: m[k] for k in ("value", "unit", "ms_per_step", "steps", "n_gpus", "scaling",
                                                      "e2e", "peak_hbm_gb", "final_loss")}
                also["c5_model"]["config"] = m["config"]
                line["also"] = also
        if rank == 0:
            print(json.dumps(line))
    finally:
        if dist is not None:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
