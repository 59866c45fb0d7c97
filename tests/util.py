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


def check(a, b, dtype, what, abs32=2e-3, abs16=2e-2, rel16=1e-2, scale_abs=True):
    """fp32: max-abs <= abs32 (the reference's fp32 gates are 2e-3..4e-3).
    bf16: max-abs <= abs16 * max(1, max|b|) and relative L2 <= rel16 against the fp32 oracle."""
    ma, rl = err(a, b)
    assert not torch.isnan(a.float()).any(), what + ": NaN"
    if dtype == torch.float32:
        assert ma <= abs32, f"{what}: max-abs {ma:.3e} > {abs32}"
    else:
        mag = max(1.0, b.abs().max().item()) if scale_abs else 1.0
        assert ma <= abs16 * mag, f"{what}: max-abs {ma:.3e} > {abs16 * mag:.3e}"
        assert rl <= rel16, f"{what}: rel-L2 {rl:.3e} > {rel16}"


def load_golden(name):
    z = np.load(os.path.join(GOLD, name))
    return {k: torch.from_numpy(z[k]) for k in z.files}
