"""CPU oracle for the NSA attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 torch on the CPU, the algorithm of the
reference's pure-torch NSA path.  It exists so that the CUDA kernels can be
checked against it; nothing in the shipped package imports it.  Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  Every function below is checked (tests/test_oracle.py)
against golden input/output vectors that were produced by importing the
reference's own functions (tests/golden/make_golden.py holds the generator).

Two families of functions live here:

* ``ref_*``  - dense O(T^2) restatements that follow the reference line by
  line (score matrix, boolean keep mask, finite-min fill, softmax, zeroing of
  fully masked rows).  They are differentiable torch code, so autograd gives
  the reference's backward.  They are what the CPU baseline times.
* ``stream_*`` - row-chunked restatements with an analytic backward, for shapes
  whose dense score matrix does not fit in host memory.  They are validated
  against the ``ref_*`` family at small sizes.

Reference citations are ``file:line`` inside the reference project.
"""

from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import numpy as np
import torch

MODE_WINDOW = 0      # nsa_fused_kernel.py:46
MODE_COMPRESS = 1    # nsa_fused_kernel.py:47
LSE_EMPTY = -1.0e9   # nsa_selection_kernel.py:134,171  (finite sentinel of empty rows)


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------
def _masked_softmax(scores: torch.Tensor, keep: torch.Tensor) -> torch.Tensor:
    """nsa_model.py:70-82 - finite-min fill, softmax, zero fully masked rows."""
    neg = torch.finfo(scores.dtype).min
    scores = scores.masked_fill(~keep, neg)
    attn = torch.softmax(scores, dim=-1)
    return attn * keep.any(dim=-1, keepdim=True)


def _expand_kv(x: torch.Tensor, group: int) -> torch.Tensor:
    """nsa_model.py:85-93 - query head h reads kv head h // group."""
    return x.repeat_interleave(group, dim=1)


# ---------------------------------------------------------------------------
# keep masks of the three branches
# ---------------------------------------------------------------------------
def window_keep(t0: int, t1: int, Lk: int, window: int) -> torch.Tensor:
    """[t1-t0, Lk] bool: key j visible to query t iff j <= t and t - j < window
    (nsa_fused_kernel.py:588-589, nsa_model.py:288-290)."""
    tt = torch.arange(t0, t1)[:, None]
    jj = torch.arange(Lk)[None, :]
    return (jj <= tt) & (tt - jj < window)


def compress_keep(t0: int, t1: int, Lk: int, block_size: int, stride: int = None) -> torch.Tensor:
    """[t1-t0, Lk] bool: summary j visible iff its last token (j+1)*Bsz-1 <= t
    (nsa_fused_kernel.py:590-592, nsa_model.py:233-235).  With a stride (summaries of length
    block_size every `stride` tokens, not in the reference): last token j*stride+Bsz-1 <= t."""
    stride = block_size if stride is None else stride
    tt = torch.arange(t0, t1)[:, None]
    jj = torch.arange(Lk)[None, :]
    return (jj * stride + block_size - 1) <= tt


def n_summaries(T: int, cmp_len: int, cmp_stride: int) -> int:
    """Number of complete summary windows [j*stride, j*stride+len) inside T tokens."""
    return (T - cmp_len) // cmp_stride + 1 if T >= cmp_len else 0


def selection_keep(block_idx: torch.Tensor, t0: int, t1: int, T: int,
                   block_size: int, clamp_tail: bool = False) -> torch.Tensor:
    """[B,Hkv,t1-t0,T] bool keep mask of the selection branch for query rows
    t0..t1 (nsa_selection_kernel.py:73-84): token j is kept for query i iff
    block(j) is listed for i (slots < 0 are padding) and j <= i.

    When T is not a multiple of block_size the reference's dense function and its
    kernels disagree about the tail tokens: the dense one assigns them to block
    n_blk-1 (the clamp at nsa_selection_kernel.py:78), the kernels attend exactly
    pos = blk*block_size+n < T (nsa_selection_kernel.py:142-144).  clamp_tail=True
    gives the former, the default gives the kernels' rule, which is the one the
    drop-in must keep.  The reference's gates only use T % block_size == 0, where
    the two coincide."""
    B, Hkv, _, S = block_idx.shape
    n_blk = T // block_size if clamp_tail else -(-T // block_size)
    idx = block_idx[:, :, t0:t1].long()
    valid = (idx >= 0) & (idx < max(n_blk, 1))
    oh = torch.zeros(B, Hkv, t1 - t0, S, max(n_blk, 1), dtype=torch.bool)
    oh.scatter_(-1, idx.clamp(min=0).unsqueeze(-1), valid.unsqueeze(-1))
    chosen = oh.any(dim=3)                                   # [B,Hkv,rows,n_blk]
    blk_of_tok = (torch.arange(T) // block_size).clamp(max=max(n_blk - 1, 0))
    keep = chosen[..., blk_of_tok]                           # [B,Hkv,rows,T]
    causal = torch.arange(T)[None, :] <= torch.arange(t0, t1)[:, None]
    return keep & causal[None, None]



# ---------------------------------------------------------------------------
# ref_* : dense, differentiable, line-by-line restatements
# ---------------------------------------------------------------------------
def ref_selection_forward(q, k, v, block_idx, block_size):
    """nsa_selection_kernel.py:55-92 (selection_forward_reference)."""
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    scale = D ** -0.5
    kexp = _expand_kv(k.float(), G)
    vexp = _expand_kv(v.float(), G)
    s = torch.matmul(q.float(), kexp.transpose(-1, -2)) * scale
    keep = selection_keep(block_idx, 0, T, T, block_size, clamp_tail=True).repeat_interleave(G, dim=1)
    s = s.masked_fill(~keep, torch.finfo(s.dtype).min)
    row_has = keep.any(dim=-1, keepdim=True)
    p = torch.softmax(s, dim=-1) * row_has
    return torch.matmul(p, vexp).to(q.dtype)


def ref_range_attn(q, k, v, mode, window, block_size):
    """nsa_fused_kernel.py:576-597 (_range_attn_reference)."""
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    Lk = k.shape[2]
    scale = D ** -0.5
    kexp = _expand_kv(k.float(), G)
    vexp = _expand_kv(v.float(), G)
    s = torch.matmul(q.float(), kexp.transpose(-1, -2)) * scale
    if mode == MODE_WINDOW:
        keep = window_keep(0, T, Lk, window)
    else:
        keep = compress_keep(0, T, Lk, block_size)
    keep = keep[None, None].expand(B, Hq, T, Lk)
    s = s.masked_fill(~keep, torch.finfo(s.dtype).min)
    row_has = keep.any(dim=-1, keepdim=True)
    p = torch.softmax(s, dim=-1) * row_has
    return torch.matmul(p, vexp).to(q.dtype)


def ref_block_mean_pool(x, block_size):
    """nsa_fused_kernel.py:549-554 (block_mean_pool)."""
    B, H, T, D = x.shape
    n_blk = T // block_size
    x = x[:, :, :n_blk * block_size].reshape(B, H, n_blk, block_size, D)
    return x.mean(dim=3)


def _windows(x, block_size, stride):
    """[B,H,T,D] -> [B,H,n,block_size,D]: the complete windows of block_size tokens every
    `stride` tokens (a view of the blocks when stride == block_size)."""
    B, H, T, D = x.shape
    n = n_summaries(T, block_size, stride)
    if n == 0:
        return x.new_zeros(B, H, 0, block_size, D)
    return x.unfold(2, block_size, stride)[:, :, :n].permute(0, 1, 2, 4, 3)


def ref_block_compressor(x, intra_pos, pool_logits, proj_weight, block_size, stride=None):
    """nsa_model.py:118-123 (BlockCompressor.forward) applied to the block view
    of x [B,Hkv,T,D] taken at nsa_model.py:217-220: softmax-weighted sum over the
    positions of each block of (x + intra_pos), then a bias-free D x D linear.
    stride < block_size (overlapping windows) is not expressible in the reference."""
    xb = _windows(x, block_size, block_size if stride is None else stride)
    xb = xb + intra_pos
    w = torch.softmax(pool_logits, dim=0)
    pooled = (xb * w[:, None]).sum(dim=-2)
    return torch.matmul(pooled, proj_weight.t())


def ref_gate_combine(o_cmp, o_slc, o_win, gate_logits):
    """nsa_model.py:297-301 / nsa_fused_kernel.py:572-573."""
    g = torch.sigmoid(gate_logits)
    return g[..., 0:1] * o_cmp + g[..., 1:2] * o_slc + g[..., 2:3] * o_win


def ref_nsa_fused(q, kc, vc, ks, vs, kw, vw, gate_logits, block_idx, block_size, window):
    """nsa_fused_kernel.py:600-609 (nsa_fused_reference)."""
    k_cmp = ref_block_mean_pool(kc, block_size)
    v_cmp = ref_block_mean_pool(vc, block_size)
    o_cmp = ref_range_attn(q, k_cmp, v_cmp, MODE_COMPRESS, 0, block_size)
    o_slc = ref_selection_forward(q, ks, vs, block_idx, block_size)
    o_win = ref_range_attn(q, kw, vw, MODE_WINDOW, window, 0)
    return ref_gate_combine(o_cmp, o_slc, o_win, gate_logits)


def ref_importance(q, k_cmp, block_size):
    """nsa_model.py:343-353: group-summed compression probabilities
    imp[B,Hkv,T,n_blk] (fp32) and the causal validity mask [T,n_blk]."""
    B, Hq, T, D = q.shape
    Hkv, n_blk = k_cmp.shape[1], k_cmp.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5
    s = torch.matmul(q.float(), _expand_kv(k_cmp.float(), G).transpose(-1, -2)) * scale
    valid = compress_keep(0, T, n_blk, block_size)
    p = _masked_softmax(s, valid[None, None].expand(B, Hq, T, n_blk))
    imp = p.view(B, Hkv, G, T, n_blk).sum(dim=2)
    return imp, valid


def ref_topk_blocks(q, k_cmp, block_size, n_sel):
    """nsa_model.py:343-355 exactly: torch.topk over importance with non-causal
    blocks filled with finfo.min.  Slots beyond the number of causally valid
    blocks hold whatever torch.topk returns among the masked entries."""
    imp, valid = ref_importance(q, k_cmp, block_size)
    imp = imp.masked_fill(~valid[None, None], torch.finfo(imp.dtype).min)
    k_top = min(n_sel, k_cmp.shape[2])
    return torch.topk(imp, k_top, dim=-1).indices.to(torch.int32)


def canonical_topn(imp: torch.Tensor, valid: torch.Tensor, n_sel: int) -> torch.Tensor:
    """Deterministic form of the reference's pick (nsa_model.py:352-355): the
    n_sel causally valid blocks of largest importance, ordered by (importance
    descending, block index ascending); slots with no valid block hold -1.
    On rows with at least n_sel valid blocks and no exact ties this is the same
    set torch.topk returns."""
    B, Hkv, T, n_blk = imp.shape
    k_top = min(n_sel, n_blk)
    if n_blk == 0:
        return torch.full((B, Hkv, T, n_sel), -1, dtype=torch.int32)
    key = imp.masked_fill(~valid[None, None], -1.0)      # probabilities are >= 0
    # stable sort of -key keeps the lower index first among equal values
    order = torch.sort(-key, dim=-1, stable=True).indices[..., :k_top]
    picked_valid = torch.gather(valid[None, None].expand(B, Hkv, T, n_blk), -1, order)
    out = torch.where(picked_valid, order, torch.full_like(order, -1)).to(torch.int32)
    if k_top < n_sel:
        pad = torch.full((B, Hkv, T, n_sel - k_top), -1, dtype=torch.int32)
        out = torch.cat([out, pad], dim=-1)
    return out


FORCED_INIT_KEY = float(1 << 20)     # rank keys of forced blocks: above every importance (<= G)
FORCED_LOCAL_KEY = float(1 << 19)


def forced_topn(imp: torch.Tensor, valid: torch.Tensor, n_sel: int, T: int, block_size: int,
                n_init: int, n_local: int) -> torch.Tensor:
    """canonical_topn with forced blocks, the selection rule of the published NSA recipe
    ("always the initial block and the local blocks").  PARITY UNPINNED: the reference's
    scorer has no forced blocks (nsa_model.py:257-258 is a plain topk), so nothing of the
    reference checks this function; with n_init = n_local = 0 it equals canonical_topn,
    which is pinned.  For query t with cur = t // block_size the list holds, in this order:
    blocks j < n_init (j <= cur) ascending; blocks cur, cur-1, ... (n_local of them) not
    already listed; then causally complete blocks by (importance descending, index
    ascending); -1 in unused slots."""
    B, Hkv, _, n_blk = imp.shape
    n_all = (T + block_size - 1) // block_size
    key = torch.full((B, Hkv, T, n_all), -1.0)
    if n_blk:
        key[..., :n_blk] = imp.masked_fill(~valid[None, None], -1.0)
    cur = (torch.arange(T) // block_size)[:, None]
    j = torch.arange(n_all)[None, :]
    is_init = (j < n_init) & (j <= cur)
    is_local = (j <= cur) & (j > cur - n_local) & ~is_init
    key = torch.where(is_init[None, None], FORCED_INIT_KEY - j.float(), key)
    key = torch.where(is_local[None, None], FORCED_LOCAL_KEY - (cur - j).float(), key)
    k_top = min(n_sel, n_all)
    order = torch.sort(-key, dim=-1, stable=True).indices[..., :k_top]
    picked = torch.gather(key, -1, order)
    out = torch.where(picked >= 0, order, torch.full_like(order, -1)).to(torch.int32)
    if k_top < n_sel:
        out = torch.cat([out, torch.full((B, Hkv, T, n_sel - k_top), -1, dtype=torch.int32)], dim=-1)
    return out


def build_block_to_query_csr(block_idx, block_size):
    """nsa_fsa.py:14-64.  Pairs (query i, block j) with j >= 0 and j*Bsz <= i,
    grouped by (b, hkv, j), queries ascending inside a group.  Returns int32
    numpy arrays q_of_block[P], block_offsets[B,Hkv,n_blk+1], pair_bh[P]."""
    idx = np.asarray(block_idx.cpu() if isinstance(block_idx, torch.Tensor) else block_idx,
                     dtype=np.int64)
    B, Hkv, T, S = idx.shape
    n_blk = T // block_size
    qpos = np.arange(T).reshape(1, 1, T, 1)
    valid = (idx >= 0) & (idx * block_size <= qpos)
    bh, ti, si = np.nonzero(valid.reshape(B * Hkv, T, S))
    jj = idx.reshape(B * Hkv, T, S)[bh, ti, si]
    key = bh * n_blk + jj
    order = np.argsort(key, kind="stable")           # row-major nonzero => query ascending
    counts = np.bincount(key, minlength=B * Hkv * n_blk)
    off = np.zeros(B * Hkv * n_blk + 1, dtype=np.int64)
    off[1:] = np.cumsum(counts)
    rows = (np.arange(B * Hkv)[:, None] * n_blk + np.arange(n_blk + 1)[None, :])
    block_offsets = off[rows].reshape(B, Hkv, n_blk + 1).astype(np.int32)
    return ti[order].astype(np.int32), block_offsets, bh[order].astype(np.int32)


# ---------------------------------------------------------------------------
# stream_* : row-chunked forward with LSE and analytic backward
# ---------------------------------------------------------------------------
KeepFn = Callable[[int, int], torch.Tensor]   # rows t0..t1 -> bool [rows,Lk] or [B,Hkv,rows,Lk]


def _keep_for(keep_fn: KeepFn, t0, t1, B, Hkv, G, Lk):
    keep = keep_fn(t0, t1)
    if keep.dim() == 2:
        keep = keep[None, None].expand(B, Hkv, t1 - t0, Lk)
    return keep[:, :, None].expand(B, Hkv, G, t1 - t0, Lk)       # [B,Hkv,G,rows,Lk]


def stream_attn_forward(q, k, v, keep_fn: KeepFn, chunk: int = 512):
    """Masked softmax attention computed in chunks of query rows.

    q [B,Hq,T,D]; k,v [B,Hkv,Lk,D] (any float dtype; arithmetic in fp32).
    Returns o [B,Hq,T,D] fp32 and lse [B,Hq,T] fp32 (natural log of the softmax
    denominator plus the row maximum; LSE_EMPTY on rows with nothing kept, whose
    output is 0 - nsa_selection_kernel.py:165-171)."""
    B, Hq, T, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5
    qf = q.float().view(B, Hkv, G, T, D)
    kf, vf = k.float(), v.float()
    o = torch.zeros(B, Hkv, G, T, D)
    lse = torch.full((B, Hkv, G, T), LSE_EMPTY)
    for t0 in range(0, T if Lk > 0 else 0, chunk):
        t1 = min(T, t0 + chunk)
        keep = _keep_for(keep_fn, t0, t1, B, Hkv, G, Lk)
        s = torch.einsum("bhgtd,bhjd->bhgtj", qf[:, :, :, t0:t1], kf) * scale
        s = s.masked_fill(~keep, -float("inf"))
        m = s.max(dim=-1, keepdim=True).values
        has = keep.any(dim=-1, keepdim=True)
        m = torch.where(has, m, torch.zeros_like(m))
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        l_safe = torch.where(has, l, torch.ones_like(l))
        o[:, :, :, t0:t1] = torch.einsum("bhgtj,bhjd->bhgtd", p / l_safe, vf)
        lse[:, :, :, t0:t1] = torch.where(has, m + torch.log(l_safe),
                                          torch.full_like(m, LSE_EMPTY)).squeeze(-1)
    return o.view(B, Hq, T, D), lse.view(B, Hq, T)


def stream_attn_backward(q, k, v, o, lse, do, keep_fn: KeepFn, chunk: int = 512):
    """Analytic backward of stream_attn_forward (nsa_selection_backward.py:12-20):
    delta = sum_d dO*O; p = exp(s - lse); dP = dO V^T; dS = p (dP - delta);
    dQ = scale dS K; dK = scale dS^T Q; dV = p^T dO.  All fp32."""
    B, Hq, T, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5
    qf = q.float().view(B, Hkv, G, T, D)
    dof = do.float().view(B, Hkv, G, T, D)
    of = o.float().view(B, Hkv, G, T, D)
    lsef = lse.float().view(B, Hkv, G, T)
    kf, vf = k.float(), v.float()
    dq = torch.zeros(B, Hkv, G, T, D)
    dk = torch.zeros(B, Hkv, Lk, D)
    dv = torch.zeros(B, Hkv, Lk, D)
    for t0 in range(0, T if Lk > 0 else 0, chunk):
        t1 = min(T, t0 + chunk)
        keep = _keep_for(keep_fn, t0, t1, B, Hkv, G, Lk)
        s = torch.einsum("bhgtd,bhjd->bhgtj", qf[:, :, :, t0:t1], kf) * scale
        p = torch.exp(s - lsef[:, :, :, t0:t1, None])
        p = torch.where(keep, p, torch.zeros_like(p))
        delta = (dof[:, :, :, t0:t1] * of[:, :, :, t0:t1]).sum(-1, keepdim=True)
        dp = torch.einsum("bhgtd,bhjd->bhgtj", dof[:, :, :, t0:t1], vf)
        ds = p * (dp - delta)
        dq[:, :, :, t0:t1] = torch.einsum("bhgtj,bhjd->bhgtd", ds, kf) * scale
        dk += torch.einsum("bhgtj,bhgtd->bhjd", ds, qf[:, :, :, t0:t1]) * scale
        dv += torch.einsum("bhgtj,bhgtd->bhjd", p, dof[:, :, :, t0:t1])
    return dq.view(B, Hq, T, D), dk, dv


def window_keep_fn(Lk, window) -> KeepFn:
    return lambda t0, t1: window_keep(t0, t1, Lk, window)


def compress_keep_fn(Lk, block_size, stride=None) -> KeepFn:
    return lambda t0, t1: compress_keep(t0, t1, Lk, block_size, stride)


def selection_keep_fn(block_idx, T, block_size) -> KeepFn:
    return lambda t0, t1: selection_keep(block_idx, t0, t1, T, block_size)


def stream_importance(q, k_cmp, block_size, chunk: int = 512, stride=None):
    """Row-chunked form of ref_importance: imp [B,Hkv,T,n_blk] fp32, valid [T,n_blk]."""
    B, Hq, T, D = q.shape
    Hkv, n_blk = k_cmp.shape[1], k_cmp.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5
    qf = q.float().view(B, Hkv, G, T, D)
    kf = k_cmp.float()
    imp = torch.zeros(B, Hkv, T, n_blk)
    for t0 in range(0, T if n_blk > 0 else 0, chunk):
        t1 = min(T, t0 + chunk)
        keep = compress_keep(t0, t1, n_blk, block_size, stride)[None, None, None].expand(
            B, Hkv, G, t1 - t0, n_blk)
        s = torch.einsum("bhgtd,bhjd->bhgtj", qf[:, :, :, t0:t1], kf) * scale
        imp[:, :, t0:t1] = _masked_softmax(s, keep).sum(dim=2)
    return imp, compress_keep(0, T, n_blk, block_size, stride)


def block_importance(imp_cmp, T, cmp_len, cmp_stride, sel_block):
    """Importance of selection blocks from the importance of summaries when the summary grid
    (length cmp_len every cmp_stride tokens) differs from the selection grid (sel_block
    tokens): a block takes the sum over the summaries that overlap it, and is a candidate
    for query t as soon as the first of them is visible.  PARITY UNPINNED (the reference
    only has cmp_len = cmp_stride = sel_block, where this is the identity on the complete
    blocks).  cmp_len and sel_block must be multiples of cmp_stride.
    Returns (imp_blk [B,Hkv,T,n_sblk], valid [T,n_sblk]) with n_sblk = ceil(T / sel_block)."""
    assert cmp_len % cmp_stride == 0 and sel_block % cmp_stride == 0
    B, Hkv, _, n_cmp = imp_cmp.shape
    r, o = sel_block // cmp_stride, cmp_len // cmp_stride
    n_sblk = (T + sel_block - 1) // sel_block
    imp_blk = torch.zeros(B, Hkv, T, n_sblk)
    valid = torch.zeros(T, n_sblk, dtype=torch.bool)
    tt = torch.arange(T)
    for b in range(n_sblk):
        j0, j1 = max(0, r * b - o + 1), min(n_cmp - 1, r * b + r - 1)
        if j0 > j1:
            continue
        imp_blk[..., b] = imp_cmp[..., j0:j1 + 1].sum(-1)
        valid[:, b] = tt >= j0 * cmp_stride + cmp_len - 1
    return imp_blk, valid


# ---------------------------------------------------------------------------
# pooling / gate backward (analytic, fp32)
# ---------------------------------------------------------------------------
def mean_pool_backward(d_pooled, T, block_size):
    """Backward of ref_block_mean_pool: every token of a complete block receives
    d_pooled / block_size; tokens past the last complete block receive 0."""
    B, H, n_blk, D = d_pooled.shape
    dx = torch.zeros(B, H, T, D)
    dx[:, :, :n_blk * block_size] = (d_pooled.float()[:, :, :, None, :] / block_size).expand(
        B, H, n_blk, block_size, D).reshape(B, H, n_blk * block_size, D)
    return dx


def compressor_backward(x, intra_pos, pool_logits, proj_weight, block_size, d_out, stride=None):
    """Analytic backward of ref_block_compressor.  Returns
    (dx [B,H,T,D], d_intra_pos [Bsz,D], d_pool_logits [Bsz], d_proj_weight [D,D])."""
    B, H, T, D = x.shape
    stride = block_size if stride is None else stride
    n_blk = n_summaries(T, block_size, stride)
    xb = _windows(x.float(), block_size, stride) + intra_pos.float()
    w = torch.softmax(pool_logits.float(), dim=0)
    pooled = (xb * w[:, None]).sum(dim=-2)                         # [B,H,n,D]
    d_out = d_out.float()
    d_proj = torch.einsum("bhno,bhni->oi", d_out, pooled)          # out = pooled @ W^T
    d_pooled = torch.matmul(d_out, proj_weight.float())            # [B,H,n,D]
    d_xb = d_pooled[:, :, :, None, :] * w[None, None, None, :, None]
    d_intra = d_xb.sum(dim=(0, 1, 2))
    d_w = (d_pooled[:, :, :, None, :] * xb).sum(dim=(0, 1, 2, 4))  # [Bsz]
    d_logits = w * (d_w - (d_w * w).sum())
    dx = torch.zeros(B, H, T, D)
    for r in range(block_size if n_blk else 0):     # position r of window j is token j*stride + r
        dx[:, :, r:r + (n_blk - 1) * stride + 1:stride] += d_xb[:, :, :, r]
    return dx, d_intra, d_logits, d_proj


def gate_combine_backward(o_cmp, o_slc, o_win, gate_logits, d_out):
    """Backward of ref_gate_combine.  Returns (do_cmp, do_slc, do_win, d_gate_logits)."""
    g = torch.sigmoid(gate_logits.float())
    d_out = d_out.float()
    outs = (o_cmp.float(), o_slc.float(), o_win.float())
    d_branches = tuple(g[..., i:i + 1] * d_out for i in range(3))
    d_g = torch.stack([(d_out * outs[i]).sum(-1) for i in range(3)], dim=-1)
    d_logits = d_g * g * (1.0 - g)
    return d_branches + (d_logits,)


# ---------------------------------------------------------------------------
# the whole op (pooling -> compression -> top-n -> selection -> window -> gate)
# ---------------------------------------------------------------------------
def stream_nsa_forward(q, kc, vc, ks, vs, kw, vw, gate_logits, block_size, n_sel, window,
                       block_idx=None, compressor=None, chunk: int = 512, cmp_len=None,
                       cmp_stride=None, n_init=0, n_local=0):
    """Forward of the full op in fp32.  `compressor` is None for mean pooling
    (nsa_fused_kernel.py:560-573) or a dict with keys k_intra,k_logits,k_proj,
    v_intra,v_logits,v_proj for the learned pooling of the model
    (nsa_model.py:336-337).  When block_idx is None it is chosen by
    canonical_topn over the compression probabilities (nsa_model.py:343-355).
    Returns a dict with out, the three branch outputs and LSEs, k_cmp, v_cmp,
    block_idx and (when computed) importance.
    cmp_len / cmp_stride (default block_size: the reference's geometry) give summaries of
    cmp_len tokens every cmp_stride tokens, selection blocks staying block_size tokens;
    n_init / n_local force blocks into every list (see forced_topn).  Both generalisations
    are parity-unpinned restatements of the published NSA recipe."""
    T = q.shape[2]
    cl = block_size if cmp_len is None else cmp_len
    cs = cl if cmp_stride is None else cmp_stride
    general = (cl, cs) != (block_size, block_size)
    if compressor is None:
        assert not general, "mean pooling is defined on the aligned grid only"
        k_cmp = ref_block_mean_pool(kc.float(), block_size)
        v_cmp = ref_block_mean_pool(vc.float(), block_size)
    else:
        k_cmp = ref_block_compressor(kc.float(), compressor["k_intra"].float(),
                                     compressor["k_logits"].float(),
                                     compressor["k_proj"].float(), cl, cs)
        v_cmp = ref_block_compressor(vc.float(), compressor["v_intra"].float(),
                                     compressor["v_logits"].float(),
                                     compressor["v_proj"].float(), cl, cs)
    n_blk = k_cmp.shape[2]
    res = {"k_cmp": k_cmp, "v_cmp": v_cmp}
    o_cmp, lse_cmp = stream_attn_forward(q, k_cmp, v_cmp, compress_keep_fn(n_blk, cl, cs), chunk)
    if block_idx is None:
        imp, valid = stream_importance(q, k_cmp, cl, chunk, cs)
        if general:
            imp, valid = block_importance(imp, T, cl, cs, block_size)
        if general or n_init or n_local:
            block_idx = forced_topn(imp, valid, n_sel, T, block_size, n_init, n_local)
        else:
            block_idx = canonical_topn(imp, valid, n_sel)
        res["importance"] = imp
    o_slc, lse_slc = stream_attn_forward(q, ks, vs, selection_keep_fn(block_idx, T, block_size), chunk)
    o_win, lse_win = stream_attn_forward(q, kw, vw, window_keep_fn(T, window), chunk)
    res.update(out=ref_gate_combine(o_cmp, o_slc, o_win, gate_logits.float()),
               o_cmp=o_cmp, o_slc=o_slc, o_win=o_win, lse_cmp=lse_cmp, lse_slc=lse_slc,
               lse_win=lse_win, block_idx=block_idx)
    return res


def stream_nsa_backward(q, kc, vc, ks, vs, kw, vw, gate_logits, block_size, window, fwd, d_out,
                        compressor=None, chunk: int = 512, cmp_len=None, cmp_stride=None):
    """Analytic backward of stream_nsa_forward given its result dict `fwd`.
    Returns a dict of gradients: q, kc, vc, ks, vs, kw, vw, gate and, for the
    learned compressor, k_intra,k_logits,k_proj,v_intra,v_logits,v_proj."""
    T = q.shape[2]
    cl = block_size if cmp_len is None else cmp_len
    cs = cl if cmp_stride is None else cmp_stride
    n_blk = fwd["k_cmp"].shape[2]
    do_cmp, do_slc, do_win, d_gate = gate_combine_backward(
        fwd["o_cmp"], fwd["o_slc"], fwd["o_win"], gate_logits, d_out)
    dq1, dk_cmp, dv_cmp = stream_attn_backward(q, fwd["k_cmp"], fwd["v_cmp"], fwd["o_cmp"],
                                               fwd["lse_cmp"], do_cmp,
                                               compress_keep_fn(n_blk, cl, cs), chunk)
    dq2, dks, dvs = stream_attn_backward(q, ks, vs, fwd["o_slc"], fwd["lse_slc"], do_slc,
                                         selection_keep_fn(fwd["block_idx"], T, block_size), chunk)
    dq3, dkw, dvw = stream_attn_backward(q, kw, vw, fwd["o_win"], fwd["lse_win"], do_win,
                                         window_keep_fn(T, window), chunk)
    g = {"q": dq1 + dq2 + dq3, "ks": dks, "vs": dvs, "kw": dkw, "vw": dvw, "gate": d_gate}
    if compressor is None:
        g["kc"] = mean_pool_backward(dk_cmp, T, block_size)
        g["vc"] = mean_pool_backward(dv_cmp, T, block_size)
    else:
        g["kc"], g["k_intra"], g["k_logits"], g["k_proj"] = compressor_backward(
            kc, compressor["k_intra"], compressor["k_logits"], compressor["k_proj"],
            cl, dk_cmp, cs)
        g["vc"], g["v_intra"], g["v_logits"], g["v_proj"] = compressor_backward(
            vc, compressor["v_intra"], compressor["v_logits"], compressor["v_proj"],
            cl, dv_cmp, cs)
    return g


# ---------------------------------------------------------------------------
# input generators used by the reference's own gates, restated
# ---------------------------------------------------------------------------
def make_block_idx(B, Hkv, T, block_size, S, seed=0):
    """test_kernel.py:39-58: random causally valid block lists, -1 padded."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blk = T // block_size
    valid = (torch.arange(n_blk)[None, :] + 1) * block_size <= (torch.arange(T)[:, None] + 1)
    score = torch.rand(B, Hkv, T, n_blk, generator=g).masked_fill(~valid[None, None], -1.0)
    k = min(S, n_blk)
    topv, topi = score.topk(k, dim=-1)
    sel = torch.where(topv >= 0, topi.to(torch.int32), torch.full_like(topi, -1, dtype=torch.int32))
    idx = torch.full((B, Hkv, T, S), -1, dtype=torch.int32)
    idx[..., :k] = sel
    return idx


def make_block_idx_recent(B, Hkv, T, block_size, S):
    """bench_kernel.py:43-53: the S most recent complete blocks, -1 padded."""
    n_valid = (torch.arange(T) + 1) // block_size
    blk = (n_valid[:, None] - 1) - torch.arange(S)[None, :]
    blk = torch.where(blk >= 0, blk, torch.full_like(blk, -1))
    return blk[None, None].expand(B, Hkv, T, S).contiguous().to(torch.int32)


def make_block_idx_forced(B, Hkv, T, block_size, S, n_init=1, n_local=2, seed=0):
    """Block lists of the published NSA recipe's shape: the first n_init blocks and the n_local
    most recent blocks (the one holding t and the ones before it) in every query's list, the
    remaining slots random causally valid blocks; no duplicates, -1 padded.  Not a reference
    generator (the reference has no forced blocks): it makes block 0 a block that every
    query lists, the case the work-list split of the block-outer kernels exists for."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blk = (T + block_size - 1) // block_size
    t = torch.arange(T)
    cur = t // block_size
    j = torch.arange(n_blk)
    score = torch.rand(B, Hkv, T, n_blk, generator=g)
    forced = (j[None, :] < n_init) | ((j[None, :] <= cur[:, None]) & (j[None, :] > cur[:, None] - n_local))
    valid = j[None, :] <= cur[:, None]
    score = torch.where(forced[None, None], score + 2.0, score)
    score = score.masked_fill(~valid[None, None], -1.0)
    k = min(S, n_blk)
    topv, topi = score.topk(k, dim=-1)
    sel = torch.where(topv >= 0, topi.to(torch.int32), torch.full_like(topi, -1, dtype=torch.int32))
    idx = torch.full((B, Hkv, T, S), -1, dtype=torch.int32)
    idx[..., :k] = sel
    return idx


def attended_keys(block_idx, T, block_size, window, n_cmp_keys=None):
    """Exact count of (query, key) pairs each branch attends, per kv head summed
    over batch: used for the algorithmic FLOP figure 4*D*N (forward) and
    14*D*N (forward+backward) per query head."""
    t = torch.arange(T)
    n_blk = T // block_size if n_cmp_keys is None else n_cmp_keys
    n_cmp = torch.clamp((t + 1) // block_size, max=n_blk).sum().item()
    n_win = torch.clamp(t + 1, max=window).sum().item()
    idx = block_idx.long()
    start = idx * block_size
    end = torch.minimum(start + block_size - 1, t.view(1, 1, T, 1).expand_as(idx))
    cnt = torch.where((idx >= 0) & (start <= t.view(1, 1, T, 1)), end - start + 1,
                      torch.zeros_like(idx))
    return {"cmp": n_cmp * block_idx.shape[0] * block_idx.shape[1],
            "win": n_win * block_idx.shape[0] * block_idx.shape[1],
            "slc": int(cnt.sum().item())}
