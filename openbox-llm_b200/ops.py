"""Host side of the NSA attention path: the reference's operator interface on top of the
C-ABI library.

Names, argument meaning and error behaviour follow the reference modules they replace:
  selection_forward_triton, selection_forward_reference   nsa_selection_kernel.py:55-213
  selection_backward_triton, SelectionAttnTriton,
  selection_attn_triton                                    nsa_selection_backward.py:156-369
  build_block_to_query_csr                                 nsa_fsa.py:14-64
  _RangeAttn, window_attn_triton, compression_attn_triton,
  block_mean_pool, nsa_fused_forward                       nsa_fused_kernel.py:521-573
`nsa_attention` is the one addition: the whole op (pooling, compression attention, block
scoring + top-n, selection, window, gate) behind one autograd.Function.
"""
import torch

from . import _lib as L

MODE_WINDOW = L.MODE_WINDOW
MODE_COMPRESS = L.MODE_COMPRESS
MODE_COMPRESS_STRIDED = L.MODE_COMPRESS_STRIDED

_impl = "auto"
_dq_accumulator = False


def set_impl(name: str):
    """Choose the kernel family: 'auto' (tcgen05 where the shape fits), 'simt' or 'tc'."""
    global _impl
    assert name in L.IMPL
    _impl = name


def get_impl() -> str:
    return _impl


def set_dq_accumulator(on: bool):
    """Whole-op backward on tcgen05 shapes.  False (default): every branch keeps bf16 dQ partials
    (one slot per key tile a query attends) and one kernel adds them in a fixed order: dq is
    bit-reproducible, at the price of the partial buffers.  True: the window and compression
    branches add their dQ tiles into one fp32 accumulator by TMA reduce-add instead: no partial
    buffers for them (23 GB less at B=8, T=32K; the way to run compression strides that would need
    dozens of slots), but the L2 reduction rate bounds those kernels (they run about 1.7 times
    longer) and the order of the adds, hence the last bits of dq, varies from run to run."""
    global _dq_accumulator
    _dq_accumulator = bool(on)


def get_dq_accumulator() -> bool:
    return _dq_accumulator


def set_option(name: str, value: int):
    """Library tuning switch (see nsa_set_option in include/nsa_b200.h)."""
    L.check(L.lib().nsa_set_option(name.encode(), int(value)))


def tc_supported(B, Hq, Hkv, T, D, dtype, block_size=64) -> bool:
    code = L.DTYPE_BF16 if dtype == torch.bfloat16 else L.DTYPE_F32
    return bool(L.lib().nsa_tc_supported(L.dims(B, Hq, Hkv, T, D, code), block_size))


def _check_qkv(q, k, v):
    B, Hq, T, D = q.shape
    assert k.shape == v.shape and k.shape[0] == B and k.shape[3] == D
    assert Hq % k.shape[1] == 0, "GQA needs Hq divisible by Hkv"
    assert D in (16, 32, 64, 128), "head dim must be a power of two <= 128"
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert q.dtype == k.dtype == v.dtype
    return B, Hq, k.shape[1], T, D


# ---------------------------------------------------------------------------------------
# raw launch wrappers
# ---------------------------------------------------------------------------------------
@L.on_device
def range_attn_forward(q, k, v, mode, window, block_size, out=None):
    """o, lse of the window (mode 0) or compression (mode 1) branch.  `out` = (o, lse) makes the
    kernel write into existing contiguous tensors (the whole op keeps its three branches' outputs
    and statistics in one tensor each)."""
    B, Hq, Hkv, T, D = _check_qkv(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o, lse = out if out is not None else (
        torch.empty_like(q), torch.empty(B, Hq, T, device=q.device, dtype=torch.float32))
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    L.check(L.lib().nsa_range_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse), d,
                                       k.shape[2], mode, int(window), int(block_size),
                                       L.IMPL[_impl], L.stream()))
    return o, lse


@L.on_device
def range_attn_backward(q, k, v, o, lse, do, mode, window, block_size, row_scale=None, row_dot=None,
                        defer_dq=False):
    """dq, dk, dv of a range branch.  With row_scale / row_dot (see nsa_gate_combine_bwd_rows) `do`
    is the whole op's upstream gradient and the gate factor is applied inside the kernel.
    defer_dq (tcgen05 shapes only): returns (workspace, dk, dv), the dQ partials staying in the
    workspace for nsa_dq_reduce3."""
    B, Hq, Hkv, T, D = _check_qkv(q, k, v)
    q, k, v, o, do = (t.contiguous() for t in (q, k, v, o, do))
    dq = None if defer_dq else torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    nws = L.lib().nsa_range_attn_bwd_workspace_bytes(d, k.shape[2], mode, int(window), L.IMPL[_impl])
    ws = L.workspace(nws, q.device)
    L.check(L.lib().nsa_range_attn_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse),
                                       L.ptr(do), L.ptr(dq), L.ptr(dk), L.ptr(dv), d, k.shape[2],
                                       mode, int(window), int(block_size), L.ptr(row_scale),
                                       L.ptr(row_dot), L.ptr(ws), nws, L.IMPL[_impl], L.stream()))
    return (ws if defer_dq else dq), dk, dv


@L.on_device
def range_attn_backward_acc(q, k, v, o, lse, do, mode, window, block_size, row_scale, row_dot, dq_acc):
    """dk, dv of a gated range branch on a tcgen05 shape; its dQ is added to dq_acc
    [B*Hkv, T, G, D] float32 (see nsa_range_attn_bwd_acc)."""
    B, Hq, Hkv, T, D = _check_qkv(q, k, v)
    q, k, v, do = (t.contiguous() for t in (q, k, v, do))
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    nws = L.lib().nsa_range_attn_bwd_acc_workspace_bytes(d, k.shape[2], mode, int(window))
    ws = L.workspace(nws, q.device)
    L.check(L.lib().nsa_range_attn_bwd_acc(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse), L.ptr(do),
                                           L.ptr(dq_acc), L.ptr(dk), L.ptr(dv), d, k.shape[2], mode,
                                           int(window), int(block_size), L.ptr(row_scale),
                                           L.ptr(row_dot), L.ptr(ws), nws, L.stream()))
    return dk, dv


@L.on_device
def selection_plan(q, k, block_idx, block_size):
    """The index structures the tcgen05 selection kernels walk (CSR, pair map, work list), built
    once for a block list so that forward and backward need not each build them; None when the
    shape is not served by those kernels.  Opaque uint8 tensor."""
    B, Hq, T, D = q.shape
    S = block_idx.shape[-1]
    if _impl == "simt" or S == 0:
        return None
    d = L.dims(B, Hq, k.shape[1], T, D, L.dtype_code(q))
    n = L.lib().nsa_selection_plan_bytes(d, S, int(block_size))
    if n == 0:
        return None
    idx = block_idx.to(torch.int32).contiguous()
    plan = torch.empty(n, dtype=torch.uint8, device=q.device)
    L.check(L.lib().nsa_selection_plan_build(L.ptr(idx), d, S, int(block_size), L.ptr(plan), n, L.stream()))
    return plan


@L.on_device
def selection_forward_triton(q, k, v, block_idx, block_size, return_lse=False, out=None, plan=None):
    """nsa_selection_kernel.py:175-213.  q [B,Hq,T,D], k/v [B,Hkv,T,D], block_idx [B,Hkv,T,S].
    `out` = (o, lse): write into existing contiguous tensors; `plan`: see selection_plan (neither
    is in the reference's signature)."""
    B, Hq, Hkv, T, D = _check_qkv(q, k, v)
    S = block_idx.shape[-1]
    assert block_idx.shape[:3] == (B, Hkv, T)
    assert block_size >= 16, "block_size must be >= 16 (tl.dot inner dim)"
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    idx = block_idx.to(torch.int32).contiguous()
    o, lse = out if out is not None else (
        torch.empty_like(q), torch.empty(B, Hq, T, device=q.device, dtype=torch.float32))
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    nws = L.lib().nsa_selection_fwd_workspace_bytes(d, S, block_size, L.IMPL[_impl])
    ws = L.workspace(nws, q.device)
    if plan is not None:
        L.check(L.lib().nsa_selection_fwd_planned(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(idx), L.ptr(o),
                                                  L.ptr(lse), d, S, int(block_size), L.ptr(ws), nws,
                                                  L.ptr(plan), L.stream()))
    else:
        L.check(L.lib().nsa_selection_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(idx), L.ptr(o),
                                          L.ptr(lse), d, S, int(block_size), L.ptr(ws), nws,
                                          L.IMPL[_impl], L.stream()))
    return (o, lse) if return_lse else o


@L.on_device
def _selection_backward(q, k, v, block_idx, block_size, do, o, lse, row_scale=None, row_dot=None,
                        defer_dq=False, plan=None):
    B, Hq, Hkv, T, D = _check_qkv(q, k, v)
    S = block_idx.shape[-1]
    assert block_size >= 16
    q, k, v, o, do = (t.contiguous() for t in (q, k, v, o, do))
    idx = block_idx.to(torch.int32).contiguous()
    dq = None if defer_dq else torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    nws = L.lib().nsa_selection_bwd_workspace_bytes(d, S, block_size, L.IMPL[_impl])
    ws = L.workspace(nws, q.device)
    if plan is not None:
        L.check(L.lib().nsa_selection_bwd_planned(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(idx), L.ptr(o),
                                                  L.ptr(lse), L.ptr(do), L.ptr(dq), L.ptr(dk), L.ptr(dv), d, S,
                                                  int(block_size), L.ptr(row_scale), L.ptr(row_dot), L.ptr(ws),
                                                  nws, L.ptr(plan), L.stream()))
    else:
        L.check(L.lib().nsa_selection_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(idx), L.ptr(o),
                                          L.ptr(lse), L.ptr(do), L.ptr(dq), L.ptr(dk), L.ptr(dv), d, S,
                                          int(block_size), L.ptr(row_scale), L.ptr(row_dot), L.ptr(ws),
                                          nws, L.IMPL[_impl], L.stream()))
    return (ws if defer_dq else dq), dk, dv


def selection_backward_triton(q, k, v, block_idx, block_size, do, o):
    """nsa_selection_backward.py:156-189: dq, dk, dv from (q,k,v,block_idx,dO,O); the softmax
    statistics are recomputed by a forward pass because this signature carries no LSE."""
    _, lse = selection_forward_triton(q, k, v, block_idx, block_size, return_lse=True)
    return _selection_backward(q, k, v, block_idx, block_size, do, o, lse)


@torch.no_grad()
@L.on_device
def build_block_to_query_csr(block_idx, block_size):
    """nsa_fsa.py:14-64: (q_of_block [P], block_offsets [B,Hkv,n_blk+1], pair_bh [P]), int32."""
    B, Hkv, T, S = block_idx.shape
    idx = block_idx.to(torch.int32).contiguous()
    n_blk = T // block_size
    dev = idx.device
    cap = max(B * Hkv * T * S, 1)
    q_of_block = torch.empty(cap, dtype=torch.int32, device=dev)
    pair_bh = torch.empty(cap, dtype=torch.int32, device=dev)
    offsets = torch.zeros(B, Hkv, n_blk + 1, dtype=torch.int32, device=dev)
    nws = L.lib().nsa_csr_workspace_bytes(B, Hkv, T, S, block_size)
    ws = L.workspace(nws, dev)
    L.check(L.lib().nsa_build_block_to_query_csr(L.ptr(idx), B, Hkv, T, S, int(block_size),
                                                 L.ptr(q_of_block), L.ptr(offsets), L.ptr(pair_bh),
                                                 L.ptr(ws), nws, L.stream()))
    P = int(offsets.view(-1)[-1].item()) if offsets.numel() else 0
    return q_of_block[:P], offsets, pair_bh[:P]


def _pool_dims(x, block_size):
    B, H, T, D = x.shape
    return B, H, T, D, T // block_size


@L.on_device
def _mean_pool_fwd(x, block_size):
    B, H, T, D, n_blk = _pool_dims(x, block_size)
    x = x.contiguous()
    out = torch.empty(B, H, n_blk, D, device=x.device, dtype=x.dtype)
    L.check(L.lib().nsa_block_mean_pool_fwd(L.ptr(x), L.ptr(out), B, H, T, D, int(block_size),
                                            L.dtype_code(x), L.stream()))
    return out


@L.on_device
def _mean_pool_bwd(d_out, T, block_size):
    B, H, n_blk, D = d_out.shape
    d_out = d_out.contiguous()
    dx = torch.empty(B, H, T, D, device=d_out.device, dtype=d_out.dtype)
    L.check(L.lib().nsa_block_mean_pool_bwd(L.ptr(d_out), L.ptr(dx), B, H, T, D, int(block_size),
                                            L.dtype_code(d_out), L.stream()))
    return dx


def n_summaries(T, cmp_len, cmp_stride):
    """Complete windows of cmp_len tokens every cmp_stride tokens inside T tokens."""
    return (T - cmp_len) // cmp_stride + 1 if T >= cmp_len else 0


@L.on_device
def _compress_fwd(x, intra, logits, proj, block_size, stride=None):
    stride = block_size if stride is None else stride
    B, H, T, D = x.shape
    x = x.contiguous()
    out = torch.empty(B, H, n_summaries(T, block_size, stride), D, device=x.device, dtype=x.dtype)
    L.check(L.lib().nsa_block_compress_strided_fwd(L.ptr(x), L.ptr(intra), L.ptr(logits), L.ptr(proj),
                                                   L.ptr(out), B, H, T, D, int(block_size), int(stride),
                                                   L.dtype_code(x), L.stream()))
    return out


@L.on_device
def _compress_bwd(x, intra, logits, proj, d_out, block_size, stride=None):
    stride = block_size if stride is None else stride
    B, H, T, D = x.shape
    x, d_out = x.contiguous(), d_out.contiguous()
    dx = torch.empty_like(x)
    d_intra, d_logits, d_proj = (torch.empty_like(t) for t in (intra, logits, proj))
    nws = L.lib().nsa_block_compress_strided_bwd_workspace_bytes(B, H, T, D, int(block_size), int(stride))
    ws = L.workspace(nws, x.device)
    L.check(L.lib().nsa_block_compress_strided_bwd(
        L.ptr(x), L.ptr(intra), L.ptr(logits), L.ptr(proj), L.ptr(d_out), L.ptr(dx), L.ptr(d_intra),
        L.ptr(d_logits), L.ptr(d_proj), B, H, T, D, int(block_size), int(stride), L.dtype_code(x),
        L.ptr(ws), nws, L.stream()))
    return dx, d_intra, d_logits, d_proj


@torch.no_grad()
@L.on_device
def topn_blocks(q, k_cmp, lse_cmp, block_size, n_sel, return_importance=False, n_init_blocks=0,
                n_local_blocks=0, cmp_len=None, cmp_stride=None):
    """Block scoring + top-n (nsa_model.py:343-355): block_idx [B,Hkv,T,n_sel] int32, ordered by
    (importance descending, index ascending), -1 where fewer than n_sel blocks are causally
    valid.  lse_cmp is the LSE of the compression branch for the same q, k_cmp.
    Not in the reference: n_init_blocks / n_local_blocks put the first blocks and the most
    recent blocks, the one holding t included, ahead of the scored ones; cmp_len / cmp_stride
    (default block_size) say that k_cmp are summaries of cmp_len tokens every cmp_stride tokens
    while the selection blocks stay block_size tokens."""
    B, Hq, T, D = q.shape
    Hkv, n_cmp = k_cmp.shape[1], k_cmp.shape[2]
    cl = int(block_size if cmp_len is None else cmp_len)
    cs = int(cl if cmp_stride is None else cmp_stride)
    aligned = cl == cs == int(block_size)
    q, k_cmp, lse_cmp = q.contiguous(), k_cmp.contiguous(), lse_cmp.contiguous()
    idx = torch.empty(B, Hkv, T, n_sel, device=q.device, dtype=torch.int32)
    cols = n_cmp if aligned else (T + int(block_size) - 1) // int(block_size)
    imp = torch.empty(B, Hkv, T, cols, device=q.device, dtype=torch.float32) if return_importance else None
    d = L.dims(B, Hq, Hkv, T, D, L.dtype_code(q))
    L.check(L.lib().nsa_topn_blocks_general(L.ptr(q), L.ptr(k_cmp), L.ptr(lse_cmp), L.ptr(idx), L.ptr(imp),
                                            d, n_cmp, cl, cs, int(block_size), int(n_sel),
                                            int(n_init_blocks), int(n_local_blocks), L.IMPL[_impl],
                                            L.stream()))
    return (idx, imp) if return_importance else idx


@L.on_device
def _gate_fwd(o_cmp, o_slc, o_win, gate):
    B, Hq, T, D = o_cmp.shape
    out = torch.empty_like(o_cmp)
    d = L.dims(B, Hq, 1, T, D, L.dtype_code(o_cmp))
    L.check(L.lib().nsa_gate_combine_fwd(L.ptr(o_cmp), L.ptr(o_slc), L.ptr(o_win), L.ptr(gate),
                                         L.ptr(out), d, L.stream()))
    return out


@L.on_device
def _gate_bwd(o_cmp, o_slc, o_win, gate, d_out):
    B, Hq, T, D = o_cmp.shape
    d_out = d_out.contiguous()
    dc, ds, dw = (torch.empty_like(o_cmp) for _ in range(3))
    dg = torch.empty_like(gate)
    d = L.dims(B, Hq, 1, T, D, L.dtype_code(o_cmp))
    L.check(L.lib().nsa_gate_combine_bwd(L.ptr(o_cmp), L.ptr(o_slc), L.ptr(o_win), L.ptr(gate),
                                         L.ptr(d_out), L.ptr(dc), L.ptr(ds), L.ptr(dw), L.ptr(dg),
                                         d, L.stream()))
    return dc, ds, dw, dg


# ---------------------------------------------------------------------------------------
# autograd boundary (same classes and callables as the reference)
# ---------------------------------------------------------------------------------------
class _RangeAttn(torch.autograd.Function):
    """nsa_fused_kernel.py:521-534; additionally keeps the LSE so backward is one pass."""

    @staticmethod
    def forward(ctx, q, k, v, mode, window, block_size):
        o, lse = range_attn_forward(q, k, v, mode, window, block_size)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.mode, ctx.window, ctx.block_size = mode, window, block_size
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = range_attn_backward(q, k, v, o, lse, do, ctx.mode, ctx.window, ctx.block_size)
        return dq, dk, dv, None, None, None


def window_attn_triton(q, k, v, window):
    return _RangeAttn.apply(q, k, v, MODE_WINDOW, window, 0)


def compression_attn_triton(q, k_cmp, v_cmp, block_size, stride=0):
    """nsa_fused_kernel.py:541-543.  stride (not in the reference): the summaries are windows of
    block_size tokens every `stride` tokens; 0 = block_size."""
    if stride:
        return _RangeAttn.apply(q, k_cmp, v_cmp, MODE_COMPRESS_STRIDED, stride, block_size)
    return _RangeAttn.apply(q, k_cmp, v_cmp, MODE_COMPRESS, 0, block_size)


class SelectionAttnTriton(torch.autograd.Function):
    """nsa_selection_backward.py:337-365: block_idx and block_size get no gradient."""

    @staticmethod
    def forward(ctx, q, k, v, block_idx, block_size):
        # the index structures of the block list are built once for forward and backward (the
        # reference builds its CSR in each: nsa_selection_kernel.py:199-201, nsa_selection_backward.py:356-358)
        plan = None
        if q.is_cuda and q.dtype == torch.bfloat16 and any(ctx.needs_input_grad[:3]):
            plan = selection_plan(q, k, block_idx, block_size)
        o, lse = selection_forward_triton(q, k, v, block_idx, block_size, return_lse=True, plan=plan)
        ctx.save_for_backward(q, k, v, block_idx, o, lse)
        ctx.block_size, ctx.sel_plan = block_size, plan
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, block_idx, o, lse = ctx.saved_tensors
        dq, dk, dv = _selection_backward(q, k, v, block_idx, ctx.block_size, do, o, lse, plan=ctx.sel_plan)
        return dq, dk, dv, None, None


def selection_attn_triton(q, k, v, block_idx, block_size):
    return SelectionAttnTriton.apply(q, k, v, block_idx, block_size)


class _MeanPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, block_size):
        ctx.T, ctx.block_size = x.shape[2], block_size
        return _mean_pool_fwd(x, block_size)

    @staticmethod
    def backward(ctx, d_out):
        return _mean_pool_bwd(d_out, ctx.T, ctx.block_size), None


def block_mean_pool(x, block_size):
    """nsa_fused_kernel.py:549-554: [B,Hkv,T,D] -> [B,Hkv,n_blk,D]."""
    return _MeanPool.apply(x, block_size)


class _BlockCompress(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, intra_pos, pool_logits, proj_weight, block_size, stride):
        intra, logits, proj = (t.detach().float().contiguous() for t in (intra_pos, pool_logits, proj_weight))
        ctx.save_for_backward(x, intra, logits, proj)
        ctx.block_size, ctx.stride = block_size, stride
        ctx.param_dtypes = (intra_pos.dtype, pool_logits.dtype, proj_weight.dtype)
        return _compress_fwd(x, intra, logits, proj, block_size, stride)

    @staticmethod
    def backward(ctx, d_out):
        x, intra, logits, proj = ctx.saved_tensors
        dx, di, dl, dp = _compress_bwd(x, intra, logits, proj, d_out, ctx.block_size, ctx.stride)
        a, b, c = ctx.param_dtypes
        return dx, di.to(a), dl.to(b), dp.to(c), None, None


def block_compress(x, intra_pos, pool_logits, proj_weight, block_size, stride=None):
    """BlockCompressor.forward (nsa_model.py:118-123) on the block view of x [B,Hkv,T,D];
    with stride < block_size on overlapping windows (not in the reference)."""
    return _BlockCompress.apply(x, intra_pos, pool_logits, proj_weight, block_size, stride)


class _GateCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o_cmp, o_slc, o_win, gate_logits):
        o_cmp, o_slc, o_win = (t.contiguous() for t in (o_cmp, o_slc, o_win))
        gate = gate_logits.to(o_cmp.dtype).contiguous()
        ctx.save_for_backward(o_cmp, o_slc, o_win, gate)
        ctx.gate_dtype = gate_logits.dtype
        return _gate_fwd(o_cmp, o_slc, o_win, gate)

    @staticmethod
    def backward(ctx, d_out):
        o_cmp, o_slc, o_win, gate = ctx.saved_tensors
        dc, ds, dw, dg = _gate_bwd(o_cmp, o_slc, o_win, gate, d_out)
        return dc, ds, dw, dg.to(ctx.gate_dtype)


def gate_combine(o_cmp, o_slc, o_win, gate_logits):
    """sigmoid(gate)[...,0]*o_cmp + [...,1]*o_slc + [...,2]*o_win (nsa_model.py:366-368)."""
    return _GateCombine.apply(o_cmp, o_slc, o_win, gate_logits)


# ---------------------------------------------------------------------------------------
# projection glue of the layer (nsa_model.py:192-194, 325-329, 358-359, 366-369)
# ---------------------------------------------------------------------------------------
def fused_projection_width(Hq, Hkv, D):
    """Row width of the fused projection: q, six K/V projections, 3*Hq gate logits padded to 8."""
    return int(L.lib().nsa_fused_projection_width(Hq, Hkv, D))


@L.on_device
def _split_heads_launch(y, q, kv, gate, Hq, Hkv, D, merge):
    B, T = y.shape[0], y.shape[1]
    fn = L.lib().nsa_merge_heads if merge else L.lib().nsa_split_heads
    if merge:
        L.check(fn(L.ptr(q), L.ptr(kv), L.ptr(gate), L.ptr(y), B, T, Hq, Hkv, D, L.dtype_code(y), L.stream()))
    else:
        L.check(fn(L.ptr(y), L.ptr(q), L.ptr(kv), L.ptr(gate), B, T, Hq, Hkv, D, L.dtype_code(y), L.stream()))


class _SplitHeads(torch.autograd.Function):
    """Rows [B,T,W] of the fused projection -> q [B,Hq,T,D], kv [6,B,Hkv,T,D] (kc, vc, ks, vs, kw,
    vw), gate logits [B,Hq,T,3], in one pass; backward assembles the gradient rows in one pass."""

    @staticmethod
    def forward(ctx, y, Hq, Hkv, D):
        B, T, W = y.shape
        assert W == fused_projection_width(Hq, Hkv, D), "row width does not match the head counts"
        y = y.contiguous()
        q = torch.empty(B, Hq, T, D, device=y.device, dtype=y.dtype)
        kv = torch.empty(6, B, Hkv, T, D, device=y.device, dtype=y.dtype)
        gate = torch.empty(B, Hq, T, 3, device=y.device, dtype=y.dtype)
        _split_heads_launch(y, q, kv, gate, Hq, Hkv, D, False)
        ctx.cfg = (Hq, Hkv, D, W)
        return q, kv, gate

    @staticmethod
    def backward(ctx, dq, dkv, dgate):
        Hq, Hkv, D, W = ctx.cfg
        B, _, T, _ = dq.shape
        dq, dkv, dgate = dq.contiguous(), dkv.contiguous(), dgate.contiguous()
        dy = torch.empty(B, T, W, device=dq.device, dtype=dq.dtype)
        _split_heads_launch(dy, dq, dkv, dgate, Hq, Hkv, D, True)
        return dy, None, None, None


def split_heads(y, Hq, Hkv, D):
    return _SplitHeads.apply(y, Hq, Hkv, D)


@L.on_device
def _swap_heads_tokens(x, to_tokens):
    if to_tokens:
        B, H, T, D = x.shape
        out = torch.empty(B, T, H, D, device=x.device, dtype=x.dtype)
    else:
        B, T, H, D = x.shape
        out = torch.empty(B, H, T, D, device=x.device, dtype=x.dtype)
    L.check(L.lib().nsa_swap_heads_tokens(L.ptr(x), L.ptr(out), B, H, T, D, L.dtype_code(x), int(to_tokens),
                                          L.stream()))
    return out


class _HeadsToTokens(torch.autograd.Function):
    """[B,H,T,D] -> [B,T,H*D] (what out_proj reads, nsa_model.py:369); backward the other way."""

    @staticmethod
    def forward(ctx, x):
        ctx.D = x.shape[3]
        out = _swap_heads_tokens(x.contiguous(), True)
        return out.view(out.shape[0], out.shape[1], -1)

    @staticmethod
    def backward(ctx, d_out):
        B, T, HD = d_out.shape
        return _swap_heads_tokens(d_out.contiguous().view(B, T, HD // ctx.D, ctx.D), False)


def heads_to_tokens(x):
    return _HeadsToTokens.apply(x)


def nsa_fused_forward(q, kc, vc, ks, vs, kw, vw, gate_logits, block_idx, block_size, window):
    """nsa_fused_kernel.py:560-573: the three branches with a given block_idx, mean pooling."""
    k_cmp = block_mean_pool(kc, block_size)
    v_cmp = block_mean_pool(vc, block_size)
    o_cmp = compression_attn_triton(q, k_cmp, v_cmp, block_size)
    o_slc = selection_attn_triton(q, ks, vs, block_idx, block_size)
    o_win = window_attn_triton(q, kw, vw, window)
    return gate_combine(o_cmp, o_slc, o_win, gate_logits)


class _NSAAttention(torch.autograd.Function):
    """The whole op in one node: pooling -> compression attention (+LSE) -> block scoring and
    top-n -> selection attention -> window attention -> gate combine.  Saves q once."""

    @staticmethod
    @L.on_device
    def forward(ctx, q, kc, vc, ks, vs, kw, vw, gate_logits, block_size, n_sel, window,
                block_idx, forced, k_intra, k_logits, k_proj, v_intra, v_logits, v_proj):
        learned = k_intra is not None
        n_init, n_local, cl, cs = forced          # cl, cs: length and stride of the summaries
        if learned:
            cp = [t.detach().float().contiguous() for t in
                  (k_intra, k_logits, k_proj, v_intra, v_logits, v_proj)]
            k_cmp = _compress_fwd(kc, cp[0], cp[1], cp[2], cl, cs)
            v_cmp = _compress_fwd(vc, cp[3], cp[4], cp[5], cl, cs)
        else:
            assert cl == cs == block_size, "mean pooling is defined on the aligned grid only"
            cp = []
            k_cmp = _mean_pool_fwd(kc, block_size)
            v_cmp = _mean_pool_fwd(vc, block_size)
        # the three branches' outputs and softmax statistics live in one tensor each
        q = q.contiguous()
        o3 = torch.empty((3,) + tuple(q.shape), device=q.device, dtype=q.dtype)
        lse3 = torch.empty((3,) + tuple(q.shape[:3]), device=q.device, dtype=torch.float32)
        o_cmp, lse_cmp = range_attn_forward(q, k_cmp, v_cmp, MODE_COMPRESS_STRIDED, cs, cl, out=(o3[0], lse3[0]))
        if block_idx is None:
            block_idx = topn_blocks(q, k_cmp, lse_cmp, block_size, n_sel, n_init_blocks=n_init,
                                    n_local_blocks=n_local, cmp_len=cl, cmp_stride=cs)
        else:
            block_idx = block_idx.to(torch.int32).contiguous()
        # CSR, pair map and work list of the block list: built once, used by forward and backward
        plan = selection_plan(q, ks, block_idx, block_size) if q.dtype == torch.bfloat16 else None
        o_slc, _ = selection_forward_triton(q, ks, vs, block_idx, block_size, return_lse=True,
                                            out=(o3[1], lse3[1]), plan=plan)
        o_win, _ = range_attn_forward(q, kw, vw, MODE_WINDOW, window, 0, out=(o3[2], lse3[2]))
        gate = gate_logits.to(q.dtype).contiguous()
        out = _gate_fwd(o_cmp, o_slc, o_win, gate)
        ctx.save_for_backward(q, kc, vc, ks, vs, kw, vw, gate, k_cmp, v_cmp, o3, lse3, block_idx, *cp)
        ctx.sel_plan = plan          # (an opaque byte buffer: kept on the context, not a differentiable input)
        ctx.cfg = (block_size, window, learned, gate_logits.dtype,
                   tuple(t.dtype for t in (k_intra, k_logits, k_proj, v_intra, v_logits, v_proj))
                   if learned else None, cl, cs)
        ctx.mark_non_differentiable(block_idx)
        if L.CHECK_STATUS_EVERY_CALL:
            L.check_device_status()
        return out, block_idx

    @staticmethod
    @L.on_device
    def backward(ctx, d_out, _d_idx):
        (q, kc, vc, ks, vs, kw, vw, gate, k_cmp, v_cmp, o3, lse3, block_idx, *cp) = ctx.saved_tensors
        (o_cmp, o_slc, o_win), (lse_cmp, lse_slc, lse_win) = o3, lse3
        block_size, window, learned, gate_dtype, pdt, cl, cs = ctx.cfg
        T = q.shape[2]
        # gate backward as per-row statistics; the branch kernels apply the gate factor themselves
        B, Hq = q.shape[0], q.shape[1]
        d_out = d_out.contiguous()
        rs = torch.empty(3, B, Hq, T, device=q.device, dtype=torch.float32)
        rd = torch.empty(3, B, Hq, T, device=q.device, dtype=torch.float32)
        d_gate = torch.empty_like(gate)
        L.check(L.lib().nsa_gate_combine_bwd_rows(
            L.ptr(o_cmp), L.ptr(o_slc), L.ptr(o_win), L.ptr(gate), L.ptr(d_out), L.ptr(rs), L.ptr(rd),
            L.ptr(d_gate), L.dims(B, Hq, 1, T, q.shape[3], L.dtype_code(q)), L.stream()))
        S = block_idx.shape[-1]
        # tcgen05 shapes: the three branches leave their dQ partials in their workspaces and one
        # kernel adds them all; otherwise three dq tensors and a sum
        fused = (_impl != "simt" and S > 0 and q.dtype == torch.bfloat16 and
                 tc_supported(B, Hq, ks.shape[1], T, q.shape[3], q.dtype, block_size))
        dq_sum = torch.empty_like(q)
        dm = L.dims(B, Hq, ks.shape[1], T, q.shape[3], L.dtype_code(q))
        n_cmp = k_cmp.shape[2]
        if fused and _dq_accumulator:
            # window and compression add their dQ into one fp32 accumulator; only the selection
            # branch keeps partials (its rows are gathered, the adds would miss L2)
            G = Hq // ks.shape[1]
            dq_acc = torch.zeros(B * ks.shape[1], T, G, q.shape[3], device=q.device, dtype=torch.float32)
            if n_cmp > 0:
                dk_cmp, dv_cmp = range_attn_backward_acc(q, k_cmp, v_cmp, o_cmp, lse_cmp, d_out,
                                                         MODE_COMPRESS_STRIDED, cs, cl, rs[0], rd[0], dq_acc)
            else:
                dk_cmp, dv_cmp = torch.zeros_like(k_cmp), torch.zeros_like(v_cmp)
            dkw, dvw = range_attn_backward_acc(q, kw, vw, o_win, lse_win, d_out, MODE_WINDOW, window, 0,
                                               rs[2], rd[2], dq_acc)
            ws2, dks, dvs = _selection_backward(q, ks, vs, block_idx, block_size, d_out, o_slc, lse_slc,
                                                rs[1], rd[1], defer_dq=True, plan=ctx.sel_plan)
            L.check(L.lib().nsa_dq_finish(dm, S, int(block_size), L.ptr(dq_acc), L.ptr(ws2), L.ptr(dq_sum),
                                          L.stream()))
            del ws2, dq_acc
        else:
            dq, dk_cmp, dv_cmp = range_attn_backward(q, k_cmp, v_cmp, o_cmp, lse_cmp, d_out,
                                                     MODE_COMPRESS_STRIDED, cs, cl, rs[0], rd[0],
                                                     defer_dq=fused)
            dq2, dks, dvs = _selection_backward(q, ks, vs, block_idx, block_size, d_out, o_slc, lse_slc,
                                                rs[1], rd[1], defer_dq=fused, plan=ctx.sel_plan)
            dq3, dkw, dvw = range_attn_backward(q, kw, vw, o_win, lse_win, d_out, MODE_WINDOW, window, 0,
                                                rs[2], rd[2], defer_dq=fused)
            if fused:
                L.check(L.lib().nsa_dq_reduce3(dm, n_cmp, int(cl), int(cs), S, int(block_size), int(window),
                                               L.ptr(dq) if n_cmp > 0 else None, L.ptr(dq2), L.ptr(dq3),
                                               L.ptr(dq_sum), L.stream()))
            else:
                L.check(L.lib().nsa_sum3(L.ptr(dq), L.ptr(dq2), L.ptr(dq3), L.ptr(dq_sum), dq.numel(),
                                         L.dtype_code(dq), L.stream()))
            del dq, dq2, dq3
        dq = dq_sum
        pgrads = [None] * 6
        if learned:
            dkc, a, b, c = _compress_bwd(kc, cp[0], cp[1], cp[2], dk_cmp, cl, cs)
            dvc, d, e, f = _compress_bwd(vc, cp[3], cp[4], cp[5], dv_cmp, cl, cs)
            pgrads = [g.to(t) for g, t in zip((a, b, c, d, e, f), pdt)]
        else:
            dkc = _mean_pool_bwd(dk_cmp, T, block_size)
            dvc = _mean_pool_bwd(dv_cmp, T, block_size)
        if L.CHECK_STATUS_EVERY_CALL:
            L.check_device_status()
        return (dq, dkc, dvc, dks, dvs, dkw, dvw, d_gate.to(gate_dtype), None, None, None, None, None,
                *pgrads)


@torch.no_grad()
def select_blocks(q, kc, vc, block_size, n_sel, compressor=None, n_init_blocks=0, n_local_blocks=0,
                  cmp_len=None, cmp_stride=None):
    """The block lists [B,Hkv,T,n_sel] the whole op picks for q (pooling, compression attention,
    block scoring + top-n; nsa_model.py:336-355), without the rest of the op.  The scores sum over
    all query heads of a kv head, so a caller that deals the query heads of one group out over
    several devices computes the lists from the whole group on each and passes them to
    nsa_attention(..., block_idx=...) with its share of the heads."""
    cl = int(block_size if cmp_len is None else cmp_len)
    cs = int(cl if cmp_stride is None else cmp_stride)
    if compressor is not None:
        cp = [compressor[n].detach().float().contiguous()
              for n in ("k_intra", "k_logits", "k_proj", "v_intra", "v_logits", "v_proj")]
        k_cmp = _compress_fwd(kc, cp[0], cp[1], cp[2], cl, cs)
        v_cmp = _compress_fwd(vc, cp[3], cp[4], cp[5], cl, cs)
    else:
        assert cl == cs == block_size, "mean pooling is defined on the aligned grid only"
        k_cmp, v_cmp = _mean_pool_fwd(kc, block_size), _mean_pool_fwd(vc, block_size)
    _, lse_cmp = range_attn_forward(q, k_cmp, v_cmp, MODE_COMPRESS_STRIDED, cs, cl)
    return topn_blocks(q, k_cmp, lse_cmp, block_size, n_sel, n_init_blocks=n_init_blocks,
                       n_local_blocks=n_local_blocks, cmp_len=cl, cmp_stride=cs)


def nsa_attention(q, kc, vc, ks, vs, kw, vw, gate_logits, block_size, n_sel, window,
                  block_idx=None, compressor=None, return_block_idx=False, n_init_blocks=0,
                  n_local_blocks=0, cmp_len=None, cmp_stride=None):
    """Full NSA attention (pre out_proj) as one differentiable op.

    q [B,Hq,T,D]; kc..vw [B,Hkv,T,D]; gate_logits [B,Hq,T,3].  `compressor` is None for mean
    pooling or a dict k_intra,k_logits,k_proj,v_intra,v_logits,v_proj holding the parameters
    of the two BlockCompressor modules (nsa_model.py:180-181).  With block_idx=None the blocks
    are picked by the scorer (nsa_model.py:343-355 semantics, deterministic tie order);
    n_init_blocks / n_local_blocks force the first blocks and the most recent blocks into every
    list ahead of the scored ones (the published NSA recipe; the reference has no such option).
    cmp_len / cmp_stride (learned pooling only; default block_size, the reference's grid) make
    the summaries windows of cmp_len tokens every cmp_stride tokens, e.g. 32 / 16 with 64-token
    selection blocks; the compressor parameters then have cmp_len positions.
    With NSA_B200_CHECK_STATUS=1 in the environment the device status word is read (one stream
    synchronisation) after every forward and backward and a give-up raises NsaError."""
    cp = [None] * 6
    if compressor is not None:
        cp = [compressor[n] for n in ("k_intra", "k_logits", "k_proj", "v_intra", "v_logits", "v_proj")]
    cl = int(block_size if cmp_len is None else cmp_len)
    cs = int(cl if cmp_stride is None else cmp_stride)
    out, idx = _NSAAttention.apply(q, kc, vc, ks, vs, kw, vw, gate_logits, block_size, n_sel,
                                   window, block_idx, (int(n_init_blocks), int(n_local_blocks), cl, cs), *cp)
    return (out, idx) if return_block_idx else out
