"""NSA attention layer on the CUDA path with the parameter names of the reference module.

`NSAAttentionB200` has the same constructor arguments and state_dict keys as the reference's
NSAAttention (nsa_model.py:126-190), so one snapshot loads into either; its forward does
what NSAAttention._forward_fused does (nsa_model.py:306-370) through `nsa_attention`, with
the learned block pooling, block scoring and gate blend inside the fused op.

Projection glue (nsa_model.py:325-329, 358-359, 366-369): the reference runs q, six K/V and the
gate projection as eight GEMMs, each followed by its own transpose + copy.  Here the eight weights
(still eight parameters with the reference's names) are applied as one GEMM, one kernel pass turns
its rows into the head-major tensors the attention kernels read and one pass brings the output back
for out_proj; the backward likewise (one pass assembling the gradient rows, one dgrad and one wgrad
GEMM).  `fused_projection=False` keeps the eight separate projections.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .ops import fused_projection_width, heads_to_tokens, nsa_attention, split_heads


class _Compressor(nn.Module):
    """Parameter holder named like BlockCompressor (nsa_model.py:100-116)."""

    def __init__(self, block_size, d_head):
        super().__init__()
        self.block_size = block_size
        self.intra_pos = nn.Parameter(torch.zeros(block_size, d_head))
        self.pool_logits = nn.Parameter(torch.zeros(block_size))
        self.proj = nn.Linear(d_head, d_head, bias=False)


class NSAAttentionB200(nn.Module):
    def __init__(self, d_model, n_q_heads, n_kv_heads, block_size=16, n_selected_blocks=4,
                 window=32, n_init_blocks=0, n_local_blocks=0, cmp_len=None, cmp_stride=None,
                 fused_projection=True):
        super().__init__()
        assert n_q_heads % n_kv_heads == 0, "GQA needs n_q_heads divisible by n_kv_heads"
        self.d_model, self.Hq, self.Hkv = d_model, n_q_heads, n_kv_heads
        self.dh = d_model // n_q_heads
        self.block_size, self.n_sel, self.window = block_size, n_selected_blocks, window
        self.fused_projection = fused_projection
        # forced selection blocks (not in the reference module; 0, 0 reproduces it)
        self.n_init_blocks, self.n_local_blocks = n_init_blocks, n_local_blocks
        # summaries of cmp_len tokens every cmp_stride tokens (default: the reference's block grid)
        self.cmp_len = block_size if cmp_len is None else cmp_len
        self.cmp_stride = self.cmp_len if cmp_stride is None else cmp_stride
        kv_dim = self.Hkv * self.dh
        self.q_proj = nn.Linear(d_model, self.Hq * self.dh, bias=False)
        self.k_cmp = nn.Linear(d_model, kv_dim, bias=False)
        self.v_cmp = nn.Linear(d_model, kv_dim, bias=False)
        self.k_slc = nn.Linear(d_model, kv_dim, bias=False)
        self.v_slc = nn.Linear(d_model, kv_dim, bias=False)
        self.k_win = nn.Linear(d_model, kv_dim, bias=False)
        self.v_win = nn.Linear(d_model, kv_dim, bias=False)
        self.comp_k = _Compressor(self.cmp_len, self.dh)
        self.comp_v = _Compressor(self.cmp_len, self.dh)
        self.gate = nn.Linear(d_model, self.Hq * 3, bias=True)
        self.out_proj = nn.Linear(self.Hq * self.dh, d_model, bias=False)

    def _split(self, x, n_heads):
        B, T, _ = x.shape
        return x.view(B, T, n_heads, self.dh).transpose(1, 2).contiguous()

    def forward(self, x, block_idx=None):
        """x [B,T,d_model] -> [B,T,d_model].  `block_idx` overrides the scorer's pick."""
        B, T, _ = x.shape
        fused = self.fused_projection and x.is_cuda and self.dh % 8 == 0
        if fused:
            # one GEMM for the eight projections, one pass to head-major layout
            ws = [p.weight for p in (self.q_proj, self.k_cmp, self.v_cmp, self.k_slc, self.v_slc,
                                     self.k_win, self.v_win, self.gate)]
            width = fused_projection_width(self.Hq, self.Hkv, self.dh)
            n_attn = (self.Hq + 6 * self.Hkv) * self.dh
            pad = width - n_attn - 3 * self.Hq
            w = torch.cat(ws + [ws[0].new_zeros(pad, self.d_model)] if pad else ws, dim=0)
            bias = torch.cat([self.gate.bias.new_zeros(n_attn), self.gate.bias, self.gate.bias.new_zeros(pad)])
            q, kv6, gate = split_heads(F.linear(x, w, bias), self.Hq, self.Hkv, self.dh)
            kv = list(kv6.unbind(0))
        else:
            q = self._split(self.q_proj(x), self.Hq)
            kv = [self._split(p(x), self.Hkv) for p in
                  (self.k_cmp, self.v_cmp, self.k_slc, self.v_slc, self.k_win, self.v_win)]
            gate = self.gate(x).view(B, T, self.Hq, 3).permute(0, 2, 1, 3).contiguous()
        comp = dict(k_intra=self.comp_k.intra_pos, k_logits=self.comp_k.pool_logits,
                    k_proj=self.comp_k.proj.weight, v_intra=self.comp_v.intra_pos,
                    v_logits=self.comp_v.pool_logits, v_proj=self.comp_v.proj.weight)
        out = nsa_attention(q, *kv, gate.to(q.dtype), self.block_size, self.n_sel, self.window,
                            block_idx=block_idx, compressor=comp, n_init_blocks=self.n_init_blocks,
                            n_local_blocks=self.n_local_blocks, cmp_len=self.cmp_len,
                            cmp_stride=self.cmp_stride)
        if fused:
            return self.out_proj(heads_to_tokens(out))
        out = out.transpose(1, 2).contiguous().view(B, T, self.Hq * self.dh)
        return self.out_proj(out)
