"""Decoder-only transformer around the NSA attention layer, with the reference's module tree and
parameter names (nsa_model.py:435-506: tok_emb, pos_emb, blocks.N.{ln1,attn,ln2,ffn.0,ffn.2},
ln_f, lm_head tied to tok_emb), so a snapshot written by the reference's train.py:159-166 loads
with load_state_dict.  Only the attention math runs on this library's kernels; embeddings,
LayerNorm, the FFN and the tied head are plain torch modules (library GEMMs)."""
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .module import NSAAttentionB200


class Block(nn.Module):
    """nsa_model.py:435-452: pre-LayerNorm residual block, GELU FFN of ffn_mult * d_model."""

    def __init__(self, d_model, n_q_heads, n_kv_heads, ffn_mult=4, **nsa_kw):
        super().__init__()
        self.ln1 = nn.LayerNorm(d_model)
        self.attn = NSAAttentionB200(d_model, n_q_heads, n_kv_heads, **nsa_kw)
        self.ln2 = nn.LayerNorm(d_model)
        hidden = ffn_mult * d_model
        self.ffn = nn.Sequential(nn.Linear(d_model, hidden), nn.GELU(), nn.Linear(hidden, d_model))

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        return x + self.ffn(self.ln2(x))


class NSATransformerB200(nn.Module):
    """nsa_model.py:455-506 with attn_type="nsa" served by NSAAttentionB200."""

    def __init__(self, vocab_size, d_model=512, n_layers=8, n_q_heads=8, n_kv_heads=2,
                 max_seq_len=256, ffn_mult=4, block_size=16, n_selected_blocks=4, window=32, **nsa_kw):
        super().__init__()
        self.max_seq_len = max_seq_len
        self.grad_checkpoint = False          # nsa_model.py:464: recompute block activations in backward
        self.tok_emb = nn.Embedding(vocab_size, d_model)
        self.pos_emb = nn.Embedding(max_seq_len, d_model)
        self.blocks = nn.ModuleList([
            Block(d_model, n_q_heads, n_kv_heads, ffn_mult=ffn_mult, block_size=block_size,
                  n_selected_blocks=n_selected_blocks, window=window, **nsa_kw)
            for _ in range(n_layers)])
        self.ln_f = nn.LayerNorm(d_model)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False)
        self.lm_head.weight = self.tok_emb.weight            # weight tying (nsa_model.py:477)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        """N(0, 0.02) weights for every Linear and Embedding, zero Linear biases (nsa_model.py:479-486)."""
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, idx, targets=None):
        B, T = idx.shape
        assert T <= self.max_seq_len
        pos = torch.arange(T, device=idx.device)
        x = self.tok_emb(idx) + self.pos_emb(pos)[None]
        for blk in self.blocks:
            if self.grad_checkpoint and self.training:
                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        loss = None
        if targets is not None:
            loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1))
        return logits, loss
