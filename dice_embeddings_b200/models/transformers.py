"""Transformer-based models: CoKE (bidirectional encoder over ``[h, r, MASK]``) and BytE (GPT-style
language model over sub-word tokens).

Module and parameter names follow the reference so checkpoints interchange:
``Block{ln_1, attn{c_attn, c_proj}, ln_2, mlp{c_fc, c_proj}}``
(``dicee/models/transformers.py:115-210``), CoKE ``pos_emb / mask_emb / blocks.N / ln_f``
(``dicee/models/real.py:134-275``), BytE ``transformer.{wte, wpe, h.N, ln_f}`` + tied ``lm_head``
(``dicee/models/transformers.py:18-112``).  Sequences are 3 (CoKE) or ``block_size`` ≤ 8 (BytE) tokens
long, so attention goes through PyTorch's fused SDPA; no custom kernel is warranted.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.nn import functional as F

from .base import BaseKGE, IdentityClass


class LayerNorm(nn.Module):
    """LayerNorm with an optional bias."""

    def __init__(self, ndim: int, bias: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.bias = nn.Parameter(torch.zeros(ndim)) if bias else None

    def forward(self, x):
        return F.layer_norm(x, self.weight.shape, self.weight, self.bias, 1e-5)


class SelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=config.bias)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=config.bias)
        self.attn_dropout = nn.Dropout(config.dropout)
        self.resid_dropout = nn.Dropout(config.dropout)
        self.n_head = config.n_head
        self.n_embd = config.n_embd
        self.dropout = config.dropout
        self.causal = config.causal

    def forward(self, x):
        B, T, C = x.size()
        q, k, v = self.c_attn(x).split(self.n_embd, dim=2)
        hs = C // self.n_head
        q = q.view(B, T, self.n_head, hs).transpose(1, 2)
        k = k.view(B, T, self.n_head, hs).transpose(1, 2)
        v = v.view(B, T, self.n_head, hs).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None,
                                           dropout_p=self.dropout if self.training else 0.0,
                                           is_causal=self.causal)
        y = y.transpose(1, 2).contiguous().view(B, T, C)
        return self.resid_dropout(self.c_proj(y))


class MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, bias=config.bias)
        self.gelu = nn.GELU()
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=config.bias)
        self.dropout = nn.Dropout(config.dropout)

    def forward(self, x):
        return self.dropout(self.c_proj(self.gelu(self.c_fc(x))))


class Block(nn.Module):
    """Pre-norm transformer block."""

    def __init__(self, config):
        super().__init__()
        self.ln_1 = LayerNorm(config.n_embd, bias=config.bias)
        self.attn = SelfAttention(config)
        self.ln_2 = LayerNorm(config.n_embd, bias=config.bias)
        self.mlp = MLP(config)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


@dataclass
class GPTConfig:
    block_size: int = 1024
    vocab_size: int = 50304
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.0
    bias: bool = False
    causal: bool = True


@dataclass
class CoKEConfig:
    block_size: int = 3
    vocab_size: int = None
    n_layer: int = 6
    n_head: int = 8
    n_embd: int = None
    dropout: float = 0.3
    bias: bool = True
    causal: bool = False


class CoKE(BaseKGE):
    """Contextualised KG embedding: the hidden state of the MASK position scores all entities.  That hidden state is
    the query vector of the bilinear contract (``compose``), so the tensor-core scoring function and the ranking kernel
    apply whenever the tail normaliser is the identity (its default)."""

    @property
    def bilinear(self) -> bool:
        return isinstance(self.normalize_tail_entity_embeddings, IdentityClass)

    def compose(self, h: torch.Tensor, r: torch.Tensor):
        return self._encode(h, r), None

    def __init__(self, args, config: CoKEConfig = None):
        super().__init__(args)
        config = config or CoKEConfig()
        self.config = config
        config.vocab_size = self.num_entities + self.num_relations
        config.n_embd = self.embedding_dim
        self.pos_emb = nn.Embedding(config.block_size, self.embedding_dim)
        self.mask_emb = nn.Parameter(torch.zeros(self.embedding_dim))
        self.blocks = nn.ModuleList([Block(config) for _ in range(config.n_layer)])
        self.ln_f = nn.LayerNorm(self.embedding_dim)
        self.coke_dropout = nn.Dropout(config.dropout)

    def _encode(self, h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
        b = h.size(0)
        seq = torch.stack([h, r, self.mask_emb.unsqueeze(0).expand(b, -1)], dim=1)
        x = seq + self.pos_emb(torch.arange(3, device=h.device)).unsqueeze(0)
        for blk in self.blocks:
            x = blk(x)
        return self.coke_dropout(self.ln_f(x)[:, 2, :])

    def forward_k_vs_all(self, x: torch.Tensor):
        h, r = self.get_head_relation_representation(x)
        E = self.normalize_tail_entity_embeddings(self.entity_embeddings.weight)
        return self._encode(h, r).mm(E.t())

    def score(self, emb_h, emb_r, emb_t):
        return torch.einsum("bd,bd->b", self._encode(emb_h, emb_r), emb_t)

    def forward_k_vs_sample(self, x, target_entity_idx):
        h, r = self.get_head_relation_representation(x)
        return torch.einsum("bd,bkd->bk", self._encode(h, r), self.entity_embeddings(target_entity_idx))


class BytE(BaseKGE):
    """Next-token language model over the token stream ``h␠r␠t.``; cross-entropy loss."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        vocab = self.args.get("num_tokens")
        if vocab is None:
            from ..data.bpe import get_tokenizer
            vocab = get_tokenizer().n_vocab
        n_head = 4 if self.embedding_dim % 4 == 0 else 1
        if self.block_size is None:  # the Python API leaves it unset (reference ``config.py:157``); the CLI default is 8
            self.block_size = 8
        self.config = GPTConfig(block_size=self.block_size, vocab_size=vocab, n_layer=4, n_head=n_head,
                                n_embd=self.embedding_dim, dropout=0.0, bias=False)
        self.temperature = 0.5
        self.topk = 2
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(self.config.vocab_size, self.config.n_embd),
            wpe=nn.Embedding(self.config.block_size, self.config.n_embd),
            drop=nn.Dropout(self.config.dropout),
            h=nn.ModuleList([Block(self.config) for _ in range(self.config.n_layer)]),
            ln_f=LayerNorm(self.config.n_embd, bias=self.config.bias),
        ))
        self.lm_head = nn.Linear(self.config.n_embd, self.config.vocab_size, bias=False)
        self.transformer.wte.weight = self.lm_head.weight  # weight tying

    def loss_function(self, yhat_batch, y_batch):
        return F.cross_entropy(yhat_batch.view(-1, yhat_batch.size(-1)), y_batch.reshape(-1), ignore_index=-1)

    def forward(self, x: torch.Tensor):
        b, t = x.size()
        assert t <= self.config.block_size, f"sequence of length {t} exceeds block size {self.config.block_size}"
        pos = torch.arange(0, t, dtype=torch.long, device=x.device)
        h = self.transformer.drop(self.transformer.wte(x) + self.transformer.wpe(pos))
        for blk in self.transformer.h:
            h = blk(h)
        return self.lm_head(self.transformer.ln_f(h))

    def get_embeddings(self):
        return self.transformer.wte.weight.data.detach(), None

    @torch.no_grad()
    def generate(self, idx, max_new_tokens, temperature=1.0, top_k=None):
        """Autoregressive sampling: append ``max_new_tokens`` tokens to ``idx [b, t]``."""
        for _ in range(max_new_tokens):
            cond = idx if idx.size(1) <= self.config.block_size else idx[:, -self.config.block_size:]
            logits = self(cond)[:, -1, :] / temperature
            if top_k is not None:
                v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < v[:, [-1]]] = -float("inf")
            nxt = torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)
            idx = torch.cat((idx, nxt), dim=1)
        return idx

    def estimate_mfu(self, fwdbwd_per_iter: float, dt: float, peak_flops: float = 2.25e15) -> float:
        """Model-FLOPs utilisation against a peak (default: B200 dense bf16)."""
        n = sum(p.numel() for p in self.parameters())
        cfg = self.config
        flops_per_token = 6 * n + 12 * cfg.n_layer * cfg.n_head * (cfg.n_embd // cfg.n_head) * cfg.block_size
        return flops_per_token * cfg.block_size * fwdbwd_per_iter / dt / peak_flops
