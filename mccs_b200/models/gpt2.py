"""GPT-2 shaped decoder-only transformer (pre-LN, learned positions, GELU MLP, tied
output embedding). ``gpt2_medium()`` is the 24-layer, d_model 1024, 16-head, FFN 4096,
vocabulary 50257 model (~355 M parameters) that the reference only has as a traffic
trace ("GPT" rows of ``workloads/setup-1_gpt_*.toml``: one 711,839,744-byte AllReduce,
i.e. 355.9 M fp16 gradients, per iteration)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    d_ff: int = 4096
    max_seq: int = 1024
    dropout: float = 0.0


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        self.fc = nn.Linear(cfg.d_model, cfg.d_ff)
        self.out = nn.Linear(cfg.d_ff, cfg.d_model)
        self.n_head = cfg.n_head

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.n_head, d // self.n_head).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, d))
        x = x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))
        return x


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.apply(self._init)
        for blk in self.blocks:   # scaled init of the residual projections, as GPT-2 does
            nn.init.normal_(blk.proj.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))
            nn.init.normal_(blk.out.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor | None = None):
        b, t = ids.shape
        pos = torch.arange(t, device=ids.device)
        x = self.wte(ids) + self.wpe(pos)[None]
        for blk in self.blocks:
            x = blk(x)
        x = self.ln_f(x)
        logits = x @ self.wte.weight.t()
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().reshape(-1, logits.size(-1)), targets.reshape(-1))


def gpt2_medium() -> GPT2:
    return GPT2(GPT2Config())


def gpt2_tiny() -> GPT2:
    """Small stand-in with the same code path (tests and CPU runs)."""
    return GPT2(GPT2Config(vocab_size=512, n_layer=2, n_head=4, d_model=64, d_ff=256, max_seq=64))
