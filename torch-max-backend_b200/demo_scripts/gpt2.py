"""GPT-2 forward used as the model definition of the benchmark configurations.

Architecture of the reference's demo model (demo_scripts/gpt2.py:15-249: nanoGPT-style blocks,
pre-LayerNorm eps 1e-5, fused QKV projection, learned positional embeddings, tied LM head) with
the choices the benchmark configurations pin down: tanh-approximated GELU through
`F.gelu(x, approximate="tanh")` (so that `aten.gelu` itself is exercised), logits for every
position, N(0, 0.02) weights with zero biases and LayerNorm gamma=1 / beta=0 from a seed, and
two attention formulations: `F.scaled_dot_product_attention(is_causal=True)` and the explicit
`masked_fill -> softmax` form of the reference demo.

`precision="bf16"` is the mixed policy the bf16 parity bar needs: GEMM and attention operands
(weights, embeddings, activations entering a GEMM) are bf16 with fp32 accumulation, while the
residual stream, LayerNorm and the logits stay fp32.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    block_size: int = 1024
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768

    @staticmethod
    def small() -> "GPTConfig":
        return GPTConfig(n_layer=12, n_head=12, n_embd=768)

    @staticmethod
    def xl() -> "GPTConfig":
        return GPTConfig(n_layer=48, n_head=25, n_embd=1600)


class CausalSelfAttention(nn.Module):
    def __init__(self, config: GPTConfig, attention: str):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=True)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=True)
        self.n_head = config.n_head
        self.n_embd = config.n_embd
        self.attention = attention
        if attention == "masked_softmax":
            self.register_buffer(
                "bias",
                torch.tril(torch.ones(config.block_size, config.block_size)).view(
                    1, 1, config.block_size, config.block_size
                ),
                persistent=False,
            )

    def forward(self, x):
        B, T, C = x.size()
        q, k, v = self.c_attn(x).split(self.n_embd, dim=2)
        k = k.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        q = q.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        v = v.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        if self.attention == "sdpa":
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            att = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(k.size(-1)))
            att = att.masked_fill(self.bias[:, :, :T, :T] == 0, float("-inf"))
            att = F.softmax(att, dim=-1)
            y = att @ v
        y = y.transpose(1, 2).contiguous().view(B, T, C)
        return self.c_proj(y)


class MLP(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, bias=True)
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=True)

    def forward(self, x):
        return self.c_proj(F.gelu(self.c_fc(x), approximate="tanh"))


class Block(nn.Module):
    def __init__(self, config: GPTConfig, attention: str):
        super().__init__()
        self.ln_1 = nn.LayerNorm(config.n_embd, eps=1e-5)
        self.attn = CausalSelfAttention(config, attention)
        self.ln_2 = nn.LayerNorm(config.n_embd, eps=1e-5)
        self.mlp = MLP(config)
        self.compute_dtype = None  # set by GPT2.set_precision

    def forward(self, x):
        cd = self.compute_dtype
        if cd is None:
            x = x + self.attn(self.ln_1(x))
            x = x + self.mlp(self.ln_2(x))
            return x
        # mixed policy: fp32 residual stream and LayerNorm, `cd` operands for GEMM / attention
        x = x + self.attn(self.ln_1(x).to(cd)).float()
        x = x + self.mlp(self.ln_2(x).to(cd)).float()
        return x


class GPT2(nn.Module):
    def __init__(self, config: GPTConfig, attention: str = "sdpa"):
        super().__init__()
        assert attention in ("sdpa", "masked_softmax")
        self.config = config
        self.wte = nn.Embedding(config.vocab_size, config.n_embd)
        self.wpe = nn.Embedding(config.block_size, config.n_embd)
        self.h = nn.ModuleList([Block(config, attention) for _ in range(config.n_layer)])
        self.ln_f = nn.LayerNorm(config.n_embd, eps=1e-5)
        self.compute_dtype = None

    def init_weights(self, seed: int = 0) -> "GPT2":
        """N(0, 0.02) for every weight matrix and embedding, zero biases, LayerNorm gamma=1 /
        beta=0, drawn from a CPU generator so that the values do not depend on the device."""
        gen = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("bias"):
                    p.zero_()
                elif ".ln_" in name or name.startswith("ln_f"):
                    p.fill_(1.0)
                else:
                    p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, 0.02, generator=gen))
        return self

    def set_precision(self, precision: str) -> "GPT2":
        """"fp32": everything fp32. "bf16": mixed policy (see module docstring)."""
        assert precision in ("fp32", "bf16")
        if precision == "fp32":
            self.float()
            cd = None
        else:
            cd = torch.bfloat16
            for module in self.modules():
                if isinstance(module, (nn.Linear, nn.Embedding)):
                    module.to(cd)
                elif isinstance(module, nn.LayerNorm):
                    module.float()
        self.compute_dtype = cd
        for block in self.h:
            block.compute_dtype = cd
        return self

    def forward(self, idx):
        B, T = idx.size()
        pos = torch.arange(0, T, dtype=torch.long, device=idx.device)
        x = self.wte(idx).float() + self.wpe(pos).float()
        for block in self.h:
            x = block(x)
        x = self.ln_f(x)
        if self.compute_dtype is not None:
            x = x.to(self.compute_dtype)
        # tied LM head: logits = x @ wte^T, kept in fp32
        return F.linear(x, self.wte.weight).float()


def flops_per_token(config: GPTConfig, seq_len: int) -> float:
    """Forward FLOPs per token: 2 x (block GEMM weights + LM head) + causal attention."""
    d, L = config.n_embd, config.n_layer
    block = L * (d * 3 * d + d * d + d * 4 * d + 4 * d * d)
    head = d * config.vocab_size
    attn = 4 * seq_len * d * L / 2
    return 2.0 * (block + head) + attn
