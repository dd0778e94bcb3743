"""GPT-style decoder stages for the PipeDream-2BW configuration (24 layers, hidden 1024, 16 heads, sequence
512, vocabulary 50257).  The reference tree holds no transformer stage files (its 2BW branch lives elsewhere),
so these are written from the architecture description: pre-LayerNorm blocks, learned position embeddings,
tanh-GELU MLP of width 4h, untied output projection.  They are plain torch modules - the CPU oracle runs them
as they are, StageRuntime swaps their leaves (Linear, LayerNorm, GELU, Embedding, Dropout and the attention core)
for native ones.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


class CausalAttentionCore(nn.Module):
    """softmax(Q K^T / sqrt(d)) V with a causal mask, per head, on the fused projection's output [B, T, 3 * hidden]
    (q, k, v each [heads, d] per token).  A module of its own so that StageRuntime can swap it like any other leaf
    (layers.NativeCausalAttentionCore); this form is what the CPU oracle runs."""

    def __init__(self, heads):
        super().__init__()
        self.heads = heads

    def forward(self, qkv):
        B, T, C3 = qkv.shape
        C = C3 // 3
        qkv = qkv.view(B, T, 3, self.heads, C // self.heads)
        q, k, v = qkv[:, :, 0].transpose(1, 2), qkv[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return y.transpose(1, 2).reshape(B, T, C)


class CausalSelfAttention(nn.Module):
    def __init__(self, hidden, heads, dropout):
        super().__init__()
        assert hidden % heads == 0
        self.heads = heads
        self.c_attn = nn.Linear(hidden, 3 * hidden)
        self.core = CausalAttentionCore(heads)
        self.c_proj = nn.Linear(hidden, hidden)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        return self.drop(self.c_proj(self.core(self.c_attn(x))))


class Block(nn.Module):
    def __init__(self, hidden, heads, dropout):
        super().__init__()
        self.ln_1 = nn.LayerNorm(hidden)
        self.attn = CausalSelfAttention(hidden, heads, dropout)
        self.ln_2 = nn.LayerNorm(hidden)
        self.fc = nn.Linear(hidden, 4 * hidden)
        self.act = nn.GELU(approximate="tanh")
        self.proj = nn.Linear(4 * hidden, hidden)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.drop(self.proj(self.act(self.fc(self.ln_2(x)))))


class Embed(nn.Module):
    def __init__(self, vocab, seq_len, hidden, dropout):
        super().__init__()
        self.wte = nn.Embedding(vocab, hidden)
        self.wpe = nn.Embedding(seq_len, hidden)
        self.drop = nn.Dropout(dropout)

    def forward(self, tokens):
        pos = torch.arange(tokens.shape[1], device=tokens.device, dtype=torch.int64).unsqueeze(0).expand_as(tokens)
        return self.drop(self.wte(tokens) + self.wpe(pos))


class Head(nn.Module):
    def __init__(self, hidden, vocab):
        super().__init__()
        self.ln_f = nn.LayerNorm(hidden)
        self.lm_head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, x):
        return self.lm_head(self.ln_f(x)).view(-1, self.lm_head.out_features)


class GptStage(nn.Module):
    def __init__(self, parts):
        super().__init__()
        self.parts = nn.ModuleList(parts)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)
                if isinstance(m, nn.Linear) and m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, input0):
        out = input0
        for p in self.parts:
            out = p(out)
        return out
