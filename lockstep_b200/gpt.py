"""Decoder-only transformer used to measure the FP4 linear layer inside a
training step (structure of lockstep's train.py:38-71: pre-norm blocks, fused
qkv, GELU MLP, learned positions, tied dense head, cross-entropy).  Every block
linear is built by the `linear` factory, so passing fp4_linear.MXFP4Linear puts
the four GEMMs of each block on the MXFP4 tensor-core path; the head stays
dense, as in the reference.  Harness code: attention, norms and the optimizer
are torch's."""

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, dim, heads, linear):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv = linear(dim, 3 * dim, bias=False)
        self.proj = linear(dim, dim, bias=False)
        self.fc = linear(dim, 4 * dim, bias=False)
        self.out = linear(4 * dim, dim, bias=False)

    def forward(self, x):
        b, t, c = x.shape
        q, k, v = (z.view(b, t, self.heads, -1).transpose(1, 2) for z in self.qkv(self.ln1(x)).split(c, 2))
        att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(att.transpose(1, 2).reshape(b, t, c))
        return x + self.out(F.gelu(self.fc(self.ln2(x))))


class GPT(nn.Module):
    def __init__(self, layers, dim, heads, seq, vocab, linear):
        super().__init__()
        self.vocab = vocab
        self.wte, self.wpe = nn.Embedding(vocab, dim), nn.Embedding(seq, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, linear) for _ in range(layers))
        self.ln = nn.LayerNorm(dim)
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                std = 0.02 / math.sqrt(2 * layers) if name.endswith(("proj.weight", "out.weight")) else 0.02
                nn.init.normal_(p, std=std)

    def forward(self, idx, targets):
        h = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
        for blk in self.blocks:
            h = blk(h)
        logits = self.ln(h) @ self.wte.weight.t()
        return F.cross_entropy(logits.float().view(-1, self.vocab), targets.reshape(-1))


def training_step_time(layers=12, dim=1024, heads=16, seq=1024, batch=16, vocab=32000, backward="mxfp4",
                       steps=5, warmup=2, device="cuda", dense=False):
    """Seconds per optimizer step (CUDA events) of the model above with every
    block linear an MXFP4Linear (or nn.Linear with dense=True): bf16 autocast,
    synthetic token ids uniform in [0, vocab) from seed 0, fused AdamW."""
    from . import fp4_linear
    torch.manual_seed(0)
    if dense:
        linear = nn.Linear
    else:
        def linear(i, o, bias=False):
            return fp4_linear.MXFP4Linear(i, o, bias=bias, backward=backward)
    model = GPT(layers, dim, heads, seq, vocab, linear).to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=6e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    g = torch.Generator(device=device).manual_seed(0)
    ids = torch.randint(0, vocab, (batch, seq + 1), device=device, generator=g)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()

    def step():
        with torch.autocast("cuda", torch.bfloat16):
            loss = model(x, y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(warmup):
        loss = step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps / 1e3, float(loss.detach())
