"""Training-step harness for the FP4 linear layer (benchmark code, not part of the package).

A small decoder-only language model with the layer plan lockstep's train.py uses for
its own measurements (pre-norm residual blocks, one fused query/key/value projection,
a GELU feed-forward of width 4 x d, learned position embeddings, an output head tied
to the token embedding, cross-entropy on the next token), so that tokens/s is measured
where the reference measures it.  Everything that is not one of the four block
projections is torch's: attention, layer norm, softmax, the optimizer.

The four projections of every block come from `make_linear`:
  "dense"   nn.Linear (cuBLAS bf16 under autocast)             -- the comparison point
  "ste"     MXFP4Linear, straight-through bf16 backward        -- lockstep's fp4_linear.py
  "mxfp4"   MXFP4Linear with MXFP4 dgrad / wgrad as well
  "nvfp4"   NVFP4Linear (blocks of 16 under E4M3 scales), straight-through backward

    python train_bench.py --kind mxfp4            # tokens/s
    python train_bench.py --kind mxfp4 --kernels  # device time per kernel of one step

Gradient sync follows train.py:100-105,124-138: all gradients live in one flat fp32
buffer that a `wire.Wire` averages in place after the backward pass.
"""

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def make_linear(kind):
    from lockstep_b200 import fp4_linear
    if kind == "dense":
        return lambda fan_in, fan_out: nn.Linear(fan_in, fan_out, bias=False)
    if kind == "nvfp4":
        return lambda fan_in, fan_out: fp4_linear.NVFP4Linear(fan_in, fan_out, bias=False)
    return lambda fan_in, fan_out: fp4_linear.MXFP4Linear(fan_in, fan_out, bias=False, backward=kind)


class CausalSelfAttention(nn.Module):
    """Pre-norm attention branch: proj(attention(qkv(norm(x)))).  `normed_qkv` builds the norm
    and the qkv projection together (the fused LayerNorm + quantize module) or separately."""

    def __init__(self, width, heads, linear, normed_qkv):
        super().__init__()
        self.heads = heads
        self.qkv = normed_qkv(width, 3 * width)
        self.proj = linear(width, width)

    def forward(self, x):
        batch, steps, width = x.shape
        # three views of the projection's output, each [batch, heads, steps, head_dim]; no copy here, and one
        # concatenation of the three gradients in backward (train.py:47-48 splits the same way)
        q, k, v = (part.view(batch, steps, self.heads, width // self.heads).transpose(1, 2)
                   for part in self.qkv(x).split(width, dim=2))
        mixed = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(mixed.transpose(1, 2).reshape(batch, steps, width))


class NormThen(nn.Module):
    """norm followed by a module: the unfused form of the fused norm + projection modules."""

    def __init__(self, width, inner):
        super().__init__()
        self.norm = nn.LayerNorm(width)
        self.inner = inner

    def forward(self, x):
        return self.inner(self.norm(x))


class FeedForward(nn.Module):
    def __init__(self, width, linear):
        super().__init__()
        self.fc = linear(width, 4 * width)
        self.out = linear(4 * width, width)

    def forward(self, x):
        return self.out(F.gelu(self.fc(x)))


def make_parts(kind, fused):
    """(linear, normed_qkv, normed_mlp) factories for a block.  fused (MXFP4 kinds only): the
    LayerNorm in front of qkv and fc is fused with the quantization of its output, and with
    kind "mxfp4" the feed-forward half keeps its activation in MXFP4 between its two GEMMs."""
    from lockstep_b200 import fp4_linear
    linear = make_linear(kind)
    if fused and kind not in ("dense", "nvfp4"):
        return (linear,
                lambda width, out: fp4_linear.MXFP4NormLinear(width, out, backward=kind),
                lambda width: fp4_linear.MXFP4MLP(width, 4 * width, backward=kind, norm=True))
    return (linear,
            lambda width, out: NormThen(width, linear(width, out)),
            lambda width: NormThen(width, FeedForward(width, linear)))


class Block(nn.Module):
    def __init__(self, width, heads, parts):
        super().__init__()
        linear, normed_qkv, normed_mlp = parts
        self.attn = CausalSelfAttention(width, heads, linear, normed_qkv)
        self.mlp = normed_mlp(width)

    def forward(self, x):
        x = x + self.attn(x)
        return x + self.mlp(x)


class Decoder(nn.Module):
    def __init__(self, layers, width, heads, context, vocab, parts):
        super().__init__()
        self.vocab = vocab
        self.tokens = nn.Embedding(vocab, width)
        self.positions = nn.Embedding(context, width)
        self.blocks = nn.ModuleList([Block(width, heads, parts) for _ in range(layers)])
        self.norm = nn.LayerNorm(width)
        # N(0, 0.02) for every matrix; the two projections that write into the residual
        # stream are scaled down by sqrt(2 * layers), as train.py:66-69 does
        shrink = 1.0 / math.sqrt(2 * layers)
        for name, p in self.named_parameters():
            if p.dim() < 2:
                continue
            residual_writer = name.endswith("attn.proj.weight") or name.endswith("out.weight")
            nn.init.normal_(p, std=0.02 * (shrink if residual_writer else 1.0))

    def forward(self, ids, targets):
        where = torch.arange(ids.shape[1], device=ids.device)
        h = self.tokens(ids) + self.positions(where)
        for block in self.blocks:
            h = block(h)
        logits = F.linear(self.norm(h), self.tokens.weight)          # tied head, dense
        return F.cross_entropy(logits.float().view(-1, self.vocab), targets.reshape(-1))


class Trainer:
    """Model + fused AdamW + a flat fp32 gradient buffer averaged by the FP4 wire.

    overlap=False: one Wire over the whole buffer, called after the backward pass
    (train.py:124-138).  overlap=True: the buffer is cut into `buckets` contiguous slices at
    parameter boundaries, each with its own Wire; as soon as the last gradient of a slice
    has been accumulated, that slice's send phase (encode + push to the owners) is queued
    on a side stream and runs under the rest of the backward pass; the owner and decode
    phases follow after the backward pass."""

    def __init__(self, kind="mxfp4", layers=12, width=1024, heads=16, context=1024, batch=16, vocab=32000,
                 device="cuda", wire_method="mxfp4ef", world=1, rank=0, overlap=False, buckets=4, fused=True):
        from lockstep_b200 import wire
        torch.manual_seed(0)
        self.model = Decoder(layers, width, heads, context, vocab, make_parts(kind, fused)).to(device)
        self.params = list(self.model.parameters())
        self.flat = torch.zeros(sum(p.numel() for p in self.params), device=device)
        at, spans = 0, []
        for p in self.params:                                  # every gradient is a view of the flat buffer
            p.grad = self.flat[at:at + p.numel()].view_as(p)
            spans.append((at, at + p.numel()))
            at += p.numel()
        self.overlap = bool(overlap and wire_method)
        self.sync, self.parts = None, []
        if wire_method and not self.overlap:
            self.sync = wire.Wire(wire_method, self.flat.numel(), world, rank)
        elif self.overlap:
            # contiguous groups of parameters of about equal size; a slice starts on a 32-byte boundary
            target, lo, members = self.flat.numel() / buckets, 0, []
            for i, (a, b) in enumerate(spans):
                members.append(i)
                last = i == len(spans) - 1
                if last or (b - lo >= target and b % 8 == 0 and len(self.parts) < buckets - 1):
                    w = wire.Wire(wire_method, b - lo, world, rank)
                    w.set_mode("launches", device=torch.device(device) if not isinstance(device, torch.device) else device)
                    self.parts.append({"wire": w, "grad": self.flat[lo:b], "members": members, "pending": 0,
                                       "sent": torch.cuda.Event()})
                    lo, members = b, []
            self.side = torch.cuda.Stream()
            self.ready = torch.cuda.Event()
            for part in self.parts:
                for i in part["members"]:
                    self.params[i].register_post_accumulate_grad_hook(self._hook(part))
        decay = [p for p in self.params if p.dim() >= 2]
        rest = [p for p in self.params if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                                     lr=6e-4, betas=(0.9, 0.95), fused=True)
        gen = torch.Generator(device=device).manual_seed(rank)
        ids = torch.randint(0, vocab, (batch, context + 1), device=device, generator=gen)
        self.x, self.y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        self.tokens_per_step = batch * context

    def _hook(self, part):
        def fire(_param):
            part["pending"] -= 1
            if part["pending"] == 0:                          # the slice is final: send it under the rest of backward
                main = torch.cuda.current_stream()
                self.ready.record(main)
                with torch.cuda.stream(self.side):
                    self.side.wait_event(self.ready)
                    part["wire"].send(part["grad"])
                    part["sent"].record(self.side)
        return fire

    def step(self):
        self.flat.zero_()
        for part in self.parts:
            part["pending"] = len(part["members"])
        with torch.autocast("cuda", torch.bfloat16):
            loss = self.model(self.x, self.y)
        loss.backward()
        if self.sync is not None:
            self.sync(self.flat)
        main = torch.cuda.current_stream()
        for part in reversed(self.parts):                      # the order the slices were sent in
            main.wait_event(part["sent"])
            part["wire"].reduce()
            part["wire"].finish(part["grad"])
        torch.nn.utils.clip_grad_norm_(self.params, 1.0)
        self.opt.step()
        return loss

    def time(self, steps=5, warmup=2):
        """(seconds per step by CUDA events, last loss)."""
        for _ in range(warmup):
            loss = self.step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            loss = self.step()
        b.record()
        torch.cuda.synchronize()
        for w in [self.sync] + [part["wire"] for part in self.parts]:
            if w is not None:
                w.status()
        return a.elapsed_time(b) / steps / 1e3, float(loss.detach())

    def close(self):
        for w in [self.sync] + [part["wire"] for part in self.parts]:
            if w is not None:
                w.close()


def training_step_time(kind="mxfp4", steps=5, warmup=2, **kw):
    t = Trainer(kind, **kw)
    out = t.time(steps, warmup)
    t.close()
    return out


def report(device, steps=5, warmup=2, world=1, rank=0):
    """The `train_step` object of the benchmark line: tokens/s of the 12-layer configuration
    with each kind of block projection (one rank only), and the step time with the gradient
    sync after the backward pass against the bucketed sync that sends under it."""
    out = {}
    runs = (("dense", "dense", False), ("ste", "ste", True), ("ste_unfused", "ste", False), ("mxfp4", "mxfp4", True),
            ("mxfp4_unfused", "mxfp4", False), ("nvfp4_ste_unfused", "nvfp4", False)) if world == 1 else (("mxfp4", "mxfp4", True),)
    for name, kind, fused in runs:
        torch.cuda.empty_cache()
        t = Trainer(kind, device=device, world=world, rank=rank, fused=fused)
        sec, loss = t.time(steps, warmup)
        out[name] = {"tokens_per_s": world * t.tokens_per_step / sec, "ms_per_step": sec * 1e3, "loss": loss}
        t.close()
        del t
    torch.cuda.empty_cache()
    t = Trainer("mxfp4", device=device, world=world, rank=rank, overlap=True)
    sec, loss = t.time(steps, warmup)
    t.close()
    res = {"model": "decoder-only 12L d1024 h16 ffn4096 seq1024 batch16 per rank vocab32000, bf16 autocast, fused AdamW, "
                    "synthetic ids seeded by rank; gradients in one flat fp32 buffer averaged by Wire('mxfp4ef') every step",
           "block_linears": out,
           "fused": "ste / mxfp4: LayerNorm fused with the quantization of its output in front of qkv and fc "
                    "(fp4_linear.MXFP4NormLinear); mxfp4: the feed-forward half is fp4_linear.MXFP4MLP (GELU applied "
                    "inside the quantizer of the second GEMM's input; the activation never exists in HBM); "
                    "*_unfused: separate LayerNorm, GELU and quantizer passes",
           "sync": {"after_backward_ms": out["mxfp4"]["ms_per_step"], "sent_under_backward_ms": sec * 1e3,
                    "buckets": len(t.parts), "loss": loss}}
    if world == 1:
        res["mxfp4_vs_dense"] = out["mxfp4"]["tokens_per_s"] / out["dense"]["tokens_per_s"]
        res["ste_vs_dense"] = out["ste"]["tokens_per_s"] / out["dense"]["tokens_per_s"]
    return res


def kernel_table(kind="mxfp4", fused=True, steps=3, top=24, device=None):
    """Device time per kernel of one training step (torch profiler, CUDA activity only): a list of
    (microseconds per step, launches per step, kernel name) sorted by time, and the total."""
    from torch.profiler import ProfilerActivity, profile
    device = device or torch.device("cuda", 0)
    t = Trainer(kind, device=device, fused=fused)
    for _ in range(3):
        t.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            t.step()
        torch.cuda.synchronize()
    t.close()
    rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in rows) / steps
    return [(e.device_time_total / steps, e.count // steps, e.key) for e in rows[:top]], total


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="tokens/s of the 12-layer configuration, or the kernel list of one step")
    ap.add_argument("--kind", default="mxfp4", choices=["dense", "ste", "mxfp4", "nvfp4"])
    ap.add_argument("--unfused", action="store_true", help="separate LayerNorm, GELU and quantizer passes")
    ap.add_argument("--kernels", action="store_true", help="print device time per kernel of one step instead")
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args()
    if a.kernels:
        rows, total = kernel_table(a.kind, not a.unfused)
        print(f"{total:10.1f} us of device time per step ({a.kind}, {'unfused' if a.unfused else 'fused'})")
        for us, n, name in rows:
            print(f"{us:10.1f} us  x{n:4d}  {name[:120]}")
    else:
        t = Trainer(a.kind, device=torch.device("cuda", 0), fused=not a.unfused)
        sec, loss = t.time(a.steps, 2)
        t.close()
        print(f"{a.kind}: {t.tokens_per_step / sec:.0f} tokens/s, {sec * 1e3:.2f} ms per step, loss {loss:.4f}")
