"""A re-statement of the reference's O2 training step on LIBRARY kernels only - NOT the reference, and none of
this repository's kernels, models or engine.

It exists to answer one question on the same box: what do the hand-written and fused sm_100a kernels buy end to
end over the step sequence the reference runs (msamp/nn/functional.py:19-125, msamp/optim/adamw.py:148-199,
msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:404-496, 659-853) when every piece is a stock kernel?

* FP8 linear: ``abs().max()`` → power-of-two scale → cast to ``torch.float8_e4m3fn`` / ``e5m2`` → materialised
  transposes → cuBLASLt FP8 GEMMs through ``torch._scaled_mm`` (forward, dgrad, wgrad) → wgrad amax → e4m3 cast;
* LayerNorm, GeLU (tanh), cross-entropy, embedding: ATen; attention: ``scaled_dot_product_attention``;
* optimizer: per parameter, two stages (update in fp32, amax of the new moments read back to the host, then
  quantise m to e4m3 and keep v in fp16, scaled fp16 master weight) as the reference's LBAdamW does;
* data parallel (ZeRO-2 shape): FP8 weight gradients agree on a scale by a MAX all-reduce, are summed as FP8
  numbers by NCCL (``float8`` dtypes) into the owner rank, the owner updates its parameters and the FP8 weights
  are all-gathered; high-precision gradients are all-reduced in one flat bucket.

``python bench.py --impl unfused`` times it with the same clock, steps, warm-up and data as the repository's own arm.
"""
import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
FMAX = {E4M3: 448.0, E5M2: 57344.0}


def _scale_from_amax(amax, fmax):
    """Power-of-two scale rule (tensor ops, no host sync)."""
    exp = torch.floor(torch.log2(fmax / amax)).clamp(-126, 126)
    sf = torch.exp2(exp)
    return torch.where((amax > 0) & torch.isfinite(amax), sf, torch.ones_like(sf))


def _quantize(x, dtype, group=None):
    """in-time scaling: amax pass, scale, cast pass.  Returns (bytes, scale_inv)."""
    amax = x.abs().max().float()
    if group is not None:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    scale = _scale_from_amax(amax, FMAX[dtype])
    x8 = (x.float() * scale).clamp(-FMAX[dtype], FMAX[dtype]).to(dtype)
    return x8, scale.reciprocal()


def _mm(a8, b8_kn_colmajor, sa, sb, out_dtype, bias=None):
    return torch._scaled_mm(a8, b8_kn_colmajor, scale_a=sa, scale_b=sb, out_dtype=out_dtype, bias=bias)


class _FP8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        x8, x_sinv = _quantize(x, E4M3)
        x8t = x8.t().contiguous()                      # kept for wgrad
        w8, w8t, w_sinv = layer.fp8_weight()
        bias = layer.bias.to(x.dtype) if layer.bias is not None else None
        y = _mm(x8, w8.t(), x_sinv, w_sinv, x.dtype, bias)
        ctx.save_for_backward(x8t, x_sinv, w8t, w_sinv)
        ctx.layer = layer
        return y

    @staticmethod
    def backward(ctx, dy):
        x8t, x_sinv, w8t, w_sinv = ctx.saved_tensors
        layer = ctx.layer
        dy = dy.contiguous()
        dy8, dy_sinv = _quantize(dy, E5M2)
        dy8t = dy8.t().contiguous()
        dx = _mm(dy8, w8t.t(), dy_sinv, w_sinv, dy.dtype)
        wgrad = _mm(dy8t, x8t.t(), dy_sinv, x_sinv, dy.dtype)
        if layer.bias is not None:
            g = dy.sum(0, dtype=torch.float32)
            layer.bias.grad = g if layer.bias.grad is None else layer.bias.grad + g
        layer.deliver_wgrad(wgrad)
        return dx, None


class Linear(torch.nn.Module):
    """FP8 linear of the O2 recipe: scaled fp16 master weight, e4m3 weight gradient."""
    def __init__(self, k, n, bias, std, dev, group=None):
        super().__init__()
        w = torch.randn(n, k, device=dev) * std
        self.w_amax = w.abs().max()
        self.w_scale = _scale_from_amax(self.w_amax, 65504.0 / 2)    # master = w * scale in fp16
        self.master = (w * self.w_scale).half()
        self.bias = torch.nn.Parameter(torch.zeros(n, device=dev)) if bias else None
        self.grad8 = None
        self.grad_sinv = None
        self.group = group
        self._cache = None
        # optimizer state: m in e4m3 with a scale, v in fp16 with a scale
        self.m8 = torch.zeros(n, k, device=dev, dtype=E4M3)
        self.m_sinv = torch.ones((), device=dev)
        self.v16 = torch.zeros(n, k, device=dev, dtype=torch.float16)
        self.v_sinv = torch.ones((), device=dev)

    def fp8_weight(self):
        if self._cache is None:
            scale = _scale_from_amax(self.w_amax, FMAX[E4M3])
            w8 = (self.master.float() * (scale / self.w_scale)).clamp(-448, 448).to(E4M3)
            self._cache = (w8, w8.t().contiguous(), scale.reciprocal())
        return self._cache

    def deliver_wgrad(self, wgrad):
        # the amax is agreed across the data-parallel group so that the FP8 bytes can be summed directly
        self.grad8, self.grad_sinv = _quantize(wgrad, E4M3, self.group if (self.group is not None and dist.get_world_size(self.group) > 1) else None)

    def forward(self, x):
        return _FP8Linear.apply(x, self)


class Block(torch.nn.Module):
    def __init__(self, h, f, nh, n_layer, dev, group):
        super().__init__()
        self.nh = nh
        self.ln1 = torch.nn.LayerNorm(h, device=dev, dtype=torch.bfloat16)
        self.ln2 = torch.nn.LayerNorm(h, device=dev, dtype=torch.bfloat16)
        self.qkv = Linear(h, 3 * h, True, 0.02, dev, group)
        self.proj = Linear(h, h, True, 0.02 / math.sqrt(2 * n_layer), dev, group)
        self.fc1 = Linear(h, f, True, 0.02, dev, group)
        self.fc2 = Linear(f, h, True, 0.02 / math.sqrt(2 * n_layer), dev, group)

    def forward(self, x, B, S):
        qkv = self.qkv(self.ln1(x)).view(B, S, 3, self.nh, -1)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B * S, -1)
        x = x + self.proj(o)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate='tanh'))


class UnfusedGPT(torch.nn.Module):
    def __init__(self, cfg, dev, group=None):
        super().__init__()
        h = cfg.hidden
        self.cfg = cfg
        self.wte = torch.nn.Embedding(cfg.vocab_size, h, device=dev, dtype=torch.bfloat16)
        self.wpe = torch.nn.Embedding(cfg.max_seq, h, device=dev, dtype=torch.bfloat16)
        self.blocks = torch.nn.ModuleList(Block(h, cfg.ffn_hidden, cfg.n_head, cfg.n_layer, dev, group) for _ in range(cfg.n_layer))
        self.ln_f = torch.nn.LayerNorm(h, device=dev, dtype=torch.bfloat16)
        self.lm_head = Linear(h, cfg.vocab_size, False, 0.02, dev, group)
        with torch.no_grad():
            self.wte.weight.normal_(0, 0.02)
            self.wpe.weight.normal_(0, 0.02)

    def forward(self, tok, lab):
        B, S = tok.shape
        x = (self.wte(tok) + self.wpe(torch.arange(S, device=tok.device))).view(B * S, -1)
        for blk in self.blocks:
            x = blk(x, B, S)
        logits = self.lm_head(self.ln_f(x))
        return F.cross_entropy(logits.float(), lab.reshape(-1))


class UnfusedTrainer:
    """forward + backward + gradient exchange + per-parameter two-stage low-bit AdamW."""
    def __init__(self, model, lr=1e-4, betas=(0.9, 0.95), wd=0.1, eps=1e-8, group=None):
        self.model, self.lr, self.betas, self.wd, self.eps = model, lr, betas, wd, eps
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.fp8 = [m for m in model.modules() if isinstance(m, Linear)]
        self.hp = [p for p in model.parameters()]
        self.hp_opt = torch.optim.AdamW(self.hp, lr=lr, betas=betas, weight_decay=wd)
        # ZeRO-2 shape: FP8 parameters are dealt to ranks largest first
        order = sorted(range(len(self.fp8)), key=lambda i: -self.fp8[i].master.numel())
        load = [0] * self.world
        self.owner = {}
        for i in order:
            r = load.index(min(load))
            self.owner[i] = r
            load[r] += self.fp8[i].master.numel()
        self.t = 0

    def _adam_fp8(self, lin):
        b1, b2 = self.betas
        g = lin.grad8.float() * (lin.grad_sinv / self.world)
        m = lin.m8.float() * lin.m_sinv
        v = lin.v16.float() * lin.v_sinv
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        bc1, bc2 = 1 - b1**self.t, 1 - b2**self.t
        w = lin.master.float() / lin.w_scale
        w = w * (1 - self.lr * self.wd) - (self.lr / bc1) * m / ((v / bc2).sqrt() + self.eps)
        # stage boundary: the amaxes of the new moments and weight come back to the host (the reference's two syncs)
        am_m, am_v = m.abs().max().item(), v.abs().max().item()
        am_w = w.abs().max()
        ms = 2.0**math.floor(math.log2(448.0 / am_m)) if am_m > 0 else 1.0
        vs = 2.0**math.floor(math.log2(65504.0 / am_v)) if am_v > 0 else 1.0
        lin.m8 = (m * ms).clamp(-448, 448).to(E4M3)
        lin.m_sinv.fill_(1.0 / ms)
        lin.v16 = (v * vs).half()
        lin.v_sinv.fill_(1.0 / vs)
        lin.w_amax = am_w
        lin.w_scale = _scale_from_amax(am_w, 65504.0 / 2)
        lin.master = (w * lin.w_scale).half()
        lin._cache = None
        lin.grad8 = None

    def step(self, tok, lab):
        self.t += 1
        for p in self.hp:
            p.grad = None
        loss = self.model(tok, lab)
        loss.backward()
        if self.world > 1:
            works = []
            for i, lin in enumerate(self.fp8):    # FP8 sum into the owner, one reduce per parameter
                works.append(dist.reduce(lin.grad8.view(-1), dst=dist.get_global_rank(self.group, self.owner[i]), group=self.group, async_op=True))
            grads = [p.grad for p in self.hp if p.grad is not None]
            flat = torch.cat([g.reshape(-1).float() for g in grads])
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world)
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
            for w in works:
                w.wait()
        for i, lin in enumerate(self.fp8):
            if self.owner[i] == self.rank:
                self._adam_fp8(lin)
        self.hp_opt.step()
        if self.world > 1:
            for i, lin in enumerate(self.fp8):    # updated weights (scaled fp16 master stands in for the FP8 all-gather + scale_inv gather)
                src = dist.get_global_rank(self.group, self.owner[i])
                w8, _, sinv = lin.fp8_weight() if self.owner[i] == self.rank else (torch.empty_like(lin.m8), None, torch.empty((), device=lin.m8.device))
                dist.broadcast(w8.view(torch.uint8), src=src, group=self.group)
                dist.broadcast(sinv, src=src, group=self.group)
                if self.owner[i] != self.rank:
                    lin._cache = (w8, w8.t().contiguous(), sinv)
                    lin.grad8 = None
        return loss.detach()
