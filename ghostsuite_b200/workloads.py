"""Synthetic workloads with the architectures the benchmarks are quoted on (random init, random
token ids; no datasets or checkpoints are involved).

``GPT2Like`` is a GPT-2-architecture decoder built from the layer types the ghost hooks support
(nn.Embedding, nn.LayerNorm, Hugging Face ``Conv1D`` for the four projections per block, nn.Linear
for the LM head tied to the token embedding) so the whole model is covered by the engine without
any forward patching: position ids are always expanded to ``[batch, T]``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

try:
    from transformers.pytorch_utils import Conv1D
except Exception:  # pragma: no cover - transformers is part of the supported environment
    class Conv1D(nn.Module):
        """``y = x @ W + b`` with ``W`` stored ``[in, out]`` (Hugging Face GPT-2 convention)."""

        def __init__(self, nf: int, nx: int):
            super().__init__()
            self.nf = nf
            self.weight = nn.Parameter(torch.empty(nx, nf))
            self.bias = nn.Parameter(torch.zeros(nf))
            nn.init.normal_(self.weight, std=0.02)

        def forward(self, x):
            size_out = x.size()[:-1] + (self.nf,)
            return torch.addmm(self.bias, x.view(-1, x.size(-1)), self.weight).view(size_out)


class _FusedTokenLoss(torch.autograd.Function):
    """Mean next-token cross-entropy over the first ``valid_cols`` logit columns from the library's
    streaming kernels.  When the logits need a gradient and their rows are dense, the forward kernel
    reads them once from HBM and also writes the gradient for an upstream gradient of 1 (in the
    logits' dtype); the backward only rescales it in place, a no-op for ``loss.backward()``.
    Otherwise the gradient comes from a second kernel in the backward.  The usual fp32-copy +
    log-softmax formulation moves the tensor through HBM about ten times."""

    @staticmethod
    def forward(ctx, logits2d, target, valid_cols):
        from . import ops
        n_valid = (target != -100).sum().to(torch.float32)
        vec = 8 if logits2d.dtype == torch.bfloat16 else 4
        fuse = ctx.needs_input_grad[0] and logits2d.shape[1] % vec == 0
        ctx.valid_cols = valid_cols
        ctx.fused = fuse
        if fuse:
            inv = (1.0 / n_valid).reshape(1)
            _, loss_rows, dlogits = ops.ce_forward(logits2d, target, valid_cols, grad_scale=inv)
            # kept on the context, not through save_for_backward: both are updated in place by the
            # backward.  `applied` is the factor already folded into dlogits, so that a second
            # backward through a retained graph rescales by the ratio, not by the upstream again
            ctx.dlogits = dlogits
            ctx.applied = torch.ones(1, dtype=torch.float32, device=dlogits.device)
        else:
            lse, loss_rows = ops.ce_forward(logits2d, target, valid_cols)
            ctx.save_for_backward(logits2d, target, lse, n_valid)
        return loss_rows.sum() / n_valid

    @staticmethod
    def backward(ctx, grad_out):
        from . import ops
        if ctx.fused:
            dlogits, applied = ctx.dlogits, ctx.applied
            up = grad_out.to(torch.float32).reshape(1)
            factor = up / applied
            applied.copy_(up)
            return ops.ce_rescale_(dlogits, factor), None, None
        logits2d, target, lse, n_valid = ctx.saved_tensors
        scale = (grad_out.to(torch.float32) / n_valid).reshape(1).contiguous()
        return ops.ce_backward(logits2d, target, ctx.valid_cols, lse, scale), None, None


def _fused_loss_ok(flat: torch.Tensor) -> bool:
    from . import ops
    return ops.ce_supported(flat)


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    tie_weights: bool = True
    #: rows of the token-embedding / LM-head table are padded to a multiple of this (GPT-2's 50257
    #: becomes 50304, as nanoGPT-style trainers and the reference's own model factory do): an odd
    #: vocabulary size makes every cuBLAS GEMM on the logits fall back to unaligned legacy kernels.
    #: Token ids stay below vocab_size and the padded logits never enter the loss.
    pad_vocab_to: int = 64
    #: on a GPU the loss comes from the library's fused cross-entropy kernels; False = torch ops
    fused_loss: bool = True

    @property
    def padded_vocab(self) -> int:
        m = max(1, self.pad_vocab_to)
        return (self.vocab_size + m - 1) // m * m


class _Attention(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head = cfg.n_head
        self.c_attn = Conv1D(3 * cfg.n_embd, cfg.n_embd)
        self.c_proj = Conv1D(cfg.n_embd, cfg.n_embd)

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.c_attn(x).split(C, dim=2)
        hd = C // self.n_head
        q = q.view(B, T, self.n_head, hd).transpose(1, 2)
        k = k.view(B, T, self.n_head, hd).transpose(1, 2)
        v = v.view(B, T, self.n_head, hd).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.c_proj(y.transpose(1, 2).reshape(B, T, C))


class _MLP(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.c_fc = Conv1D(4 * cfg.n_embd, cfg.n_embd)
        self.c_proj = Conv1D(cfg.n_embd, 4 * cfg.n_embd)

    def forward(self, x):
        return self.c_proj(F.gelu(self.c_fc(x), approximate="tanh"))


class _Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln_1 = nn.LayerNorm(cfg.n_embd)
        self.attn = _Attention(cfg)
        self.ln_2 = nn.LayerNorm(cfg.n_embd)
        self.mlp = _MLP(cfg)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class GPT2Like(nn.Module):
    """GPT-2 architecture; ``forward(input_ids, labels=None)`` returns ``(loss, logits)``."""

    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.padded_vocab, cfg.n_embd)
        self.wpe = nn.Embedding(cfg.n_positions, cfg.n_embd)
        self.h = nn.ModuleList(_Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.n_embd)
        self.lm_head = nn.Linear(cfg.n_embd, cfg.padded_vocab, bias=False)
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * cfg.n_layer))
        if cfg.tie_weights:
            self.lm_head.weight = self.wte.weight

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, Conv1D)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def ghost_prepare(self):
        """Called by the ghost engines: embeddings get the one-element dummy bias that keeps the
        autograd graph alive when every real parameter has requires_grad=False."""
        from .ghostEngines.transformers_support import _add_dummy_bias
        _add_dummy_bias(self.wte)
        _add_dummy_bias(self.wpe)

    def forward(self, input_ids, labels=None):
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device).unsqueeze(0).expand(B, T)
        x = self.wte(input_ids) + self.wpe(pos)
        for blk in self.h:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        loss = None
        if labels is not None:
            # next-token loss in fp32 without copying the logits for the shift: the targets are
            # shifted instead and the last position of every sequence is ignored
            V = self.cfg.vocab_size
            target = torch.cat((labels[:, 1:], labels.new_full((B, 1), -100)), dim=1).reshape(-1)
            flat = logits.reshape(-1, logits.size(-1))
            if self.cfg.fused_loss and flat.is_cuda and _fused_loss_ok(flat):
                loss = _FusedTokenLoss.apply(flat, target, V)
            else:
                # an fp32 copy that is safe to edit in place (for an fp32 model .float() is a no-op view)
                flat = flat.float() if flat.dtype != torch.float32 else flat.clone()
                if flat.size(-1) != V:
                    flat[:, V:] = float("-inf")        # padded classes take no probability mass
                loss = F.cross_entropy(flat, target, ignore_index=-100)
        return loss, logits


def make_mlp(in_dim: int = 512, hidden: int = 1024, out_dim: int = 10) -> nn.Sequential:
    """The Linear+ReLU MLP of the fp32 GradDotProd configuration (512 -> 1024 -> 1024 -> 10)."""
    return nn.Sequential(nn.Linear(in_dim, hidden), nn.ReLU(), nn.Linear(hidden, hidden), nn.ReLU(),
                         nn.Linear(hidden, out_dim))
