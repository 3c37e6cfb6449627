"""CPU engine that drives the oracle layer functions from autograd hooks.  TEST INFRASTRUCTURE ONLY.

It follows the control flow of the reference's hook plumbing
(ghostEngines/autograd_grad_sample_dotprod.py:23-196 and ghostEngines/graddotprod_engine.py:64-230)
with the layer math of ``oracle.ghost_oracle``: the ``*_reference`` functions by default (the
reference's own arithmetic, including its 2*T^2 <= numel path rule), or the float64 ``*_exact``
matrices with ``exact=True``.  Used to check whole-model results of the CUDA engine and as the
timed CPU baseline; the shipped package never imports it.
"""
from __future__ import annotations

import torch
from torch import nn

from . import ghost_oracle as O

try:
    from transformers.pytorch_utils import Conv1D as _HFConv1D
except Exception:  # pragma: no cover
    _HFConv1D = ()


def _is_conv1d(layer) -> bool:
    return layer.__class__.__name__ == "Conv1D"


def _supported(layer) -> bool:
    return isinstance(layer, (nn.Linear, nn.Embedding, nn.LayerNorm)) or _is_conv1d(layer)


class OracleDotProdEngine:
    """``attach()`` / ``detach()`` / ``prepare_gradients()`` / ``clear_gradients()`` like the real
    engine.  After a backward pass every hooked parameter carries ``grad_dot_prod`` (and, with
    ``exact=True``, ``grad_dot_prod_matrix``) and ``train_grad``; ``records`` maps
    ``(module_name, 'weight'|'bias')`` to the value computed in that module's hook, which is what
    parity is checked on when parameters are tied."""

    def __init__(self, module: nn.Module, val_batch_size: int, use_dummy_bias: bool = False,
                 exact: bool = False):
        self.module = module
        self.n_val = val_batch_size
        self.exact = exact
        self.handles = []
        self.records = {}
        for p in module.parameters():
            p.initially_requires_grad = bool(p.requires_grad)
            p.requires_grad = not use_dummy_bias
        prep = getattr(module, "ghost_prepare", None)
        if callable(prep):
            prep()

    def attach(self):
        for name, layer in self.module.named_modules():
            if _supported(layer) and any(getattr(p, "initially_requires_grad", False) for p in layer.parameters()):
                self.handles.append(layer.register_forward_hook(self._fwd))
                self.handles.append(layer.register_full_backward_hook(self._make_bwd(name)))

    def detach(self):
        for h in self.handles:
            h.remove()
        self.handles.clear()

    @staticmethod
    def _fwd(layer, inputs, output):
        layer._oracle_A = inputs[0].detach()

    def _store(self, name, role, param, value):
        self.records[(name, role)] = value
        if value.dim() == 2:
            param.grad_dot_prod_matrix = value
            param.grad_dot_prod = value.sum(0)
        else:
            param.grad_dot_prod = value

    @staticmethod
    def _acc(param, grad):
        if hasattr(param, "train_grad"):
            param.train_grad.add_(grad)
        else:
            param.train_grad = grad

    def _make_bwd(self, name):
        def bwd(layer, grad_input, grad_output):
            B = grad_output[0].detach()
            A = layer._oracle_A
            if A.is_floating_point() and A.dtype != B.dtype:
                common = torch.promote_types(A.dtype, B.dtype)
                A, B = A.to(common), B.to(common)
            nv = self.n_val
            N = B.shape[0]
            Bs = B * N
            if isinstance(layer, nn.Linear) or _is_conv1d(layer):
                T = O.flatten_tokens(A).shape[1]
                ghost = O.use_gram_rule(T, layer.weight.numel())
                if self.exact:
                    w = O.linear_dot_exact(A, B, nv)
                elif _is_conv1d(layer):
                    w = O.conv1d_dot_reference(A, B, nv, ghost)
                else:
                    w = O.linear_dot_reference(A, B, nv, ghost)
                self._store(name, "weight", layer.weight, w)
                if layer.bias is not None:
                    b = O.bias_dot_exact(B, nv) if self.exact else O.bias_dot_reference(
                        B.to(torch.bfloat16) if _is_conv1d(layer) else B, nv)
                    self._store(name, "bias", layer.bias, b)
                if layer.weight.initially_requires_grad:
                    g = O.conv1d_train_grad(A, Bs, nv) if _is_conv1d(layer) else O.linear_train_grad(A, Bs, nv)
                    self._acc(layer.weight, g)
                if layer.bias is not None and layer.bias.initially_requires_grad:
                    self._acc(layer.bias, O.bias_train_grad(Bs.clone(), nv))
            elif isinstance(layer, nn.Embedding):
                vocab = layer.weight.shape[0]
                w = O.embedding_dot_exact(A, B, nv) if self.exact else O.embedding_dot_reference(A, B, nv, vocab)
                self._store(name, "weight", layer.weight, w)
                if layer.weight.initially_requires_grad:
                    self._acc(layer.weight, O.embedding_train_grad(A, Bs, nv, vocab, sequential=False))
            elif isinstance(layer, nn.LayerNorm):
                if self.exact:
                    w, b = O.layernorm_dot_exact(A, B, nv, layer.eps)
                else:
                    w, b = O.layernorm_dot_reference(A, B, nv, layer.eps)
                self._store(name, "weight", layer.weight, w)
                self._store(name, "bias", layer.bias, b)
                gw, gb = O.layernorm_train_grad(A, Bs, nv, layer.eps)
                self._acc(layer.weight, gw)
                self._acc(layer.bias, gb)
            del layer._oracle_A
        return bwd

    def prepare_gradients(self):
        for name, p in self.module.named_parameters():
            if p.initially_requires_grad and "dummy_bias" not in name and hasattr(p, "train_grad"):
                p.grad = p.train_grad

    def clear_gradients(self):
        for p in self.module.parameters():
            for attr in ("train_grad", "grad_dot_prod", "grad_dot_prod_matrix"):
                if hasattr(p, attr):
                    delattr(p, attr)

    def aggregate(self):
        total = None
        for _, p in self.module.named_parameters():
            if hasattr(p, "grad_dot_prod") and p.initially_requires_grad:
                total = p.grad_dot_prod.clone().float() if total is None else total + p.grad_dot_prod.float()
        return total
