"""Forward/backward hooks that compute Kronecker-projected per-sample gradients.

Drop-in for GhostSuite's ``ghostEngines/gradProjection/autograd_gradproj.py``: ``GradProjHooks``
keeps its constructor and hook methods (:47-118), ``module._ghost_A_raw`` / ``module._ghost_grad_proj``
keep their meaning, ``create_projection_hooks`` keeps its layer-type rules (:239-283).  The dense
projection (:120-165) runs in one fused kernel that streams the activations and output gradients
once; when the engine supplies a destination (``bind_output``) the result is written straight into
that layer's column slice of the engine's ``[B, total_proj_dim]`` buffer, so collecting a batch
needs no reshape/cat pass.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn

from ... import ops


def _flatten_tokens(x: torch.Tensor) -> torch.Tensor:
    """``[B, D] -> [B, 1, D]``; ``[B, ..., D] -> [B, T, D]``."""
    if x.dim() <= 2:
        return x.unsqueeze(1)
    return x.reshape(x.shape[0], -1, x.shape[-1])


def _extract_batch_size(x: torch.Tensor) -> int:
    return 1 if x.dim() == 0 else x.shape[0]


class GradProjHooks:
    """Projection matrices of one layer plus the two hook functions."""

    def __init__(self, P_i: torch.Tensor, P_o: torch.Tensor, layer_name: str, layer_type: str):
        self.P_i = P_i            # [k_i, n_i] float32
        self.P_o = P_o            # [k_o, n_o] float32
        self.layer_name = layer_name
        self.layer_type = layer_type
        self._handle_forward = None
        self._handle_backward = None
        self._kernel_P = {}       # split flag -> (P_i, P_o) in the kernel's bf16 layout
        self._P_i_t = None        # embedding layers: float32 [vocab, k_i] transpose of P_i
        self._out_fn: Optional[Callable[[int], torch.Tensor]] = None

    # -- engine integration ------------------------------------------------------------------
    def bind_output(self, out_fn: Optional[Callable[[int], torch.Tensor]]) -> None:
        """``out_fn(batch_size)`` returns the float32 ``[B, k_i*k_o]`` view this layer writes to."""
        self._out_fn = out_fn

    def _prepared(self, split: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        if split not in self._kernel_P:
            # an embedding's P_i [k_i, vocab] is gathered by token id, never multiplied: no bf16 copy
            P_i = None if self.layer_type == "Embedding" else ops.prepare_projection(self.P_i, split)
            self._kernel_P[split] = (P_i, ops.prepare_projection(self.P_o, split))
        return self._kernel_P[split]

    # -- hooks -----------------------------------------------------------------------------------
    def forward_hook_store_inputs(self, module: nn.Module, inputs: Tuple[torch.Tensor, ...],
                                  output: torch.Tensor) -> None:
        # Under activation checkpointing (re-entrant form) the first forward runs without autograd
        # and the layer is run again inside the backward pass: only that second run is followed by
        # the backward hook, so only it keeps the input alive.
        if not torch.is_grad_enabled():
            return
        module._ghost_A_raw = inputs[0].detach()

    def backward_hook_compute_proj(self, module: nn.Module, grad_input, grad_output) -> None:
        A_raw = getattr(module, "_ghost_A_raw", None)
        if A_raw is None:
            raise RuntimeError(f"Missing cached activations for GradProjection in {self.layer_name}")
        B_out = grad_output[0]
        if B_out is None:
            module._ghost_grad_proj = None
            delattr(module, "_ghost_A_raw")
            return
        B_out = B_out.detach()
        if self.layer_type == "Embedding":
            self._compute_embedding_proj(module, A_raw, B_out)
        else:
            self._compute_dense_proj(module, A_raw, B_out)
        delattr(module, "_ghost_A_raw")

    def _compute_dense_proj(self, module: nn.Module, A_raw: torch.Tensor, B_out: torch.Tensor) -> None:
        """``module._ghost_grad_proj[b] = batch_size * (P_o grad W_b P_i^T)`` as ``[B, k_o, k_i]`` float32
        for nn.Linear.  HF Conv1D follows the reference's convention: ``P_i`` projects the out-grad,
        ``P_o`` the activations, result ``[B, k_i, k_o]``."""
        is_conv1d = module.__class__.__name__ == "Conv1D"
        A = _flatten_tokens(A_raw)
        B = _flatten_tokens(B_out)
        if A.dtype != B.dtype:
            common = torch.promote_types(A.dtype, B.dtype)
            A, B = A.to(common), B.to(common)
        batch = A.shape[0]
        if B.shape[0] != batch or B.shape[1] != A.shape[1]:
            raise RuntimeError(f"Batch size mismatch between activations and gradients in {self.layer_name}")
        split = A.dtype == torch.float32
        P_i, P_o = self._prepared(split)
        k_i, k_o = self.P_i.shape[0], self.P_o.shape[0]
        if is_conv1d:
            P_r, P_c, k_r, k_c = P_i, P_o, k_i, k_o
        else:
            P_r, P_c, k_r, k_c = P_o, P_i, k_o, k_i
        out = self._out_fn(batch) if self._out_fn is not None else \
            torch.empty((batch, k_r * k_c), dtype=torch.float32, device=A.device)
        ops.gradproj_dense(B, A, P_r, P_c, k_r, k_c, float(batch), out)
        module._ghost_grad_proj = out.view(batch, k_r, k_c)

    def _compute_embedding_proj(self, module: nn.Module, indices: torch.Tensor,
                                grad_output: torch.Tensor) -> None:
        """Embedding projection ``module._ghost_grad_proj[b] = sum_t (P_o g_t)(P_i[:, id_t])^T`` as
        ``[B, k_o, k_i]`` float32 (reference :167-222, a Python loop over every token there): one
        kernel that streams the out-grad rows once and gathers the rows of ``P_i^T`` by token id."""
        batch = indices.shape[0]
        ids = indices.reshape(batch, -1)
        g = grad_output.reshape(batch, ids.shape[1], grad_output.shape[-1])
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        split = g.dtype == torch.float32
        _, P_o = self._prepared(split)
        if self._P_i_t is None:
            self._P_i_t = ops.prepare_embedding_projection(self.P_i.to(g.device))
        k_i, k_o = self.P_i.shape[0], self.P_o.shape[0]
        out = self._out_fn(batch) if self._out_fn is not None else \
            torch.empty((batch, k_o * k_i), dtype=torch.float32, device=g.device)
        ops.gradproj_embedding(ids, g, P_o, self._P_i_t, k_o, k_i, 1.0, out)
        module._ghost_grad_proj = out.view(batch, k_o, k_i)

    def attach(self, module: nn.Module) -> None:
        self._handle_forward = module.register_forward_hook(self.forward_hook_store_inputs)
        self._handle_backward = module.register_full_backward_hook(self.backward_hook_compute_proj)

    def detach(self) -> None:
        for attr in ("_handle_forward", "_handle_backward"):
            handle = getattr(self, attr)
            if handle is not None:
                handle.remove()
                setattr(self, attr, None)


def create_projection_hooks(module: nn.Module, layer_name: str, P_i: torch.Tensor,
                            P_o: torch.Tensor) -> GradProjHooks:
    """Build (not attach) the hooks for ``module``; same layer-type rules as the reference."""
    layer_type = module.__class__.__name__
    if layer_type == "Conv1D":
        layer_type = "Linear"
    elif isinstance(module, nn.Conv1d):
        raise NotImplementedError(
            f"Conv1d layers are not yet supported for gradient projection. Layer '{layer_name}' is a "
            f"Conv1d layer. Please exclude Conv1d layers from proj_layers pattern.")
    elif isinstance(module, nn.Conv2d):
        raise NotImplementedError(
            f"Conv2d layers are not yet supported for gradient projection. Layer '{layer_name}' is a "
            f"Conv2d layer. Please exclude Conv2d layers from proj_layers pattern or set include_conv2d=False.")
    elif isinstance(module, nn.Linear):
        layer_type = "Linear"
    elif isinstance(module, nn.Embedding):
        layer_type = "Embedding"
    else:
        raise ValueError(f"Unsupported layer type: {layer_type}")
    return GradProjHooks(P_i, P_o, layer_name, layer_type)
