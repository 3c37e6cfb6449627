"""Forward/backward hook plumbing for the gradient-dot-product engine.

Drop-in for GhostSuite's ``ghostEngines/autograd_grad_sample_dotprod.py`` (``add_hooks`` :23-81,
``remove_hooks`` :84-89, ``_capture_activations`` :92-94, ``backward_hook`` closure :58-71): same
names, signatures, attributes (``layer.activations``, ``layer.backprops``, ``layer.name``,
``model.autograd_grad_sample_hooks``) and exceptions.  The hook bodies call the CUDA-backed layer
functions of ``supported_layers_grad_samplers_dotprod``.

One deliberate difference inside the hook: the reference multiplies the whole out-grad tensor by
the batch size (a full extra read and write per layer, :132-134) before the train-gradient pass.
Here the raw out-grad is kept and the factor is recorded in ``layer._ghost_backprop_scale``; the
kernels fold it into their epilogue scale.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn as nn

from .. import ops
from . import supported_layers_grad_samplers_dotprod as _layers
from .supported_layers_grad_samplers_dotprod import (
    _supported_layers_dotprod,
    _create_or_accumulate_train_grad,
)


#: optional ``fn(layer, A, B, n_val_local) -> (A_full, B_full, n_val_global)`` applied to every hooked
#: layer's operands before its layer functions run.  The data-parallel layer installs one when the
#: validation batch is split over ranks: it appends the other ranks' validation rows (an all-gather
#: into local memory), so the kernels see ``cat(train_local, val_global)`` without every rank having
#: run the whole validation batch through the model.
VALIDATION_GATHER = None


def requires_grad(module: nn.Module) -> bool:
    """True if any parameter of ``module`` was trainable when the engine was built."""
    return any(getattr(p, "initially_requires_grad", p.requires_grad) for p in module.parameters())


def add_hooks(model: nn.Module, val_batch_size: int, loss_reduction: str = "mean"):
    """Register the activation-capture and dot-product/train-gradient hooks on every supported
    layer that has a trainable parameter.  Calling it twice on one model raises ValueError."""
    if hasattr(model, "autograd_grad_sample_hooks"):
        raise ValueError("Trying to add hooks twice to the same model")
    if loss_reduction not in ("mean", "sum"):
        raise ValueError(f"loss_reduction must be 'mean' or 'sum', got {loss_reduction!r}")

    handles = []
    for name, layer in model.named_modules():
        if type(layer) not in _supported_layers_dotprod and getattr(layer, "weight", None) is not None \
                and layer.weight.dim() == 1:
            _layers.maybe_register_rmsnorm(type(layer))
        if type(layer) in _supported_layers_dotprod and requires_grad(layer):
            layer.name = name
            handles.append(layer.register_forward_hook(_capture_activations))

            def backward_hook(this_layer, grad_input, grad_output):
                _prepare_sample_grad_or_dotprod(this_layer, grad_output, val_batch_size, loss_reduction)
                _apply_train_grad(this_layer, val_batch_size)
                return None

            handles.append(layer.register_full_backward_hook(backward_hook))
        elif not list(layer.children()) and requires_grad(layer):
            print(f"WARNING: Skipping atomic layer '{name}' of type {type(layer)} because it is not supported.")

    model.__dict__.setdefault("autograd_grad_sample_hooks", []).extend(handles)


def remove_hooks(model: nn.Module):
    """Remove everything ``add_hooks`` registered."""
    _layers.finalize_pending_dots()
    if hasattr(model, "autograd_grad_sample_hooks"):
        for handle in model.autograd_grad_sample_hooks:
            handle.remove()
        del model.autograd_grad_sample_hooks


def _capture_activations(layer: nn.Module, inputs: Tuple, outputs: Tuple):
    """Forward hook: keep the layer input for the backward hook.  A forward without autograd
    (evaluation, or the first pass of re-entrant activation checkpointing) is followed by no
    backward hook and keeps nothing alive."""
    if not torch.is_grad_enabled():
        return
    layer.activations = inputs[0].detach()


def _prepare_sample_grad_or_dotprod(layer: nn.Module, grad_output: Tuple[torch.Tensor],
                                    val_batch_size: int, loss_reduction: str = "mean"):
    """Backward hook, part 1: dot products of this layer's parameters (reference :97-137)."""
    backprops = grad_output[0].detach()
    if not hasattr(layer, "activations"):
        layer.activations = None
    A = layer.activations
    dot_fn, _ = _supported_layers_dotprod[type(layer)]

    # mixed precision: bring both operands to the common floating type (ids stay integer)
    if A is not None and A.is_floating_point() and A.dtype != backprops.dtype:
        common = torch.promote_types(A.dtype, backprops.dtype)
        A = A.to(common)
        backprops = backprops.to(common)
        layer.activations = A

    # 'mean' losses carry a 1/batch factor (the batch this process ran); the train-gradient kernels
    # undo it in their epilogue
    layer._ghost_backprop_scale = float(backprops.shape[0]) if loss_reduction == "mean" else 1.0
    # the per-parameter [n_train] vectors are reduced in one batched op when the backward pass ends
    if _layers.begin_deferred_dots():
        try:
            torch.autograd.Variable._execution_engine.queue_callback(_layers.finalize_pending_dots)
        except Exception:
            _layers.finalize_pending_dots()      # not inside a backward pass: reduce immediately
    exchange = _layers.VALIDATION_EXCHANGE
    if exchange is not None and VALIDATION_GATHER is not None and A is not None and A.is_floating_point():
        # validation batch split over ranks: the ranks exchange validation gradients where the layer
        # type allows it ...
        layer._ghost_val_batch = val_batch_size
        try:
            handled = _layers.dot_product_with_exchange(layer, A, backprops, val_batch_size, exchange)
        except BaseException:
            _layers.finalize_pending_dots()
            raise
        if handled:
            layer.backprops = backprops
            return
    if VALIDATION_GATHER is not None and A is not None:
        # ... and validation operands everywhere else
        A, backprops, val_batch_size = VALIDATION_GATHER(layer, A, backprops, val_batch_size)
        layer.activations = A
    layer._ghost_val_batch = val_batch_size
    try:
        dot_fn(layer, A, backprops, val_batch_size=val_batch_size)
    except BaseException:
        _layers.finalize_pending_dots()          # a failed pass may never reach its callback
        raise
    layer.backprops = backprops


def _apply_train_grad(layer: nn.Module, val_batch_size: int, loss_reduction: str = "mean"):
    """Backward hook, part 2: averaged train gradients into ``param.train_grad`` (reference :140-196)."""
    _, train_grad_fn = _supported_layers_dotprod.get(type(layer), (None, None))
    val_batch_size = layer.__dict__.get("_ghost_val_batch", val_batch_size)
    if not train_grad_fn:
        raise ValueError(
            f"Layer {layer.__class__.__name__} is not supported for training gradient computation. "
            "Ensure it is included in the _supported_layers_dotprod dictionary.")
    try:
        if type(layer) in _layers._SELF_APPLYING or isinstance(layer, nn.LayerNorm):
            train_grad_fn(layer, layer.activations, layer.backprops, val_batch_size)
        else:
            weight = getattr(layer, "weight", None)
            if weight is not None and getattr(weight, "initially_requires_grad", weight.requires_grad):
                grad_weight = train_grad_fn(layer, layer.activations, layer.backprops, val_batch_size)
                if grad_weight is None:
                    raise ValueError(
                        f"Layer {layer.__class__.__name__} returned None for weight gradient. "
                        "Ensure the compute_layer_train_grad function is implemented correctly.")
                if grad_weight is not _layers.DEFERRED:      # else: handed over by the launch that makes it
                    _create_or_accumulate_train_grad(weight, grad_weight)
            bias = getattr(layer, "bias", None)
            if bias is not None and getattr(bias, "initially_requires_grad", bias.requires_grad):
                _train_grad_bias_from_layer(layer, val_batch_size, loss_reduction)
    finally:
        for attr in ("activations", "backprops", "_ghost_backprop_scale", "_ghost_val_batch", "_ghost_colsums",
                     "_ghost_cached_train_grad", "_ghost_ln_cache", "_ghost_conv_tokens"):
            layer.__dict__.pop(attr, None)


def _train_grad_bias_from_layer(layer: nn.Module, val_batch_size: int, loss_reduction: str) -> None:
    """Bias train gradient from the per-sample column sums the dot-product pass already made, added to
    ``layer.bias.train_grad`` (inside a backward pass: by the batched launch at its end)."""
    B = layer.backprops
    n_train = B.size(0) - val_batch_size
    if n_train <= 0:
        raise ValueError("No training samples to compute gradients, check batch sizes.")
    colsums = layer.__dict__.get("_ghost_colsums")
    if colsums is None:
        if isinstance(layer, nn.Conv2d):      # features are dim 1 there: [N, p, H, W] -> [N, H*W, p]
            B = B.reshape(B.size(0), B.size(1), -1).transpose(1, 2).contiguous()
        colsums = ops.colsum(B)
    scale = float(getattr(layer, "_ghost_backprop_scale", 1.0))
    if loss_reduction == "mean":
        scale /= n_train
    out_dtype = layer.bias.dtype if layer.bias.dtype in (torch.float32, torch.bfloat16) else torch.float32
    _layers._train_grad_from_vectors(layer.bias, colsums, n_train, scale, out_dtype)


def _compute_train_grad_bias(B: torch.Tensor, val_batch_size: int, loss_reduction: str = "mean") -> torch.Tensor:
    """Sum (or, for 'mean', average over the train samples) of the already scaled out-grad over
    batch and tokens -> ``[features]`` (reference :199-222)."""
    n_train = B.size(0) - val_batch_size
    if n_train <= 0:
        raise ValueError("No training samples to compute gradients, check batch sizes.")
    colsums = ops.colsum(B)
    out_dtype = B.dtype if B.dtype in (torch.float32, torch.bfloat16) else torch.float32
    return ops.rows_sum(colsums, n_train, 1.0 / n_train if loss_reduction == "mean" else 1.0, out_dtype)
