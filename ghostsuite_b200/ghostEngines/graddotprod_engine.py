"""GradDotProdEngine: lifecycle around the dot-product hooks.

Drop-in for GhostSuite's ``ghostEngines/graddotprod_engine.py`` (class at :17-272): same
constructor, methods and on-disk artefacts (``valset.pt``, ``dot_prod_log_iter_{n}.pt`` holding a
list of ``{dot_product, X_train, Y_train, iter_num, batch_idx}`` dicts).  Additions: the aggregated
full matrix is kept next to the vector (``dot_product_matrix`` in each log entry) and
``aggregate_and_log`` checks the device error word that kernels set when a bounded wait ran out.
"""
from __future__ import annotations

import os
import warnings
from typing import Optional

import torch
from torch import nn

from .. import _lib
from . import autograd_grad_sample_dotprod
from . import supported_layers_grad_samplers_dotprod as _layers
from . import transformers_support


class GradDotProdEngine:
    """Computes, inside one ordinary backward pass over ``cat(train, val)``, the dot product of
    every validation sample's gradient with every train sample's gradient, and recovers the
    averaged train gradient for the optimizer."""

    def __init__(self, module: nn.Module, val_batch_size: int, loss_reduction: str = "mean",
                 use_dummy_bias: bool = False, dot_prod_save_path: Optional[str] = None):
        self.module = module
        self.val_batch_size = val_batch_size
        self.loss_reduction = loss_reduction
        self.dot_prod_save_path = dot_prod_save_path
        self.named_params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        self._grad_creation_locked = False
        self.dot_product_log = []
        self.batch_idx_lst = []
        self.X_train = self.Y_train = None
        self.iter_num = None
        self.batch_idx = None

        # remember what was trainable; in dummy-bias mode autograd then only computes
        # activation gradients (the hooks produce every weight gradient themselves)
        for name, param in module.named_parameters():
            if name.endswith("dummy_bias"):
                # left behind by an earlier engine on the same model: it is what keeps the autograd
                # graph alive in dummy-bias mode, so it stays trainable
                param.initially_requires_grad = True
                param.requires_grad = True
                continue
            param.initially_requires_grad = bool(param.requires_grad)
            param.requires_grad = not use_dummy_bias
        transformers_support.forward_swapper(module=module)

    # ------------------------------------------------------------------ attach / detach
    def attach(self, optimizer: torch.optim.Optimizer):
        self.optimizer = optimizer
        autograd_grad_sample_dotprod.add_hooks(model=self.module, val_batch_size=self.val_batch_size,
                                               loss_reduction=self.loss_reduction)
        optimizer.grad_dot_prod_engine = self

    def detach(self):
        optimizer = self.optimizer
        if hasattr(optimizer, "grad_dot_prod_engine"):
            del optimizer.grad_dot_prod_engine
        autograd_grad_sample_dotprod.remove_hooks(self.module)
        self.module.zero_grad()
        for param in self.module.parameters():
            for attr in ("train_grad", "grad_dot_prod", "grad_dot_prod_matrix", "activations", "backprops"):
                if hasattr(param, attr):
                    delattr(param, attr)

    # ------------------------------------------------------------------ gradients
    def _lock_grad_creation(self):
        self._grad_creation_locked = True

    def _unlock_grad_creation(self):
        self._grad_creation_locked = False

    def _prepare_and_apply_train_grad(self):
        if self._grad_creation_locked:
            return
        for name, param in self.module.named_parameters():
            if not param.initially_requires_grad or "dummy_bias" in name:
                continue
            if not hasattr(param, "train_grad"):
                raise ValueError(f"Parameter {name} requires grad but does not have 'train_grad' attribute. ")
            if param.train_grad is None:
                raise ValueError(f"Parameter {name} requires grad has no accumulated training gradient. ")
            param.grad = param.train_grad
        self._lock_grad_creation()

    def _clear_train_grad(self):
        for param in self.module.parameters():
            if hasattr(param, "train_grad"):
                del param.train_grad
        self._unlock_grad_creation()

    def prepare_gradients(self):
        """Move ``param.train_grad`` into ``param.grad`` for the optimizer."""
        self._prepare_and_apply_train_grad()

    def clear_gradients(self):
        """Drop the stored train gradients after the optimizer step."""
        self._clear_train_grad()

    # ------------------------------------------------------------------ dot products
    def aggregate_and_log(self):
        self._aggregate_and_log_dot_products()

    def _aggregate_and_log_dot_products(self):
        """Sum of the dot products over all parameters (reference :195-262), as one stacked
        reduction instead of one in-place add per parameter."""
        _layers.finalize_pending_dots()
        vectors, matrices = [], []
        for _, param in self.module.named_parameters():
            if hasattr(param, "grad_dot_prod") and param.initially_requires_grad:
                if param.grad_dot_prod.numel() > 0:
                    m = getattr(param, "grad_dot_prod_matrix", None)
                    if m is not None:
                        matrices.append(m)
                    else:
                        vectors.append(param.grad_dot_prod)
                delattr(param, "grad_dot_prod")
                if hasattr(param, "grad_dot_prod_matrix"):
                    delattr(param, "grad_dot_prod_matrix")
        total = None
        total_matrix = None
        if matrices:
            total_matrix = torch.stack(matrices).sum(dim=0)
            total = total_matrix.sum(dim=0)
        if vectors:
            extra = torch.stack(vectors).sum(dim=0)
            total = extra if total is None else total + extra
            total_matrix = None          # a parameter without a matrix makes the summed matrix partial
        if total is None:
            warnings.warn("No gradient dot products computed for this iteration.")
            return
        # device -> host: all copies are queued first and waited for once (this is also the step's
        # sync point); the train batch is copied once when inputs and labels are one tensor
        x_cpu = _to_host_async(self.X_train)
        y_cpu = x_cpu if self.Y_train is self.X_train else _to_host_async(self.Y_train)
        entry = {
            "dot_product": _to_host_async(total),
            "X_train": x_cpu,
            "Y_train": y_cpu,
            "iter_num": self.iter_num,
            "batch_idx": self.batch_idx,
        }
        if total_matrix is not None:
            entry["dot_product_matrix"] = _to_host_async(total_matrix)
        if total.is_cuda:
            torch.cuda.current_stream(total.device).synchronize()
            _lib.poll_kernel_error()
        self.dot_product_log.append(entry)

    def save_dot_product_log(self, iter_num: int):
        if not self.dot_product_log:
            raise ValueError("No gradient dot products found to save for this iteration.")
        print(f"[INFO] Saving dot product log at iteration {iter_num} ...")
        path = os.path.join(self.dot_prod_save_path, f"dot_prod_log_iter_{iter_num}.pt")
        torch.save(self.dot_product_log, path)
        self.dot_product_log.clear()

    def attach_and_store_valset(self, X_val, Y_val):
        path = os.path.join(self.dot_prod_save_path, "valset.pt")
        torch.save({"X_val": to_device(X_val, "cpu"), "Y_val": to_device(Y_val, "cpu")}, path)
        print(f"[INFO] Saved validation set to {path}")

    def attach_train_batch(self, X_train, Y_train, iter_num, batch_idx=None):
        self.X_train = X_train
        self.Y_train = Y_train
        self.iter_num = iter_num
        self.batch_idx = batch_idx


def _to_host_async(data):
    """Queue a device -> host copy (pinned destination) without waiting; the caller synchronises
    the stream once after queueing all of them.  Host data is passed through."""
    if data is None:
        return None
    if isinstance(data, dict):
        return {k: _to_host_async(v) if hasattr(v, "to") else v for k, v in data.items()}
    if hasattr(data, "is_cuda") and data.is_cuda:
        return data.to("cpu", non_blocking=True)
    return data


def to_device(data, device):
    """Move a tensor or a dict of tensors to ``device``."""
    if isinstance(data, dict):
        return {k: (v.to(device) if hasattr(v, "to") else v) for k, v in data.items()}
    if hasattr(data, "to"):
        return data.to(device)
    raise TypeError(f"Unsupported data type for moving to GPU: {type(data)}. Expected tensor or dict of tensors.")
