"""GhostEngineManager: one facade over the ghost engines for training loops.

Drop-in for GhostSuite's ``ghostEngines/engine_manager.py`` (class at :18-253): the engine is chosen
by ``config.method`` in {'GradDotProd', 'GradProjLora', 'Regular'} and every public method keeps
its name and meaning.  ``ddp_info`` may be omitted (single process: this process is the master).
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch
from torch import nn

from .graddotprod_engine import GradDotProdEngine
from .gradProjection.gradproj_engine import GradProjLoraEngine


class GhostEngineManager:
    def __init__(self, config, model: nn.Module, optimizer: torch.optim.Optimizer,
                 ddp_info: Optional[Dict[str, Any]] = None, val_data=None):
        self.config = config
        self.model = model
        self.optimizer = optimizer
        self.ddp_info = ddp_info if ddp_info is not None else {"master_process": True}
        self.engine = None
        self.X_val, self.Y_val = val_data if val_data is not None else (None, None)
        self._initialize_engine()

    # ------------------------------------------------------------------ construction
    def _initialize_engine(self):
        method = self.config.method
        if method == "GradDotProd":
            self._initialize_graddotprod_engine()
        elif method == "GradProjLora":
            self._initialize_gradproj_engine()
        elif method == "Regular":
            print("[INFO] Regular training mode - no ghost engine required.")
        else:
            print(f"[WARNING] Unknown method '{method}' - no ghost engine initialized.")

    def _initialize_graddotprod_engine(self):
        print("[INFO] Initializing GradDotProdEngine ...")
        save_path = os.path.join(self.config.result_dir, "grad_dotprods")
        if self.ddp_info["master_process"]:
            os.makedirs(save_path, exist_ok=True)
        self.engine = GradDotProdEngine(module=self.model, val_batch_size=self.config.val_batch_size,
                                        loss_reduction="mean", use_dummy_bias=True,
                                        dot_prod_save_path=save_path)
        self.engine.attach(self.optimizer)
        if self.X_val is None or self.Y_val is None:
            raise ValueError("X_val and Y_val are required for GradDotProd method")
        self.engine.attach_and_store_valset(self.X_val, self.Y_val)
        print("[INFO] GradDotProdEngine initialized successfully.")

    def _initialize_gradproj_engine(self):
        print("[INFO] Initializing GradProjLoraEngine ...")
        proj_dir = os.path.join(self.config.result_dir, "projections")
        if self.ddp_info["master_process"]:
            os.makedirs(proj_dir, exist_ok=True)
        cfg = self.config
        default_interval = getattr(cfg, "dot_prod_save_interval", 1)
        extra = {}
        if getattr(cfg, "proj_dims_override", None) is not None:
            extra["proj_dims_override"] = cfg.proj_dims_override
        self.engine = GradProjLoraEngine(
            module=self.model,
            proj_layers=getattr(cfg, "proj_layers", "mlp,attn"),
            proj_rank_total=getattr(cfg, "proj_rank_total", 256),
            proj_rank_min=getattr(cfg, "proj_rank_min", 8),
            proj_seed=getattr(cfg, "proj_seed", 42),
            proj_dtype=getattr(cfg, "proj_dtype", getattr(cfg, "train_dtype", "float32")),
            proj_dir=proj_dir,
            proj_save_interval=getattr(cfg, "proj_save_interval", default_interval),
            include_embeddings=getattr(cfg, "include_embeddings", False),
            **extra)
        self.engine.attach()
        print("[INFO] GradProjLoraEngine initialized successfully.")

    # ------------------------------------------------------------------ queries
    def is_active(self) -> bool:
        return self.engine is not None

    def get_method(self) -> str:
        return self.config.method

    def get_validation_data(self):
        return self.X_val, self.Y_val

    # ------------------------------------------------------------------ per-step calls
    def _call(self, name: str, *args, **kwargs):
        fn = getattr(self.engine, name, None) if self.engine else None
        if fn is not None:
            return fn(*args, **kwargs)
        return None

    def attach_train_batch(self, X_train, Y_train, iter_num, batch_idx=None):
        self._call("attach_train_batch", X_train, Y_train, iter_num, batch_idx)

    def prepare_gradients(self):
        self._call("prepare_gradients")

    def aggregate_and_log(self):
        self._call("aggregate_and_log")

    def clear_gradients(self):
        self._call("clear_gradients")

    def prepare_forward_input(self, X_train, Y_train):
        """GradDotProd: forward on ``cat(train, val)`` (validation LAST); otherwise unchanged."""
        if self.config.method != "GradDotProd" or self.X_val is None:
            return X_train, Y_train
        if isinstance(self.X_val, dict):
            X_cat = {key: torch.cat((X_train[key], self.X_val[key]), dim=0)
                     for key in ("input_ids", "pixel_values", "attention_mask")}
        else:
            X_cat = torch.cat((X_train, self.X_val), dim=0)
        return X_cat, torch.cat((Y_train, self.Y_val), dim=0)

    # ------------------------------------------------------------------ saving
    def should_save_metrics(self, iter_num: int) -> bool:
        if iter_num <= 0:
            return False
        if self.config.method == "GradDotProd":
            return iter_num % self.config.dot_prod_save_interval == 0
        if self.config.method == "GradProjLora":
            interval = getattr(self.config, "proj_save_interval",
                               getattr(self.config, "dot_prod_save_interval", 1))
            return iter_num % interval == 0
        return False

    def save_metrics(self, iter_num: int):
        if not self.engine:
            return
        if self.config.method == "GradDotProd":
            self.engine.save_dot_product_log(iter_num=iter_num)
        elif self.config.method == "GradProjLora":
            self._call("save_projections", iter_num=iter_num)

    # ------------------------------------------------------------------ evaluation / shutdown
    def detach_for_evaluation(self):
        if self.engine:
            if hasattr(self.engine, "detach"):
                self.engine.detach()
            elif hasattr(self.engine, "disable_hooks"):
                self.engine.disable_hooks()

    def reattach_after_evaluation(self):
        if not self.engine:
            return
        if isinstance(self.engine, GradProjLoraEngine):
            self.engine.reattach_after_evaluation()
        elif hasattr(self.engine, "attach"):
            self.engine.attach(self.optimizer)
        elif hasattr(self.engine, "enable_hooks"):
            self.engine.enable_hooks()

    def cleanup(self):
        """Save whatever is pending and detach; never raises (called from ``finally`` blocks)."""
        if not self.engine:
            return
        if self.config.method == "GradDotProd" and getattr(self.engine, "dot_product_log", None):
            try:
                self.engine.save_dot_product_log(iter_num=-1)
            except Exception as e:
                print(f"Error saving remaining dot products during cleanup: {e}")
        elif self.config.method == "GradProjLora" and hasattr(self.engine, "cleanup"):
            try:
                self.engine.cleanup()
            except Exception as e:
                print(f"Error during GradProjLora cleanup: {e}")
        try:
            if hasattr(self.engine, "detach"):
                self.engine.detach()
            elif hasattr(self.engine, "disable_hooks"):
                self.engine.disable_hooks()
        except Exception as e:
            print(f"Error detaching ghost engine during cleanup: {e}")
