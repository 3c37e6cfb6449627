"""GradProjLoraEngine: per-sample Kronecker-projected gradients for a set of layers.

Drop-in for GhostSuite's ``ghostEngines/gradProjection/gradproj_engine.py`` (class at :29-434,
factory :437-457): same constructor arguments, attributes (``matched_layers``,
``projection_matrices``, ``projection_dims``, ``slice_ranges``, ``total_proj_dim``, ``metadata``,
``iteration``, ``batch_count``), methods and files (``metadata.json`` once,
``proj_iter_{06d}.pt`` = ``{'proj', 'iter', 'batch_size'[, 'batch_idx']}`` per saved iteration).

What is different underneath:

* every layer's hook writes its ``[B, k_o*k_i]`` block directly into that layer's column range
  (sorted-name order, as the reference concatenates) of ONE device buffer ``[B, total_proj_dim]``,
  so ``collect_batch`` has nothing to reshape or concatenate;
* saving does not block the GPU: the batch is copied device -> pinned host on a side stream into a
  small ring of pinned slots and a writer thread does the ``torch.save``; ``flush()`` / ``detach()``
  / ``cleanup()`` wait for it.  A slot that does not free up within ``slot_timeout_s`` raises
  instead of hanging;
* optional keyword ``proj_dims_override`` -- ``(k_i, k_o)`` for every layer or a
  ``{layer_name: (k_i, k_o)}`` dict -- replaces the ``choose_ki_ko`` heuristic where given (the
  heuristic does not produce ``k_i == k_o`` for non-square layers);
* optional keyword ``freeze_weights=True``: while the engine is attached no model parameter requires
  grad, so autograd computes activation gradients only (the reference's loop,
  ``Examples/GradProj_LM/gradproj_loop.py:66``, computes every weight gradient and throws it away --
  about a third of the backward flops).  A one-element ``dummy_bias`` on the input embedding keeps
  the autograd graph alive; ``detach()`` removes it and restores every ``requires_grad`` flag.
"""
from __future__ import annotations

import json
import queue
import threading
import time
from collections import OrderedDict
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from .projection_utils import choose_ki_ko, get_projection_initializer, compute_projection_metadata
from .autograd_gradproj import create_projection_hooks
from .supported_layers_gradproj import (
    find_matching_layers,
    validate_layer_selection,
    get_layer_dimensions,
    compute_total_projection_size,
    get_layer_slice_ranges,
)


class _HostStreamer:
    """Ring of pinned host slots fed by a side stream and drained by a writer thread."""

    def __init__(self, slots: int = 3, slot_timeout_s: float = 60.0):
        self.n_slots = slots
        self.timeout = slot_timeout_s
        self._slots: List[Optional[torch.Tensor]] = [None] * slots
        self._free = [threading.Event() for _ in range(slots)]
        for e in self._free:
            e.set()
        self._cursor = 0
        self._stream = None
        self._queue: "queue.Queue" = queue.Queue()
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    def _worker(self):
        while True:
            job = self._queue.get()
            if job is None:
                self._queue.task_done()
                return
            slot_idx, event, rows, save_dict, path = job
            try:
                event.synchronize()
                if callable(path):                      # raw format: the engine appends the rows itself
                    path(self._slots[slot_idx][:rows], save_dict)
                else:
                    save_dict["proj"] = self._slots[slot_idx][:rows].clone()
                    torch.save(save_dict, path)
            except BaseException as exc:   # surfaced on the next submit()/flush()
                self._error = exc
            finally:
                self._free[slot_idx].set()
                self._queue.task_done()

    def submit(self, dev: torch.Tensor, save_dict: dict, path: Path) -> None:
        if self._error is not None:
            err, self._error = self._error, None
            raise RuntimeError(f"projection writer failed: {err}")
        if self._thread is None:
            self._thread = threading.Thread(target=self._worker, name="gradproj-writer", daemon=True)
            self._thread.start()
        idx = self._cursor
        self._cursor = (self._cursor + 1) % self.n_slots
        if not self._free[idx].wait(self.timeout):
            raise RuntimeError(f"pinned host slot {idx} was not released within {self.timeout} s")
        self._free[idx].clear()
        slot = self._slots[idx]
        if slot is None or slot.dtype != dev.dtype or slot.shape[1] != dev.shape[1] or slot.shape[0] < dev.shape[0]:
            slot = torch.empty(dev.shape, dtype=dev.dtype, pin_memory=True)
            self._slots[idx] = slot
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=dev.device)
        self._stream.wait_stream(torch.cuda.current_stream(dev.device))
        with torch.cuda.stream(self._stream):
            slot[:dev.shape[0]].copy_(dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record(self._stream)
        dev.record_stream(self._stream)
        self._queue.put((idx, event, dev.shape[0], save_dict, path))

    def flush(self) -> None:
        self._queue.join()
        if self._error is not None:
            err, self._error = self._error, None
            raise RuntimeError(f"projection writer failed: {err}")

    def close(self) -> None:
        if self._thread is not None:
            self._queue.put(None)
            self._thread.join(timeout=self.timeout)
            self._thread = None


class GradProjLoraEngine:
    """Computes per-sample projected gradients ``P_o grad W P_i^T`` in backward hooks without
    touching the model's forward pass or its training dynamics."""

    def __init__(self, module: nn.Module, proj_layers: Union[str, List[str]], proj_rank_total: int,
                 proj_rank_min: int, proj_seed: int, proj_dtype: str, proj_dir: str,
                 proj_row_orthonormal: bool = False, include_embeddings: bool = False,
                 include_conv2d: bool = False, proj_save_interval: int = 1, **kwargs):
        self.module = module
        self.proj_layers = proj_layers
        self.proj_rank_total = proj_rank_total
        self.proj_rank_min = proj_rank_min
        self.proj_seed = proj_seed
        self.proj_dir = Path(proj_dir)
        self.proj_save_interval = proj_save_interval
        dtype_map = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
        if proj_dtype not in dtype_map:
            raise ValueError(f"proj_dtype must be one of {list(dtype_map.keys())}, got {proj_dtype}")
        self.proj_dtype = dtype_map[proj_dtype]
        self.proj_method = "orthonormal" if proj_row_orthonormal else "gaussian"
        self.include_embeddings = include_embeddings
        self.include_conv2d = include_conv2d
        self.proj_dims_override = kwargs.get("proj_dims_override")
        self.async_save = bool(kwargs.get("async_save", True))
        # 'pt': one torch.save file per saved iteration, as the reference writes them.
        # 'bin': rows appended to one flat file (proj.bin, row-major [rows, total_proj_dim] in
        # proj_dtype) plus index.json, which a reader memory-maps (load_projection_bin): no pickling
        # on the writer thread, so one host thread keeps up with several GPUs.
        self.proj_format = str(kwargs.get("proj_format", "pt"))
        if self.proj_format not in ("pt", "bin"):
            raise ValueError(f"proj_format must be 'pt' or 'bin', got {self.proj_format}")
        self._bin_file = None
        self._bin_rows = 0
        self._bin_index: List[dict] = []
        self.freeze_weights = bool(kwargs.get("freeze_weights", False))
        self._frozen_flags: Optional[Dict[int, Tuple[torch.Tensor, bool]]] = None
        self._frozen_embeddings: List[nn.Embedding] = []

        self.matched_layers = OrderedDict()
        self.projection_matrices = {}
        self.projection_dims = {}
        self.hooks = {}
        self.slice_ranges = {}
        self.total_proj_dim = 0
        self.metadata = {}
        self.is_attached = False
        self.iteration = 0
        self.batch_count = 0
        self._buffer: Optional[torch.Tensor] = None
        self._streamer = _HostStreamer(slots=int(kwargs.get("host_slots", 3)),
                                       slot_timeout_s=float(kwargs.get("slot_timeout_s", 60.0)))
        self._initialize_projections()

    # ------------------------------------------------------------------ setup
    def _dims_for(self, name: str, n_i: int, n_o: int) -> Tuple[int, int]:
        ov = self.proj_dims_override
        if isinstance(ov, dict):
            ov = ov.get(name)
        if ov is not None:
            k_i, k_o = int(ov[0]), int(ov[1])
            if not (1 <= k_i <= n_i and 1 <= k_o <= n_o):
                raise ValueError(f"proj_dims_override {ov} does not fit layer {name} ({n_i} -> {n_o})")
            return k_i, k_o
        return choose_ki_ko(n_i, n_o, self.proj_rank_total, self.proj_rank_min)

    def _initialize_projections(self):
        self.matched_layers = find_matching_layers(self.module, self.proj_layers,
                                                   self.include_embeddings, self.include_conv2d)
        validate_layer_selection(self.matched_layers, self.proj_layers)
        device = next(self.module.parameters()).device
        init_fn = get_projection_initializer(self.proj_method)
        torch.manual_seed(self.proj_seed)
        # seeds follow TRAVERSAL order (layer_idx), slices follow SORTED-name order
        for layer_idx, (name, layer) in enumerate(self.matched_layers.items()):
            n_i, n_o = get_layer_dimensions(layer)
            k_i, k_o = self._dims_for(name, n_i, n_o)
            self.projection_dims[name] = (k_i, k_o)
            seed = self.proj_seed + layer_idx
            P_i = init_fn(k_i, n_i, dtype=torch.float32, device=device, seed=seed)
            P_o = init_fn(k_o, n_o, dtype=torch.float32, device=device, seed=seed + 1000)
            self.projection_matrices[name] = (P_i, P_o)
            print(f"  Projection dims: k_i={k_i}, k_o={k_o} (k_total={k_i*k_o})")
        self.slice_ranges = get_layer_slice_ranges(self.matched_layers, self.projection_dims)
        self.total_proj_dim = compute_total_projection_size(self.matched_layers, self.projection_dims)
        print(f"Total projection dimension: {self.total_proj_dim}")
        self._prepare_metadata()

    def _prepare_metadata(self):
        self.metadata = {
            "engine": "GradProjLora",
            "proj_seed": self.proj_seed,
            "proj_dtype": str(self.proj_dtype).split(".")[-1],
            "proj_method": self.proj_method,
            "proj_rank_total": self.proj_rank_total,
            "proj_rank_min": self.proj_rank_min,
            "total_proj_dim": self.total_proj_dim,
            "layers": [],
        }
        for name in sorted(self.matched_layers.keys()):
            k_i, k_o = self.projection_dims[name]
            meta = compute_projection_metadata(name, self.matched_layers[name], k_i, k_o)
            meta["slice_start"], meta["slice_end"] = self.slice_ranges[name]
            self.metadata["layers"].append(meta)

    # ------------------------------------------------------------------ device buffer
    def _slice_for(self, name: str):
        start, end = self.slice_ranges[name]

        def out_fn(batch: int) -> torch.Tensor:
            buf = self._buffer
            device = next(self.module.parameters()).device
            if buf is None or buf.shape[0] != batch or buf.device != device:
                buf = torch.empty((batch, self.total_proj_dim), dtype=torch.float32, device=device)
                self._buffer = buf
            return buf[:, start:end]

        return out_fn

    def _attach_hooks(self):
        for name, layer in self.matched_layers.items():
            P_i, P_o = self.projection_matrices[name]
            hooks = create_projection_hooks(layer, name, P_i, P_o)
            hooks.bind_output(self._slice_for(name))
            hooks.attach(layer)
            self.hooks[name] = hooks

    # ------------------------------------------------------------------ frozen weights
    def _input_embeddings(self) -> List[nn.Embedding]:
        """The embeddings that start the autograd graph: ``get_input_embeddings()`` of a Hugging Face
        model, else every nn.Embedding of the module."""
        getter = getattr(self.module, "get_input_embeddings", None)
        if callable(getter):
            try:
                emb = getter()
            except Exception:
                emb = None
            if isinstance(emb, nn.Embedding):
                return [emb]
        return [m for m in self.module.modules() if isinstance(m, nn.Embedding)]

    def _freeze(self) -> None:
        if self._frozen_flags is not None:
            return
        from ..transformers_support import _add_dummy_bias
        embeddings = self._input_embeddings()
        if not embeddings:
            raise RuntimeError("freeze_weights=True needs an nn.Embedding at the model's input: with no "
                               "trainable parameter upstream of the projected layers, backward hooks "
                               "would never fire")
        self._frozen_flags = {id(p): (p, bool(p.requires_grad)) for p in self.module.parameters()}
        for p, _ in self._frozen_flags.values():
            p.requires_grad = False
        for emb in embeddings:
            if not hasattr(emb, "dummy_bias"):
                _add_dummy_bias(emb)
                self._frozen_embeddings.append(emb)

    def _unfreeze(self) -> None:
        if self._frozen_flags is None:
            return
        for emb in self._frozen_embeddings:
            handle = emb.__dict__.pop("_ghost_dummy_bias_handle", None)
            if handle is not None:
                handle.remove()
            if "dummy_bias" in emb._parameters:
                del emb._parameters["dummy_bias"]
        self._frozen_embeddings = []
        for p, flag in self._frozen_flags.values():
            p.requires_grad = flag
        self._frozen_flags = None

    # ------------------------------------------------------------------ attach / detach
    def attach(self):
        if self.is_attached:
            return
        if self.freeze_weights:
            self._freeze()
        self._attach_hooks()
        self.is_attached = True
        print(f"Attached projection hooks to {len(self.matched_layers)} layers")

    def detach(self):
        if not self.is_attached:
            return
        self.flush()
        self._unfreeze()
        for name, hooks in self.hooks.items():
            hooks.detach()
            layer = self.matched_layers[name]
            for attr in ("_ghost_A_raw", "_ghost_grad_proj"):
                if hasattr(layer, attr):
                    delattr(layer, attr)
        self.hooks.clear()
        self.is_attached = False
        print(f"Detached projection hooks from {len(self.matched_layers)} layers")

    # ------------------------------------------------------------------ collect / save
    def collect_batch(self, batch_indices: Optional[List[int]] = None) -> torch.Tensor:
        """Concatenated projections ``[B, total_proj_dim]`` in ``proj_dtype`` for the last backward
        pass; saved every ``proj_save_interval`` iterations."""
        if not self.is_attached:
            raise RuntimeError("Engine is not attached. Call attach() first.")
        batch_size = None
        pieces = []
        in_buffer = True
        for name in sorted(self.matched_layers.keys()):
            grad_proj = getattr(self.matched_layers[name], "_ghost_grad_proj", None)
            if grad_proj is None:
                raise RuntimeError(f"No projected gradient found for layer {name}")
            B = grad_proj.shape[0]
            if batch_size is None:
                batch_size = B
            elif B != batch_size:
                raise RuntimeError(f"Batch size mismatch: expected {batch_size}, got {B} for {name}")
            buf = self._buffer
            if buf is None or grad_proj.untyped_storage().data_ptr() != buf.untyped_storage().data_ptr():
                in_buffer = False
            pieces.append(grad_proj)
        if in_buffer and self._buffer is not None and self._buffer.shape[0] == batch_size:
            full = self._buffer
            self._buffer = None        # the next backward gets a fresh buffer; `full` stays valid
        else:                          # embeddings or foreign hooks: fall back to concatenation
            full = torch.cat([p.reshape(batch_size, -1) for p in pieces], dim=1)
        full = full.to(self.proj_dtype)
        from ... import _lib
        if full.is_cuda and (self.iteration % 64 == 0):
            _lib.poll_kernel_error()
        if self.iteration % self.proj_save_interval == 0:
            self._save_projection(full, batch_indices)
        self.iteration += 1
        self.batch_count += batch_size
        return full

    def _save_projection(self, projection: torch.Tensor, batch_indices: Optional[List[int]] = None):
        self.proj_dir.mkdir(parents=True, exist_ok=True)
        meta_path = self.proj_dir / "metadata.json"
        if not meta_path.exists():
            with open(meta_path, "w") as f:
                json.dump(self.metadata, f, indent=2)
            print(f"Saved metadata to {meta_path}")
        save_dict = {"iter": self.iteration, "batch_size": projection.shape[0]}
        if batch_indices is not None:
            save_dict["batch_idx"] = batch_indices
        if self.proj_format == "bin":
            if projection.is_cuda and self.async_save:
                self._streamer.submit(projection, save_dict, self._append_bin)
            else:
                self._append_bin(projection.cpu(), save_dict)
            return
        path = self.proj_dir / f"proj_iter_{self.iteration:06d}.pt"
        if projection.is_cuda and self.async_save:
            self._streamer.submit(projection, save_dict, path)
        else:
            save_dict = {"proj": projection.cpu(), **save_dict}
            torch.save(save_dict, path)

    def _append_bin(self, rows_host: torch.Tensor, info: dict) -> None:
        """Append one batch of rows to proj.bin (called in submission order, by the writer thread
        when saving is asynchronous)."""
        if self._bin_file is None:
            self._bin_file = open(self.proj_dir / "proj.bin", "wb")
        data = rows_host.contiguous()
        if data.dtype == torch.bfloat16:
            data = data.view(torch.int16)
        self._bin_file.write(data.numpy().tobytes())
        entry = {"iter": info["iter"], "row0": self._bin_rows, "rows": int(rows_host.shape[0])}
        if "batch_idx" in info:
            entry["batch_idx"] = [int(i) for i in info["batch_idx"]]
        self._bin_index.append(entry)
        self._bin_rows += int(rows_host.shape[0])

    def _write_bin_index(self) -> None:
        if self.proj_format != "bin" or self._bin_file is None:
            return
        self._bin_file.flush()
        with open(self.proj_dir / "index.json", "w") as f:
            json.dump({"dtype": str(self.proj_dtype).split(".")[-1], "total_proj_dim": self.total_proj_dim,
                       "rows": self._bin_rows, "batches": self._bin_index}, f)

    def flush(self):
        """Wait until every queued projection has been written to disk."""
        self._streamer.flush()
        self._write_bin_index()

    def get_projection_metadata(self) -> dict:
        return self.metadata.copy()

    # ------------------------------------------------------------------ GhostEngineManager shims
    def attach_train_batch(self, X_train, Y_train, iter_num, batch_idx=None):
        self.current_iter_num = iter_num
        self.current_batch_idx = batch_idx

    def prepare_gradients(self):
        """Projections are produced inside the backward hooks: nothing to do."""

    def aggregate_and_log(self, result_dict: Optional[dict] = None):
        """With a dict: add counters to it.  Without: collect (and possibly save) this batch."""
        if result_dict is not None:
            result_dict["proj_iteration"] = self.iteration
            result_dict["proj_batch_count"] = self.batch_count
            result_dict["proj_total_dim"] = self.total_proj_dim
            return
        self.collect_batch(batch_indices=getattr(self, "current_batch_idx", None))

    def clear_gradients(self):
        for layer in self.matched_layers.values():
            for attr in ("_ghost_A_raw", "_ghost_grad_proj"):
                if hasattr(layer, attr):
                    delattr(layer, attr)

    def attach_with_optimizer(self, optimizer):
        self.attach()

    def detach_for_evaluation(self):
        self.detach()

    def reattach_after_evaluation(self):
        if not self.is_attached:
            if self.freeze_weights:
                self._freeze()
            self._attach_hooks()
            self.is_attached = True

    def cleanup(self):
        self.detach()
        self._streamer.flush()
        self._write_bin_index()
        if self._bin_file is not None:
            self._bin_file.close()
            self._bin_file = None
        self._streamer.close()
        self.projection_matrices.clear()

    def save_projections(self, iter_num: int):
        """Projections are saved by ``collect_batch``; kept for the manager's ``save_metrics``."""

    def __repr__(self):
        return (f"GradProjLoraEngine(layers={len(self.matched_layers)}, "
                f"total_dim={self.total_proj_dim}, attached={self.is_attached})")


#: spelling used in some descriptions of the engine
GradProjLoRAEngine = GradProjLoraEngine


def load_projection_bin(proj_dir: str):
    """Reader for ``proj_format='bin'``: ``(rows, index)`` with ``rows`` a read-only numpy memory map
    of shape ``[n_rows, total_proj_dim]`` (bfloat16 data is exposed as int16 bit patterns) and
    ``index`` the parsed index.json (per saved batch: iter, row0, rows, batch_idx)."""
    import numpy as np
    with open(Path(proj_dir) / "index.json") as f:
        index = json.load(f)
    np_dtype = {"float32": np.float32, "float16": np.float16, "bfloat16": np.int16}[index["dtype"]]
    rows = np.memmap(Path(proj_dir) / "proj.bin", dtype=np_dtype, mode="r",
                     shape=(index["rows"], index["total_proj_dim"]))
    return rows, index


def create_gradproj_engine(model: nn.Module, config: dict) -> GradProjLoraEngine:
    """Build the engine from a config dict (all six projection keys are required)."""
    for key in ("proj_layers", "proj_rank_total", "proj_rank_min", "proj_seed", "proj_dtype", "proj_dir"):
        if key not in config:
            raise ValueError(f"Missing required parameter: {key}")
    return GradProjLoraEngine(model, **config)
