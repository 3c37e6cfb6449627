"""Layer discovery and bookkeeping for GradProj.

Drop-in for GhostSuite's ``ghostEngines/gradProjection/supported_layers_gradproj.py``:
substring matching of layer names (:104-143), ``(n_i, n_o)`` per layer type (:62-101, including
the HF Conv1D convention ``n_i = weight.shape[1]``, ``n_o = weight.shape[0]``), and slice ranges in
sorted-name order (:188-208).
"""
from __future__ import annotations

from typing import Dict, List, Tuple, Union

import torch.nn as nn

SUPPORTED_DENSE_LAYERS = (nn.Linear, nn.Conv1d)
SUPPORTED_EMBEDDING_LAYERS = (nn.Embedding,)
IGNORED_LAYERS = (nn.LayerNorm, nn.BatchNorm1d, nn.BatchNorm2d)


def is_transformers_conv1d(module: nn.Module) -> bool:
    return module.__class__.__name__ == "Conv1D"


def is_supported_layer(module: nn.Module, include_embeddings: bool = True,
                       include_conv2d: bool = False) -> bool:
    if isinstance(module, SUPPORTED_DENSE_LAYERS) or is_transformers_conv1d(module):
        return True
    if include_embeddings and isinstance(module, SUPPORTED_EMBEDDING_LAYERS):
        return True
    return bool(include_conv2d and isinstance(module, nn.Conv2d))


def get_layer_dimensions(module: nn.Module) -> Tuple[int, int]:
    """``(n_i, n_o)`` as GhostSuite defines them for each layer type."""
    if isinstance(module, nn.Linear):
        return module.in_features, module.out_features
    if is_transformers_conv1d(module):
        shape = module.weight.shape
        return shape[1], shape[0]
    if isinstance(module, nn.Conv1d):
        return module.in_channels * module.kernel_size[0], module.out_channels
    if isinstance(module, nn.Conv2d):
        return module.in_channels * module.kernel_size[0] * module.kernel_size[1], module.out_channels
    if isinstance(module, nn.Embedding):
        return module.num_embeddings, module.embedding_dim
    raise ValueError(f"Unsupported layer type: {module.__class__.__name__}")


def find_matching_layers(module: nn.Module, layer_patterns: Union[str, List[str]],
                         include_embeddings: bool = True,
                         include_conv2d: bool = False) -> Dict[str, nn.Module]:
    """Supported layers whose qualified name contains any of the patterns, in traversal order."""
    if isinstance(layer_patterns, str):
        patterns = [p.strip() for p in layer_patterns.split(",")]
    else:
        patterns = layer_patterns
    matched = {}
    for name, sub in module.named_modules():
        if is_supported_layer(sub, include_embeddings, include_conv2d) and \
                any(pat in name for pat in patterns):
            matched[name] = sub
    return matched


def validate_layer_selection(matched_layers: Dict[str, nn.Module],
                             layer_patterns: Union[str, List[str]]) -> None:
    if len(matched_layers) == 0:
        raise ValueError(f"No layers matched patterns: {layer_patterns}")
    print(f"Found {len(matched_layers)} layers for projection:")
    for name in sorted(matched_layers):
        layer = matched_layers[name]
        try:
            n_i, n_o = get_layer_dimensions(layer)
            print(f"  - {name} ({layer.__class__.__name__}): {n_i} -> {n_o}")
        except Exception:
            print(f"  - {name} ({layer.__class__.__name__})")


def compute_total_projection_size(matched_layers: Dict[str, nn.Module],
                                  projection_dims: Dict[str, Tuple[int, int]]) -> int:
    return sum(projection_dims[n][0] * projection_dims[n][1] for n in matched_layers)


def get_layer_slice_ranges(matched_layers: Dict[str, nn.Module],
                           projection_dims: Dict[str, Tuple[int, int]]) -> Dict[str, Tuple[int, int]]:
    """``name -> (start, end)`` inside the concatenated projection vector, sorted-name order."""
    ranges, cursor = {}, 0
    for name in sorted(matched_layers):
        k_i, k_o = projection_dims[name]
        ranges[name] = (cursor, cursor + k_i * k_o)
        cursor += k_i * k_o
    return ranges
