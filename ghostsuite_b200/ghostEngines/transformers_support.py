"""Model-side preparation so that every hooked layer sees a batch dimension.

GhostSuite's ``ghostEngines/transformers_support.py`` replaces whole Hugging Face forward methods
(copied per model family, tied to one transformers release) for two effects only:

1. position (and similar) embeddings must be looked up with ids of shape ``[batch, T]`` rather than
   ``[1, T]``, otherwise the out-grad that reaches the embedding's backward hook is already summed
   over the batch (``swap_gpt2_model_forward``, :171-267 there);
2. in dummy-bias mode every real parameter has ``requires_grad=False``; a one-element
   ``dummy_bias`` on each embedding keeps the autograd graph alive so that backward hooks fire
   (``_add_dummy_bias``, :17-37).

Both are done here with hooks that do not depend on the transformers version: a forward
pre-hook on the GPT-2 backbone injects batch-expanded ``position_ids``, and a forward hook on each
embedding adds ``dummy_bias * 0`` to its output.
"""
from __future__ import annotations

import torch
from torch import nn


def _add_dummy_bias(embedding: nn.Embedding):
    """Give ``embedding`` a one-element trainable ``dummy_bias`` that is added (times zero) to its
    output, and freeze its weight.  Idempotent."""
    if hasattr(embedding, "dummy_bias"):
        return
    embedding.register_parameter(
        "dummy_bias", nn.Parameter(torch.zeros(1, device=embedding.weight.device)))

    def add_bias(module, inputs, output):
        return output + module.dummy_bias.to(dtype=output.dtype, device=output.device) * 0

    embedding._ghost_dummy_bias_handle = embedding.register_forward_hook(add_bias)
    embedding.weight.requires_grad = False
    embedding.dummy_bias.initially_requires_grad = True


def _expand_position_ids(module, args, kwargs):
    """Forward pre-hook (with kwargs) for GPT-2 style backbones: supply ``position_ids`` of shape
    ``[batch, T]`` when the caller left them out."""
    if kwargs.get("position_ids") is not None:
        return None
    input_ids = kwargs.get("input_ids")
    if input_ids is None and args:
        input_ids = args[0]
    embeds = kwargs.get("inputs_embeds")
    if input_ids is not None:
        batch, seq = input_ids.shape[0], input_ids.shape[-1]
        device = input_ids.device
    elif embeds is not None:
        batch, seq = embeds.shape[0], embeds.shape[1]
        device = embeds.device
    else:
        return None
    if kwargs.get("past_key_values") is not None:
        return None   # generation with a cache: leave the model's own bookkeeping alone
    kwargs = dict(kwargs)
    kwargs["position_ids"] = torch.arange(seq, device=device).unsqueeze(0).expand(batch, seq).contiguous()
    return args, kwargs


def swap_gpt2_model_forward(backbone: nn.Module):
    """GPT-2 backbone (``GPT2Model``): batch-shaped position ids + dummy biases on wte / wpe."""
    if not hasattr(backbone, "_ghost_posid_handle"):
        backbone._ghost_posid_handle = backbone.register_forward_pre_hook(
            _expand_position_ids, with_kwargs=True)
    for name in ("wte", "wpe"):
        emb = getattr(backbone, name, None)
        if isinstance(emb, nn.Embedding):
            _add_dummy_bias(emb)


def forward_swapper(module: nn.Module):
    """Prepare ``module`` for per-sample hooks.  Plain nn.Modules are left alone; Hugging Face GPT-2
    heads get :func:`swap_gpt2_model_forward`; a module can opt in by defining
    ``ghost_prepare(self)`` (used by the synthetic workloads of this package)."""
    prepare = getattr(module, "ghost_prepare", None)
    if callable(prepare):
        prepare()
        return
    try:
        import transformers
    except Exception:  # pragma: no cover
        return
    if not isinstance(module, transformers.PreTrainedModel):
        return
    if isinstance(module, (transformers.GPT2LMHeadModel, transformers.GPT2DoubleHeadsModel)):
        swap_gpt2_model_forward(module.transformer)
        return
    # other families: make sure at least the embeddings keep the graph alive in dummy-bias mode
    for sub in module.modules():
        if isinstance(sub, nn.Embedding):
            _add_dummy_bias(sub)
