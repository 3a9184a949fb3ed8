"""generate() wiring of the paged KV cache.

Only the part of the reference's ``python/barqtrain/patch_models.py`` that calls the paged-cache
path is here: ``_patch_generate_with_paged_kv`` (patch_models.py:235-261), reached through
``patch_inference`` (patch_models.py:319-329).  The reference's other patchers (RMSNorm, chunked
loss, attention backend selection) belong to training ops outside this package's scope.
"""

from __future__ import annotations

import types

import torch


def _patch_generate_with_paged_kv(model: torch.nn.Module, model_label: str) -> torch.nn.Module:
    """Wrap ``model.generate`` once so that calls without a cache get a ``BarqPagedKVCache``.

    Sets the same attributes as the reference: ``_barqtrain_generate_paged_kv_patched``,
    ``_barqtrain_paged_kv_supported`` and, per call, ``_barqtrain_last_generate_used_paged_kv``.
    """
    if getattr(model, "_barqtrain_generate_paged_kv_patched", False) or not hasattr(model, "generate"):
        return model

    from . import kv_cache

    inner_generate = model.generate

    def generate(self, *args, **kwargs):
        new_kwargs, used = kv_cache.maybe_prepare_paged_kv_generate_kwargs(self, args, kwargs)
        self._barqtrain_last_generate_used_paged_kv = used
        return inner_generate(*args, **new_kwargs)

    model.generate = types.MethodType(generate, model)
    model._barqtrain_generate_paged_kv_patched = True
    model._barqtrain_paged_kv_supported = kv_cache.paged_kv_supported_for_model(model)
    if model._barqtrain_paged_kv_supported:
        print(f"BarqTrain: Enabled paged KV-cache injection for {model_label}")
    return model


def patch_inference(model: torch.nn.Module) -> torch.nn.Module:
    """Inference-side patching: here, the paged KV-cache injection into ``generate()``."""
    label = getattr(getattr(model, "config", None), "model_type", None) or type(model).__name__
    return _patch_generate_with_paged_kv(model, str(label))


__all__ = ["patch_inference"]
