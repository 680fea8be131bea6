"""apply() / reset(): swap the four Qwen3 hot-path ops of HF transformers for the
sm_100a kernels and back.

Mirrors src/bastile/core.py:79-205 of the reference: same keyword arguments,
same returned names in the same order (registry patches in registration order,
then the literal ``"fused_linear_cross_entropy"``), patch failures logged and
not raised, idempotent re-application, and a warm-up at the end of ``apply``.

One deliberate difference: the reference overwrites
``Qwen3ForCausalLM.forward`` without keeping the original, so its ``reset()``
cannot undo the fused-loss patch (core.py:136-146 vs :179-200).  Here the
original ``forward`` is kept and ``reset()`` with no arguments, or with
``"fused_linear_cross_entropy"`` in ``names``, puts it back - the state that
``reset()`` leaves is then the unpatched HF eager model.  The return value of
``reset()`` and of ``get_patched_ops()`` still lists registry patches only, as
in the reference.

One addition, off by default: ``apply(fused_layers=True)`` also replaces
``Qwen3DecoderLayer.forward`` and ``Qwen3Attention.forward`` with versions that
fold the residual adds into the norm / down-projection kernels and run
q/k-norm + RoPE as one kernel (``ops/fused_layers.py``).  With it the q/k/v
projections keep their library GEMMs but let those GEMMs accumulate the shared
input gradient (``gemm_projections="acc"``, the default; ``"off"`` leaves
``nn.Linear`` alone; ``"dx"``, ``"all"`` and ``"qkv"`` move the input gradient, every
product, or the stacked q|k|v product to the library's own GEMM); the names
``"decoder_layer_qwen3"`` and ``"attention_qwen3"`` are then appended to the
returned list, and ``reset()`` restores both methods.
"""

from __future__ import annotations

import importlib
import logging
from typing import Any

from .registry import PatchInfo, get_registry

log = logging.getLogger(__name__)

_QWEN3 = "transformers.models.qwen3.modeling_qwen3"
_LCE_NAME = "fused_linear_cross_entropy"
_lce_original_forward: Any = None

# apply()'s boolean switches and the registry names they govern.  A switch
# governs a patch when its key occurs in the patch name or the name starts with
# the key's first word (core.py:123-129) - first matching switch wins.
_SWITCH_ORDER = ("rms_norm", "swiglu", "rope")


def _module(path: str):
    try:
        return importlib.import_module(path)
    except ImportError as exc:
        log.warning("Could not import %s: %s", path, exc)
        return None


def _install(patch: PatchInfo) -> bool:
    if patch.is_applied:
        return True
    mod = _module(patch.target_module)
    if mod is None or not hasattr(mod, patch.target_attr):
        log.warning("Could not apply patch '%s': %s.%s not found", patch.name, patch.target_module, patch.target_attr)
        return False
    original = getattr(mod, patch.target_attr)
    setattr(mod, patch.target_attr, patch.replacement)
    get_registry().mark_applied(patch.name, original)
    log.info("Applied patch: %s (%s)", patch.name, patch.description)
    return True


def _uninstall(patch: PatchInfo) -> bool:
    if not patch.is_applied:
        return True
    if patch.original is None:
        log.warning("Cannot reset patch '%s': original not stored", patch.name)
        return False
    mod = _module(patch.target_module)
    if mod is None:
        return False
    setattr(mod, patch.target_attr, patch.original)
    get_registry().mark_reset(patch.name)
    log.info("Reset patch: %s", patch.name)
    return True


def _switch_for(name: str, switches: dict[str, bool]) -> bool:
    for key in _SWITCH_ORDER:
        if key in name or name.startswith(key.split("_")[0]):
            return switches[key]
    return True


def apply(rms_norm: bool = True, swiglu: bool = True, rope: bool = True,
          fused_linear_cross_entropy: bool = True, model_type: str | None = None, **kwargs) -> list[str]:
    """Patch HF Qwen3 with the B200 kernels; returns the names applied.

    Call before constructing the model: ``Qwen3RMSNorm`` and ``Qwen3MLP`` are
    classes looked up at construction time.
    """
    global _lce_original_forward
    from . import ops  # noqa: F401  (import registers the patches)

    reg = get_registry()
    switches = {"rms_norm": rms_norm, "swiglu": swiglu, "rope": rope}
    if model_type:
        candidates = reg.get_for_model(model_type)
    else:
        candidates = [p for p in (reg.get(n) for n in reg.list_all()) if p is not None]

    applied: list[str] = []
    for patch in candidates:
        if _switch_for(patch.name, switches) and _install(patch):
            applied.append(patch.name)

    if kwargs.get("fused_layers", False) and rms_norm and (model_type in (None, "qwen3")):
        try:
            from .ops import fused_layers

            applied.extend(fused_layers.install(importlib.import_module(_QWEN3), decoder_layer=True,
                                                attention=bool(rope),
                                                projections=kwargs.get("gemm_projections", "acc")))
        except Exception as exc:  # patch failures are reported, not raised
            log.warning("Could not apply the fused decoder-layer forwards: %s", exc)

    if fused_linear_cross_entropy:
        try:
            qwen3 = importlib.import_module(_QWEN3)
            from .ops.fused_linear_cross_entropy import bastile_lce_forward

            current = qwen3.Qwen3ForCausalLM.forward
            if current is not bastile_lce_forward:
                _lce_original_forward = current
                qwen3.Qwen3ForCausalLM.forward = bastile_lce_forward
            applied.append(_LCE_NAME)
            log.info("Applied fused linear cross-entropy (logits are never materialised)")
        except Exception as exc:  # patch failures are reported, not raised
            log.warning("Could not apply fused linear cross-entropy: %s", exc)

    try:
        from .autotune import warmup_all_kernels

        warmup_all_kernels()
    except Exception as exc:
        log.debug("Warmup skipped: %s", exc)
    return applied


def apply_to_model(model: Any, **kwargs) -> list[str]:
    """``apply`` filtered by ``model.config.model_type`` (classes are patched, not
    the instance: modules that already exist keep their original ops)."""
    model_type = getattr(getattr(model, "config", None), "model_type", None)
    log.info("Applying patches for model type: %s", model_type)
    return apply(model_type=model_type, **kwargs)


def _restore_lce_forward() -> None:
    global _lce_original_forward
    if _lce_original_forward is None:
        return
    qwen3 = _module(_QWEN3)
    if qwen3 is not None:
        qwen3.Qwen3ForCausalLM.forward = _lce_original_forward
    _lce_original_forward = None


def _restore_fused_layers(names: list[str] | None) -> None:
    from .ops import fused_layers

    if fused_layers.installed():
        qwen3 = _module(_QWEN3)
        if qwen3 is not None:
            fused_layers.uninstall(qwen3, names)


def reset(names: list[str] | None = None) -> list[str]:
    """Undo patches (all when ``names`` is None); returns the registry names reset."""
    reg = get_registry()
    _restore_fused_layers(names)
    if names is None:
        _restore_lce_forward()
        names = reg.get_applied()
    elif _LCE_NAME in names:
        _restore_lce_forward()
    done = []
    for name in names:
        patch = reg.get(name)
        if patch and _uninstall(patch):
            done.append(name)
    return done


def get_patched_ops() -> list[str]:
    return get_registry().get_applied()
