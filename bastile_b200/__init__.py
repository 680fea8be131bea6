"""bastile_b200 - the four Qwen3 training ops of aghilann/bastile as hand-written
sm_100a CUDA behind the same patch API.

    import bastile_b200 as bastile
    bastile.apply()            # before the model is constructed
    model = Qwen3ForCausalLM(config)

The public names, defaults and return values are those of the reference
package (src/bastile/__init__.py:18-33).
"""

from .autotune import clear_cache as clear_autotune_cache
from .autotune import warmup_all_kernels
from .core import apply, apply_to_model, get_patched_ops, reset
from .registry import list_patches, register_patch

__version__ = "0.1.0"
__all__ = [
    "apply",
    "apply_to_model",
    "clear_autotune_cache",
    "get_patched_ops",
    "list_patches",
    "register_patch",
    "reset",
    "warmup_all_kernels",
]
