"""ctypes binding of ``libbastile_b200.so`` (declarations: ``include/bastile_b200.h``).

The library is the only implementation of the ops: when it cannot be loaded the
ops raise, they never fall back to torch or the CPU.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import torch

BT_BF16, BT_FP16, BT_FP32 = 0, 1, 2

_DTYPES = {torch.bfloat16: BT_BF16, torch.float16: BT_FP16, torch.float32: BT_FP32}

_lock = threading.Lock()
_lib = None

class GemmDesc(ctypes.Structure):
    """``bt_gemm_desc`` of include/bastile_b200.h."""

    _fields_ = [("A", c_void_p), ("B", c_void_p), ("lda", c_int64), ("ldb", c_int64), ("K", c_int64),
                ("A1", c_void_p), ("B1", c_void_p), ("lda1", c_int64), ("ldb1", c_int64), ("K1", c_int64),
                ("D", c_void_p), ("ldd", c_int64), ("M", c_int64), ("N", c_int64),
                ("a_kmajor", ctypes.c_int32), ("b_kmajor", ctypes.c_int32),
                ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
                ("addend", c_void_p), ("ld_addend", c_int64), ("addend_t", c_void_p), ("ld_addend_t", c_int64),
                ("alpha", c_void_p),
                ("A2", c_void_p), ("lda2", c_int64), ("K2", c_int64),
                ("a_split", ctypes.c_int32), ("d_split", ctypes.c_int32), ("M0", c_int64), ("M1", c_int64),
                ("D1", c_void_p), ("D2", c_void_p), ("ldd1", c_int64), ("ldd2", c_int64), ("N0", c_int64),
                ("N1", c_int64)]


I64x3 = c_int64 * 3
I64x2 = c_int64 * 2

# name -> (restype, argtypes); mirrors include/bastile_b200.h one to one.
SIGNATURES = {
    "bt_version": (c_int, []),
    "bt_last_error": (c_char_p, []),
    "bt_sm_count": (c_int, []),
    "bt_device_wait_errors": (c_int, []),
    "bt_set_wait_limit_ms": (c_int, [c_int64]),
    "bt_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                               c_float, c_int, c_void_p]),
    "bt_rmsnorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "bt_rmsnorm_bwd_ws_bytes": (c_int64, [c_int64]),
    "bt_add_rmsnorm_fwd": (c_int, [c_void_p] * 6 + [c_int64] * 6 + [c_float, c_int, c_void_p]),
    "bt_add_rmsnorm_bwd": (c_int, [c_void_p] * 8 + [c_int64] * 6 + [c_int, c_void_p]),
    "bt_qk_norm_rope_fwd": (c_int, [c_void_p] * 10 + [c_int64] * 5 + [POINTER(c_int64)] * 5 +
                            [c_int64, c_float, c_float, c_int, c_void_p]),
    "bt_qk_norm_rope_bwd": (c_int, [c_void_p] * 16 + [c_int64] * 5 + [POINTER(c_int64)] * 7 +
                            [c_int64, c_int, c_void_p]),
    "bt_rmsnorm_bwd_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int, c_void_p]),
    "bt_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                        c_int64, c_int64, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                        POINTER(c_int64), POINTER(c_int64), c_int64, c_int, c_int, c_void_p]),
    "bt_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                              c_void_p]),
    "bt_swiglu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                              c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "bt_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                        c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "bt_gemm_ex": (c_int, [POINTER(GemmDesc), c_void_p, c_void_p]),
    "bt_set_gemm_cta_pairs": (c_int, [c_int]),
    "bt_set_gemm_dynamic_tiles": (c_int, [c_int]),
    "bt_set_gemm_tile_stores": (c_int, [c_int]),
    "bt_set_gemm_group_rows": (c_int, [c_int]),
    "bt_set_dependent_launch": (c_int, [c_int]),
    "bt_mlp_fwd": (c_int, [c_void_p] * 8 + [c_int64] * 4 + [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "bt_mlp_bwd": (c_int, [c_void_p] * 14 + [c_int64] * 6 + [c_int, c_void_p, c_void_p]),
    "bt_lce_logits_stats": (c_int, [c_void_p] * 6 + [c_int64] * 7 + [c_int, c_void_p, c_void_p]),
    "bt_lce_num_vtiles": (c_int64, [c_int64]),
    "bt_lce_row_stats": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "bt_lce_stats_combine": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bt_lce_dlogits": (c_int, [c_void_p] * 5 + [c_int64] * 5 + [c_int, c_int, c_void_p]),
    "bt_lce_count_valid": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p,
                                   c_void_p]),
    "bt_lce_reduce_loss": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "bt_adamw_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_float,
                              c_float, c_float, c_int64, c_int, c_int, c_void_p]),
    "bt_adamw_master_step": (c_int, [c_void_p] * 5 + [c_int64] + [c_float] * 5 + [c_int64, c_float, c_int, c_int,
                                     c_void_p]),
    "bt_scale_cast": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]),
}


def lib_path() -> Path:
    env = os.environ.get("BASTILE_B200_LIB")
    return Path(env) if env else Path(__file__).resolve().parent / "libbastile_b200.so"


def get_lib() -> ctypes.CDLL:
    """Load (once) and return the shared library; raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = lib_path()
            if not path.exists():
                raise RuntimeError(
                    f"{path} is missing: build it with `python -m bastile_b200.build` "
                    "(bastile_b200 has no fallback implementation)"
                )
            lib = ctypes.CDLL(str(path))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError here = library older than the header
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


class BastileB200Error(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = get_lib().bt_last_error().decode(errors="replace")
        raise BastileB200Error(f"{what} failed (code {rc}): {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"bastile_b200: unsupported dtype {dtype}") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t.device.type != "cuda":
            raise RuntimeError(
                "bastile_b200 ops run on CUDA (sm_100a) tensors only; got a tensor on "
                f"'{t.device}'. There is no CPU implementation."
            )
        if t.device != dev:
            raise RuntimeError(f"bastile_b200: tensors on different devices ({dev} vs {t.device})")
    return dev


def stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


class device_of:
    """Make ``dev`` the current CUDA device for the duration of a launch."""

    def __init__(self, dev: torch.device):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


# Where the gradient of a weight should be written, keyed by the weight's data pointer.  An
# optimizer that keeps gradients in flat buckets (optim.ShardedAdamW) registers its bucket views
# here; the ops that allocate weight gradients themselves (MLP block, fused loss) then write
# straight into the bucket instead of into a fresh tensor that would be copied there afterwards.
_grad_sinks: dict[int, torch.Tensor] = {}


def register_grad_sink(weight: torch.Tensor, destination: torch.Tensor) -> None:
    _grad_sinks[weight.data_ptr()] = destination


def unregister_grad_sinks(destinations) -> None:
    ids = {id(d) for d in destinations}
    for key in [k for k, v in _grad_sinks.items() if id(v) in ids]:
        del _grad_sinks[key]


def grad_sink(weight: torch.Tensor, dtype: torch.dtype):
    """The registered destination for ``weight``'s gradient if it fits (shape, dtype, device)."""
    dest = _grad_sinks.get(weight.data_ptr())
    if dest is None or dest.shape != weight.shape or dest.dtype != dtype or dest.device != weight.device:
        return None
    # a FRESH view object: autograd only adopts an incoming gradient without cloning it when nothing
    # else holds a reference to that tensor object (the registry keeps the original)
    return dest.view(dest.shape)


# Per (device, stream) scratch that must start zeroed and that kernels leave zeroed.
_zero_ws: dict[tuple[int, int], torch.Tensor] = {}
# Per (device, stream) int32 status word for the bounded waits of the GEMM kernels.
_status: dict[tuple[int, int], torch.Tensor] = {}


def zero_workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    key = (dev.index or 0, stream_ptr(dev))
    buf = _zero_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=dev)
        _zero_ws[key] = buf
    return buf


def status_word(dev: torch.device) -> torch.Tensor:
    key = (dev.index or 0, stream_ptr(dev))
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = buf
    return buf


# ---------------------------------------------------------------------------
# Instrumentation used by the benchmark: a count of kernels launched by the ops
# and, when switched on, CUDA-event pairs around the calls into the library
# (recorded on the stream the kernels run on).  Off by default; the ops pay one
# attribute test per call.
class _Instrumentation:
    def __init__(self):
        self.enabled = False
        self.launches = 0
        self.events: dict[str, list] = {}

    def reset(self, enabled: bool) -> None:
        self.enabled = enabled
        self.launches = 0
        self.events = {}

    def elapsed_ms(self) -> dict[str, tuple[int, float]]:
        """name -> (calls, total milliseconds); synchronises."""
        torch.cuda.synchronize()
        return {k: (len(v), sum(a.elapsed_time(b) for a, b in v)) for k, v in self.events.items()}


instr = _Instrumentation()


class timed:
    """``with timed("mlp_fwd", n_kernels, dev):`` around a library call."""

    __slots__ = ("name", "n", "dev", "start")

    def __init__(self, name: str, n_kernels: int, dev: torch.device):
        self.name, self.n, self.dev, self.start = name, n_kernels, dev, None

    def __enter__(self):
        if instr.enabled:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, *exc):
        instr.launches += self.n
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.dev))
            instr.events.setdefault(self.name, []).append((self.start, end))
        return False


STATUS_WAIT_MASK, STATUS_BAD_LABEL = 0x0F, 0x10  # BT_STATUS_* of include/bastile_b200.h


def _describe_status(v: int) -> str:
    parts = []
    if v & STATUS_WAIT_MASK:
        parts.append(f"a bounded device-side wait ran out (bits {v & STATUS_WAIT_MASK:#x}): results are invalid")
    if v & STATUS_BAD_LABEL:
        parts.append("fused_linear_cross_entropy got a label that is neither ignore_index nor a vocabulary row")
    return "; ".join(parts) or f"status {v:#x}"


def _reset_zero_workspaces() -> None:
    """A kernel that gave up may have left its 'zero on entry, zero on exit' scratch dirty."""
    for buf in _zero_ws.values():
        buf.zero_()


def check_status(dev: torch.device, what: str) -> None:
    """Synchronising read of the current stream's status word on ``dev``; raises if it is set."""
    st = status_word(dev)
    v = int(st.item())
    if v != 0:
        st.zero_()
        if v & STATUS_WAIT_MASK:
            _reset_zero_workspaces()
        raise BastileB200Error(f"{what}: {_describe_status(v)}")


def check_all_status() -> None:
    """Synchronising check of every status word the ops have handed to the kernels and of the
    bulk-copy wait flag of the RMSNorm kernels.  Raises if a bounded device-side wait ever ran out
    (the results of that call were invalid) or a loss call saw an out-of-range label; after a wait
    error every cached zero-scratch buffer is cleared again, so that later calls start from the
    state they expect.  The ops never call this themselves - they do not synchronise - so a
    training loop calls it where it syncs anyway (``AdamW(check_device_status=True)`` does it at
    the end of ``step()``; reading the loss with ``.item()`` is another natural place)."""
    bad, waits = [], False
    for (dev_idx, _stream), word in _status.items():
        v = int(word.item())
        if v:
            word.zero_()
            waits |= bool(v & STATUS_WAIT_MASK)
            bad.append(f"cuda:{dev_idx}: {_describe_status(v)}")
    if _lib is not None and torch.cuda.is_available():
        v = int(_lib.bt_device_wait_errors())
        if v:
            waits = True
            bad.append(f"RMSNorm bulk-copy wait flag {v:#x}")
    if waits:
        _reset_zero_workspaces()
    if bad:
        raise BastileB200Error("; ".join(bad))
