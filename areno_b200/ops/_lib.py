"""ctypes loader for ``libareno_kernels.so`` (the sm_100a kernel library).

The library exposes a flat C ABI (see ``csrc/launch.h``).  Python passes raw device pointers
(``tensor.data_ptr()``) and the current CUDA stream handle; nothing here allocates.

On a machine with a GPU a missing library is a hard error: ops never fall back to eager
PyTorch for CUDA tensors.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Any

import torch

_SIG_CODES = {
    "p": ctypes.c_void_p,
    "i": ctypes.c_int,
    "l": ctypes.c_longlong,
    "f": ctypes.c_float,
}

# name -> argument type codes (p = pointer, i = int, l = long long, f = float); all return int.
_SIGNATURES: dict[str, str] = {
    "areno_gemm_bf16": "ppppiiillliiiiplpp",
    "areno_rmsnorm_fwd": "pppifppplifp",
    "areno_gemm_bf16_partials": "pppiiilllplppp",
    "areno_gemm_bf16_gated": "pppiiilllipp",
    "areno_splitk_residual_rmsnorm": "pilppifpplifp",
    "areno_rmsnorm_bwd_blocks": "l",
    "areno_rmsnorm_bwd": "pppifpppppilip",
    "areno_gated_act_fwd": "ppliip",
    "areno_gated_act_bwd": "pppliip",
    "areno_unary_act": "pppliip",
    "areno_rope": "pppliiilffip",
    "areno_embedding_fwd": "ppplillfp",
    "areno_embedding_bwd": "ppplillfp",
    "areno_accumulate_bf16": "pplp",
    "areno_attn_fwd": "pppppppp" + "iiiii" + "llll" + "fiip",
    "areno_attn_fwd_tc": "pppppppp" + "iiiii" + "llllll" + "fi" + "pp",
    "areno_attn_bwd": "pppppppppp" + "pppp" + "iii" + "l" + "iii" + "llllllll" + "fiiplp",
    "areno_gemm_workspace_bytes": "iii",
    "areno_headnorm_fwd": "plpifplpliifp",
    "areno_headnorm_bwd_blocks": "l",
    "areno_headnorm_bwd": "plplpifpplppiliip",
    "areno_page_size": "",
    "areno_rope_append_kv": "pppppppp" + "l" + "iiii" + "f" + "iii" + "p",
    "areno_fold_rope_append_kv": "pil" + "ppppppppp" + "l" + "iiii" + "f" + "iii" + "pp" + "i" + "ff" + "p",
    "areno_paged_decode": "pppppppppp" + "iiiii" + "ll" + "f" + "iiii" + "p",
    "areno_logprob_stats": "pilliplppppp",
    "areno_logprob_bwd": "pilliplppppp",
    "areno_sample": "pilliippififlpppp" + "pip",
    "areno_adamw_fp32": "ppppplfffffifpp",
    "areno_adamw_8bit": "ppppppplfffffifpp",
    "areno_sumsq_blocks": "",
    "areno_sumsq": "plppip",
    "areno_scale_f32": "plpfp",
    "areno_cast_f32_bf16": "pplp",
    "areno_policy_loss": "ppppppppplfffip",
}

_lock = threading.Lock()
_cdll: ctypes.CDLL | None = None
_load_error: str | None = None


def register_signature(name: str, codes: str) -> None:
    """Declare the argument types of another exported symbol (used by sibling op modules)."""
    _SIGNATURES[name] = codes


def _load() -> ctypes.CDLL:
    global _cdll, _load_error
    if _cdll is not None:
        return _cdll
    with _lock:
        if _cdll is not None:
            return _cdll
        from areno_b200 import build

        path = build.kernels_lib_path()
        try:
            build.build_kernels()
        except Exception as exc:  # pragma: no cover - depends on toolchain
            if not path.exists():
                _load_error = f"kernel library is not built and could not be built: {exc}"
                raise RuntimeError(_load_error) from exc
        _cdll = ctypes.CDLL(str(path))
        return _cdll


def available() -> bool:
    """True when the kernel library can be loaded (does not require a GPU)."""
    try:
        _load()
        return True
    except Exception:
        return False


_fn_cache: dict[str, Any] = {}


def fn(name: str):
    f = _fn_cache.get(name)
    if f is None:
        lib = _load()
        f = getattr(lib, name)
        codes = _SIGNATURES[name]
        f.argtypes = [_SIG_CODES[c] for c in codes]
        f.restype = ctypes.c_int
        _fn_cache[name] = f
    return f


# Kernel launches issued through this module (an entry point may launch more than one kernel).
_KERNELS_PER_CALL = {"areno_attn_bwd": 4, "areno_paged_decode": 2, "areno_rmsnorm_bwd": 2, "areno_sumsq": 2,
                     "areno_headnorm_bwd": 2}
launch_count = 0


def call(name: str, *args) -> int:
    """Invoke an entry point and raise on a non-zero return code."""
    global launch_count
    launch_count += _KERNELS_PER_CALL.get(name, 1)
    rc = fn(name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    return rc


# Debug mode ``ARENO_BOUNDS_CHECK=1``: every data-dependent index a kernel is about to use (cache slots, page ids,
# token ids, targets, expert ids, row maps) is range-checked on the host BEFORE the launch, and the wrappers
# verify canary words that they place behind their scratch buffers after it.  A violation raises here, with the
# name of the operand, instead of reaching the GPU as an out-of-range access.  Costs a device synchronisation per
# checked operand, so it is for tests and for chasing a fault, not for production runs.
BOUNDS_CHECK = os.environ.get("ARENO_BOUNDS_CHECK", "0").lower() in {"1", "true", "yes", "on"}
CANARY = 0x5AFEC0DE


def check_index(name: str, index: torch.Tensor | None, limit: int, *, low: int = 0, enabled: bool | None = None) -> None:
    """Raise ``IndexError`` unless every element of ``index`` lies in ``[low, limit)`` (``low=-1`` admits the
    "skip" marker used by slot mappings and row maps).  A no-op unless the checked mode is on."""
    if not (BOUNDS_CHECK if enabled is None else enabled) or index is None or index.numel() == 0:
        return
    lo, hi = int(index.min()), int(index.max())
    if lo < low or hi >= limit:
        bad = int(((index < low) | (index >= limit)).sum())
        raise IndexError(f"{name}: {bad} of {index.numel()} indices outside [{low}, {limit}) (min {lo}, max {hi})")


def with_canary(nbytes: int, device) -> torch.Tensor:
    """uint8 scratch of ``nbytes`` followed by a 16-byte canary (checked mode); plain scratch otherwise."""
    if not BOUNDS_CHECK:
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    padded = (nbytes + 15) // 16 * 16
    buf = torch.empty(padded + 16, dtype=torch.uint8, device=device)
    buf[padded:].view(torch.int32).fill_(CANARY if CANARY < 2**31 else CANARY - 2**32)
    return buf


def check_canary(name: str, buf: torch.Tensor) -> None:
    if not BOUNDS_CHECK or buf.numel() < 16:
        return
    tail = buf[-16:].view(torch.int32)
    want = CANARY if CANARY < 2**31 else CANARY - 2**32
    if not bool((tail == want).all()):
        raise RuntimeError(f"{name}: a kernel wrote past the end of its scratch buffer (canary overwritten)")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_status: dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] status words written by kernels whose bounded waits ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = buf
    return buf


def check_status(device: torch.device | None = None) -> None:
    """Synchronising check of the status words; raises if any kernel reported an error."""
    for idx, buf in list(_status.items()):
        if device is not None and device.index not in (None, idx):
            continue
        vals = buf.tolist()
        if vals[0] != 0:
            buf.zero_()
            raise RuntimeError(f"device kernel reported status code={vals[0]} block={vals[1]} stage={vals[2]}")
