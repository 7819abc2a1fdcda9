"""Python faces of the CUDA kernels: each takes torch tensors on a CUDA device, checks what the
kernel assumes (types, shapes, contiguity), and launches on torch's current stream.

There is no other implementation behind these functions.  If the library cannot be built or
loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import build as _build

F32, BF16 = 0, 1
STATUS_BAD_TOKEN, STATUS_BAD_PAGE, STATUS_TIMEOUT = 1, 2, 4

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
_c_ull = ctypes.c_ulonglong

_SIGNATURES = {
    "bg_embed_gather": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "bg_softcap": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "bg_fill_normal": [_c_void_p, _c_int, _c_ll, _c_ull, _c_ll, _c_float, _c_float, _c_void_p],
    "bg_add_rmsnorm": [_c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_float, _c_void_p, _c_int,
                       _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_add_residual": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "bg_swiglu": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_activation": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_ll, _c_int, _c_void_p],
    "bg_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "bg_rope_kv_append": [_c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_attention_plan": [_c_int, _c_int, _c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "bg_attention_partial": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int,
                             _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_void_p],
    "bg_attention_merge": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_rmsnorm_add": [_c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int,
                       _c_int, _c_void_p],
    "bg_rmsnorm_add_routed": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_float, _c_void_p,
                              _c_int, _c_int, _c_int, _c_void_p],
    "bg_cast_rows": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "bg_qk_norm_rope_append": [_c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                               _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                               _c_void_p],
    "bg_route_logits": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_route_topk": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p],
    "bg_route": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float,
                 _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "bg_route_combine_ext": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p,
                             _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_glu_clamped": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p],
    "bg_lane_step": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                     _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "bg_lane_fill": [_c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p],
    "bg_rglru_scan": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll,
                      _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_rglru_scan_chunked": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll,
                              _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                              _c_int, _c_int, _c_void_p],
    "bg_rglru_softplus": [_c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_void_p],
    "bg_rglru_split": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_route_sort": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "bg_route_gather": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_route_combine": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_gemm_grouped": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                        _c_int, _c_int, _c_int, _c_void_p],
    "bg_gemm_grouped_tc": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                           _c_void_p, _c_int, _c_void_p, _c_void_p],
    "bg_sigmoid_gate": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_ll,
                        _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_decay_attention": [_c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll, _c_void_p,
                           _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_decay_attention_chunk_plan": [_c_int, _c_int, ctypes.POINTER(_c_int)],
    "bg_decay_attention_chunked": [_c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll,
                                   _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                   _c_void_p],
    "bg_add_terms_norm": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "bg_attention_mma_plan": [_c_int, _c_int, _c_int, ctypes.POINTER(_c_int)],
    "bg_attention_mma_partial": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                 _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                 _c_int, _c_float, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "bg_attention_tc_plan": [_c_int, _c_int, _c_int, ctypes.POINTER(_c_int)],
    "bg_attention_tc": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                        _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p, _c_void_p],
    "bg_attention_tc_ext": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                            _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_float,
                            _c_void_p, _c_void_p],
    "bg_attention_tc_sink": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                             _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p, _c_void_p],
    "bg_gemm_f32_nt": [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_void_p],
    "bg_gemm_bf16_tn": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                        _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_gemm_pair": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int,
                     _c_void_p, _c_void_p],
    "bg_gemm_fused": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                      _c_void_p, _c_float, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                      _c_void_p, _c_void_p],
    "bg_gemm_fused_rope": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                           _c_void_p, _c_float, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                           _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                           _c_void_p],
    "bg_add_layernorm": [_c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_float, _c_void_p, _c_int,
                         _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "bg_depth_mix": [_c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_ll, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p],
    "bg_xielu": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_void_p, _c_int, _c_ll, _c_void_p],
    "bg_rmsnorm_slice": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_int, _c_int,
                         _c_int, _c_void_p],
    "bg_gate_heads": [_c_void_p, _c_int, _c_ll, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                      _c_int, _c_void_p],
    "bg_latent_attention_plan": [_c_int, _c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "bg_latent_append": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_float, _c_void_p,
                         _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                         _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "bg_latent_attention_partial": [_c_void_p, _c_int, _c_ll, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                    _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                                    _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                    _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "bg_latent_attention_merge": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int,
                                  _c_int, _c_int, _c_int, _c_void_p],
    "bg_latent_attention_mma_plan": [_c_int, _c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "bg_latent_attention_mma_partial": [_c_void_p, _c_ll, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                                        _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                        _c_void_p, _c_void_p],
    "bg_latent_gather": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                         _c_void_p],
    "bg_latent_expand": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_rotate_q": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p],
    "bg_conv_silu": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_ll,
                     _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "bg_ssm_scan": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                    _c_ll, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_gated_group_rmsnorm": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_int,
                               _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "bg_gemm_f32_nt_batched": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_int, _c_ll, _c_void_p, _c_int, _c_ll, _c_int, _c_int,
                               _c_int, _c_int, _c_void_p],
    "bg_sample": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "bg_sample_feed": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_void_p],
}

_lib = None


class KernelError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        handle = _build.load()
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise KernelError(f"the kernel library lacks '{name}'") from e
            fn.argtypes = argtypes
            fn.restype = _c_int
        _lib = handle
    return _lib


def available() -> bool:
    """True when a CUDA device is present.  (The library itself builds without one.)"""
    return torch.cuda.is_available()


_ARG_ERRORS = {-1: "unsupported element type", -2: "unsupported shape", -3: "misaligned tensor",
               -4: "sizes that this kernel does not take"}


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or recorded into a graph) so far."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels that a replayed CUDA graph launched."""
    global _launches
    _launches += n


def _check(rc: int, name: str) -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc < 0:
        raise KernelError(f"{name}: refused: {_ARG_ERRORS.get(rc, rc)}")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


# ------------------------------------------------------------------------------------------------
# Phase timers (the reference's QWEN_PROF, qwen_infer.c:1224-1235): while a profile is open, every kernel
# class is bracketed by two CUDA events on the launching stream; `profile_end` adds up the device time
# between them per class.  Closed, `phase` hands out one shared do-nothing context.
class _NoPhase:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


class _Phase:
    __slots__ = ("name", "start")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        _profile.append((self.name, self.start, end))
        return False


_NO_PHASE = _NoPhase()
_profile = None            # None: closed; a list of (class, start event, end event) while open
_depth = 0


def phase(name: str):
    """Context for the launches of one kernel class.  Phases do not nest: inside an open phase an inner
    one is part of it."""
    if _profile is None:
        return _NO_PHASE
    return _Outer(name)


class _Outer(_Phase):
    def __enter__(self):
        global _depth
        _depth += 1
        if _depth == 1:
            super().__enter__()

    def __exit__(self, *exc):
        global _depth
        if _depth == 1:
            super().__exit__(*exc)
        _depth -= 1
        return False


def profile_begin() -> None:
    global _profile, _depth
    _profile, _depth = [], 0


def profile_end() -> dict:
    """Close the profile: {kernel class: (device milliseconds, brackets)} in order of first use.  Waits for
    the device."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    out = {}
    for name, start, end in records:
        ms, n = out.get(name, (0.0, 0))
        out[name] = (ms + start.elapsed_time(end), n + 1)
    return out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensors must be float32 or bfloat16, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("beglin_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The raw handle of torch's current stream on the current device (a cheap call; the public
    torch.cuda.current_stream() costs several microseconds, which counts at hundreds of launches a step)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _i32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def new_status(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor) -> None:
    """Read the status word (this waits for the device) and raise if a kernel recorded a fault."""
    v = int(status.item())
    if v == 0:
        return
    status.zero_()
    what = []
    if v & STATUS_BAD_TOKEN:
        what.append("a token id outside the vocabulary")
    if v & STATUS_BAD_PAGE:
        what.append("a block-table entry outside the page pool")
    if v & STATUS_TIMEOUT:
        what.append("a bounded wait inside a kernel ran out")
    raise KernelError("a kernel recorded: " + "; ".join(what or [f"status {v}"]))


# ------------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor],
                 scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32; an id outside the table sets BG_STATUS_BAD_TOKEN."""
    _cuda(table, ids, out)
    _i32(ids, "ids")
    T, d = ids.numel(), table.shape[1]
    if out.dtype != torch.float32 or tuple(out.shape) != (T, d) or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed_gather: out must be contiguous float32 [T, d] and the table contiguous")
    with phase("emb_gather"):
        _check(lib().bg_embed_gather(_p(table), _dt(table), _p(ids), _p(out), T, d, table.shape[0], float(scale), _p(status),
                                     _stream()), "embed_gather")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out (contiguous, float32 or bfloat16) = mean + std * x(key, first + i) for its elements i in storage order: the
    counter-based generator of weights/counter_random.py on the device, with the same bits."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_normal: a contiguous tensor")
    _check(lib().bg_fill_normal(_p(out), _dt(out), out.numel(), int(key) & ((1 << 64) - 1), int(first), float(mean), float(std),
                                _stream()), "fill_normal")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place; x contiguous float32 (logits)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0.0:
        raise KernelError("softcap: contiguous float32 values and a positive cap")
    _check(lib().bg_softcap(_p(x), x.numel(), float(cap), _stream()), "softcap")


def _parts(t: torch.Tensor, what: str):
    """(number of partial sums, elements between them) of a product's result: [T, N], or
    [parts, T, N] float32 from a split-K product."""
    if t.dim() == 2:
        return 1, 0
    if t.dim() == 3 and t.is_contiguous():
        return t.shape[0], t.shape[1] * t.shape[2]
    raise KernelError(f"{what} must be [T, N] or contiguous [parts, T, N]")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, update: bool = True) -> None:
    """v = x[s] (+ delta[s], or the sum over p of delta[p][s]); x[s] = v when update;
    out[r] = rmsnorm(v) * weight, s = rows[r] or r."""
    _cuda(x, delta, weight, out, rows)
    d = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or not weight.is_contiguous():
        raise KernelError("add_rmsnorm: x must be contiguous float32; out and weight contiguous")
    if tuple(out.shape) != (n, d) or weight.numel() != d:
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, expected {(n, d)}; weight has {weight.numel()} of {d}")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = _parts(delta, "add_rmsnorm: delta")
        if tuple(delta.shape[-2:]) != tuple(x.shape) or not delta.is_contiguous():
            raise KernelError("add_rmsnorm: delta must be contiguous and shaped like x")
    if rows is not None:
        _i32(rows, "rows")
    with phase("rmsnorm"):
        _check(lib().bg_add_rmsnorm(_p(x), _p(delta), _dt(delta) if delta is not None else F32, parts, stride, _p(weight),
                                    _dt(weight), float(eps), _p(out), _dt(out), _p(rows), n, d, 1 if update else 0,
                                    _stream()), "add_rmsnorm")


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _cuda(x, delta)
    if x.dtype != torch.float32 or x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous():
        raise KernelError("add_residual: x must be contiguous float32 and delta shaped like it")
    with phase("residuals"):
        _check(lib().bg_add_residual(_p(x), _p(delta), _dt(delta), x.numel(), _stream()), "add_residual")


GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0, activation: str = "silu") -> None:
    """out[t, i] = act(g[t, i]) * g[t, im + i], g = gate_up or the sum of its partial sums; act is silu or the tanh form
    of GELU.  With `block` > 0 the columns of g are interleaved in blocks of that many: gate, up, gate, up, ..."""
    if activation not in GLU_ACTIVATIONS:
        raise KernelError(f"swiglu: unknown activation '{activation}' ({', '.join(GLU_ACTIVATIONS)})")
    _cuda(gate_up, out)
    parts, stride = _parts(gate_up, "swiglu: gate_up")
    rows, two_im = gate_up.shape[-2:]
    im = two_im // 2
    if two_im != 2 * im or tuple(out.shape) != (rows, im):
        raise KernelError("swiglu: gate_up must be [rows, 2*im] and out [rows, im]")
    if not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("swiglu: tensors must be contiguous")
    if block < 0 or (block > 0 and im % block):
        raise KernelError(f"swiglu: blocks of {block} do not divide {im} features")
    with phase("swiglu"):
        _check(lib().bg_swiglu(_p(gate_up), _dt(gate_up), parts, stride, _p(out), _dt(out), rows, im, block,
                               GLU_ACTIVATIONS[activation], _stream()), "swiglu")


def activation(z: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out = act(z), z [rows, n] or its float partial sums [parts, rows, n]; act is silu or the tanh form of GELU."""
    if activation not in GLU_ACTIVATIONS:
        raise KernelError(f"activation: unknown activation '{activation}' ({', '.join(GLU_ACTIVATIONS)})")
    _cuda(z, out)
    parts, stride = _parts(z, "activation: z")
    if tuple(out.shape) != tuple(z.shape[-2:]) or not z.is_contiguous() or not out.is_contiguous():
        raise KernelError("activation: z and out contiguous and of one shape")
    with phase("swiglu"):
        _check(lib().bg_activation(_p(z), _dt(z), parts, stride, _p(out), _dt(out), out.numel(), GLU_ACTIVATIONS[activation],
                                   _stream()), "activation")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, amplitude: float = 1.0) -> None:
    """out[t, i] = amplitude * (cos, sin)(positions[t] * inv_freq[i]); out is float32 [T, half, 2]."""
    _cuda(positions, inv_freq, out)
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    if inv_freq.dtype != torch.float32 or out.dtype != torch.float32 or tuple(out.shape) != (T, half, 2) \
            or not out.is_contiguous() or not inv_freq.is_contiguous():
        raise KernelError("rope_table: inv_freq float32 [half], out contiguous float32 [T, half, 2]")
    with phase("rope"):
        _check(lib().bg_rope_table(_p(positions), _p(inv_freq), _p(out), T, half, float(amplitude), _stream()), "rope_table")


def rope_kv_append(src: torch.Tensor, q_out: torch.Tensor, n_rows: int, nh: int, nkv: int, hd: int, rot: int,
                   interleaved: bool, cos_sin: Optional[torch.Tensor], positions: torch.Tensor, row_req: torch.Tensor,
                   block_table: torch.Tensor, kv_pool: Optional[torch.Tensor], page_size: int,
                   status: Optional[torch.Tensor]) -> None:
    """Rows [q | k | v] of `src` ([T, W], or partial sums [parts, T, W]): rotate q into q_out [T, nh*hd],
    rotate k and store k and v into kv_pool [num_pages, 2, nkv, page_size, hd] through the block table
    [B, max_pages].  With kv_pool None the rows hold q only."""
    _cuda(src, q_out, cos_sin, positions, row_req, block_table, kv_pool)
    _i32(positions, "positions"); _i32(row_req, "row_req"); _i32(block_table, "block_table")
    parts, stride = _parts(src, "rope_kv_append: src")
    width = src.shape[-1]
    need = nh * hd + (2 * nkv * hd if kv_pool is not None else 0)
    if src.stride(-1) != 1 or width < need:
        raise KernelError(f"rope_kv_append: rows of {width} features cannot hold q, k, v ({need})")
    if q_out.data_ptr() == src.data_ptr() or q_out.stride(1) != 1 or q_out.shape[1] < nh * hd or q_out.shape[0] < n_rows:
        raise KernelError("rope_kv_append: q_out must be a separate [T, nh*hd] tensor")
    num_pages = 0
    if kv_pool is not None:
        if tuple(kv_pool.shape[1:]) != (2, nkv, page_size, hd) or not kv_pool.is_contiguous():
            raise KernelError(f"rope_kv_append: kv_pool is {tuple(kv_pool.shape)}, expected [pages, 2, {nkv}, {page_size}, {hd}]")
        num_pages = kv_pool.shape[0]
    if rot > 0 and (cos_sin is None or cos_sin.shape[0] < n_rows or cos_sin.shape[1] != rot // 2 or cos_sin.dtype != torch.float32):
        raise KernelError("rope_kv_append: cos_sin must be float32 [T, rot/2, 2]")
    with phase("rope+kv_write"):
        _check(lib().bg_rope_kv_append(_p(src), _dt(src), src.stride(-2), parts, stride, _p(q_out), _dt(q_out),
                                       q_out.stride(0), _p(cos_sin), _p(positions), _p(row_req), _p(block_table),
                                       block_table.shape[1], _p(kv_pool), _dt(kv_pool) if kv_pool is not None else F32,
                                       num_pages, page_size, n_rows, nh, nkv, hd, rot, 1 if interleaved else 0,
                                       _p(status), _stream()), "rope_kv_append")



# choices of `prefer` under which prompt portions run the tcgen05 kernel
def attention_wide_from(keys: int = 0) -> int:
    """The number of keys from which the tcgen05 prompt attention walks tiles of 128 keys instead of 64 (measured
    default 24,576; BEGLIN_B200_ATTN_WIDE_FROM overrides it).  A positive `keys` sets it; the old value is returned."""
    fn = lib().bg_attention_tc_wide_from
    fn.argtypes, fn.restype = [_c_int], _c_int
    return int(fn(int(keys)))


TC_ROWS_FOR = ("auto", "tcgen05")
TC_OPTIONS = ("softcap", "sink_weight")        # options of the softmax that the tcgen05 kernel knows besides the plain one
MMA_OPTIONS = ("softcap", "sink_weight")       # ... and the mma kernels (the sink's share is added where partial results merge)
SINK_KERNELS = ("generic", "tc_rows", "mma_keys", "mma_rows")   # every kernel can take the enlarged denominator (`sink`)


def attention_plan(group: int, hd: int, dtype: torch.dtype = torch.float32, decode_only: bool = False,
                   prefer: str = "auto", page_size: int = 64, vd: Optional[int] = None, softcap: bool = False,
                   learned_sink: bool = False) -> Tuple[str, int, int]:
    """(kernel, rows per query block, keys per tile) for these sizes.  Kernels: "mma_keys" (tensor
    cores, one token per block, for steps of single tokens), "mma_rows" (tensor cores, up to 64 rows
    per block) and "generic" (CUDA cores, every size up to head_dim 256, float or bfloat16)."""
    L = lib()
    if prefer not in ("auto", "generic", "mma", "tcgen05"):
        raise KernelError(f"unknown attention kernel choice '{prefer}'")
    vd = hd if vd is None else vd
    tc_knows = (not softcap or "softcap" in TC_OPTIONS) and (not learned_sink or "sink_weight" in TC_OPTIONS)
    if prefer == "tcgen05" and not tc_knows:
        raise KernelError("the tcgen05 attention kernel knows neither squashed scores nor a learned sink")
    if vd != hd:
        if prefer in ("mma", "tcgen05"):
            raise KernelError(f"the tensor-core attention kernels take values of the keys' size ({hd}), not {vd}")
        prefer = "generic"
    if dtype == torch.bfloat16 and not decode_only and prefer in TC_ROWS_FOR and tc_knows:
        bq = _c_int(0)
        if L.bg_attention_tc_plan(group, hd, page_size, ctypes.byref(bq)) == 0:
            return "tc_rows", bq.value, 64
        if prefer == "tcgen05":
            raise KernelError(f"the tcgen05 attention kernel does not take head_dim {hd} with {group} query heads "
                              f"per kv head and pages of {page_size} (head_dim 64 or 128; at most 128 heads per kv head; "
                              "a page size that divides 64)")
    if dtype == torch.bfloat16 and prefer != "generic":
        bq = _c_int(0)
        if L.bg_attention_mma_plan(group, hd, 1 if decode_only else 0, ctypes.byref(bq)) == 0:
            return ("mma_keys" if decode_only else "mma_rows"), bq.value, 64
        if prefer == "mma":
            raise KernelError(f"the tensor-core attention kernel does not take head_dim {hd} with {group} query "
                              "heads per kv head (head_dim 64 or 128; at most 64 heads per kv head)")
    bq, tile = _c_int(0), _c_int(0)
    rc = L.bg_attention_plan(group, hd, vd, ctypes.byref(bq), ctypes.byref(tile))
    if rc != 0:
        raise KernelError(f"attention: head_dim {hd} (values of {vd}) with {group} query heads per kv head is not "
                          "supported (both sizes must be at most 256)")
    return "generic", bq.value, tile.value


_sm_counts = {}


def sm_count(device=None) -> int:
    """The number of SMs of `device` (default: the current CUDA device), read from the device once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


def decode_splits(n_streams: int, context: int, sms: Optional[int] = None) -> int:
    """How many CTAs share the keys of one (request, kv head) stream in the decoding kernel.  A CTA has
    a shared-memory buffer per warp and is alone on its SM, so the streams are cut to make one wave
    of CTAs (one per SM; `sms` defaults to the current device's count): more CTAs wait for a second
    wave, fewer leave SMs idle while the others walk longer ranges.  No more than one CTA per 256 keys
    of `context` (a stage of 64 for each of the four warps).  Each request's keys are spread evenly
    over its CTAs by the kernel itself, by the request's own length, so the count depends on the
    shapes of the step only."""
    if sms is None:
        sms = sm_count()
    want = max(1, min(sms // max(1, n_streams), -(-context // 256)))
    per = -(-(-(-context // want)) // 256) * 256          # what the kernel makes of it: whole multiples of 256 keys
    return -(-context // per)                             # no CTA without keys


def attention(*args, **kwargs) -> None:
    """`_attention` under the phase timer of its kernel class (the partial kernel and its merge together)."""
    with phase("attn"):
        _attention(*args, **kwargs)


def _attention(q: torch.Tensor, q_stride: int, kv_pool: torch.Tensor, block_table: torch.Tensor,
              positions: torch.Tensor, qblk: torch.Tensor, n_qblk: int, max_position: int, n_rows: int, nh: int,
              nkv: int, hd: int, window: int, split: int, tile: int, bq: int, scale: float, out: torch.Tensor,
              status: Optional[torch.Tensor], kernel: str = "generic", vd: Optional[int] = None, sink: bool = False,
              sink_weight: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Paged grouped-query attention of a step's rows; out is [T, nh*hd].  `kernel`, `bq` and `tile`
    come from `attention_plan`; `qblk` must be cut for that `bq`; `max_position` is the largest
    position among the rows (or a bound on it).

    "generic" cuts the keys into splits of `split` positions (the same boundaries for every request),
    writes partial results and merges them; "mma_keys" (decoding) spreads every request's own keys over
    `decode_splits` CTAs and merges likewise; "mma_rows" and "tc_rows" let one CTA walk all keys of its
    query block and write `out` directly.

    `sink`: the softmax's denominator also holds exp(b) for a key that has no value, b = 0, or `sink_weight`[head]
    (float32 [nh]) when given.  `softcap` c > 0: a score s becomes c tanh(s / c)."""
    _cuda(q, kv_pool, block_table, positions, qblk, out, sink_weight)
    if sink_weight is not None:
        sink = True
        if sink_weight.dtype != torch.float32 or sink_weight.numel() != nh or not sink_weight.is_contiguous():
            raise KernelError("attention: the sink's scores are contiguous float32, one per query head")
    if softcap and kernel != "generic" and "softcap" not in (TC_OPTIONS if kernel == "tc_rows" else MMA_OPTIONS):
        raise KernelError(f"attention: the kernel '{kernel}' does not squash scores")
    learned = sink_weight is not None
    _i32(positions, "positions"); _i32(block_table, "block_table")
    if qblk is not None:
        _i32(qblk, "qblk")
    elif kernel != "mma_keys" or n_qblk != n_rows:
        raise KernelError("attention: only the decoding kernel runs without a list of query blocks (block i = row i)")
    if kernel == "tc_rows" and status is None:
        raise KernelError("attention: the tcgen05 kernel wants a status word (its waits are bounded)")
    vd = hd if vd is None else int(vd)
    if vd == hd:
        num_pages, two, nkv_, page_size, hd_ = kv_pool.shape
        if (two, nkv_, hd_) != (2, nkv, hd) or not kv_pool.is_contiguous():
            raise KernelError(f"attention: kv_pool is {tuple(kv_pool.shape)}, expected [pages, 2, {nkv}, page, {hd}]")
    else:
        # values of another size than keys: a page is flat, the keys of all kv heads followed by their values
        if kernel != "generic":
            raise KernelError("attention: values of another size than keys run the CUDA-core kernel")
        if kv_pool.dim() != 2 or kv_pool.shape[1] % (nkv * (hd + vd)) or not kv_pool.is_contiguous():
            raise KernelError(f"attention: kv_pool is {tuple(kv_pool.shape)}, expected [pages, {nkv} * page * ({hd} + {vd})]")
        num_pages, page_size = kv_pool.shape[0], kv_pool.shape[1] // (nkv * (hd + vd))
    if sink and kernel not in SINK_KERNELS:
        raise KernelError(f"attention: the kernel '{kernel}' has no softmax with an enlarged denominator")
    if out.stride(1) != 1 or out.shape[1] < nh * vd or out.shape[0] < n_rows:
        raise KernelError("attention: out must be [T, nh*vd] with unit inner stride")
    L = lib()
    if kernel == "tc_rows" and learned and "sink_weight" not in TC_OPTIONS:
        raise KernelError("attention: the tcgen05 kernel knows the sink of score 0 only")
    if kernel == "tc_rows":
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention: the tcgen05 kernel takes bfloat16 queries, caches and outputs")
        if learned or softcap:
            _check(L.bg_attention_tc_ext(
                _p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table), block_table.shape[1], _p(positions),
                _p(qblk), n_qblk, _p(out), out.stride(0), nh, nkv, hd, window, float(scale), int(max_position),
                1 if sink else 0, _p(sink_weight), float(softcap), _p(status), _stream()), "attention_tcgen05")
            return
        _check((L.bg_attention_tc_sink if sink else L.bg_attention_tc)(
            _p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table), block_table.shape[1], _p(positions), _p(qblk),
            n_qblk, _p(out), out.stride(0), nh, nkv, hd, window, float(scale), int(max_position), _p(status), _stream()),
            "attention_tcgen05")
        return
    if kernel == "mma_rows" and not sink:
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention: the tensor-core kernel takes bfloat16 queries, caches and outputs")
        _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                          block_table.shape[1], _p(positions), _p(qblk), n_qblk, None, None, 1, 1,
                                          nh, nkv, hd, window, split, 0, float(scale), float(softcap), _p(out), out.stride(0),
                                          _p(status), _stream()), "attention_mma")
        return
    if kernel == "mma_keys":
        split, n_splits = 0, decode_splits(n_qblk * nkv, max_position + 1)
        if n_splits == 1 and not sink:           # one CTA walks all keys of its (request, kv head) and writes the rows
            if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
                raise KernelError("attention: the tensor-core kernel takes bfloat16 queries, caches and outputs")
            _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                              block_table.shape[1], _p(positions), _p(qblk) if qblk is not None else None,
                                              n_qblk, None, None, 1, 1, nh, nkv, hd, window, 0, 1, float(scale), float(softcap), _p(out),
                                              out.stride(0), _p(status), _stream()), "attention_mma_keys")
            return
    else:
        n_splits = max_position // split + 1
    part_o = torch.empty((n_rows * nh * n_splits, vd), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n_rows * nh * n_splits, 2), dtype=torch.float32, device=q.device)
    if kernel == "generic":
        _check(L.bg_attention_partial(_p(q), _dt(q), q_stride, _p(kv_pool), _dt(kv_pool), num_pages, page_size,
                                      _p(block_table), block_table.shape[1], _p(positions), _p(qblk), n_qblk,
                                      _p(part_o), _p(part_ml), n_splits, n_splits, nh, nkv, hd, vd, window, split, tile,
                                      bq, float(scale), float(softcap), _p(status), _stream()), "attention_partial")
    elif kernel in ("mma_keys", "mma_rows"):
        # (the kernels that write finished rows know the plain softmax only: with the enlarged denominator their rows
        # go through partial results, also when there is one range of keys, and the merge adds the sink's share)
        if q.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16:
            raise KernelError("attention: the tensor-core kernel takes bfloat16 queries and caches")
        _check(L.bg_attention_mma_partial(_p(q), q_stride, _p(kv_pool), num_pages, page_size, _p(block_table),
                                          block_table.shape[1], _p(positions), _p(qblk) if qblk is not None else None,
                                          n_qblk, _p(part_o),
                                          _p(part_ml), n_splits, n_splits, nh, nkv, hd, window, split,
                                          1 if kernel == "mma_keys" else 0,
                                          float(scale), float(softcap), None, 0, _p(status), _stream()), "attention_mma_partial")
    else:
        raise KernelError(f"unknown attention kernel '{kernel}'")
    _check(L.bg_attention_merge(_p(part_o), _p(part_ml), _p(positions), _p(out), _dt(out), out.stride(0), n_rows, nh,
                                vd, n_splits, split, window, 1 if sink else 0, _p(sink_weight), _stream()), "attention_merge")


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                accumulate: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T (+ bias), all float32, CUDA cores only."""
    _cuda(a, w, bias, out)
    for t in (a, w, out) + ((bias,) if bias is not None else ()):
        if t.dtype != torch.float32:
            raise KernelError("gemm_f32_nt takes float32 tensors")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_f32_nt: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
    if bias is not None and (bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_f32_nt: bias must have one value per output feature")
    _check(lib().bg_gemm_f32_nt(_p(a), a.stride(0), _p(w), w.stride(0), _p(bias), _p(out), out.stride(0), M, N, K,
                                1 if accumulate else 0, _stream()), "gemm_f32_nt")


def gemm_bf16_tn(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 splits: int = 1, status: Optional[torch.Tensor] = None) -> None:
    """out = x[T, K] @ w[N, K]^T (+ bias) on the tcgen05 tensor cores, bfloat16 in, float accumulation.
    `out` is [T, N] (float32 or bfloat16) for splits == 1, or float32 [splits, T, N] partial sums over
    ranges of K, which the consumer adds up in index order (the bias is in partial 0)."""
    _cuda(x, w, bias, out, status)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16_tn takes bfloat16 operands")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_bf16_tn: shapes x{tuple(x.shape)} w{tuple(w.shape)} do not fit")
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError("gemm_bf16_tn: the inner size and the row strides must be multiples of 8 (TMA wants "
                          "16-byte row strides)")
    want = (T, N) if splits == 1 else (splits, T, N)
    if tuple(out.shape) != want or not out.is_contiguous():
        raise KernelError(f"gemm_bf16_tn: out is {tuple(out.shape)}, expected contiguous {want}")
    if splits > 1 and out.dtype != torch.float32:
        raise KernelError("gemm_bf16_tn: partial sums are float32")
    if splits > (K + 63) // 64:
        raise KernelError("gemm_bf16_tn: more splits than 64-wide blocks of K")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_bf16_tn: bias must be float32 with one value per output feature")
    _check(lib().bg_gemm_bf16_tn(_p(w), N, K, w.stride(0), _p(x), T, x.stride(0), _p(bias), _p(out), _dt(out), N,
                                 splits, _p(status), _stream()), "gemm_bf16_tn")


def gemm_bf16_tn_unchecked(x: torch.Tensor, w_ptr: int, n_out: int, k: int, ldw: int, bias_ptr, out: torch.Tensor,
                           splits: int, status_ptr) -> None:
    """gemm_bf16_tn for a caller that has checked the weight once (Linear): x must be contiguous
    bfloat16 [T, k] and out contiguous [T, n_out] or float32 [splits, T, n_out]."""
    _check(_lib.bg_gemm_bf16_tn(w_ptr, n_out, k, ldw, x.data_ptr(), x.shape[0], x.stride(0), bias_ptr, out.data_ptr(),
                                F32 if out.dtype == torch.float32 else BF16, n_out, splits, status_ptr, _stream()),
           "gemm_bf16_tn")


PAIR_PLAIN, PAIR_SWIGLU, PAIR_RESIDUAL, PAIR_GEGLU = 0, 1, 2, 3       # PAIR_GEGLU: as PAIR_SWIGLU with the tanh form of GELU
PAIR_GLU = {"silu": PAIR_SWIGLU, "gelu_tanh": PAIR_GEGLU}


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = PAIR_PLAIN,
              bias: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """The product of many rows (prompt portions) with w[N, K]^T by pairs of CTAs on the tcgen05 tensor cores.
    mode PAIR_PLAIN: out bfloat16 [T, N] = product (+ bias).  mode PAIR_SWIGLU: w's rows are interleaved (64 of
    gate, then their 64 of up); out bfloat16 [T, N / 2] = silu(gate) * up.  mode PAIR_RESIDUAL: out is the float32
    residual stream [T, N]: out += product (+ bias)."""
    _cuda(x, w, out, bias, status)
    N, K = w.shape
    T = x.shape[0]
    cols = N // 2 if mode in (PAIR_SWIGLU, PAIR_GEGLU) else N
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or \
            out.dtype != (torch.float32 if mode == PAIR_RESIDUAL else torch.bfloat16):
        raise KernelError("gemm_pair takes bfloat16 operands and gives a bfloat16 result (adds to a float32 stream)")
    if x.shape[1] != K or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or tuple(out.shape) != (T, cols):
        raise KernelError(f"gemm_pair: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    if status is None:
        raise KernelError("gemm_pair wants a status word (its waits are bounded)")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_pair: bias must be float32 with one value per output feature")
    _check(lib().bg_gemm_pair(_p(w), N, K, w.stride(0), _p(x), T, x.stride(0), _p(bias), _p(out), out.stride(0), mode,
                              _p(status), _stream()), "gemm_pair")


def gemm_pair_unchecked(x: torch.Tensor, w_ptr: int, n_out: int, k: int, ldw: int, out: torch.Tensor, mode: int,
                        status_ptr, bias_ptr=None) -> None:
    """gemm_pair for a caller that has checked the weight once (Linear): x bfloat16 [T, k] with contiguous rows,
    out bfloat16 [T, n_out], with PAIR_SWIGLU [T, n_out / 2], with PAIR_RESIDUAL the float32 stream [T, n_out]."""
    if status_ptr is None:
        raise KernelError("gemm_pair wants a status word (its waits are bounded)")
    _check(_lib.bg_gemm_pair(w_ptr, n_out, k, ldw, x.data_ptr(), x.shape[0], x.stride(0), bias_ptr, out.data_ptr(),
                             out.stride(0), mode, status_ptr, _stream()), "gemm_pair")


FUSED_PLAIN, FUSED_RESIDUAL, FUSED_SWIGLU = 0, 1, 2


def gemm_fused(w: torch.Tensor, out: torch.Tensor, mode: int = FUSED_PLAIN, *, x: Optional[torch.Tensor] = None,
               xf: Optional[torch.Tensor] = None, ssq_in: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None,
               ssq_out: Optional[torch.Tensor] = None, splits: int = 1, status: Optional[torch.Tensor] = None) -> None:
    """The product of up to 64 rows with w[N, K]^T on the tcgen05 tensor cores, with its neighbours fused in.

    Left operand: `x` (bfloat16 [T, K]), or the float32 residual stream `xf` [T, K] normalised on the fly:
    bf16(xf * rstd * norm_weight), rstd = 1 / sqrt(sum_p ssq_in[p] / K + eps), ssq_in float32 [parts, >= T].
    K is cut into `splits` (1, 2, 4, 8 or 16) ranges whose CTAs add up inside a thread block cluster.
    mode FUSED_PLAIN: out[T, N] = product (+ bias), float32 or bfloat16.
    mode FUSED_RESIDUAL: out (float32 [T, N], the residual stream) += product (+ bias); ssq_out
      [ceil(N / 128) * splits, >= T] receives partial sums of squares of the new rows.
    mode FUSED_SWIGLU: w's rows are interleaved (64 of gate, then their 64 of up); out bfloat16 [T, N / 2] =
      silu(gate) * up."""
    _cuda(w, out, x, xf, ssq_in, norm_weight, bias, ssq_out, status)
    N, K = w.shape
    if w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelError("gemm_fused takes a bfloat16 weight with contiguous rows")
    if (x is None) == (xf is None):
        raise KernelError("gemm_fused takes either x (bfloat16) or xf (float32 with ssq_in and norm_weight)")
    src = x if x is not None else xf
    T = src.shape[0]
    if src.shape[1] != K or src.stride(1) != 1 or T > 64:
        raise KernelError(f"gemm_fused: the left operand is {tuple(src.shape)}, expected up to 64 rows of {K}")
    if x is not None and x.dtype != torch.bfloat16:
        raise KernelError("gemm_fused: x must be bfloat16")
    if xf is not None:
        if xf.dtype != torch.float32 or ssq_in is None or norm_weight is None:
            raise KernelError("gemm_fused: xf must be float32 and come with ssq_in and norm_weight")
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[1] < T or ssq_in.stride(1) != 1:
            raise KernelError("gemm_fused: ssq_in must be float32 [parts, >= T]")
        if norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_fused: norm_weight must be bfloat16 with one value per input feature")
    n_cols = N // 2 if mode == FUSED_SWIGLU else N
    if out.shape[0] != T or out.shape[1] != n_cols or out.stride(1) != 1:
        raise KernelError(f"gemm_fused: out is {tuple(out.shape)}, expected {(T, n_cols)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_fused: bias must be float32 with one value per output feature")
    if mode == FUSED_RESIDUAL and ssq_out is not None:
        parts = -(-N // 128) * splits
        if ssq_out.dtype != torch.float32 or ssq_out.dim() != 2 or ssq_out.shape[0] < parts or ssq_out.shape[1] < T \
                or ssq_out.stride(1) != 1:
            raise KernelError(f"gemm_fused: ssq_out must be float32 [>= {parts}, >= {T}]")
    _check(lib().bg_gemm_fused(_p(w), N, K, w.stride(0), _p(x), x.stride(0) if x is not None else 0, _p(xf),
                               xf.stride(0) if xf is not None else 0, _p(ssq_in),
                               ssq_in.shape[0] if ssq_in is not None else 0, ssq_in.stride(0) if ssq_in is not None else 0,
                               _p(norm_weight), float(eps), T, _p(bias), mode, _p(out), _dt(out), out.stride(0),
                               _p(ssq_out), ssq_out.stride(0) if ssq_out is not None else 0, splits, _p(status),
                               _stream()), "gemm_fused")


def gemm_fused_unchecked(w_ptr: int, n_out: int, k: int, ldw: int, T: int, out: torch.Tensor, mode: int, x, xf, ssq_in,
                         norm_w_ptr, eps: float, bias_ptr, ssq_out, splits: int, status_ptr) -> None:
    """gemm_fused for a caller that has checked the shapes once (Linear)."""
    _check(_lib.bg_gemm_fused(w_ptr, n_out, k, ldw, None if x is None else x.data_ptr(), 0 if x is None else x.stride(0),
                              None if xf is None else xf.data_ptr(), 0 if xf is None else xf.stride(0),
                              None if ssq_in is None else ssq_in.data_ptr(), 0 if ssq_in is None else ssq_in.shape[0],
                              0 if ssq_in is None else ssq_in.stride(0), norm_w_ptr, eps, T, bias_ptr, mode, out.data_ptr(),
                              F32 if out.dtype == torch.float32 else BF16, out.stride(0),
                              None if ssq_out is None else ssq_out.data_ptr(), 0 if ssq_out is None else ssq_out.stride(0),
                              splits, status_ptr, _stream()), "gemm_fused")


def gemm_fused_rope(w: torch.Tensor, x: Optional[torch.Tensor], bias: Optional[torch.Tensor], q_out: torch.Tensor,
                    cos_sin: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
                    kv_pool: torch.Tensor, nh: int, nkv: int, hd: int, splits: int = 1,
                    status: Optional[torch.Tensor] = None, *, xf: Optional[torch.Tensor] = None,
                    ssq_in: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                    eps: float = 0.0) -> None:
    """x [T, K] (bfloat16, up to 64 rows; or the float32 stream xf with ssq_in, norm_weight and eps, as gemm_fused)
    times w [(nh + 2 nkv) hd, K]^T (+ bias), rows [q | k | v]: queries and keys rotated by cos_sin [T, hd / 2, 2]
    (feature d with d + hd / 2), queries to q_out [T, nh hd], keys and values into kv_pool
    [pages, 2, nkv, page_size, hd] at positions[t] of request row_req[t].  hd is 32, 64 or 128."""
    _cuda(w, x, xf, ssq_in, norm_weight, bias, q_out, cos_sin, positions, row_req, block_table, kv_pool, status)
    N, K = w.shape
    if (x is None) == (xf is None):
        raise KernelError("gemm_fused_rope takes either x (bfloat16) or xf (float32 with ssq_in and norm_weight)")
    src = x if x is not None else xf
    T = src.shape[0]
    if w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16:
        raise KernelError("gemm_fused_rope takes bfloat16 weights, queries and cache")
    if x is not None and x.dtype != torch.bfloat16:
        raise KernelError("gemm_fused_rope: x must be bfloat16")
    if xf is not None:
        if xf.dtype != torch.float32 or ssq_in is None or norm_weight is None:
            raise KernelError("gemm_fused_rope: xf must be float32 and come with ssq_in and norm_weight")
        if ssq_in.dtype != torch.float32 or ssq_in.dim() != 2 or ssq_in.shape[1] < T or ssq_in.stride(1) != 1:
            raise KernelError("gemm_fused_rope: ssq_in must be float32 [parts, >= T]")
        if norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_fused_rope: norm_weight must be bfloat16 with one value per input feature")
    if N != (nh + 2 * nkv) * hd or src.shape[1] != K or w.stride(1) != 1 or src.stride(1) != 1 or T > 64:
        raise KernelError(f"gemm_fused_rope: w {tuple(w.shape)}, rows {tuple(src.shape)} for {nh}/{nkv} heads of {hd}")
    if q_out.shape[0] < T or q_out.shape[1] < nh * hd or q_out.stride(1) != 1:
        raise KernelError(f"gemm_fused_rope: q_out is {tuple(q_out.shape)}")
    if kv_pool.dim() != 5 or tuple(kv_pool.shape[1:3]) != (2, nkv) or kv_pool.shape[4] != hd or not kv_pool.is_contiguous():
        raise KernelError(f"gemm_fused_rope: the pool is {tuple(kv_pool.shape)}")
    if cos_sin.dtype != torch.float32 or tuple(cos_sin.shape) != (T, hd // 2, 2) or not cos_sin.is_contiguous():
        raise KernelError(f"gemm_fused_rope: cos_sin is {tuple(cos_sin.shape)}, expected {(T, hd // 2, 2)} float32")
    for t in (positions, row_req, block_table):
        _i32(t, "positions, row_req and block_table")
    if positions.numel() != T or row_req.numel() != T or block_table.dim() != 2 or not block_table.is_contiguous():
        raise KernelError("gemm_fused_rope: positions and row_req have one value per row, block_table is [requests, pages]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise KernelError("gemm_fused_rope: bias must be float32 with one value per output feature")
    gemm_fused_rope_unchecked(w.data_ptr(), K, w.stride(0), T, q_out, x, xf, ssq_in,
                              None if norm_weight is None else norm_weight.data_ptr(), float(eps),
                              None if bias is None else bias.data_ptr(), cos_sin, positions, row_req, block_table, kv_pool,
                              kv_pool.shape[3], nh, nkv, hd, splits, None if status is None else status.data_ptr())


def gemm_fused_rope_unchecked(w_ptr: int, k: int, ldw: int, T: int, q_out: torch.Tensor, x, xf, ssq_in, norm_w_ptr,
                              eps: float, bias_ptr, cos_sin: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                              block_table: torch.Tensor, kv_pool: torch.Tensor, page_size: int, nh: int, nkv: int, hd: int,
                              splits: int, status_ptr) -> None:
    """The q/k/v product of up to 64 rows with rotation and cache append behind it (left operand as gemm_fused):
    q_out bfloat16 [T, nh hd] receives the rotated queries, kv_pool [pages, 2, nkv, page_size, hd] (bfloat16) the
    rotated keys and the values at each row's position.  For a caller that has checked the shapes (Attention);
    head sizes other than 32, 64 and 128 raise."""
    _check(_lib.bg_gemm_fused_rope(w_ptr, k, ldw, None if x is None else x.data_ptr(), 0 if x is None else x.stride(0),
                                   None if xf is None else xf.data_ptr(), 0 if xf is None else xf.stride(0),
                                   None if ssq_in is None else ssq_in.data_ptr(), 0 if ssq_in is None else ssq_in.shape[0],
                                   0 if ssq_in is None else ssq_in.stride(0), norm_w_ptr, eps, T, bias_ptr,
                                   q_out.data_ptr(), q_out.stride(0), cos_sin.data_ptr(), positions.data_ptr(),
                                   row_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], kv_pool.data_ptr(),
                                   kv_pool.shape[0], page_size, nh, nkv, hd, splits, status_ptr, _stream()),
           "gemm_fused_rope")


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
           out: torch.Tensor, feed_tokens: Optional[torch.Tensor] = None, feed_positions: Optional[torch.Tensor] = None,
           advance: Optional[torch.Tensor] = None) -> None:
    """out[r] = first argmax of logits[r] when temperature[r] <= 0 (or temperature is None), else the
    index where the cumulative softmax(logits[r] / temperature[r]) first exceeds uniform[r].  For a decoding
    step that is replayed on the device: the token also goes to feed_tokens[r] (the step's input buffer), and
    feed_positions[r] grows by advance[r] (by 1 without `advance`)."""
    _cuda(logits, temperature, uniform, out, feed_tokens, feed_positions, advance)
    for t in (feed_tokens, feed_positions, advance):
        if t is not None:
            _i32(t, "feed_tokens, feed_positions and advance")
            if t.numel() != logits.shape[0]:
                raise KernelError("sample: feed_tokens, feed_positions and advance have one value per row")
    n, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("sample: logits must be contiguous float32 [n, V]")
    _i32(out, "out")
    for t in (temperature, uniform):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError("sample: temperature and uniform must be float32 [n]")
    scratch = torch.empty(n * 64 * 3, dtype=torch.float32, device=logits.device)
    with phase("sample"):
        _check(lib().bg_sample_feed(_p(logits), n, V, _p(temperature), _p(uniform), _p(out), _p(scratch), _p(feed_tokens),
                                    _p(feed_positions), _p(advance), _stream()), "sample")
    global _launches
    _launches += 1            # two kernels


# ------------------------------------------------------------------------------------------------
# Layer norm, depth-weighted average, xIELU, norms of slices, output gates
def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None, update: bool = True) -> None:
    """As add_rmsnorm, with a layer norm (mean taken off, no bias): v = x[s] (+ delta[s], or the sum of its
    partial sums); x[s] = v when update; out[r] = (v - mean) / sqrt(var + eps) * weight, s = rows[r] or r."""
    _cuda(x, delta, weight, out, rows)
    d = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or not weight.is_contiguous():
        raise KernelError("add_layernorm: x must be contiguous float32; out and weight contiguous")
    if tuple(out.shape) != (n, d) or weight.numel() != d:
        raise KernelError(f"add_layernorm: out is {tuple(out.shape)}, expected {(n, d)}; weight has {weight.numel()} of {d}")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = _parts(delta, "add_layernorm: delta")
        if tuple(delta.shape[-2:]) != tuple(x.shape) or not delta.is_contiguous():
            raise KernelError("add_layernorm: delta must be contiguous and shaped like x")
    if rows is not None:
        _i32(rows, "rows")
    with phase("layernorm"):
        _check(lib().bg_add_layernorm(_p(x), _p(delta), _dt(delta) if delta is not None else F32, parts, stride, _p(weight),
                                      _dt(weight), float(eps), _p(out), _dt(out), _p(rows), n, d, 1 if update else 0,
                                      _stream()), "add_layernorm")


def depth_mix(x: torch.Tensor, delta: Optional[torch.Tensor], history: torch.Tensor, weight: torch.Tensor, terms: int) -> None:
    """v = x (+ delta or the sum of its partial sums); history[terms - 1] = v; x = sum_{j < terms} weight[j] history[j],
    added in the order of j.  x float32 [T, d]; history float32 [slots >= terms, T, d]."""
    _cuda(x, delta, history, weight)
    if x.dtype != torch.float32 or history.dtype != torch.float32 or not x.is_contiguous() or not history.is_contiguous():
        raise KernelError("depth_mix: x and history must be contiguous float32")
    if history.dim() != 3 or tuple(history.shape[1:]) != tuple(x.shape) or not 1 <= terms <= history.shape[0]:
        raise KernelError(f"depth_mix: history is {tuple(history.shape)} for {terms} terms of {tuple(x.shape)}")
    if weight.numel() != terms or not weight.is_contiguous():
        raise KernelError(f"depth_mix: {weight.numel()} weights for {terms} terms")
    parts, stride = 0, 0
    if delta is not None:
        parts, stride = _parts(delta, "depth_mix: delta")
        if tuple(delta.shape[-2:]) != tuple(x.shape) or not delta.is_contiguous():
            raise KernelError("depth_mix: delta must be contiguous and shaped like x")
    with phase("residuals"):
        _check(lib().bg_depth_mix(_p(x), _p(delta), _dt(delta) if delta is not None else F32, parts, stride, _p(history),
                                  x.numel(), _p(weight), _dt(weight), terms, x.numel(), _stream()), "depth_mix")


def xielu(z: torch.Tensor, act: torch.Tensor, out: torch.Tensor) -> None:
    """out = xIELU(z): with a_pos = softplus(act[0]) and a_neg = 1/2 + softplus(act[1]), z (a_pos z + 1/2) above zero
    and a_neg (expm1(z) - z) + z/2 elsewhere.  z is [T, n] or float partial sums [parts, T, n]."""
    _cuda(z, act, out)
    parts, stride = _parts(z, "xielu: z")
    if tuple(out.shape) != tuple(z.shape[-2:]) or not z.is_contiguous() or not out.is_contiguous() or act.numel() != 2:
        raise KernelError("xielu: z [T, n] (or its partial sums), out [T, n], act with two numbers, all contiguous")
    with phase("activation"):
        _check(lib().bg_xielu(_p(z), _dt(z), parts, stride, _p(act), _dt(act), _p(out), _dt(out), out.numel(), _stream()), "xielu")


def rmsnorm_slice(src: torch.Tensor, col0: int, n: int, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[r] = RMS norm of src[r, col0 : col0 + n] times weight."""
    _cuda(src, weight, out)
    if src.dim() != 2 or src.stride(1) != 1 or col0 < 0 or col0 + n > src.shape[1]:
        raise KernelError(f"rmsnorm_slice: columns {col0}..{col0 + n} of rows of {tuple(src.shape)}")
    if tuple(out.shape) != (src.shape[0], n) or out.stride(1) != 1 or weight.numel() != n or not weight.is_contiguous():
        raise KernelError("rmsnorm_slice: out is [rows, n] and weight has n values")
    with phase("rmsnorm"):
        _check(lib().bg_rmsnorm_slice(_p(src), _dt(src), src.stride(0), col0, n, _p(weight), _dt(weight), float(eps), _p(out),
                                      _dt(out), out.stride(0), src.shape[0], _stream()), "rmsnorm_slice")


def gate_heads(src: torch.Tensor, gate: Optional[torch.Tensor], gate_col0: int, out: torch.Tensor) -> None:
    """out[t, h * vd + j] = src[h, t, j] * sigmoid(gate[t, gate_col0 + h]); src is [H, T, vd].  Without `gate` the heads
    are put row by row as they are."""
    _cuda(src, gate, out)
    H, T, vd = src.shape
    if src.stride(2) != 1 or (gate is not None and (gate.stride(1) != 1 or gate_col0 + H > gate.shape[1] or gate.shape[0] < T)):
        raise KernelError("gate_heads: src [H, T, vd] with unit inner stride, gate rows that hold H values from gate_col0")
    if tuple(out.shape) != (T, H * vd) or not out.is_contiguous():
        raise KernelError(f"gate_heads: out is {tuple(out.shape)}, expected {(T, H * vd)}")
    with phase("activation"):
        _check(lib().bg_gate_heads(_p(src), _dt(src), src.stride(0), src.stride(1), _p(gate), _dt(gate) if gate is not None else F32,
                                   gate.stride(0) if gate is not None else 0, gate_col0, _p(out), _dt(out), T, H, vd, _stream()),
               "gate_heads")


def gemm_f32_nt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] @ w[b]^T for a [B, M, K], w [B, N, K], out [B, M, N], float32 views of any batch and row
    strides with unit inner stride.  CUDA cores only."""
    _cuda(a, w, out)
    for t in (a, w, out):
        if t.dtype != torch.float32 or t.dim() != 3 or t.stride(2) != 1:
            raise KernelError("gemm_f32_nt_batched takes float32 [B, rows, cols] views with unit inner stride")
    B, M, K = a.shape
    N = w.shape[1]
    if w.shape[0] != B or w.shape[2] != K or tuple(out.shape) != (B, M, N):
        raise KernelError(f"gemm_f32_nt_batched: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
    _check(lib().bg_gemm_f32_nt_batched(_p(a), a.stride(1), a.stride(0), _p(w), w.stride(1), w.stride(0), _p(out),
                                        out.stride(1), out.stride(0), B, M, N, K, _stream()), "gemm_f32_nt_batched")


# ------------------------------------------------------------------------------------------------
# Attention through a latent
def latent_attention_plan(rank: int, rot: int) -> Tuple[int, int]:
    """(rows per CTA, keys per tile) of the latent attention kernel for a cache row of rank + rot features."""
    rows, tile = _c_int(0), _c_int(0)
    if lib().bg_latent_attention_plan(rank, rot, ctypes.byref(rows), ctypes.byref(tile)) != 0:
        raise KernelError(f"latent attention: a cache row of {rank} + {rot} features does not fit a CTA's shared memory")
    return rows.value, tile.value


def latent_attention_mma_plan(rank: int, rot: int) -> Optional[Tuple[int, int]]:
    """(rows per CTA, stages) of the tensor-core latent attention kernel, or None when it does not take a cache row of
    rank + rot features (a multiple of 32, rank a multiple of 8 up to 512)."""
    rows, stages = _c_int(0), _c_int(0)
    if lib().bg_latent_attention_mma_plan(rank, rot, ctypes.byref(rows), ctypes.byref(stages)) != 0:
        return None
    return rows.value, stages.value


def latent_append(src: torch.Tensor, col0: int, rank: int, rot: int, rot_dims: int, weight: torch.Tensor, eps: float,
                  cos_sin: Optional[torch.Tensor], positions: torch.Tensor, row_req: torch.Tensor,
                  block_table: torch.Tensor, pool: torch.Tensor, status: Optional[torch.Tensor],
                  q_norm: Optional[tuple] = None) -> None:
    """For every row t of src: pool[page, slot] = [rmsnorm(src[t, col0 : col0+rank]) * weight |
    rotate(src[t, col0+rank : col0+rank+rot])] at positions[t] of request row_req[t]; pool is
    [pages, page_size, rank + rot].  The first rot_dims features of the key part turn in pairs (2i, 2i+1) by
    cos_sin [T, rot_dims/2, 2].  With q_norm = (q_col0, q_weight, q_out) the same launch also writes
    q_out[t] = rmsnorm(src[t, q_col0 : q_col0 + q_rank]) * q_weight, q_out [T, q_rank], the weights of one type."""
    _cuda(src, weight, cos_sin, positions, row_req, block_table, pool, status)
    _i32(positions, "positions"); _i32(row_req, "row_req"); _i32(block_table, "block_table")
    T = positions.numel()
    if src.dim() != 2 or src.stride(1) != 1 or src.shape[0] < T or col0 + rank + rot > src.shape[1]:
        raise KernelError(f"latent_append: rows of {tuple(src.shape)} cannot hold {rank} + {rot} features from {col0}")
    if pool.dim() != 3 or pool.shape[2] != rank + rot or not pool.is_contiguous():
        raise KernelError(f"latent_append: the pool is {tuple(pool.shape)}, expected [pages, page, {rank + rot}]")
    if weight.numel() != rank or not weight.is_contiguous():
        raise KernelError("latent_append: one norm weight per latent feature")
    if rot_dims > 0 and (cos_sin is None or cos_sin.dtype != torch.float32 or cos_sin.shape[0] < T
                         or cos_sin.shape[1] != rot_dims // 2 or not cos_sin.is_contiguous()):
        raise KernelError("latent_append: cos_sin must be float32 [T, rot_dims/2, 2]")
    q_col0, q_rank, q_w, q_out = 0, 0, None, None
    if q_norm is not None:
        q_col0, q_w, q_out = q_norm
        _cuda(q_w, q_out)
        q_rank = q_w.numel()
        if q_w.dtype != weight.dtype or not q_w.is_contiguous() or tuple(q_out.shape) != (T, q_rank) or not q_out.is_contiguous() \
                or q_col0 < 0 or q_col0 + q_rank > src.shape[1]:
            raise KernelError("latent_append: the query latent's norm wants q_out [T, q_rank] and a weight of the other's type")
    with phase("rope+kv_write"):
        _check(lib().bg_latent_append(_p(src), _dt(src), src.stride(0), col0, rank, rot, rot_dims, _p(weight), _dt(weight),
                                      float(eps), _p(cos_sin), _p(positions), _p(row_req), _p(block_table),
                                      block_table.shape[1], _p(pool), _dt(pool), pool.shape[0], pool.shape[1], T, _p(status),
                                      q_col0, q_rank, _p(q_w), _p(q_out), _dt(q_out) if q_out is not None else F32, _stream()),
               "latent_append")


def latent_attention(q_lat: torch.Tensor, q_raw: torch.Tensor, dim: int, rot: int, rot_dims: int,
                     cos_sin: Optional[torch.Tensor], pool: torch.Tensor, block_table: torch.Tensor,
                     positions: torch.Tensor, qblk: torch.Tensor, n_qblk: int, max_position: int, bq: int, hc: int,
                     tile: int, split: int, scale: float, out: torch.Tensor, status: Optional[torch.Tensor],
                     mma_stages: int = 0, window: int = 0) -> None:
    """Causal attention of a step's rows over the latent cache.  q_lat float32 [H, T, rank]: the queries carried into
    the latent space; q_raw [T, H * (dim + rot)]: the query product's rows, whose rot part is rotated here; pool
    [pages, page_size, rank + rot]; out [H, T, rank] receives, per head, the softmax-weighted sum of the cached
    latents.  `qblk` is cut for `bq` rows; a CTA takes `hc` heads; keys are cut into splits of `split` positions.
    With `mma_stages` 1 or 2 the products run on the tensor cores (bfloat16 q_raw and pool, bq * hc at most 64, sizes as
    `latent_attention_mma_plan` says); else on the CUDA cores in float, for every size and type.  `window` w > 0: a row
    sees itself and the w - 1 positions before it."""
    _cuda(q_lat, q_raw, cos_sin, pool, block_table, positions, qblk, out, status)
    _i32(positions, "positions"); _i32(block_table, "block_table"); _i32(qblk, "qblk")
    H, T, rank = q_lat.shape
    if q_lat.dtype != torch.float32 or q_lat.stride(2) != 1 or tuple(out.shape) != (H, T, rank) or out.stride(2) != 1:
        raise KernelError("latent_attention: q_lat float32 [H, T, rank] and out [H, T, rank] with unit inner stride")
    if q_raw.dim() != 2 or q_raw.stride(1) != 1 or q_raw.shape[1] != H * (dim + rot) or q_raw.shape[0] < T:
        raise KernelError(f"latent_attention: q_raw is {tuple(q_raw.shape)} for {H} heads of {dim} + {rot}")
    if pool.dim() != 3 or pool.shape[2] != rank + rot or not pool.is_contiguous():
        raise KernelError(f"latent_attention: the pool is {tuple(pool.shape)}, expected [pages, page, {rank + rot}]")
    if rot_dims > 0 and (cos_sin is None or cos_sin.dtype != torch.float32 or cos_sin.shape[0] < T
                         or cos_sin.shape[1] != rot_dims // 2 or not cos_sin.is_contiguous()):
        raise KernelError("latent_attention: cos_sin must be float32 [T, rot_dims/2, 2]")
    n_splits = max_position // split + 1
    part_o = torch.empty((T * H * n_splits, rank), dtype=torch.float32, device=q_lat.device)
    part_ml = torch.empty((T * H * n_splits, 2), dtype=torch.float32, device=q_lat.device)
    L = lib()
    with phase("attn"):
        if mma_stages:
            if q_raw.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
                raise KernelError("latent_attention: the tensor-core kernel takes bfloat16 query rows and caches")
            _check(L.bg_latent_attention_mma_partial(_p(q_lat), q_lat.stride(0), q_lat.stride(1), _p(q_raw), q_raw.stride(0),
                                                     dim + rot, dim, _p(cos_sin), _p(pool), pool.shape[0], pool.shape[1],
                                                     _p(block_table), block_table.shape[1], _p(positions), _p(qblk), n_qblk,
                                                     _p(part_o), _p(part_ml), n_splits, n_splits, H, hc, rank, rot, rot_dims,
                                                     split, bq, mma_stages, int(window), float(scale), _p(status), _stream()),
                   "latent_attention_mma_partial")
        else:
            _check(L.bg_latent_attention_partial(_p(q_lat), _dt(q_lat), q_lat.stride(0), q_lat.stride(1), _p(q_raw), _dt(q_raw),
                                                 q_raw.stride(0), dim + rot, dim, _p(cos_sin), _p(pool), _dt(pool), pool.shape[0],
                                                 pool.shape[1], _p(block_table), block_table.shape[1], _p(positions), _p(qblk),
                                                 n_qblk, _p(part_o), _p(part_ml), n_splits, n_splits, H, hc, rank, rot, rot_dims,
                                                 split, tile, bq, int(window), float(scale), _p(status), _stream()), "latent_attention_partial")
        _check(L.bg_latent_attention_merge(_p(part_o), _p(part_ml), _p(positions), _p(out), _dt(out), out.stride(0),
                                           out.stride(1), T, H, rank, n_splits, split, int(window), _stream()), "latent_attention_merge")


def latent_gather(pool: torch.Tensor, block_table: torch.Tensor, req: int, rank: int, lat: torch.Tensor, kr: torch.Tensor,
                  first: int = 0) -> None:
    """lat[s] and kr[s] = the latent and the rotated key part of the cached row of position first + s, s < S, of the step's
    request `req` (zeros where it holds no page); pool [pages, page_size, rank + rot], lat [S, rank], kr [S, rot], bfloat16."""
    _cuda(pool, block_table, lat, kr)
    _i32(block_table, "block_table")
    S, rot = lat.shape[0], pool.shape[2] - rank
    if pool.dtype != torch.bfloat16 or lat.dtype != torch.bfloat16 or kr.dtype != torch.bfloat16 or pool.dim() != 3 \
            or not pool.is_contiguous() or tuple(lat.shape) != (S, rank) or tuple(kr.shape) != (S, rot) \
            or not lat.is_contiguous() or (rot and not kr.is_contiguous()) or not 0 <= req < block_table.shape[0] or first < 0:
        raise KernelError("latent_gather: a bfloat16 pool [pages, page, rank + rot], lat [S, rank] and kr [S, rot]")
    with phase("kv_expand"):
        _check(lib().bg_latent_gather(_p(pool), _p(block_table), block_table.shape[1], req, pool.shape[0], pool.shape[1],
                                      rank, rot, S, int(first), _p(lat), _p(kr), _stream()), "latent_gather")


def latent_expand(kv: torch.Tensor, kr: torch.Tensor, H: int, dim: int, pages: torch.Tensor) -> None:
    """Per-head keys and values of S positions laid out as pages of 64 positions for the grouped-query kernels:
    kv [S, H dim + H (dim + rot)] = [plain key parts | values], kr [S, rot] the rotated key part; pages
    [ceil(S / 64), 2, H, 64, dim + rot] receives keys [plain | rotated part] and values.  dim and rot are multiples of 8."""
    _cuda(kv, kr, pages)
    S, rot = kv.shape[0], kr.shape[1]
    hd = dim + rot
    for t in (kv, kr, pages):
        if t.dtype != torch.bfloat16:
            raise KernelError("latent_expand takes bfloat16 tensors")
    if kv.stride(1) != 1 or kv.shape[1] != H * dim + H * hd or kr.shape[0] != S or (rot and not kr.is_contiguous()) or dim % 8 or rot % 8 \
            or kv.stride(0) % 8 or kv.data_ptr() % 16:
        raise KernelError(f"latent_expand: kv is {tuple(kv.shape)}, kr {tuple(kr.shape)}")
    if tuple(pages.shape) != (-(-S // 64), 2, H, 64, hd) or not pages.is_contiguous():
        raise KernelError(f"latent_expand: pages are {tuple(pages.shape)}")
    with phase("kv_expand"):
        _check(lib().bg_latent_expand(_p(kv), kv.stride(0), _p(kr), H, dim, rot, S, _p(pages), _stream()), "latent_expand")


def rotate_q(q: torch.Tensor, H: int, head: int, off: int, rot_dims: int, cos_sin: torch.Tensor) -> None:
    """In place: of every head (of `head` features) of the rows of q, features off + 2i and off + 2i + 1 turn by
    cos_sin [T, rot_dims / 2, 2]."""
    _cuda(q, cos_sin)
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or q.stride(1) != 1 or q.shape[1] < H * head or off + rot_dims > head:
        raise KernelError("rotate_q: bfloat16 rows of H heads")
    if cos_sin.dtype != torch.float32 or cos_sin.shape[0] < T or cos_sin.shape[1] != rot_dims // 2 or not cos_sin.is_contiguous():
        raise KernelError("rotate_q: cos_sin must be float32 [T, rot_dims/2, 2]")
    with phase("rope"):
        _check(lib().bg_rotate_q(_p(q), q.stride(0), head, off, rot_dims, H, _p(cos_sin), T, _stream()), "rotate_q")


# ------------------------------------------------------------------------------------------------
# The Mamba-2 recurrence
def conv_silu(src: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor, state: torch.Tensor,
              conv_off: int, slots: torch.Tensor, row_req: torch.Tensor, reqs: torch.Tensor, n_req: int,
              out: torch.Tensor, activation: str = "silu", src_bias: Optional[torch.Tensor] = None) -> None:
    """The causal convolution per channel with SiLU (`activation` "none": without it) over src[:, col0 : col0 + channels],
    continued from and into the slots' conv state (`src_bias` float32 [channels], when given, is added to the rows' inputs,
    and the state keeps them with it).  weight [channels, taps] (last column the current token's), bias [channels]; state float32
    [slots, slot size] with the conv state, (taps - 1) x channels, at conv_off; reqs int32 [n_req, 3] = (request,
    first row, rows); out float32 [T, channels]."""
    _cuda(src, weight, bias, state, slots, row_req, reqs, out)
    _i32(slots, "slots"); _i32(row_req, "row_req"); _i32(reqs, "reqs")
    T = row_req.numel()
    taps = weight.shape[1]
    if src.dim() != 2 or src.stride(1) != 1 or src.shape[0] < T or col0 + channels > src.shape[1]:
        raise KernelError(f"conv_silu: rows of {tuple(src.shape)} cannot hold {channels} channels from {col0}")
    if tuple(weight.shape) != (channels, taps) or bias.numel() != channels or weight.dtype != bias.dtype \
            or not weight.is_contiguous() or not bias.is_contiguous():
        raise KernelError("conv_silu: weight [channels, taps] and bias [channels] of one type")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or conv_off + (taps - 1) * channels > state.shape[1]:
        raise KernelError(f"conv_silu: the state is {tuple(state.shape)}")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, channels) or not out.is_contiguous():
        raise KernelError("conv_silu: out is float32 [T, channels]")
    if activation not in ("silu", "none"):
        raise KernelError(f"conv_silu: unknown activation '{activation}' (silu, none)")
    if src_bias is not None:
        _cuda(src_bias)
        if src_bias.dtype != torch.float32 or src_bias.numel() != channels or not src_bias.is_contiguous():
            raise KernelError("conv_silu: src_bias is contiguous float32 [channels]")
    with phase("conv"):
        _check(lib().bg_conv_silu(_p(src), _dt(src), src.stride(0), col0, channels, taps, _p(weight), _p(bias), _dt(weight),
                                  _p(state), state.stride(0), conv_off, _p(slots), _p(row_req), _p(reqs), n_req, _p(out), T,
                                  1 if activation == "silu" else 0, _p(src_bias), _stream()), "conv_silu")
    if taps > 1:
        count_launches(1)


def ssm_scan(xbc: torch.Tensor, src: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, slots: torch.Tensor, reqs: torch.Tensor, n_req: int, y: torch.Tensor, H: int, P: int,
             N: int, G: int) -> None:
    """The recurrence over each request's rows, from and into the slots' state S [H, P, N] (float32, at the start of
    a slot): dt = softplus(src[t, dt_col + h] + dt_bias[h]); S = exp(-exp(A_log[h]) dt) S + dt B_t x_t^T;
    y_t = S^T C_t + D[h] x_t.  xbc float32 [T, H P + 2 G N] = [x | B | C]; y float32 [T, H P]."""
    _cuda(xbc, src, dt_bias, A_log, D, state, slots, reqs, y)
    _i32(slots, "slots"); _i32(reqs, "reqs")
    T = xbc.shape[0]
    if xbc.dtype != torch.float32 or not xbc.is_contiguous() or xbc.shape[1] != H * P + 2 * G * N:
        raise KernelError(f"ssm_scan: xbc is {tuple(xbc.shape)}")
    if src.dim() != 2 or src.stride(1) != 1 or dt_col + H > src.shape[1] or src.shape[0] < T:
        raise KernelError("ssm_scan: the rows hold no step sizes there")
    if not (dt_bias.dtype == A_log.dtype == D.dtype) or dt_bias.numel() != H or A_log.numel() != H or D.numel() != H:
        raise KernelError("ssm_scan: dt_bias, A_log and D have one value per head, of one type")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * N * P:
        raise KernelError(f"ssm_scan: the state is {tuple(state.shape)}")
    if y.dtype != torch.float32 or tuple(y.shape) != (T, H * P) or not y.is_contiguous():
        raise KernelError("ssm_scan: y is float32 [T, H P]")
    with phase("scan"):
        _check(lib().bg_ssm_scan(_p(xbc), xbc.shape[1], _p(src), _dt(src), src.stride(0), dt_col, _p(dt_bias), _p(A_log), _p(D),
                                 _dt(D), _p(state), state.stride(0), _p(slots), _p(reqs), n_req, _p(y), H, P, N, G, _stream()),
               "ssm_scan")


def gated_group_rmsnorm(y: torch.Tensor, src: torch.Tensor, z_col: int, weight: torch.Tensor, eps: float, groups: int,
                        out: torch.Tensor, gate_after: bool = False) -> None:
    """out = RMS norm, in `groups` equal parts of a row, of y * silu(src[:, z_col : z_col + inner]), times weight.  With
    `gate_after` the gate stands behind the norm and is a sigmoid: out = norm(y) * weight * sigmoid(src[:, z_col : ...])."""
    _cuda(y, src, weight, out)
    T, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or tuple(out.shape) != (T, inner) or not out.is_contiguous():
        raise KernelError("gated_group_rmsnorm: y float32 [T, inner], out [T, inner]")
    if src.dim() != 2 or src.stride(1) != 1 or z_col + inner > src.shape[1] or src.shape[0] < T or inner % groups:
        raise KernelError("gated_group_rmsnorm: the gate's columns or the groups do not fit")
    if weight.numel() != inner or not weight.is_contiguous():
        raise KernelError("gated_group_rmsnorm: one weight per feature")
    with phase("rmsnorm"):
        _check(lib().bg_gated_group_rmsnorm(_p(y), _p(src), _dt(src), src.stride(0), z_col, _p(weight), _dt(weight), float(eps),
                                            _p(out), _dt(out), T, inner, groups, 1 if gate_after else 0, _stream()), "gated_group_rmsnorm")


def rmsnorm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, lowp: Optional[torch.Tensor] = None) -> None:
    """x += rmsnorm(y) * weight for y [T, d] or its float partial sums [parts, T, d]; statistics and sum in float.
    `lowp`, when given, receives the new rows of x rounded to its type."""
    _cuda(x, y, weight, lowp)
    T, d = x.shape
    parts, stride = _parts(y, "rmsnorm_add: y")
    if x.dtype != torch.float32 or not x.is_contiguous() or tuple(y.shape[-2:]) != (T, d) or not y.is_contiguous():
        raise KernelError("rmsnorm_add: x contiguous float32 [T, d], y shaped like it (or its partial sums)")
    if parts > 1 and y.dtype != torch.float32:
        raise KernelError("rmsnorm_add: partial sums are float32")
    if weight.numel() != d or not weight.is_contiguous():
        raise KernelError(f"rmsnorm_add: weight has {weight.numel()} of {d} values")
    if lowp is not None and (tuple(lowp.shape) != (T, d) or not lowp.is_contiguous()):
        raise KernelError("rmsnorm_add: lowp must be contiguous and shaped like x")
    with phase("rmsnorm"):
        _check(lib().bg_rmsnorm_add(_p(x), _p(y), _dt(y), parts, stride, _p(weight), _dt(weight), float(eps), _p(lowp),
                                    _dt(lowp) if lowp is not None else F32, T, d, _stream()), "rmsnorm_add")


def rmsnorm_add_routed(x: torch.Tensor, yp: torch.Tensor, row_of: torch.Tensor, weights: torch.Tensor, top: int, scale: bool,
                       weight: torch.Tensor, eps: float, lowp: Optional[torch.Tensor] = None) -> None:
    """`route_combine` and `rmsnorm_add` as one kernel: x += rmsnorm(y) * weight with y[t] the sum over j < top of
    (weights[t * top + j] *) yp[row_of[t * top + j]], ranks in index order; yp float32 [T * top, d]."""
    _cuda(x, yp, row_of, weights, weight, lowp)
    _i32(row_of, "row_of")
    T, d = x.shape
    if x.dtype != torch.float32 or yp.dtype != torch.float32 or weights.dtype != torch.float32 or not x.is_contiguous() \
            or not yp.is_contiguous() or tuple(yp.shape) != (T * top, d) or row_of.numel() != T * top or weights.numel() != T * top:
        raise KernelError("rmsnorm_add_routed: x float32 [T, d], yp float32 [T * top, d], row_of and weights [T * top]")
    if weight.numel() != d or not weight.is_contiguous():
        raise KernelError(f"rmsnorm_add_routed: weight has {weight.numel()} of {d} values")
    if lowp is not None and (tuple(lowp.shape) != (T, d) or not lowp.is_contiguous()):
        raise KernelError("rmsnorm_add_routed: lowp must be contiguous and shaped like x")
    with phase("rmsnorm"):
        _check(lib().bg_rmsnorm_add_routed(_p(x), _p(yp), _p(row_of), _p(weights), top, 1 if scale else 0, _p(weight), _dt(weight),
                                           float(eps), _p(lowp), _dt(lowp) if lowp is not None else F32, T, d, _stream()),
               "rmsnorm_add_routed")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x rounded to out's type (x float32)."""
    _cuda(x, out)
    if x.dtype != torch.float32 or x.shape != out.shape or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("cast_rows: x contiguous float32, out contiguous and shaped like it")
    with phase("residuals"):
        _check(lib().bg_cast_rows(_p(x), _p(out), _dt(out), x.numel(), _stream()), "cast_rows")


def qk_norm_rope_append(src: torch.Tensor, q_out: torch.Tensor, n_rows: int, nh: int, nkv: int, hd: int, vd: int, rot: int,
                        interleaved: bool, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos_sin: Optional[torch.Tensor], positions: torch.Tensor, row_req: torch.Tensor,
                        block_table: torch.Tensor, kv_pool: Optional[torch.Tensor], page_size: int,
                        status: Optional[torch.Tensor], stored: Optional[int] = None, per_head: bool = False) -> None:
    """Rows [q | k | v | ...] of `src` ([T, W], or float partial sums [parts, T, W]): RMS norm of the whole q row and of
    the whole k row with the float weights given (None: no norm; with `per_head` every head is normed by itself and the
    weights have hd values, shared by the heads), rotation of the first `rot` features of every head,
    q into q_out [T, nh*hd], k and v into the paged cache (a page: keys [nkv, page, hd], then values [nkv, page, vd]).
    With `stored` = D every head of q, k and v is stored D features wide, zeros behind its own."""
    qs, ks, vs = (hd, hd, vd) if stored is None else (stored, stored, stored)
    _cuda(src, q_out, q_weight, k_weight, cos_sin, positions, row_req, block_table, kv_pool)
    _i32(positions, "positions"); _i32(row_req, "row_req"); _i32(block_table, "block_table")
    parts, stride = _parts(src, "qk_norm_rope_append: src")
    need = nh * hd + (nkv * (hd + vd) if kv_pool is not None else 0)
    if src.stride(-1) != 1 or src.shape[-1] < need or src.shape[-2] < n_rows:
        raise KernelError(f"qk_norm_rope_append: rows of {src.shape[-1]} features cannot hold q, k, v ({need})")
    if q_out.stride(1) != 1 or q_out.shape[1] < nh * qs or q_out.shape[0] < n_rows:
        raise KernelError("qk_norm_rope_append: q_out must be [T, nh*hd]")
    for w, n in ((q_weight, hd if per_head else nh * hd), (k_weight, hd if per_head else nkv * hd)):
        if w is not None and (w.dtype != torch.float32 or w.numel() != n or not w.is_contiguous()):
            raise KernelError("qk_norm_rope_append: norm weights are contiguous float32 of the projection's width")
    num_pages = 0
    if kv_pool is not None:
        if not kv_pool.is_contiguous() or kv_pool[0].numel() != nkv * page_size * (ks + vs):
            raise KernelError(f"qk_norm_rope_append: a page of {tuple(kv_pool.shape)} does not hold {nkv} x {page_size} x ({ks} + {vs})")
        num_pages = kv_pool.shape[0]
    if rot > 0 and (cos_sin is None or cos_sin.shape[0] < n_rows or cos_sin.shape[1] != rot // 2 or cos_sin.dtype != torch.float32):
        raise KernelError("qk_norm_rope_append: cos_sin must be float32 [T, rot/2, 2]")
    with phase("rope+kv_write"):
        _check(lib().bg_qk_norm_rope_append(_p(src), _dt(src), src.stride(-2), parts, stride, _p(q_out), _dt(q_out), q_out.stride(0),
                                            _p(q_weight), _p(k_weight), float(eps), _p(cos_sin), _p(positions), _p(row_req),
                                            _p(block_table), block_table.shape[1], _p(kv_pool),
                                            _dt(kv_pool) if kv_pool is not None else _dt(q_out), num_pages, page_size, n_rows, nh,
                                            nkv, hd, vd, rot, 1 if interleaved else 0, qs, ks, vs, 1 if per_head else 0, _p(status), _stream()),
               "qk_norm_rope_append")


def sigmoid_gate(out: torch.Tensor, gate: torch.Tensor, col0: int, n: int, src: Optional[torch.Tensor] = None,
                 vd: Optional[int] = None, head_stride: Optional[int] = None, gate_per: int = 1) -> None:
    """out[t, j] = src[t, (j // vd) * head_stride + j % vd] * sigmoid(gate[t, col0 + j // gate_per]) for j < n; gate is [T, W]
    or its float partial sums [parts, T, W].  Without `src`, out itself is gated in place.  `gate_per` = the size of a head
    gives every head one gate."""
    _cuda(out, gate, src)
    parts, stride = _parts(gate, "sigmoid_gate: gate")
    T = out.shape[0]
    if src is None:
        src, vd, head_stride = out, n, n
    if out.dim() != 2 or out.stride(1) != 1 or out.shape[1] < n or gate.stride(-1) != 1 or gate.shape[-2] < T or col0 + -(-n // gate_per) > gate.shape[-1]:
        raise KernelError("sigmoid_gate: out [T, >= n], gate rows that hold n values from col0")
    if src.dtype != out.dtype or src.stride(1) != 1 or src.shape[0] < T or n % vd or src.shape[1] < (n // vd - 1) * head_stride + vd:
        raise KernelError("sigmoid_gate: src of out's type with n / vd heads, head_stride features apart")
    with phase("activation"):
        _check(lib().bg_sigmoid_gate(_p(out), _dt(out), out.stride(0), _p(src), src.stride(0), vd, head_stride, _p(gate), _dt(gate),
                                     gate.stride(-2), parts, stride, col0, T, n, int(gate_per), _stream()), "sigmoid_gate")


def decay_attention_chunk(n: int, nv: int) -> int:
    """The number of tokens in a chunk of the chunked kernels for heads of n x nv values, 0 when they do not take them."""
    c = _c_int(0)
    return c.value if lib().bg_decay_attention_chunk_plan(int(n), int(nv), ctypes.byref(c)) == 0 else 0


def decay_attention(src: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
                    slots: torch.Tensor, reqs: torch.Tensor, n_req: int, y: torch.Tensor, H: int, n: int, nv: int,
                    chunks: Optional[torch.Tensor] = None, n_chunks: int = 0, longs: Optional[torch.Tensor] = None,
                    n_long: int = 0) -> None:
    """Linear attention with a constant decay per head.  `src` [T, W] (or float partial sums [parts, T, W]) holds, from the
    columns given, the products for q, k ([H, n] each) and v ([H, nv]); q, k, v = silu of them.  Per request (`reqs`
    [n_req, 3] = request, first row, rows) and head, for its rows in turn: S <- decay[h] S + k v^T, y = S^T q, with S
    [n, nv] float32 at state[slots[request], h * n * nv ...], read at the start and written back at the end.

    Requests of many rows may be given apart, cut into chunks of `decay_attention_chunk(n, nv)` rows: `chunks`
    [n_chunks, 4] = (request, first row, rows, -) and `longs` [n_long, 4] = (request, first row, rows, index of the first
    chunk).  Their chunks run in parallel (sums of a chunk's own k v^T, a pass over the chunks' states, the outputs); the
    results are those of the walk token by token up to rounding.  A request stands in `reqs` or in `longs`, not both."""
    _cuda(src, decay, state, slots, reqs, y, chunks, longs)
    _i32(slots, "slots")
    if n_req:
        _i32(reqs, "reqs")
    parts, stride = _parts(src, "decay_attention: src")
    T, W = src.shape[-2:]
    if src.stride(-1) != 1 or max(q_col + H * n, k_col + H * n, v_col + H * nv) > W:
        raise KernelError("decay_attention: the rows do not hold q, k and v at the columns given")
    if decay.dtype != torch.float32 or decay.numel() != H or not decay.is_contiguous():
        raise KernelError("decay_attention: one float32 decay per head")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * n * nv:
        raise KernelError(f"decay_attention: the state slab is float32 [slots, >= {H * n * nv}]")
    if y.dtype != torch.float32 or tuple(y.shape) != (T, H * nv) or not y.is_contiguous():
        raise KernelError(f"decay_attention: y is float32 {(T, H * nv)}")
    with phase("scan"):
        if n_req:
            _check(lib().bg_decay_attention(_p(src), _dt(src), src.stride(-2), parts, stride, q_col, k_col, v_col, _p(decay),
                                            _p(state), state.stride(0), _p(slots), _p(reqs), n_req, _p(y), H, n, nv, _stream()),
                   "decay_attention")
        if n_chunks:
            _i32(chunks, "chunks"); _i32(longs, "longs")
            if chunks.shape[0] < n_chunks or longs.shape[0] < n_long or n_long < 1:
                raise KernelError("decay_attention: the lists of chunks and of long requests are shorter than their counts")
            work = torch.empty((n_chunks, H, n * nv), dtype=torch.float32, device=y.device)
            _check(lib().bg_decay_attention_chunked(_p(src), _dt(src), src.stride(-2), parts, stride, q_col, k_col, v_col, _p(decay),
                                                    _p(state), state.stride(0), _p(slots), _p(chunks), n_chunks, _p(longs), n_long,
                                                    _p(work), _p(y), H, n, nv, _stream()), "decay_attention_chunked")


def add_terms_norm(x: torch.Tensor, terms, assign: bool = False, weight1: Optional[torch.Tensor] = None,
                   weight2: Optional[torch.Tensor] = None, eps: float = 0.0, out1: Optional[torch.Tensor] = None,
                   out2: Optional[torch.Tensor] = None) -> None:
    """x (= or +=) sum_i scale_i * term_i for `terms` = [(tensor, scale), ...], each tensor [T, d] of either type or float
    partial sums [parts, T, d]; then out1 = rmsnorm(x) * weight1 and out2 = rmsnorm(x) * weight2 when given (one pass
    over the rows for the sum and both norms).  x is the float32 residual [T, d]."""
    tensors = [t for t, _ in terms]
    _cuda(x, weight1, weight2, out1, out2, *tensors)
    T, d = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("add_terms_norm: x is contiguous float32")
    if len(terms) > 6:
        raise KernelError("add_terms_norm: at most six terms")
    ptrs, dts, parts, strides, scales = [], [], [], [], []
    for t, sc in terms:
        n, st = _parts(t, "add_terms_norm: term")
        if tuple(t.shape[-2:]) != (T, d) or not t.is_contiguous():
            raise KernelError("add_terms_norm: a term is contiguous and shaped like x")
        ptrs.append(t.data_ptr()); dts.append(_dt(t)); parts.append(n); strides.append(st); scales.append(float(sc))
    for o, w in ((out1, weight1), (out2, weight2)):
        if o is not None and (w is None or w.numel() != d or not w.is_contiguous() or tuple(o.shape) != (T, d) or not o.is_contiguous()):
            raise KernelError("add_terms_norm: a normed output is [T, d] and has d weights")
    if out2 is not None and (out1 is None or out2.dtype != out1.dtype or weight2.dtype != weight1.dtype):
        raise KernelError("add_terms_norm: the second normed output comes with a first of the same types")
    k = len(terms)
    arr = lambda ct, vals: (ct * max(k, 1))(*vals) if vals else (ct * 1)()
    with phase("rmsnorm" if out1 is not None else "residuals"):
        _check(lib().bg_add_terms_norm(_p(x), T, d, 1 if assign else 0, k, arr(_c_void_p, ptrs), arr(_c_int, dts), arr(_c_int, parts),
                                       arr(_c_ll, strides), arr(_c_float, scales), _p(weight1), _p(weight2),
                                       _dt(weight1) if weight1 is not None else F32, float(eps), _p(out1), _p(out2),
                                       _dt(out1) if out1 is not None else F32, _stream()), "add_terms_norm")


# ---------------------------------------------------------------------------------------------------- routed experts
EXPERT_ACTIVATIONS = {"none": 0, "relu2": 1}


def route_logits(h: torch.Tensor, router: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, e] = sum_k h[t, k] router[e, k], float: h in either type, router and out float32.  CUDA cores."""
    _cuda(h, router, out)
    T, d = h.shape
    E = router.shape[0]
    if router.dtype != torch.float32 or out.dtype != torch.float32 or router.shape[1] != d or tuple(out.shape) != (T, E) \
            or h.stride(1) != 1 or not router.is_contiguous() or not out.is_contiguous():
        raise KernelError("route_logits: h [T, d], router float32 [E, d], out float32 [T, E]")
    with phase("router"):
        _check(lib().bg_route_logits(_p(h), _dt(h), h.stride(0), _p(router), d, _p(out), E, T, E, d, _stream()), "route_logits")


ROUTER_MODES = {"none": 0, "sigmoid": 1, "softmax": 2}


def _route_rule(E: int, sigmoid, bias: Optional[torch.Tensor], what: str) -> int:
    """The kernels' score mode from `sigmoid` (True, False, or one of ROUTER_MODES), with the choice bias checked."""
    mode = ROUTER_MODES[sigmoid] if isinstance(sigmoid, str) else (1 if sigmoid else 0)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != E or not bias.is_contiguous()):
        raise KernelError(f"{what}: the choice bias is contiguous float32, one number per expert")
    return mode


def route_topk(logits: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor, sigmoid=True,
               renorm: bool = False, bias: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """Per row of float logits [T, E]: the `top` experts of largest score into ids [T, top] (int32) and their scores
    into weights [T, top] (float32).  `sigmoid` may name the score: "none", "sigmoid" or "softmax" (over all E).  `bias`
    [E] is added to the scores for the choice only; `scale` multiplies the weights."""
    _cuda(logits, ids, weights)
    T, E = logits.shape
    _i32(ids, "ids")
    if logits.dtype != torch.float32 or weights.dtype != torch.float32 or not logits.is_contiguous() \
            or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top) or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("route_topk: logits float32 [T, E], ids int32 [T, top], weights float32 [T, top]")
    with phase("router"):
        _check(lib().bg_route_topk(_p(logits), T, E, top, _route_rule(E, sigmoid, bias, "route_topk"), 1 if renorm else 0, _p(bias),
                                   float(scale), _p(ids), _p(weights), _stream()), "route_topk")


def route(h: torch.Tensor, router: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor, sigmoid=True,
          renorm: bool = False, logits: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> None:
    """`route_logits` and `route_topk` as one kernel: h [T, d] in either type, router float32 [E, d], ids int32 [T, top],
    weights float32 [T, top]; `logits`, when given, receives the float logits [T, E]."""
    _cuda(h, router, ids, weights, logits, bias)
    T, d = h.shape
    E = router.shape[0]
    _i32(ids, "ids")
    if router.dtype != torch.float32 or router.shape[1] != d or h.stride(1) != 1 or not router.is_contiguous() \
            or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top) or weights.dtype != torch.float32 \
            or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("route: h [T, d], router float32 [E, d], ids int32 [T, top], weights float32 [T, top]")
    if logits is not None and (logits.dtype != torch.float32 or tuple(logits.shape) != (T, E) or not logits.is_contiguous()):
        raise KernelError("route: logits float32 [T, E]")
    with phase("router"):
        _check(lib().bg_route(_p(h), _dt(h), h.stride(0), _p(router), T, d, E, top, _route_rule(E, sigmoid, bias, "route"),
                              1 if renorm else 0, _p(bias), float(scale), _p(ids), _p(weights), _p(logits), _stream()), "route")


def route_sort(ids: torch.Tensor, E: int, offsets: torch.Tensor, row_of: torch.Tensor, src_of: torch.Tensor) -> None:
    """The assignments ids [A] laid out expert by expert: offsets int32 [E + 1], row_of [A] (where each went), src_of [A]."""
    _cuda(ids, offsets, row_of, src_of)
    for t, n in ((ids, "ids"), (offsets, "offsets"), (row_of, "row_of"), (src_of, "src_of")):
        _i32(t, n)
    A = ids.numel()
    if offsets.numel() != E + 1 or row_of.numel() != A or src_of.numel() != A:
        raise KernelError("route_sort: offsets [E + 1], row_of and src_of [A]")
    with phase("router"):
        _check(lib().bg_route_sort(_p(ids), A, E, _p(offsets), _p(row_of), _p(src_of), _stream()), "route_sort")


def route_gather(x: torch.Tensor, weights: torch.Tensor, src_of: torch.Tensor, out: torch.Tensor, top: int, scale: bool) -> None:
    """out[row] = (weights[a] *) x[a // top] for a = src_of[row], rounded to out's type."""
    _cuda(x, weights, src_of, out)
    A, d = out.shape
    if not x.is_contiguous() or not out.is_contiguous() or x.shape[1] != d or weights.numel() != A or src_of.numel() != A:
        raise KernelError("route_gather: x [T, d], out [T * top, d], weights and src_of [T * top]")
    with phase("router"):
        _check(lib().bg_route_gather(_p(x), _dt(x), _p(weights), _p(src_of), _p(out), _dt(out), A, d, top, 1 if scale else 0,
                                     _stream()), "route_gather")


def route_combine(yp: torch.Tensor, weights: torch.Tensor, row_of: torch.Tensor, out: torch.Tensor, top: int, scale: bool) -> None:
    """out[t] = sum over j < top of (weights[t * top + j] *) yp[row_of[t * top + j]], ranks in index order, float."""
    _cuda(yp, weights, row_of, out)
    T, d = out.shape
    if out.dtype != torch.float32 or not yp.is_contiguous() or not out.is_contiguous() or tuple(yp.shape) != (T * top, d):
        raise KernelError("route_combine: yp [T * top, d], out float32 [T, d]")
    with phase("router"):
        _check(lib().bg_route_combine(_p(yp), _dt(yp), _p(weights), _p(row_of), _p(out), T, d, top, 1 if scale else 0, _stream()),
               "route_combine")


def route_combine_ext(yp: torch.Tensor, weights: torch.Tensor, row_of: torch.Tensor, ids: torch.Tensor, n_real: int, h: torch.Tensor,
                      out: torch.Tensor, top: int, shared: Optional[torch.Tensor] = None, sg: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over j < top of weights[t top + j] * (yp[row_of[t top + j]] if ids[t top + j] < n_real else h[t])
    + sigmoid(sg[t]) * shared[t]: experts from n_real on return their input h [T, d] (either type, unit inner stride).
    `shared` float32 [T, d] contiguous and `sg` [T] (either type, any stride) may be absent; without sg the shared rows are added
    as they are."""
    _cuda(yp, weights, row_of, ids, h, out, shared, sg)
    _i32(row_of, "row_of"); _i32(ids, "ids")
    T, d = out.shape
    if out.dtype != torch.float32 or not yp.is_contiguous() or not out.is_contiguous() or tuple(yp.shape) != (T * top, d) \
            or tuple(h.shape) != (T, d) or h.stride(1) != 1 or ids.numel() != T * top or weights.numel() != T * top \
            or weights.dtype != torch.float32:
        raise KernelError("route_combine_ext: yp [T * top, d], h [T, d], out float32 [T, d], ids and weights [T * top]")
    if shared is not None and (shared.dtype != torch.float32 or tuple(shared.shape) != (T, d) or not shared.is_contiguous()):
        raise KernelError("route_combine_ext: shared float32 [T, d]")
    if sg is not None and (shared is None or sg.dim() != 1 or sg.numel() != T):
        raise KernelError("route_combine_ext: sg [T] beside shared rows")
    with phase("router"):
        _check(lib().bg_route_combine_ext(_p(yp), _dt(yp), _p(weights), _p(row_of), _p(ids), int(n_real), _p(h), _dt(h), h.stride(0),
                                          _p(shared), _p(sg), _dt(sg) if sg is not None else F32,
                                          sg.stride(0) if sg is not None else 0, _p(out), T, d, top, _stream()), "route_combine_ext")


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float = 1.702) -> None:
    """out[r, i] = g sigmoid(alpha g) (u + 1) with g = min(gate_up[r, i], limit), u = clamp(gate_up[r, n + i], -limit, limit),
    n = out.shape[1]: gate_up [rows, >= 2 n] of either type with unit inner stride, out contiguous [rows, n]."""
    _cuda(gate_up, out)
    rows, n = out.shape
    if gate_up.dim() != 2 or gate_up.shape[0] != rows or gate_up.shape[1] < 2 * n or gate_up.stride(1) != 1 or not out.is_contiguous() \
            or not limit > 0.0:
        raise KernelError("glu_clamped: gate_up [rows, >= 2 n], out contiguous [rows, n], a positive limit")
    with phase("swiglu"):
        _check(lib().bg_glu_clamped(_p(gate_up), _dt(gate_up), gate_up.stride(0), _p(out), _dt(out), rows, n, float(limit),
                                    float(alpha), _stream()), "glu_clamped")


# ---------------------------------------------------------------------------------------------------- a residual in lanes
def lane_fill(x: torch.Tensor, lanes: torch.Tensor) -> None:
    """lanes[a] = x for every lane a: x float32 [T, d], lanes float32 [n, T, d], both contiguous."""
    _cuda(x, lanes)
    if x.dtype != torch.float32 or lanes.dtype != torch.float32 or not x.is_contiguous() or not lanes.is_contiguous() \
            or tuple(lanes.shape[1:]) != tuple(x.shape):
        raise KernelError("lane_fill: x float32 [T, d], lanes float32 [n, T, d]")
    with phase("residuals"):
        _check(lib().bg_lane_fill(_p(x), _p(lanes), x.numel(), lanes.shape[0], _stream()), "lane_fill")


def lane_step(lanes: torch.Tensor, owed: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
              out_weights: Optional[torch.Tensor] = None, in_weights: Optional[torch.Tensor] = None,
              norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, h: Optional[torch.Tensor] = None,
              z: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """One pass over a residual kept in lanes, float32 [n, T, d].  With `owed` (a sublayer's result [T, d] in either type, or
    float partial sums [parts, T, d]) the lanes are first rewritten, all at once: lane b <- sum_a mix[a, b] lane a +
    out_weights[b] owed.  Then the read sum_a in_weights[a] lane a (ones when absent) goes to `z` (float32) as it is and/or
    to `h` RMS-normed with `norm_weight` (float32 [d]) and `eps`.  With `rows` (int32) only those rows are read, and
    nothing is written back."""
    _cuda(lanes, owed, mix, out_weights, in_weights, norm_weight, h, z, rows)
    if lanes.dtype != torch.float32 or lanes.dim() != 3 or not lanes.is_contiguous():
        raise KernelError("lane_step: the lanes are contiguous float32 [n, T, d]")
    n, T, d = lanes.shape
    for name, t, count in (("mix", mix, n * n), ("out_weights", out_weights, n), ("in_weights", in_weights, n), ("norm_weight", norm_weight, d)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != count or not t.is_contiguous()):
            raise KernelError(f"lane_step: {name} is contiguous float32 with {count} values")
    parts, stride = 0, 0
    if owed is not None:
        parts, stride = _parts(owed, "lane_step: owed")
        if tuple(owed.shape[-2:]) != (T, d) or not owed.is_contiguous() or mix is None or out_weights is None:
            raise KernelError("lane_step: the owed result is contiguous [T, d] (or [parts, T, d]) and comes with mix and out_weights")
    n_rows = T
    if rows is not None:
        _i32(rows, "rows")
        n_rows = rows.numel()
    for name, t in (("h", h), ("z", z)):
        if t is not None and (tuple(t.shape) != (n_rows, d) or not t.is_contiguous()):
            raise KernelError(f"lane_step: {name} is contiguous [{n_rows}, {d}]")
    if z is not None and z.dtype != torch.float32:
        raise KernelError("lane_step: z is float32")
    if h is not None and norm_weight is None:
        raise KernelError("lane_step: the normed read wants a norm weight")
    with phase("rmsnorm"):
        _check(lib().bg_lane_step(_p(lanes), n, T * d, _p(owed), _dt(owed) if owed is not None else F32, parts, stride, _p(mix),
                                  _p(out_weights), _p(in_weights), _p(norm_weight), float(eps), _p(h),
                                  _dt(h) if h is not None else F32, _p(z), _p(rows), n_rows, d, _stream()), "lane_step")


# ---------------------------------------------------------------------------------------------------- gated linear recurrence
def rglru_softplus(lam: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[c] = scale * softplus(lam[c]), float32."""
    _cuda(lam, out)
    if out.dtype != torch.float32 or out.numel() != lam.numel() or not lam.is_contiguous() or not out.is_contiguous():
        raise KernelError("rglru_softplus: out float32 of lam's size")
    _check(lib().bg_rglru_softplus(_p(lam), _dt(lam), float(scale), _p(out), lam.numel(), _stream()), "rglru_softplus")


def rglru_split(u: torch.Tensor, blocks: int, out: torch.Tensor) -> None:
    """out[b, t] = [bfloat16(u_b[t]) | bfloat16(u_b[t] - the first)] for the parts u_b of u's columns: u float32 [T, W],
    out bfloat16 [blocks, T, 2 W / blocks]."""
    _cuda(u, out)
    T, W = u.shape
    if u.dtype != torch.float32 or out.dtype != torch.bfloat16 or not u.is_contiguous() or not out.is_contiguous() \
            or W % blocks or tuple(out.shape) != (blocks, T, 2 * (W // blocks)):
        raise KernelError("rglru_split: u float32 [T, W], out bfloat16 [blocks, T, 2 W / blocks]")
    with phase("scan"):
        _check(lib().bg_rglru_split(_p(u), _p(out), T, W, blocks, _stream()), "rglru_split")


def rglru_scan(gates: torch.Tensor, u: torch.Tensor, src: torch.Tensor, y_col: int, gate_bias_r: torch.Tensor,
               gate_bias_i: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, reqs: torch.Tensor,
               n_req: int, out: torch.Tensor, chunked: Optional[tuple] = None, y_bias: Optional[torch.Tensor] = None) -> None:
    """The gated linear recurrence of a step.  gates float32 [blocks, T, 2 bs] (per block the recurrence gate's and the
    input gate's products), u float32 [T, W] the convolved input, src float32 rows whose columns y_col .. y_col + W are
    the other branch (`y_bias` float32 [W], when given, is added to it), the gates' biases and `decay` (= C softplus(lam)) float32 [W], state float32 [slots, size] with
    the W states first, reqs int32 [n_req, 3] = (request, first row, rows), out [T, W] in either type.  `chunked` =
    (chunks, n_chunks, longs, n_long, chunk_rows) instead of reqs: those requests' rows in chunks (`cut_long_requests`)."""
    _cuda(gates, u, src, gate_bias_r, gate_bias_i, decay, state, slots, reqs, out, y_bias)
    _i32(slots, "slots")
    T, W = u.shape
    if y_bias is not None and (y_bias.dtype != torch.float32 or y_bias.numel() != W or not y_bias.is_contiguous()):
        raise KernelError("rglru_scan: y_bias is contiguous float32 [W]")
    blocks = gates.shape[0]
    for t in (gates, u, gate_bias_r, gate_bias_i, decay):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise KernelError("rglru_scan: gates, u, biases and decay are contiguous float32")
    if W % blocks or tuple(gates.shape) != (blocks, T, 2 * (W // blocks)) or gate_bias_r.numel() != W or gate_bias_i.numel() != W \
            or decay.numel() != W:
        raise KernelError(f"rglru_scan: gates {tuple(gates.shape)} do not fit u {tuple(u.shape)}")
    if src.dtype != torch.float32 or src.dim() != 2 or src.stride(1) != 1 or src.shape[0] < T or y_col + W > src.shape[1]:
        raise KernelError("rglru_scan: src float32 rows with the other branch's W columns from y_col")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < W:
        raise KernelError(f"rglru_scan: the state is {tuple(state.shape)}")
    if tuple(out.shape) != (T, W) or not out.is_contiguous():
        raise KernelError("rglru_scan: out is contiguous [T, W]")
    with phase("scan"):
        if chunked is None:
            _i32(reqs, "reqs")
            _check(lib().bg_rglru_scan(_p(gates), _p(u), _p(src), src.stride(0), y_col, _p(y_bias), _p(gate_bias_r), _p(gate_bias_i), _p(decay),
                                       _p(state), state.stride(0), _p(slots), _p(reqs), n_req, _p(out), _dt(out), T, W, blocks,
                                       _stream()), "rglru_scan")
        else:
            chunks, n_chunks, longs, n_long, chunk_rows = chunked
            if n_chunks == 0:
                return
            pq = torch.empty((n_chunks, 2, W), dtype=torch.float32, device=u.device)
            ab = torch.empty((T, W, 2), dtype=torch.float32, device=u.device)
            _check(lib().bg_rglru_scan_chunked(_p(gates), _p(u), _p(src), src.stride(0), y_col, _p(y_bias), _p(gate_bias_r), _p(gate_bias_i),
                                               _p(decay), _p(state), state.stride(0), _p(slots), _p(chunks), n_chunks, _p(longs),
                                               n_long, chunk_rows, _p(pq), _p(ab), _p(out), _dt(out), T, W, blocks, _stream()),
                   "rglru_scan_chunked")
            count_launches(2)


def gemm_grouped(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor, activation: str = "none",
                 status: Optional[torch.Tensor] = None, tensor_cores: bool = True) -> None:
    """out[row] = act(x[row] w[e]^T) for the rows offsets[e] .. offsets[e + 1] of every expert e: x [A, K], w [E, N, K],
    out [A, N].  bfloat16 operands whose K is a multiple of 8 run the tcgen05 kernel (unless `tensor_cores` is False);
    float32 operands, and every other size, the CUDA-core kernel."""
    _cuda(x, w, offsets, out)
    _i32(offsets, "offsets")
    A, K = x.shape
    E, N, K2 = w.shape
    if K2 != K or tuple(out.shape) != (A, N) or offsets.numel() != E + 1 or x.dtype != w.dtype \
            or not x.is_contiguous() or not w.is_contiguous() or not out.is_contiguous():
        raise KernelError("gemm_grouped: x [A, K], w [E, N, K] of x's type, out [A, N], offsets [E + 1], all contiguous")
    act = EXPERT_ACTIVATIONS[activation]
    with phase("experts"):
        if tensor_cores and x.dtype == torch.bfloat16 and K % 8 == 0:
            _check(lib().bg_gemm_grouped_tc(_p(w), E, N, K, K, _p(x), A, K, _p(out), _dt(out), N, _p(offsets), act, _p(status),
                                            _stream()), "gemm_grouped_tc")
        else:
            _check(lib().bg_gemm_grouped(_p(x), _dt(x), K, _p(w), K, N * K, _p(out), _dt(out), N, _p(offsets), E, A, N, K, act,
                                         _stream()), "gemm_grouped")
