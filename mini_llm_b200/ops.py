"""The kernel library: the Python face of the CUDA sources in ``csrc/``.

Every function checks its arguments (device, dtype, layout, sizes the kernel can
take) and then calls one exported C function with raw device pointers and the
current CUDA stream.  There is no CPU fallback and no library attention or model
code behind these names: if the shared library cannot be built or loaded, or a
tensor is not on a CUDA device, the call fails with an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
SMALL_M = 64                 # rows up to which the weight-streaming product is used
SMALL_M_F32 = 64             # the same for the float32 weight-streaming product (csrc/linear_stream_f32.cu)
NORM_FUSE_M_F32 = 16         # rows up to which that product takes the norm into its loads (rows up to 2048 wide)
DECODE_SPLIT = 128           # keys per split of the decode attention (csrc/attention_decode.cu)
DECODE_CLUSTER_SPLITS = 8    # splits that can meet in one thread-block cluster (MAX_CLUSTER there)
_FLASH_HEAD_DIMS = (16, 32, 64, 128)
_DECODE_HEAD_DIMS = {torch.bfloat16: (16, 32, 64, 128, 256), torch.float32: (16, 32, 64, 128)}
_ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2}      # what the products' epilogues take
_GATE_ACT = {"gelu_tanh": 1, "gelu_erf": 2, "relu": 3, "silu": 4, "swiglu_clamp": 5}   # what gated_act takes
_UNGATED_ACT = {"relu_sq": 6}     # activations of one argument that the experts' first product takes (experts without a gate)
_lib = None

c_int, c_ll, c_float, c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def _signatures(lib):
    lib.mllm_last_error.restype = ctypes.c_char_p
    lib.mllm_abi_version.restype = c_int
    lib.mllm_set_pdl.argtypes = [c_int]
    lib.mllm_set_pdl.restype = c_int
    sig = {
        "mllm_embed": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_resolve_tokens": [c_void_p, c_int, c_void_p, c_int, c_void_p],
        "mllm_layernorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_kv_write": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                          c_void_p],
        "mllm_linear_simt": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_void_p, c_ll, c_void_p],
        "mllm_linear_simt_splits": [c_int, c_int],
        "mllm_attention_simt": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                c_ll, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_linear_smallm": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p],
        "mllm_linear_smallm_fused": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_linear_stream_f32": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_void_p],
        "mllm_linear_stream_f32_tall_rows": [c_int, c_int],
        "mllm_linear_stream_f32_kernel_of": [c_int, c_int, c_int],
        "mllm_linear_stream_f32_bind_error": [c_void_p],
        "mllm_linear_stream_f32_error": [c_void_p],
        "mllm_linear_tcgen05": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p],
        "mllm_linear_tcgen05_qkv": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_tcgen05_error": [c_void_p],
        "mllm_tcgen05_bind_error": [c_void_p],
        "mllm_attention_tcgen05_bind_error": [c_void_p],
        "mllm_attention_decode_bind_error": [c_void_p],
        "mllm_debug_report_error": [c_int, c_void_p],
        "mllm_attention_decode": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_int, c_int, c_int, c_void_p],
        "mllm_attention_decode_last_staging": [],
        "mllm_attention_flash": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                 c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_attention_tcgen05": [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_attention_tcgen05_error": [c_void_p],
        "mllm_attention_decode_error": [c_void_p],
        "mllm_attention_tiled": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                 c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_attention_tiled_wide": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                      c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_rmsnorm": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_float,
                         c_float, c_float, c_int, c_void_p],
        "mllm_gated_recurrence_wide": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p],
        "mllm_gated_act": [c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
        "mllm_paged_write": [c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_paged_write_kv": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_void_p],
        "mllm_attention_bias_split_keys": [],
        "mllm_attention_bias": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_float, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_int,
                                c_int, c_void_p],
        "mllm_qk_norm_rope": [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                              c_void_p, c_int, c_int, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_int,
                              c_int, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
        "mllm_post_norm": [c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_ll, c_void_p, c_ll, c_int,
                           c_int, c_float, c_int, c_void_p],
        "mllm_wkv_shift": [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_int, c_int, c_void_p],
        "mllm_wkv_step_ok": [c_int, c_int],
        "mllm_wkv_step": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_ll, c_void_p, c_void_p, c_ll, c_void_p, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_wkv_decay": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_wkv_scan": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_void_p,
                          c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_wkv_finish": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int,
                            c_void_p],
        "mllm_wkv_max_dim": [],
        "mllm_hyper_step": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                            c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_hyper_max_streams": [],
        "mllm_softcap": [c_void_p, c_ll, c_int, c_int, c_float, c_void_p],
        "mllm_gated_recurrence": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                  c_int, c_void_p],
        "mllm_norm_scale_add": [c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_float,
                                c_float, c_void_p, c_ll, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_latent_prepare": [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "mllm_headwise_linear": [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_void_p],
        "mllm_latent_attention": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_latent_attention_mma": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_float, c_void_p],
        "mllm_latent_mma_ok": [c_int, c_int, c_int],
        "mllm_ssd_conv": [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_ssd_scan": [c_void_p, c_int, c_int, c_int, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_ll,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_gated_group_norm": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int,
                                  c_void_p],
        "mllm_moe_route": [c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mllm_moe_grouped": [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
        "mllm_moe_combine": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_argmax": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p],
        "mllm_argmax_sliced": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mllm_sample": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


def library():
    """The loaded shared library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.ensure_built()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from e
        _signatures(lib)
        _lib = lib
        _bind_error_word(lib)
    return _lib


_error_word = None      # one int32 in pinned host memory: kernels that give up on a bounded wait write it


def _bind_error_word(lib) -> None:
    """Give the kernels that have bounded waits the address of a pinned host word (a no-op
    without a CUDA device: the library can be built and loaded on a machine that has none)."""
    global _error_word
    if _error_word is not None or not torch.cuda.is_available():
        return
    word = torch.zeros(1, dtype=torch.int32).pin_memory()
    for name in ("mllm_tcgen05_bind_error", "mllm_attention_tcgen05_bind_error", "mllm_attention_decode_bind_error",
                 "mllm_linear_stream_f32_bind_error"):
        if getattr(lib, name)(word.data_ptr()) != 0:
            raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    _error_word = word


_WHO = {1: "the tcgen05 product", 2: "the tcgen05 attention", 3: "the decode attention",
        4: "the float32 weight-streaming product"}


def raise_if_kernel_gave_up() -> None:
    """Costs one read of host memory: call it wherever the host has just waited for the
    stream (after tokens or logits were fetched).  Raises once per event."""
    if _error_word is None:
        return
    code = int(_error_word[0])
    if code:
        _error_word[0] = 0
        raise KernelError(f"{_WHO.get(code // 100, 'a kernel')} gave up on a bounded wait (code {code % 100}): "
                          "the results of the step are not valid")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it: the next kernel's
    blocks may start (and prefetch weights) while the current kernel drains."""
    library().mllm_set_pdl(int(bool(on)))


def is_loaded() -> bool:
    return _lib is not None


launches = 0       # kernels launched through this module (bench.py reports the count)


_timeline = None    # a list while time_launches() is active: (entry point, start event, end event) per launch


def _call(name: str, *args) -> None:
    global launches
    lib = library()
    launches += 1
    if _timeline is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = getattr(lib, name)(*args)
        e1.record()
        _timeline.append((name, e0, e1))
    else:
        rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.mllm_last_error().decode(errors='replace')}")


class time_launches:
    """Times every launch made inside the scope with a pair of CUDA events (eager launches only: nothing can be
    recorded inside a graph capture).  ``rows()`` afterwards gives (entry point, launches, total ms) per entry
    point in order of first use: the per-kernel share of a step, in the manner of the reference's stage timer
    (include/profiling/stage_timer.cuh:40-101), without a device synchronisation per stage."""

    def __enter__(self):
        global _timeline
        self._old, _timeline = _timeline, []
        self._mine = _timeline
        return self

    def __exit__(self, *a):
        global _timeline
        _timeline = self._old

    def rows(self):
        torch.cuda.synchronize()
        agg = {}
        for name, e0, e1 in self._mine:
            n, ms = agg.get(name, (0, 0.0))
            agg[name] = (n + 1, ms + e0.elapsed_time(e1))
        return [(k, n, ms) for k, (n, ms) in agg.items()]


def check_device_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check.  Synchronises and reads
    the kernels' own device words (the thorough check of tests and tools; the engine uses
    raise_if_kernel_gave_up, which costs nothing)."""
    code = c_int(0)
    lib = library()
    torch.cuda.synchronize()
    raise_if_kernel_gave_up()
    if lib.mllm_tcgen05_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        who = {1: "the TMA producer (no free stage)", 2: "the MMA issuer (no full stage)",
               3: "the epilogue (accumulator never ready)"}.get(code.value, "?")
        raise KernelError(f"a tcgen05 kernel gave up waiting: code {code.value}, {who}")
    if lib.mllm_attention_tcgen05_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError(f"the tcgen05 attention kernel gave up waiting: code {code.value} "
                          "(1 producer, 2-6 MMA issuer, 7-8 softmax warps)")
    if lib.mllm_attention_decode_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError("the decode attention kernel gave up waiting for a split's keys and values")
    if lib.mllm_linear_stream_f32_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError("the float32 weight-streaming product gave up waiting for its weights")


_stream_handle = None     # set by stream_scope(); None: ask torch on every call


class stream_scope:
    """Within the scope every launch goes to the stream that is current on entry, without
    asking torch again on each call (a lookup costs more than the launch itself)."""

    def __enter__(self):
        global _stream_handle
        self._old = _stream_handle
        _stream_handle = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *a):
        global _stream_handle
        _stream_handle = self._old


def _stream() -> int:
    return _stream_handle if _stream_handle is not None else torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16")


def _cuda(name: str, t: torch.Tensor, dtype=None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _rows(name: str, t: torch.Tensor):
    """A 2-D tensor whose rows are contiguous; returns its row stride in elements."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


# --------------------------------------------------------------------------- embedding
def embed(ids, positions, table, pos_table, out, copies: int = 1) -> None:
    """out[t] = table[ids[t]] (+ pos_table[positions[t]]), 32-bit; with ``copies`` > 1 a row of out holds that many
    copies of the token's row side by side (a residual of several streams at its start)."""
    _cuda("ids", ids, torch.int32)
    _cuda("table", table)
    _cuda("out", out, torch.float32)
    T, D = out.shape
    if copies < 1 or D % copies:
        raise KernelError(f"embed: {copies} copies in rows of {D}")
    D //= copies
    if ids.numel() != T or table.shape[1] != D:
        raise KernelError(f"embed: {ids.numel()} ids, table {tuple(table.shape)}, out {tuple(out.shape)}")
    pp = None
    if pos_table is not None:
        _cuda("positions", positions, torch.int32)
        _cuda("pos_table", pos_table, table.dtype)
        if pos_table.shape[1] != D or positions.numel() != T:
            raise KernelError("embed: position table or positions do not fit")
        pp = pos_table.data_ptr()
    _call("mllm_embed", ids.data_ptr(), positions.data_ptr() if pos_table is not None else None,
          table.data_ptr(), pp, out.data_ptr(), T, D, int(copies), _dt(table), _stream())


def resolve_tokens(ids, sampled) -> None:
    """In place: ids[t] = sampled[-ids[t] - 1] wherever ids[t] is negative (a token that the
    last sampling launch left on the device and the host has not read yet)."""
    _cuda("ids", ids, torch.int32)
    _cuda("sampled", sampled, torch.int32)
    _call("mllm_resolve_tokens", ids.data_ptr(), ids.numel(), sampled.data_ptr(), sampled.numel(), _stream())


# --------------------------------------------------------------------------- norm
def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[r] = LayerNorm(x[rows[r]] or x[r]); x 32-bit, out 32-bit or bfloat16."""
    _cuda("x", x, torch.float32)
    _cuda("gamma", gamma, torch.float32)
    _cuda("beta", beta, torch.float32)
    _cuda("out", out)
    D = x.shape[1]
    R = out.shape[0]
    if gamma.numel() != D or beta.numel() != D or out.shape[1] != D:
        raise KernelError(f"layernorm: width {D} against gamma {gamma.numel()}, out {tuple(out.shape)}")
    if rows is not None:
        _cuda("rows", rows, torch.int32)
        if rows.numel() != R:
            raise KernelError("layernorm: rows and out differ in length")
    elif x.shape[0] != R:
        raise KernelError("layernorm: x and out differ in rows")
    _call("mllm_layernorm", x.data_ptr(), rows.data_ptr() if rows is not None else None, gamma.data_ptr(),
          beta.data_ptr(), out.data_ptr(), R, D, float(eps), _dt(out), _stream())


def rmsnorm(x, weight, eps: float, out, rows=None, unit_offset: bool = True, weight2=None, out2=None, heads: int = 1,
            scale: float = 1.0) -> None:
    """out[r] = scale * x[r] / sqrt(mean(x[r]^2) + eps) * (weight + 1) (or * weight when ``unit_offset`` is False);
    x 32-bit, out 32-bit or bfloat16 (rows contiguous: a column slice of a wider buffer is fine).  ``weight2`` /
    ``out2``: a second norm of the same rows with other weights, from the same sum of squares.  ``heads`` > 1: a row
    is that many vectors side by side, each normed on its own with the same weights."""
    _cuda("x", x, torch.float32, contiguous=False)
    _cuda("weight", weight, torch.float32)
    _cuda("out", out, contiguous=False)
    ldx = _rows("x", x)
    ldo = _rows("out", out)
    D = x.shape[1] // heads
    R = out.shape[0]
    if weight.numel() != D or out.shape[1] != D * heads or x.shape[1] != D * heads:
        raise KernelError(f"rmsnorm: width {D} x {heads} against weight {weight.numel()}, out {tuple(out.shape)}")
    if (weight2 is None) != (out2 is None):
        raise KernelError("rmsnorm: the second weight and the second output come together")
    if weight2 is not None:
        _cuda("weight2", weight2, torch.float32)
        _cuda("out2", out2, out.dtype, contiguous=False)
        if weight2.numel() != D or tuple(out2.shape) != tuple(out.shape) or _rows("out2", out2) != ldo:
            raise KernelError("rmsnorm: the second weight or output does not fit the first")
    if rows is not None:
        _cuda("rows", rows, torch.int32)
        if rows.numel() != R:
            raise KernelError("rmsnorm: rows and out differ in length")
    elif x.shape[0] != R:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call("mllm_rmsnorm", x.data_ptr(), ldx, rows.data_ptr() if rows is not None else None, weight.data_ptr(),
          weight2.data_ptr() if weight2 is not None else None, out.data_ptr(),
          out2.data_ptr() if out2 is not None else None, ldo, int(heads), R, D, float(eps), 1.0 if unit_offset else 0.0,
          float(scale), _dt(out), _stream())


def gated_act(gu, out, act: str, limit: float = 0.0, alpha: float = 1.0) -> None:
    """out[t, c] = act(gu[t, c]) * gu[t, F + c] for gu [T, 2F]: the gate and the up half of one product.
    ``act`` "swiglu_clamp": with g the gate cut off above ``limit`` and u the up value cut off at +-``limit``,
    out = g * sigmoid(alpha * g) * (u + 1)."""
    _cuda("gu", gu, contiguous=False)
    _cuda("out", out, gu.dtype, contiguous=False)
    T, F = out.shape
    if tuple(gu.shape) != (T, 2 * F):
        raise KernelError(f"gated_act: gu {tuple(gu.shape)} against out {tuple(out.shape)}")
    if act not in _GATE_ACT:
        raise KernelError(f"gated_act: unknown activation {act!r}; known: {sorted(_GATE_ACT)}")
    if act == "swiglu_clamp" and not limit > 0:
        raise KernelError("gated_act: the clamped form needs a positive limit")
    _call("mllm_gated_act", gu.data_ptr(), _rows("gu", gu), out.data_ptr(), _rows("out", out), T, F, _GATE_ACT[act],
          float(limit), float(alpha), _dt(gu), _stream())


# --------------------------------------------------------------------------- linear
class NormedInput:
    """LayerNorm(x[rows]) not yet computed: a product that can fuse the norm into its
    loads takes it as it is, anything else calls ``materialize()``.  ``rms``: the norm
    without centring, x / sqrt(mean(x^2) + eps) * gamma (+ beta, which is then zeros);
    ``buf``: the workspace buffer a materialised result goes to."""

    def __init__(self, x, gamma, beta, eps, rows, ws, dtype, rms: bool = False, buf: str = "norm_out"):
        self.x, self.gamma, self.beta, self.eps, self.rows, self.ws, self.dtype = x, gamma, beta, eps, rows, ws, dtype
        self.rms, self.buf = bool(rms), buf
        self.shape = (x.shape[0] if rows is None else rows.shape[0], x.shape[1])
        self._out = None

    @property
    def kernel_eps(self) -> float:
        """eps as the fused products take it: negative for the norm without centring."""
        return -float(self.eps) if self.rms else float(self.eps)

    def materialize(self):
        if self._out is None:
            out = self.ws.buf(self.buf, self.shape[0], self.shape[1], self.dtype)
            if self.rms:
                rmsnorm(self.x, self.gamma, self.eps, out, rows=self.rows, unit_offset=False)
            else:
                layernorm(self.x, self.gamma, self.beta, self.eps, out, rows=self.rows)
            self._out = out
        return self._out


def decode_splits(max_ctx_len: int) -> int:
    """Key splits the decode attention is launched with: just enough for the longest context
    (launching more costs: the splits of a request form a cluster that is scheduled as a whole)."""
    return max(1, -(-int(max_ctx_len) // DECODE_SPLIT))


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sm_count


def _small_m_wins(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming kernel (mma.sync, 16 weight rows per CTA, K split over its warps) beats the
    tensor-memory kernel for M rows of bfloat16.  Measured in replayed graphs at the shapes of GPT-2 small, medium
    and XL (N = D, 3D, 4D and K = D, 4D for D = 768, 1024, 1600, and the 50,257-row head): up to 16 rows the
    streaming kernel needs one pass of its token tiles and wins everywhere (2.3-12 us against 6-27 us), except
    that a matrix as tall as a vocabulary is streamed faster by the tensor-memory kernel from 9 rows on; from 17
    to 32 rows it makes two passes and still wins while its N/16 CTAs fit the SMs in one wave (N <= 2368 on 148
    SMs: 4.4 against 5.7 us at N = 2304, 8.1 against 5.8 us at N = 3072); beyond 32 rows it loses everywhere (it
    reads its input rows from L2 again and again while the other stays near its fixed cost)."""
    if M <= 8:
        return True
    if N >= 16384:
        return False
    if M <= 16:
        return True
    if M <= 32:
        return -(-N // 16) <= sm_count()
    return False


def _fusable(weight, M, K) -> bool:
    return weight.dtype == torch.bfloat16 and M <= SMALL_M and K % 8 == 0 and weight.data_ptr() % 16 == 0


NORM_FUSE_M = 16             # rows up to which the norm is recomputed inside every CTA of the product


def _norm_ok(n: NormedInput) -> bool:
    x = n.x
    return (n.shape[0] <= NORM_FUSE_M and x.dtype == torch.float32 and x.stride(1) == 1 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0
            and n.gamma.data_ptr() % 16 == 0 and n.beta.data_ptr() % 16 == 0)


def _linear_fused(x, weight, bias, out, act, accumulate, norm: Optional[NormedInput], kv) -> None:
    """The small-M product with the norm fused on its input and/or the cache write on its output."""
    M = norm.shape[0] if norm is not None else x.shape[0]
    N, K = weight.shape
    ldo = _rows("out", out)
    if norm is not None:
        xp, ldx = None, norm.x.stride(0)
        nargs = (norm.x.data_ptr(), norm.rows.data_ptr() if norm.rows is not None else None,
                 norm.gamma.data_ptr(), norm.beta.data_ptr(), norm.kernel_eps)
    else:
        xp, ldx = x.data_ptr(), _rows("x", x)
        nargs = (None, None, None, None, 0.0)
    if kv is not None:
        k_pages, v_pages, slots, q_size = kv
        _, Hkv, ps, dh = k_pages.shape
        kargs = (k_pages.data_ptr(), v_pages.data_ptr(), slots.data_ptr(), int(q_size), Hkv, dh, ps)
    else:
        kargs = (None, None, None, 0, 0, 0, 0)
    _call("mllm_linear_smallm_fused", xp, ldx, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), _dt(out), *nargs, *kargs, _stream())


STREAM_F32_MAX_K = 12288      # the longest rows whose tiles fit the streaming product's shared memory in every case


def _stream_f32_ok(weight, M, K) -> bool:
    return (weight.dtype == torch.float32 and M <= SMALL_M_F32 and K % 4 == 0 and K <= STREAM_F32_MAX_K
            and weight.data_ptr() % 16 == 0)


def _norm_ok_f32(n: NormedInput) -> bool:
    x = n.x
    return (n.shape[0] <= NORM_FUSE_M_F32 and n.shape[1] <= 2048 and x.dtype == torch.float32 and x.stride(1) == 1
            and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and n.gamma.data_ptr() % 16 == 0
            and n.beta.data_ptr() % 16 == 0)


def _linear_stream_f32(x, weight, bias, out, act, accumulate, norm: Optional[NormedInput], kv) -> None:
    """The float32 weight-streaming product, with the norm fused on its input and/or the cache write on its output."""
    M = norm.shape[0] if norm is not None else x.shape[0]
    N, K = weight.shape
    ldo = _rows("out", out)
    if norm is not None:
        xp, ldx = None, norm.x.stride(0)
        nargs = (norm.x.data_ptr(), norm.rows.data_ptr() if norm.rows is not None else None,
                 norm.gamma.data_ptr(), norm.beta.data_ptr(), norm.kernel_eps)
    else:
        xp, ldx = x.data_ptr(), _rows("x", x)
        nargs = (None, None, None, None, 0.0)
    if kv is not None:
        k_pages, v_pages, slots, q_size = kv
        _, Hkv, ps, dh = k_pages.shape
        kargs = (k_pages.data_ptr(), v_pages.data_ptr(), slots.data_ptr(), int(q_size), Hkv, dh, ps)
    else:
        kargs = (None, None, None, 0, 0, 0, 0)
    _call("mllm_linear_stream_f32", xp, ldx, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), *nargs, *kargs, _stream())


def linear_qkv_cache(x, weight, bias, q_out, k_pages, v_pages, slot_mapping, ws):
    """Q|K|V projection whose keys and values go to their page slots; returns the queries.

    weight [q_size + 2*kv_heads*head_dim, K]; q_out [M, q_size] is where the queries may be
    put.  The cache write rides in the product's epilogue - the weight-streaming kernel's with few
    rows (which also takes a NormedInput's norm into its loads), the tensor-memory kernel's with
    many - and q_out is returned; where neither applies (32-bit, head sizes that are no multiple
    of 32) the product writes a [M, N] buffer, kv_write copies keys and values from it, and the
    buffer's query columns are returned.
    """
    M = x.shape[0]
    N, K = weight.shape
    q_size = q_out.shape[1]
    _, Hkv, ps, dh = k_pages.shape
    if N != q_size + 2 * Hkv * dh:
        raise KernelError(f"linear_qkv_cache: {N} output columns against {q_size} + 2*{Hkv}*{dh}")
    _cuda("q_out", q_out, contiguous=False)
    _cuda("k_pages", k_pages, q_out.dtype)
    _cuda("v_pages", v_pages, q_out.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    if slot_mapping.numel() != M or q_out.shape[0] != M or v_pages.shape != k_pages.shape:
        raise KernelError(f"linear_qkv_cache: {M} rows, {slot_mapping.numel()} slots, q_out {tuple(q_out.shape)}")
    norm = x if isinstance(x, NormedInput) else None
    if q_out.dtype == torch.float32 and _stream_f32_ok(weight, M, K) and q_out.stride(1) == 1 \
            and k_pages.is_contiguous() and v_pages.is_contiguous():
        # float32, few rows: the weight-streaming product writes keys and values from its epilogue
        if norm is not None and not _norm_ok_f32(norm):
            x, norm = norm.materialize(), None
        if norm is not None or (x.is_cuda and x.dtype == torch.float32 and _rows("x", x) % 4 == 0 and x.data_ptr() % 16 == 0):
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            _linear_stream_f32(None if norm is not None else x, weight, bias, q_out, None, False, norm,
                               (k_pages, v_pages, slot_mapping, q_size))
            return q_out
    if norm is not None and not _norm_ok(norm):
        x, norm = norm.materialize(), None
    if q_out.dtype == torch.bfloat16 and _fusable(weight, M, K) and _small_m_wins(M, N, K) and (
            _norm_ok(norm) if norm is not None else
            (x.is_cuda and x.dtype == torch.bfloat16 and _rows("x", x) % 8 == 0 and x.data_ptr() % 16 == 0)):
        if bias is not None:
            _cuda("bias", bias, torch.float32)
        _linear_fused(None if norm is not None else x, weight, bias, q_out, None, False, norm,
                      (k_pages, v_pages, slot_mapping, q_size))
        return q_out
    if norm is not None:
        x, norm = norm.materialize(), None
    _cuda("x", x, contiguous=False)
    if (q_out.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and not _small_m_wins(M, N, K) and q_size % 32 == 0 and dh % 32 == 0 and K % 8 == 0
            and _rows("x", x) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and _rows("q_out", q_out) % 8 == 0 and q_out.data_ptr() % 16 == 0 and k_pages.is_contiguous()
            and v_pages.is_contiguous()):
        # many rows: the tensor-memory product, whose epilogue stores keys and values into their pages
        if bias is not None:
            _cuda("bias", bias, torch.float32)
        _call("mllm_linear_tcgen05_qkv", x.data_ptr(), _rows("x", x), weight.data_ptr(),
              bias.data_ptr() if bias is not None else None, q_out.data_ptr(), _rows("q_out", q_out), M, N, K,
              k_pages.data_ptr(), v_pages.data_ptr(), slot_mapping.data_ptr(), q_size, Hkv, dh, ps, _stream())
        return q_out
    qkv = ws.buf("qkv", M, N, q_out.dtype)
    linear(x, weight, bias, out=qkv)
    kv_write(qkv[:, q_size:q_size + Hkv * dh], qkv[:, q_size + Hkv * dh:], k_pages, v_pages, slot_mapping)
    return qkv[:, :q_size]


def linear(x, weight, bias, out, act: Optional[str] = None, accumulate: bool = False, impl: Optional[str] = None):
    """out = act(x @ weight^T + bias) (+ out when ``accumulate``).

    x [M,K] rows contiguous (a column slice is fine) or a NormedInput, weight [N,K]
    contiguous, bias [N] 32-bit or None, out [M,N] rows contiguous.  float32 operands run
    the true 32-bit FMA kernel; bfloat16 operands accumulate in 32-bit.
    """
    if isinstance(x, NormedInput):
        if impl in (None, "smallm") and _fusable(weight, x.shape[0], weight.shape[1]) and _norm_ok(x) \
                and (impl == "smallm" or _small_m_wins(x.shape[0], weight.shape[0], weight.shape[1])) \
                and x.shape[1] == weight.shape[1] and tuple(out.shape) == (x.shape[0], weight.shape[0]):
            _cuda("out", out, contiguous=False)
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            if act not in _ACT:
                raise KernelError(f"linear: unknown activation {act!r}")
            _linear_fused(None, weight, bias, out, act, accumulate, x, None)
            return out
        if impl in (None, "stream_f32") and _stream_f32_ok(weight, x.shape[0], weight.shape[1]) and _norm_ok_f32(x) \
                and out.dtype == torch.float32 and x.shape[1] == weight.shape[1] \
                and tuple(out.shape) == (x.shape[0], weight.shape[0]):
            _cuda("out", out, contiguous=False)
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            if act not in _ACT:
                raise KernelError(f"linear: unknown activation {act!r}")
            _linear_stream_f32(None, weight, bias, out, act, accumulate, x, None)
            return out
        x = x.materialize()
    _cuda("x", x, contiguous=False)
    _cuda("weight", weight, x.dtype)
    _cuda("out", out, contiguous=False)
    lda = _rows("x", x)
    ldo = _rows("out", out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"linear: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _cuda("bias", bias, torch.float32)
        if bias.numel() != N:
            raise KernelError("linear: bias length")
    if act not in _ACT:
        raise KernelError(f"linear: unknown activation {act!r}")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 operands need a float32 result")
    if impl is None:
        impl = "simt"
        if x.dtype == torch.bfloat16 and K % 8 == 0 and lda % 8 == 0 \
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
            impl = "smallm" if _small_m_wins(M, N, K) else "tcgen05"
        elif x.dtype == torch.float32 and out.dtype == torch.float32 and _stream_f32_ok(weight, M, K) \
                and lda % 4 == 0 and x.data_ptr() % 16 == 0:
            impl = "stream_f32"
    if impl == "stream_f32":
        _linear_stream_f32(x, weight, bias, out, act, accumulate, None, None)
        return out
    if impl in ("smallm", "tcgen05"):
        _call("mllm_linear_" + impl, x.data_ptr(), lda, weight.data_ptr(),
              bias.data_ptr() if bias is not None else None, out.data_ptr(), ldo, M, N, K, _ACT[act],
              int(accumulate), _dt(out), _stream())
        return out
    if impl != "simt":
        raise KernelError(f"linear: unknown implementation {impl!r}")
    ws_ptr, ws_floats = None, 0
    if x.dtype == torch.float32 and M > 128:
        # many rows in 32-bit: a narrow result is computed in K slices whose partial sums need room
        splits = library().mllm_linear_simt_splits(N, K)
        if splits > 1:
            ws = _scratch("simt_splitk", x.device, splits * M * N)
            ws_ptr, ws_floats = ws.data_ptr(), ws.numel()
    _call("mllm_linear_simt", x.data_ptr(), lda, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), _dt(x), _dt(out), ws_ptr, ws_floats, _stream())
    if ws_ptr is not None:
        global launches
        launches += 1           # the finishing kernel that adds the slices
    return out


_scratch_bufs = {}


def _scratch(name: str, device, floats: int) -> torch.Tensor:
    """A float32 scratch buffer of this module that only grows (a step shape runs eagerly before it is captured as a
    graph, so a captured graph never sees the buffer replaced under it unless a larger shape comes later: sizes are
    rounded up to the next power of two to make that rare, and the runner drops its graphs when it happens)."""
    global scratch_version
    key = (name, str(device))
    buf = _scratch_bufs.get(key)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(1 << (int(floats) - 1).bit_length(), 1 << 20), dtype=torch.float32, device=device)
        _scratch_bufs[key] = buf
        scratch_version += 1
    return buf


scratch_version = 0     # bumped whenever a scratch buffer of this module is replaced


# --------------------------------------------------------------------------- cache
def kv_write(k, v, k_pages, v_pages, slot_mapping) -> None:
    """Copy rows of k and v ([T, kv_heads*head_dim], same row stride) to their slots."""
    _cuda("k", k, contiguous=False)
    _cuda("v", v, k.dtype, contiguous=False)
    _cuda("k_pages", k_pages, k.dtype)
    _cuda("v_pages", v_pages, k.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    ld = _rows("k", k)
    if _rows("v", v) != ld:
        raise KernelError("kv_write: k and v differ in row stride")
    _, Hkv, ps, dh = k_pages.shape
    T = k.shape[0]
    if k.shape[1] != Hkv * dh or slot_mapping.numel() != T or v_pages.shape != k_pages.shape:
        raise KernelError("kv_write: shapes do not fit the pages")
    _call("mllm_kv_write", k.data_ptr(), v.data_ptr(), ld, k_pages.data_ptr(), v_pages.data_ptr(),
          slot_mapping.data_ptr(), T, Hkv, dh, ps, _dt(k), _stream())


def paged_write(src, pages, slot_mapping) -> None:
    """Rows of src [T, heads * d] (rows contiguous) to their slots in pages [num_pages, heads, page_size, d]."""
    _cuda("src", src, contiguous=False)
    _cuda("pages", pages, src.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    _, heads, ps, d = pages.shape
    T = src.shape[0]
    if src.shape[1] != heads * d or slot_mapping.numel() != T:
        raise KernelError(f"paged_write: src {tuple(src.shape)} against pages {tuple(pages.shape)}")
    _call("mllm_paged_write", src.data_ptr(), _rows("src", src), pages.data_ptr(), slot_mapping.data_ptr(), T, heads, d,
          ps, _dt(src), _stream())


def paged_write_kv(k, v, k_pages, v_pages, slot_mapping) -> None:
    """Keys k [T, heads * dk] and values v [T, heads * dv] (rows contiguous) to their slots in k_pages
    [num_pages, heads, page_size, dkp] and v_pages [num_pages, heads, page_size, dv], in one launch.  dkp >= dk:
    key rows of the pages may be padded (the padding is never written and stays zero)."""
    _cuda("k", k, contiguous=False)
    _cuda("v", v, k.dtype, contiguous=False)
    _cuda("k_pages", k_pages, k.dtype)
    _cuda("v_pages", v_pages, k.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    _, heads, ps, dkp = k_pages.shape
    dv = v_pages.shape[3]
    T = k.shape[0]
    dk = k.shape[1] // heads
    if k.shape[1] != heads * dk or dk > dkp or tuple(v.shape) != (T, heads * dv) or slot_mapping.numel() != T \
            or v_pages.shape[:3] != k_pages.shape[:3]:
        raise KernelError(f"paged_write_kv: k {tuple(k.shape)}, v {tuple(v.shape)} against pages {tuple(k_pages.shape)}, "
                          f"{tuple(v_pages.shape)}")
    _call("mllm_paged_write_kv", k.data_ptr(), _rows("k", k), v.data_ptr(), _rows("v", v), k_pages.data_ptr(),
          v_pages.data_ptr(), slot_mapping.data_ptr(), T, heads, dk, dkp, dv, ps, _dt(k), _stream())


BIAS_ATTN_MMA_MAX_DIM = 128    # largest key and value size of its tensor-core kernel


def _bias_mma_ok(q, k_pages, v_pages, out, dk, dv, ldq, ldo) -> bool:
    return (q.dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and dk <= BIAS_ATTN_MMA_MAX_DIM
            and dv <= BIAS_ATTN_MMA_MAX_DIM and ldq % 8 == 0 and q.data_ptr() % 16 == 0 and ldo % 2 == 0
            and out.data_ptr() % 4 == 0 and k_pages.data_ptr() % 16 == 0 and v_pages.data_ptr() % 16 == 0)


BIAS_ATTN_MAX_DIM = 256        # largest key and value size of csrc/attention_bias.cu
_bias_split_keys = None


def biased_attention(q, k_pages, v_pages, block_table, ctx, out, *, num_heads, num_kv_heads, scale, dist_bias=None,
                     q_scale=None, out_scale: float = 1.0, window=None, chunk=None, sink=None, softcap: float = 0.0,
                     slopes=None, impl: Optional[str] = None) -> None:
    """Causal attention over the cache with keys and values of different sizes, an additive score bias
    ``dist_bias[head, i - j]`` (float32 [heads, n]) and a factor ``q_scale[position]`` (float32 [n]) on the query:
    out[t] = out_scale * softmax_j((q_t . k_j) * scale * q_scale[p_t] + dist_bias[h, p_t - j]) v_j.
    ``window``: only the last ``window`` keys are seen; ``chunk``: only keys from floor(p_t / chunk) * chunk on (block b is
    positions [b * chunk, (b + 1) * chunk) of the request); ``sink`` (float32 [heads]): exp(sink[h]) is one more
    term of the softmax's denominator and of nothing else.  ``softcap`` c > 0: the scaled product s becomes
    c * tanh(s / c) before any bias is added; ``slopes`` (float32 [heads]): slopes[h] * (p_t - j) is taken off the score.

    q [T, heads * dkq], k_pages [P, kv_heads, page_size, dk] with dk >= dkq a multiple of 8 (key rows padded with
    zeros), v_pages [P, kv_heads, page_size, dv], out [T, heads * dv] (rows contiguous; a column slice of a wider
    buffer is fine).
    """
    global _bias_split_keys
    _cuda("q", q, contiguous=False)
    _cuda("k_pages", k_pages, q.dtype)
    _cuda("v_pages", v_pages, q.dtype)
    _cuda("out", out, q.dtype, contiguous=False)
    _cuda("block_table", block_table, torch.int32, contiguous=False)
    T = q.shape[0]
    _, Hkv, ps, dk = k_pages.shape
    dv = v_pages.shape[3]
    dkq = q.shape[1] // num_heads
    if Hkv != num_kv_heads or q.shape[1] != num_heads * dkq or not (0 < dkq <= dk) or tuple(out.shape) != (T, num_heads * dv) \
            or v_pages.shape[:3] != k_pages.shape[:3]:
        raise KernelError("biased_attention: head counts or sizes do not fit the pages")
    ldq, ldo = _rows("q", q), _rows("out", out)
    if dk % 8 != 0 or dk > BIAS_ATTN_MAX_DIM or dv > BIAS_ATTN_MAX_DIM:
        raise KernelError(f"biased_attention: key rows of {dk} must be a multiple of 8, and key and value rows at most "
                          f"{BIAS_ATTN_MAX_DIM}")
    n_dist = 0
    if dist_bias is not None:
        _cuda("dist_bias", dist_bias, torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[0] != num_heads:
            raise KernelError("biased_attention: dist_bias must be [heads, distances]")
        n_dist = dist_bias.shape[1]
        if ctx.max_ctx_len > n_dist:
            raise KernelError(f"biased_attention: a context of {ctx.max_ctx_len} tokens exceeds the bias table's {n_dist} distances")
    if q_scale is not None:
        _cuda("q_scale", q_scale, torch.float32)
        if ctx.max_ctx_len > q_scale.numel():
            raise KernelError("biased_attention: a position exceeds the query-scale table")
    if sink is not None:
        _cuda("sink", sink, torch.float32)
        if sink.numel() != num_heads:
            raise KernelError("biased_attention: one sink per query head")
    if slopes is not None:
        _cuda("slopes", slopes, torch.float32)
        if slopes.numel() != num_heads:
            raise KernelError("biased_attention: one slope per query head")
    if impl is None:
        impl = "simt"
        if getattr(ctx, "decode_only", False):
            impl = "split"
        elif getattr(ctx, "n_tiles", 0) > 0:
            impl = "tiled"
            if dkq == dk and _bias_mma_ok(q, k_pages, v_pages, out, dk, dv, ldq, ldo):
                impl = "mma"       # prompt portions in bfloat16: tensor cores
    attention_launches["bias_" + impl] = attention_launches.get("bias_" + impl, 0) + 1
    part_o = part_ml = None
    nsplit = 0
    tiles, n_tiles = None, 0
    if impl == "split":
        if _bias_split_keys is None:
            _bias_split_keys = int(library().mllm_attention_bias_split_keys())
        # splits cover the longest context of the step, rounded up to a power of two so that captured graphs keep their grid
        need = max(1, -(-int(ctx.max_ctx_len) // _bias_split_keys))
        nsplit = 1 << (need - 1).bit_length()
        part_o = ctx.ws.buf("battn_part_o", T * num_heads * nsplit, dv, torch.float32).data_ptr()
        part_ml = ctx.ws.buf("battn_part_ml", T * num_heads * nsplit, 2, torch.float32).data_ptr()
    elif impl in ("tiled", "mma"):
        tiles, n_tiles = ctx.attn_tiles.data_ptr(), int(ctx.n_tiles)
        if impl == "mma" and not (dkq == dk and _bias_mma_ok(q, k_pages, v_pages, out, dk, dv, ldq, ldo)):
            raise KernelError("biased_attention: the tensor-core kernel takes bfloat16, key and value sizes that are "
                              f"multiples of 16 up to {BIAS_ATTN_MMA_MAX_DIM} and 16-byte aligned rows")
    elif impl != "simt":
        raise KernelError(f"biased_attention: unknown implementation {impl!r}")
    _call("mllm_attention_bias", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
          _rows("block_table", block_table), ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), tiles, n_tiles,
          out.data_ptr(), ldo, part_o, part_ml, nsplit, T, num_heads, num_kv_heads, dkq, dk, dv, ps, float(scale),
          float(out_scale), dist_bias.data_ptr() if dist_bias is not None else None, n_dist,
          q_scale.data_ptr() if q_scale is not None else None, int(window or 0), int(chunk or 0),
          sink.data_ptr() if sink is not None else None, float(softcap or 0.0),
          slopes.data_ptr() if slopes is not None else None, _dt(q), {"simt": 0, "tiled": 1, "split": 2, "mma": 3}[impl],
          _stream())
    if impl == "split":
        global launches
        launches += 1           # the kernel that merges the splits



# --------------------------------------------------------------------------- normed and rotated queries and keys
def qk_norm_rope(proj, q_off: int, k_off: int, v_off: int, ctx, q_out, k_pages, v_pages, slot_mapping, *, heads: int,
                 kv_heads: int, head_dim: int, v_head_dim: int, q_norm=None, k_norm=None, eps: float = 0.0, freq=None,
                 rot_dims: int = 0, interleaved: bool = True, head_norm: bool = False, v_first=None, v_lambda=None,
                 v_keep=None) -> None:
    """What stands between a Q | K | V projection and attention when queries and keys are normed and rotated.

    proj [T, .] holds a token's queries at column q_off (heads * head_dim), keys at k_off (kv_heads * head_dim) and
    values at v_off (kv_heads * v_head_dim).  ``q_norm`` / ``k_norm`` (float32, one weight per column of the WHOLE
    projection, or None): x / sqrt(mean(x^2) + eps) * w over all heads of the token at once.  Then the first
    ``rot_dims`` entries of every head turn by position * freq[i] (float32 [rot_dims / 2]); ``interleaved``: entry 2i
    pairs with 2i + 1, else i with i + rot_dims / 2.  Queries go to q_out [T, heads * head_dim]; keys (rows of the
    pages may be padded) and values go to the tokens' slots (``slot_mapping`` None: nothing is cached).  All 32-bit
    up to the final rounding.  ``head_norm`` (instead of q_norm / k_norm): after the rotation every query head and every
    key head is divided by its own root mean square (eps inside the root, no weights).  ``v_first`` [T, kv_heads *
    v_head_dim] with ``v_lambda`` (a float32 scalar on the device): the values become (1 - lambda) v + lambda v_first
    before they are cached; ``v_keep`` [T, kv_heads * v_head_dim] gets the values as they are cached."""
    _cuda("proj", proj, contiguous=False)
    _cuda("q_out", q_out, proj.dtype, contiguous=False)
    T = proj.shape[0]
    ld = _rows("proj", proj)
    nq, nk, nv = heads * head_dim, kv_heads * head_dim, kv_heads * v_head_dim
    if max(q_off + nq, k_off + nk, v_off + nv) > proj.shape[1] or tuple(q_out.shape) != (T, nq):
        raise KernelError(f"qk_norm_rope: proj {tuple(proj.shape)} against {nq} + {nk} + {nv} columns, q_out {tuple(q_out.shape)}")
    for name, w, n in (("q_norm", q_norm, nq), ("k_norm", k_norm, nk)):
        if w is not None:
            _cuda(name, w, torch.float32)
            if w.numel() != n:
                raise KernelError(f"qk_norm_rope: {name} has {w.numel()} weights for {n} columns")
    if rot_dims:
        _cuda("freq", freq, torch.float32)
        if rot_dims % 2 or rot_dims > head_dim or freq.numel() != rot_dims // 2:
            raise KernelError(f"qk_norm_rope: {rot_dims} rotated entries of {head_dim}, {freq.numel()} frequencies")
    if head_norm and (q_norm is not None or k_norm is not None):
        raise KernelError("qk_norm_rope: the per-head norm takes no weights")
    for name, t in (("v_first", v_first), ("v_keep", v_keep)):
        if t is not None:
            _cuda(name, t, proj.dtype, contiguous=False)
            if tuple(t.shape) != (T, nv):
                raise KernelError(f"qk_norm_rope: {name} {tuple(t.shape)} against {nv} value columns")
    if v_first is not None:
        _cuda("v_lambda", v_lambda, torch.float32)
        if v_lambda.numel() != 1:
            raise KernelError("qk_norm_rope: v_lambda is one number")
    dkp, ps = head_dim, 1
    if slot_mapping is not None:
        _cuda("k_pages", k_pages, proj.dtype)
        _cuda("v_pages", v_pages, proj.dtype)
        _cuda("slot_mapping", slot_mapping, torch.int32)
        _, G, ps, dkp = k_pages.shape
        if G != kv_heads or dkp < head_dim or v_pages.shape[3] != v_head_dim or v_pages.shape[:3] != k_pages.shape[:3] \
                or slot_mapping.numel() != T:
            raise KernelError(f"qk_norm_rope: pages {tuple(k_pages.shape)}, {tuple(v_pages.shape)} do not fit")
    _call("mllm_qk_norm_rope", proj.data_ptr(), ld, int(q_off), int(k_off), int(v_off), int(heads), int(kv_heads),
          int(head_dim), int(v_head_dim), q_norm.data_ptr() if q_norm is not None else None,
          k_norm.data_ptr() if k_norm is not None else None, float(eps), freq.data_ptr() if rot_dims else None,
          int(rot_dims), int(bool(interleaved)), ctx.positions.data_ptr(), q_out.data_ptr(), _rows("q_out", q_out),
          k_pages.data_ptr() if slot_mapping is not None else None, v_pages.data_ptr() if slot_mapping is not None else None,
          int(dkp), slot_mapping.data_ptr() if slot_mapping is not None else None, int(ps), int(bool(head_norm)),
          v_first.data_ptr() if v_first is not None else None, _rows("v_first", v_first) if v_first is not None else 0,
          v_lambda.data_ptr() if v_first is not None else None, v_keep.data_ptr() if v_keep is not None else None,
          _rows("v_keep", v_keep) if v_keep is not None else 0, T, _dt(proj), _stream())


# --------------------------------------------------------------------------- a residual of several streams
HYPER_MAX_STREAMS = 8


def hyper_step(x, streams: int, *, y=None, mix=None, out_weights=None, in_weights=None, gamma=None, beta=None, eps: float = 0.0,
               rows=None, h=None, sum_out=None, pairs=None) -> None:
    """One pass over a residual of ``streams`` streams, x [T, streams * D] (32-bit, changed in place).

    With ``y`` [T, D] (32-bit; the result of the sublayer that has just run), ``mix`` [streams, streams] ([from, to])
    and ``out_weights`` [streams]: x_t <- sum_s mix[s, t] x_s + out_weights[t] * y, all streams at once from the old
    ones.  ``pairs`` = (results [T * top, D], weights [T, top], top), all 32-bit: the result written is y (if given) plus
    the weighted sum over the token's ``top`` chosen experts in the order of the choices, which a routed feed-forward
    leaves to this pass.  With ``h`` [R, D] (activation dtype) and ``gamma``: h = norm(sum_s in_weights[s] x_s) of the new streams
    (``in_weights`` None: the plain sum); LayerNorm with ``beta``, an RMS norm without.  ``sum_out`` [R, D] (32-bit)
    gets the read before its norm.  ``rows`` (int32 [R]) gathers the tokens that are read; a write then takes place for
    those tokens only, on the way to the read, and x is left as it was (a step's last write, when only the wanted tokens'
    sum is read afterwards)."""
    _cuda("x", x, torch.float32)
    T = x.shape[0]
    if streams < 1 or streams > HYPER_MAX_STREAMS or x.shape[1] % streams:
        raise KernelError(f"hyper_step: {streams} streams (at most {HYPER_MAX_STREAMS}) in rows of {x.shape[1]}")
    D = x.shape[1] // streams
    R = T if rows is None else rows.numel()
    writes = y is not None or pairs is not None
    if y is not None:
        _cuda("y", y, torch.float32, contiguous=False)
        if tuple(y.shape) != (T, D):
            raise KernelError("hyper_step: y does not fit the streams")
    pair_out = pair_w = None
    top = 0
    if pairs is not None:
        pair_out, pair_w, top = pairs
        _cuda("pairs", pair_out, torch.float32)
        _cuda("pair weights", pair_w, torch.float32)
        if top < 1 or tuple(pair_out.shape) != (T * top, D) or pair_w.numel() != T * top:
            raise KernelError("hyper_step: the experts' results or weights do not fit")
    if writes:
        _cuda("mix", mix, torch.float32)
        _cuda("out_weights", out_weights, torch.float32)
        if mix.numel() != streams * streams or out_weights.numel() != streams:
            raise KernelError("hyper_step: mix or out_weights do not fit the streams")
    if rows is not None:
        _cuda("rows", rows, torch.int32)
    if in_weights is not None:
        _cuda("in_weights", in_weights, torch.float32)
        if in_weights.numel() != streams:
            raise KernelError("hyper_step: one read weight per stream")
    dt = F32
    if h is not None:
        _cuda("h", h, contiguous=False)
        _cuda("gamma", gamma, torch.float32)
        if tuple(h.shape) != (R, D) or gamma.numel() != D or (beta is not None and beta.numel() != D):
            raise KernelError(f"hyper_step: h {tuple(h.shape)} against {R} rows of {D}")
        if beta is not None:
            _cuda("beta", beta, torch.float32)
        dt = _dt(h)
    if sum_out is not None:
        _cuda("sum_out", sum_out, torch.float32)
        if tuple(sum_out.shape) != (R, D):
            raise KernelError("hyper_step: sum_out does not fit")
    _call("mllm_hyper_step", x.data_ptr(), y.data_ptr() if y is not None else None, _rows("y", y) if y is not None else 0,
          mix.data_ptr() if writes else None, out_weights.data_ptr() if writes else None,
          in_weights.data_ptr() if in_weights is not None else None, gamma.data_ptr() if h is not None else None,
          beta.data_ptr() if (h is not None and beta is not None) else None, float(eps),
          rows.data_ptr() if rows is not None else None, h.data_ptr() if h is not None else None,
          _rows("h", h) if h is not None else 0, sum_out.data_ptr() if sum_out is not None else None,
          pair_out.data_ptr() if pairs is not None else None, pair_w.data_ptr() if pairs is not None else None, int(top), R,
          int(streams), D, dt, _stream())


def softcap(logits, cap: float) -> None:
    """In place on 32-bit logits [R, V]: x <- cap * tanh(x / cap)."""
    _cuda("logits", logits, torch.float32, contiguous=False)
    _call("mllm_softcap", logits.data_ptr(), _rows("logits", logits), logits.shape[0], logits.shape[1], float(cap), _stream())


# --------------------------------------------------------------------------- joining a branch's result to the residual
def norm_scale_add(y, weight, scale, x, eps: float, *, pairs=None, pair_weights=None, top: int = 0, next_weight=None,
                   next_eps: float = 0.0, next_offset: float = 0.0, next_out=None) -> None:
    """x += (v / sqrt(mean(v^2) + eps) * weight) * scale, row by row, all 32-bit; ``scale`` (a vector) may be None.
    v = y, plus sum_k pair_weights[t, k] * pairs[t * top + k] when ``pairs`` [T * top, D] is given (the chosen experts'
    results of a routed feed-forward; y may then be None).  With ``next_weight`` the new x is also normed for the branch
    that reads it next: next_out = x / sqrt(mean(x^2) + next_eps) * (next_weight + next_offset), float32 or bfloat16."""
    _cuda("x", x, torch.float32, contiguous=False)
    _cuda("weight", weight, torch.float32)
    if scale is not None:
        _cuda("scale", scale, torch.float32)
    R, D = x.shape
    if weight.numel() != D or (scale is not None and scale.numel() != D):
        raise KernelError(f"norm_scale_add: x {tuple(x.shape)}, weight {weight.numel()}")
    if y is not None:
        _cuda("y", y, torch.float32, contiguous=False)
        if tuple(y.shape) != (R, D):
            raise KernelError(f"norm_scale_add: y {tuple(y.shape)}, x {tuple(x.shape)}")
    if pairs is not None:
        _cuda("pairs", pairs, torch.float32)
        _cuda("pair_weights", pair_weights, torch.float32)
        if tuple(pairs.shape) != (R * top, D) or pair_weights.numel() != R * top:
            raise KernelError("norm_scale_add: pairs do not fit")
    elif y is None:
        raise KernelError("norm_scale_add: nothing to add")
    if next_weight is not None:
        _cuda("next_weight", next_weight, torch.float32)
        _cuda("next_out", next_out, contiguous=False)
        if next_weight.numel() != D or tuple(next_out.shape) != (R, D):
            raise KernelError("norm_scale_add: the next norm does not fit")
    _call("mllm_norm_scale_add", y.data_ptr() if y is not None else None, _rows("y", y) if y is not None else 0,
          pairs.data_ptr() if pairs is not None else None, pair_weights.data_ptr() if pairs is not None else None, int(top),
          weight.data_ptr(), scale.data_ptr() if scale is not None else None, x.data_ptr(), _rows("x", x),
          next_weight.data_ptr() if next_weight is not None else None, float(next_offset), float(next_eps),
          next_out.data_ptr() if next_weight is not None else None, _rows("next_out", next_out) if next_weight is not None else 0,
          R, D, float(eps), _dt(next_out) if next_weight is not None else F32, _stream())


def post_norm(x, weight, eps: float, alpha: float, *, y=None, pairs=None, pair_weights=None, top: int = 0, h=None) -> None:
    """x <- (alpha * x + v) / sqrt(mean((alpha * x + v)^2) + eps) * weight, row by row, all 32-bit, in place: the join of a
    block that norms after the sum.  v = y (32-bit [T, D], or None), plus sum_k pair_weights[t, k] * pairs[t * top + k]
    when ``pairs`` [T * top, D] is given (the chosen experts' results of a routed feed-forward).  ``h`` [T, D]
    (float32 or bfloat16, or None) gets the new x for the products that read it next."""
    _cuda("x", x, torch.float32, contiguous=False)
    _cuda("weight", weight, torch.float32)
    R, D = x.shape
    if weight.numel() != D:
        raise KernelError(f"post_norm: x {tuple(x.shape)}, weight {weight.numel()}")
    if y is not None:
        _cuda("y", y, torch.float32, contiguous=False)
        if tuple(y.shape) != (R, D):
            raise KernelError(f"post_norm: y {tuple(y.shape)}, x {tuple(x.shape)}")
    if pairs is not None:
        _cuda("pairs", pairs, torch.float32)
        _cuda("pair_weights", pair_weights, torch.float32)
        if tuple(pairs.shape) != (R * top, D) or pair_weights.numel() != R * top:
            raise KernelError("post_norm: pairs do not fit")
    if h is not None:
        _cuda("h", h, contiguous=False)
        if tuple(h.shape) != (R, D):
            raise KernelError("post_norm: h does not fit x")
    _call("mllm_post_norm", y.data_ptr() if y is not None else None, _rows("y", y) if y is not None else 0,
          pairs.data_ptr() if pairs is not None else None, pair_weights.data_ptr() if pairs is not None else None, int(top),
          weight.data_ptr(), float(alpha), x.data_ptr(), _rows("x", x), h.data_ptr() if h is not None else None,
          _rows("h", h) if h is not None else 0, R, D, float(eps), _dt(h) if h is not None else F32, _stream())


# --------------------------------------------------------------------------- a recurrence with token-dependent decay
WKV_MAX_DIM = 256       # largest head size of csrc/wkv.cu


def wkv_shift(h, mu, state, prev_off: int, ctx, mixes) -> None:
    """mixes[s, t] = h[t] + (h'[t] - h[t]) * mu[s] for the step's tokens, h' the row before: the token before it in the step,
    or (for a request's first token of the step) the row kept in its state at column ``prev_off`` (zeros at position 0).
    h [T, D], mu float32 [NS, D], state float32 [slots, row], mixes [NS, T, D] in h's dtype."""
    _cuda("h", h, contiguous=False)
    _cuda("mu", mu, torch.float32)
    _cuda("state", state, torch.float32)
    _cuda("mixes", mixes, h.dtype)
    T, D = h.shape
    NS = mu.shape[0]
    if tuple(mu.shape) != (NS, D) or tuple(mixes.shape) != (NS, T, D) or state.dim() != 2 or prev_off + D > state.shape[1]:
        raise KernelError(f"wkv_shift: h {tuple(h.shape)}, mu {tuple(mu.shape)}, mixes {tuple(mixes.shape)}, state {tuple(state.shape)}")
    _call("mllm_wkv_shift", h.data_ptr(), _rows("h", h), mu.data_ptr(), state.data_ptr(), state.stride(0), int(prev_off),
          ctx.token_seq.data_ptr(), ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr(), ctx.positions.data_ptr(),
          mixes.data_ptr(), T, D, NS, _dt(h), _stream())


def wkv_decay(low, w2, w0, out) -> None:
    """out[t, c] = exp(-exp(w0[c] + sum_q w2[c, q] * tanh(low[t, q]))), 32-bit: the decays of csrc/wkv.cu's recurrence.
    low [T, R] and w2 [N, R] in one dtype, w0 float32 [N], out float32 [T, N]."""
    _cuda("low", low, contiguous=False)
    _cuda("w2", w2, low.dtype)
    _cuda("w0", w0, torch.float32)
    _cuda("out", out, torch.float32, contiguous=False)
    T, R = low.shape
    N = w2.shape[0]
    if tuple(w2.shape) != (N, R) or w0.numel() != N or tuple(out.shape) != (T, N):
        raise KernelError(f"wkv_decay: low {tuple(low.shape)}, w2 {tuple(w2.shape)}, out {tuple(out.shape)}")
    _call("mllm_wkv_decay", low.data_ptr(), _rows("low", low), w2.data_ptr(), w0.data_ptr(), out.data_ptr(), _rows("out", out),
          T, N, R, _dt(low), _stream())


def wkv_scan(r, k, v, w, u, h, state, prev_off: int, ctx, out, *, heads: int, write_state: bool = True, cols: int = 0) -> None:
    """The recurrence of csrc/wkv.cu over the step's tokens, request by request: o = (S + diag(u) k v^T)^T r;
    S <- diag(w) S + k v^T.  r, k, v [T, heads * n] in one dtype; w (the decays, ``wkv_decay``) float32 [T, heads * n];
    u float32 [heads * n]; state float32 [slots, row] with S [heads, n, n] at column 0 and the last row of h
    [T, D] of every request kept at column ``prev_off``; out float32 [T, heads * n].  ``cols``: columns of a state per CTA,
    16 or 32 (0: the library's rule by the size of the grid; the same bits either way)."""
    _cuda("r", r, contiguous=False)
    for name, t in (("k", k), ("v", v), ("h", h)):
        _cuda(name, t, r.dtype, contiguous=False)
    _cuda("w", w, torch.float32, contiguous=False)
    _cuda("u", u, torch.float32)
    _cuda("state", state, torch.float32)
    _cuda("out", out, torch.float32, contiguous=False)
    T = r.shape[0]
    n = r.shape[1] // heads
    D = h.shape[1]
    if n > WKV_MAX_DIM or r.shape[1] != heads * n or tuple(k.shape) != tuple(r.shape) or tuple(v.shape) != tuple(r.shape) \
            or tuple(out.shape) != tuple(r.shape) or tuple(w.shape) != tuple(r.shape) or u.numel() != heads * n \
            or h.shape[0] != T or state.dim() != 2 or state.shape[1] < max(heads * n * n, prev_off + D) \
            or prev_off < heads * n * n:
        raise KernelError("wkv_scan: shapes do not fit")
    _call("mllm_wkv_scan", r.data_ptr(), _rows("r", r), k.data_ptr(), _rows("k", k), v.data_ptr(), _rows("v", v),
          w.data_ptr(), _rows("w", w), u.data_ptr(), h.data_ptr(), _rows("h", h), state.data_ptr(), state.stride(0),
          int(prev_off), ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr(), out.data_ptr(), _rows("out", out), ctx.S,
          int(heads), n, D, int(write_state), int(cols), _dt(r), _stream())


def wkv_step_ok(n: int, rank: int) -> bool:
    """Whether the single-launch kernel for steps of single tokens takes heads of ``n`` entries with a decay of this rank."""
    return bool(library().mllm_wkv_step_ok(int(n), int(rank)))


def wkv_step(r, k, v, low, w2, w0, u, z, weight, h, state, prev_off: int, ctx, out, *, heads: int, eps: float,
             write_state: bool = True) -> None:
    """A step of single tokens of csrc/wkv.cu's recurrence in one launch: what ``wkv_decay``, ``wkv_scan`` and
    ``wkv_finish`` do one after the other (the same decays and the same state bit for bit; the outputs' sums over the
    state's rows meet in another grouping).  r, k, v, z, out [T, heads * n], low [T, R], w2 [heads * n, R], h [T, D] in one
    dtype; w0, u, weight float32 [heads * n]; state as for ``wkv_scan``."""
    _cuda("r", r, contiguous=False)
    for name, t in (("k", k), ("v", v), ("low", low), ("z", z), ("h", h), ("out", out)):
        _cuda(name, t, r.dtype, contiguous=False)
    _cuda("w2", w2, r.dtype)
    for name, t in (("w0", w0), ("u", u), ("weight", weight), ("state", state)):
        _cuda(name, t, torch.float32)
    T = r.shape[0]
    n = r.shape[1] // heads
    R = low.shape[1]
    D = h.shape[1]
    if r.shape[1] != heads * n or any(tuple(t.shape) != tuple(r.shape) for t in (k, v, z, out)) or tuple(w2.shape) != (heads * n, R) \
            or w0.numel() != heads * n or u.numel() != heads * n or weight.numel() != heads * n or low.shape[0] != T \
            or h.shape[0] != T or state.dim() != 2 or state.shape[1] < max(heads * n * n, prev_off + D) or prev_off < heads * n * n:
        raise KernelError("wkv_step: shapes do not fit")
    if not wkv_step_ok(n, R):
        raise KernelError(f"wkv_step: heads of {n} entries with rank {R} go through wkv_decay, wkv_scan and wkv_finish")
    _call("mllm_wkv_step", r.data_ptr(), _rows("r", r), k.data_ptr(), _rows("k", k), v.data_ptr(), _rows("v", v), low.data_ptr(),
          _rows("low", low), w2.data_ptr(), w0.data_ptr(), u.data_ptr(), z.data_ptr(), _rows("z", z), weight.data_ptr(),
          h.data_ptr(), _rows("h", h), state.data_ptr(), state.stride(0), int(prev_off), ctx.cu_q.data_ptr(),
          ctx.state_slots.data_ptr(), out.data_ptr(), _rows("out", out), ctx.S, int(heads), n, R, D, float(eps),
          int(write_state), _dt(r), _stream())


def wkv_finish(o, z, weight, out, *, heads: int, eps: float) -> None:
    """out = o / sqrt(mean(o^2) + eps) (per head) * weight * silu(z): o float32 [T, heads * n], z and out [T, heads * n] in
    the activation dtype, weight float32 [heads * n]."""
    _cuda("o", o, torch.float32, contiguous=False)
    _cuda("z", z, contiguous=False)
    _cuda("weight", weight, torch.float32)
    _cuda("out", out, z.dtype, contiguous=False)
    T, W = o.shape
    if W % heads or tuple(z.shape) != (T, W) or tuple(out.shape) != (T, W) or weight.numel() != W:
        raise KernelError("wkv_finish: shapes do not fit")
    _call("mllm_wkv_finish", o.data_ptr(), _rows("o", o), z.data_ptr(), _rows("z", z), weight.data_ptr(), out.data_ptr(),
          _rows("out", out), T, int(heads), W // heads, float(eps), _dt(z), _stream())


# --------------------------------------------------------------------------- attention over a cache of latents
LATENT_MAX_RANK, LATENT_MAX_KEY = 512, 1024      # what csrc/latent_attention.cu takes
# keys per CTA of the CUDA-core kernel: short splits when a step has single tokens only (a few long contexts must fill
# the GPU), long ones when it has prompt portions (their tokens fill it, and every split costs a partial result)
LATENT_SPAN_DECODE, LATENT_SPAN_PROMPT = 128, 1024


def latent_prepare(proj, q_off: int, dkv_off: Optional[int], ctx, slot_mapping, freq, mscale: float, norm_weight, eps: float,
                   pages, qa, *, heads: int, dim: int, rot_dim: int, rank: int, rot_dims: int, write: bool) -> None:
    """Per token of the step: the latent (columns dkv_off .. of ``proj``, RMS-normed with ``norm_weight``) and the shared
    key part rotated at the token's position go to the token's cache row [rank | rot_dim | padding] (``dkv_off`` None or
    ``write`` False: no row is written); every head's rotated query part goes, rotated, to columns rank.. of
    qa [T, heads, rank + rot_dim] (32-bit).  Angles p * freq[i], cos and sin times ``mscale``, all 32-bit."""
    _cuda("proj", proj, contiguous=False)
    _cuda("qa", qa, torch.float32)
    _cuda("freq", freq, torch.float32)
    T = proj.shape[0]
    row = 0
    if dkv_off is not None and write:
        _cuda("pages", pages, proj.dtype)
        _cuda("norm_weight", norm_weight, torch.float32)
        _cuda("slot_mapping", slot_mapping, torch.int32)
        row = pages.shape[-1]
        if pages.shape[1] != 1 or norm_weight.numel() != rank or slot_mapping.numel() != T:
            raise KernelError("latent_prepare: the cache must have one key/value head and one slot per token")
    else:
        row = rank + rot_dim
    if tuple(qa.shape) != (T, heads * (rank + rot_dim)) or freq.numel() * 2 != rot_dims:
        raise KernelError(f"latent_prepare: qa {tuple(qa.shape)} for {heads} heads of {rank} + {rot_dim}")
    wr = dkv_off is not None and write
    _call("mllm_latent_prepare", proj.data_ptr(), _rows("proj", proj), int(q_off), int(dkv_off) if wr else -1, T, heads, dim,
          rot_dim, rank, rot_dims, ctx.positions.data_ptr(), slot_mapping.data_ptr() if wr else None, freq.data_ptr(),
          float(mscale), norm_weight.data_ptr() if wr else None, float(eps), pages.data_ptr() if wr else None, row,
          qa.data_ptr(), int(wr), _dt(proj), _stream())


def headwise_linear(x, x_head: int, weight, out, out_head: int, gate=None) -> None:
    """out[t, h*out_head + n] = sum_k x[t, h*x_head + k] * weight[h, n, k], optionally times sigmoid(gate[t, h*N + n]):
    a small product per head.  Either x has the weights' dtype and out is 32-bit, or x is 32-bit and out (and the
    gate) have the weights' dtype."""
    _cuda("x", x, contiguous=False)
    _cuda("weight", weight)
    _cuda("out", out, contiguous=False)
    H, N, K = weight.shape
    T = x.shape[0]
    if out.shape[0] != T or x_head < K or out_head < N:
        raise KernelError("headwise_linear: shapes do not fit the weights")
    if x.dtype == weight.dtype and out.dtype == torch.float32 and gate is None:
        mode = 0
    elif x.dtype == torch.float32 and out.dtype == weight.dtype:
        mode = 1
        if gate is not None:
            _cuda("gate", gate, weight.dtype, contiguous=False)
    else:
        raise KernelError(f"headwise_linear: x {x.dtype}, weight {weight.dtype}, out {out.dtype}")
    _call("mllm_headwise_linear", x.data_ptr(), _rows("x", x), int(x_head), weight.data_ptr(), out.data_ptr(), _rows("out", out),
          int(out_head), gate.data_ptr() if gate is not None else None, _rows("gate", gate) if gate is not None else 0,
          T, H, N, K, mode, _dt(weight), _stream())


def latent_attention(qa, pages, block_table, ctx, out, *, heads: int, rank: int, scale: float,
                     impl: Optional[str] = None) -> None:
    """Causal softmax attention of qa [T, heads * dk] (32-bit) over cache rows pages [P, 1, page_size, row]: a token's row
    holds its key (the first dk columns) and its value (the first ``rank`` columns) for all heads.
    out[t, h] = sum_j softmax_j((qa[t, h] . row_j[:dk]) * scale) row_j[:rank], 32-bit [T, heads * rank].
    ``impl``: "split" (CUDA cores, all 32-bit, splits of 256 keys: single tokens, 32-bit caches, any size) or "mma"
    (tensor cores: steps with prompt portions over a bfloat16 cache); None picks by the step's shape."""
    _cuda("qa", qa, torch.float32)
    _cuda("pages", pages)
    _cuda("out", out, torch.float32)
    _cuda("block_table", block_table, torch.int32, contiguous=False)
    T = qa.shape[0]
    dk = qa.shape[1] // heads
    _, one, ps, row = pages.shape
    if one != 1 or qa.shape[1] != heads * dk or tuple(out.shape) != (T, heads * rank) or not (rank <= dk <= row):
        raise KernelError("latent_attention: shapes do not fit the cache rows")
    if rank > LATENT_MAX_RANK or dk > LATENT_MAX_KEY:
        raise KernelError(f"latent_attention: latent size {rank} (at most {LATENT_MAX_RANK}), key size {dk} (at most {LATENT_MAX_KEY})")
    mma_ok = pages.dtype == torch.bfloat16 and getattr(ctx, "n_tiles", 0) > 0 and library().mllm_latent_mma_ok(rank, dk, row) == 1
    if impl is None:
        impl = "mma" if mma_ok and not getattr(ctx, "decode_only", False) else "split"
    attention_launches["latent_" + impl] = attention_launches.get("latent_" + impl, 0) + 1
    if impl == "mma":
        if not mma_ok:
            raise KernelError("latent_attention: the tensor-core kernel takes a bfloat16 cache, a step with tiles, latents "
                              "that are multiples of 8 and keys that are multiples of 16")
        _call("mllm_latent_attention_mma", qa.data_ptr(), pages.data_ptr(), row, block_table.data_ptr(),
              _rows("block_table", block_table), ctx.attn_tiles.data_ptr(), int(ctx.n_tiles), ctx.positions.data_ptr(),
              out.data_ptr(), heads, rank, dk, ps, float(scale), _stream())
        return
    if impl != "split":
        raise KernelError(f"latent_attention: unknown implementation {impl!r}")
    span = LATENT_SPAN_DECODE if getattr(ctx, "decode_only", False) else LATENT_SPAN_PROMPT
    need = max(1, -(-int(ctx.max_ctx_len) // span))
    nsplit = 1 << (need - 1).bit_length()       # a power of two: few distinct grids for captured graphs
    part_o = ctx.ws.buf("latent_part_o", T * heads * nsplit, rank, torch.float32)
    part_ml = ctx.ws.buf("latent_part_ml", T * heads * nsplit, 2, torch.float32)
    _call("mllm_latent_attention", qa.data_ptr(), pages.data_ptr(), row, block_table.data_ptr(), _rows("block_table", block_table),
          ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(), nsplit, out.data_ptr(),
          T, heads, rank, dk, ps, float(scale), span, _dt(pages), _stream())
    global launches
    launches += 1           # the kernel that merges the splits


def latent_splits(max_ctx_len: int) -> int:
    """Splits of the latent attention at a context length (part of a step's shape for captured graphs)."""
    need = max(1, -(-int(max_ctx_len) // LATENT_SPAN_DECODE))
    return 1 << (need - 1).bit_length()


# --------------------------------------------------------------------------- state-space mixer
SSD_MAX_STATE_ROWS, SSD_MAX_TAPS = 256, 16       # what csrc/ssd.cu takes


def ssd_conv(proj, off: int, weight, bias, state, conv_off: int, ctx, out, *, write_state: bool = True) -> None:
    """out[t, c] = silu(bias[c] + sum_j weight[c, j] * u[t - (taps-1) + j, c]) with u = proj[:, off : off + C] within a
    request; inputs before the step's first token of a request come from state[slot, conv_off:] ([taps-1, C], oldest
    first), which afterwards holds the request's last taps - 1 inputs.  out 32-bit [T, C]."""
    _cuda("proj", proj, contiguous=False)
    _cuda("weight", weight, torch.float32)
    _cuda("bias", bias, torch.float32)
    _cuda("state", state, torch.float32)
    _cuda("out", out, torch.float32)
    C, taps = weight.shape
    T = proj.shape[0]
    if tuple(out.shape) != (T, C) or bias.numel() != C or state.dim() != 2 or conv_off + (taps - 1) * C > state.shape[1]:
        raise KernelError("ssd_conv: shapes do not fit")
    _call("mllm_ssd_conv", proj.data_ptr(), _rows("proj", proj), int(off), weight.data_ptr(), bias.data_ptr(), state.data_ptr(),
          state.stride(0), int(conv_off), ctx.token_seq.data_ptr(), ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr(),
          out.data_ptr(), T, ctx.S, C, taps, int(write_state), _dt(proj), _stream())
    if write_state and taps > 1 and T != ctx.S:
        global launches
        launches += 1       # the state's update (steps of single tokens do both in one launch)


def ssd_scan(xbc, proj, dt_off: int, dt_bias, A_log, D, state, ctx, y, *, heads: int, vdim: int, state_rows: int, groups: int,
             write_state: bool = True) -> None:
    """The selective state-space recurrence over the step's tokens, request by request and head by head:
    dt = softplus(proj[:, dt_off + h] + dt_bias[h]); S <- exp(-exp(A_log[h]) dt) S + dt B x^T; y = S^T C + D[h] x, with
    x = xbc[:, h*vdim : (h+1)*vdim], B and C the group's rows after the x columns of xbc [T, heads*vdim + 2*groups*N]
    (32-bit).  state [slots, >= heads*N*vdim] float32: S of head h at h*N*vdim, [N, vdim]; y [T, heads*vdim] 32-bit."""
    _cuda("xbc", xbc, torch.float32)
    _cuda("proj", proj, contiguous=False)
    _cuda("state", state, torch.float32)
    _cuda("y", y, torch.float32)
    for name, t in (("dt_bias", dt_bias), ("A_log", A_log), ("D", D)):
        _cuda(name, t, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"ssd_scan: {name} has {t.numel()} entries for {heads} heads")
    T = xbc.shape[0]
    inner, N = heads * vdim, state_rows
    if xbc.shape[1] != inner + 2 * groups * N or tuple(y.shape) != (T, inner) or state.dim() != 2 \
            or state.shape[1] < heads * N * vdim or proj.shape[0] != T:
        raise KernelError("ssd_scan: shapes do not fit")
    if N > SSD_MAX_STATE_ROWS:
        raise KernelError(f"ssd_scan: a state of {N} rows (at most {SSD_MAX_STATE_ROWS})")
    _call("mllm_ssd_scan", xbc.data_ptr(), xbc.shape[1], inner, inner + groups * N, proj.data_ptr(), _rows("proj", proj),
          int(dt_off), dt_bias.data_ptr(), A_log.data_ptr(), D.data_ptr(), state.data_ptr(), state.stride(0),
          ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr(), y.data_ptr(), ctx.S, heads, N, vdim, groups, int(write_state),
          _dt(proj), _stream())


def gated_group_norm(y, z, weight, out, groups: int, eps: float) -> None:
    """out = rms_norm(y * silu(z)) * weight with the norm taken over each of ``groups`` equal parts of a row on its own;
    y 32-bit [T, W], z and out in the activation dtype (column slices are fine)."""
    _cuda("y", y, torch.float32)
    _cuda("z", z, contiguous=False)
    _cuda("out", out, z.dtype, contiguous=False)
    _cuda("weight", weight, torch.float32)
    T, W = y.shape
    if tuple(z.shape) != (T, W) or tuple(out.shape) != (T, W) or weight.numel() != W or W % groups:
        raise KernelError("gated_group_norm: shapes do not fit")
    _call("mllm_gated_group_norm", y.data_ptr(), z.data_ptr(), _rows("z", z), weight.data_ptr(), out.data_ptr(),
          _rows("out", out), T, W, int(groups), float(eps), _dt(z), _stream())


# --------------------------------------------------------------------------- routed feed-forward
MOE_MAX_EXPERTS = 512
_moe_few_tokens = None


def moe_route(h, router, idx, weights, offsets, order, *, top: int, groups: int = 1, keep: int = 1, bias=None,
              mode: str = "softmax_all", group_sum: int = 1, weight_scale: float = 1.0) -> None:
    """Per row of h: softmax of the router's logits (32-bit) over all experts; the best ``keep`` of ``groups`` equal
    groups of neighbours (by their largest score); the ``top`` best experts within them -> idx [T, top] (int32) and
    weights [T, top] (scores over their sum + 1e-20).  ``bias`` (float32 [E]) is added to the logits first.  ``mode``
    "softmax_top": the ``top`` largest logits are chosen and weighted by the softmax over those alone (no groups);
    "sigmoid": the scores are sigmoid(logit), expert by expert.  ``group_sum`` 2: a group's score is the sum of its two
    largest scores.  The weights are multiplied by ``weight_scale``.
    Then the (row, choice) pairs ordered by expert: offsets [E + 1], order [T * top]."""
    _cuda("h", h, contiguous=False)
    _cuda("router", router, h.dtype)
    for name, t, dt in (("idx", idx, torch.int32), ("weights", weights, torch.float32), ("offsets", offsets, torch.int32),
                        ("order", order, torch.int32)):
        _cuda(name, t, dt)
    T, D = h.shape
    E = router.shape[0]
    if router.shape[1] != D or idx.numel() != T * top or weights.numel() != T * top or offsets.numel() != E + 1 \
            or order.numel() != T * top:
        raise KernelError("moe_route: shapes do not fit")
    if bias is not None:
        _cuda("bias", bias, torch.float32)
        if bias.numel() != E:
            raise KernelError("moe_route: one bias per expert")
    modes = {"softmax_all": 0, "softmax_top": 1, "sigmoid": 2}
    if mode not in modes:
        raise KernelError(f"moe_route: unknown mode {mode!r}")
    _call("mllm_moe_route", h.data_ptr(), _rows("h", h), router.data_ptr(), bias.data_ptr() if bias is not None else None,
          modes[mode], T, D, E, int(top), int(groups), int(keep), int(group_sum), float(weight_scale),
          idx.data_ptr(), weights.data_ptr(), offsets.data_ptr(), order.data_ptr(), _dt(h), _stream())
    global launches, _moe_few_tokens
    if _moe_few_tokens is None:
        _moe_few_tokens = int(library().mllm_moe_few_tokens())
    if T > _moe_few_tokens:
        launches += 1       # the ordering is a launch of its own


def moe_grouped(a, weight, out, offsets, order, *, top: int, first: bool, act: str = "silu", limit: float = 0.0,
                alpha: float = 1.0) -> None:
    """The experts' products over the pairs in ``order``.  ``first``: a [T, K] (row = pair // top), weight [E, 2F, K]
    (gate rows, then up rows) -> out[i] = silu(gate) * up (``act`` "swiglu_clamp": the clamped form of gated_act, with
    ``limit`` and ``alpha``) for the i-th pair in order, [T*top, F]; ``act`` "relu_sq": experts without a gate, weight
    [E, F, K], out[i] = relu(.)^2.  Otherwise: a [T*top, K]
    in that order, weight [E, N, K] -> out[pair] [T*top, N] 32-bit, by pair id."""
    _cuda("a", a, contiguous=False)
    _cuda("weight", weight, a.dtype)
    _cuda("out", out, contiguous=False)
    E, rows, K = weight.shape
    n_pairs = order.numel()
    ungated = first and act in _UNGATED_ACT
    N = rows // 2 if (first and not ungated) else rows
    if a.shape[1] != K or tuple(out.shape) != (n_pairs, N) or offsets.numel() != E + 1:
        raise KernelError("moe_grouped: shapes do not fit")
    if act not in ("silu", "swiglu_clamp", *_UNGATED_ACT) or (act == "swiglu_clamp" and not limit > 0):
        raise KernelError(f"moe_grouped: activation {act!r} (limit {limit})")
    if (first and out.dtype != a.dtype) or (not first and out.dtype != torch.float32):
        raise KernelError("moe_grouped: the first product keeps the dtype, the second gives 32-bit")
    _call("mllm_moe_grouped", a.data_ptr(), _rows("a", a), weight.data_ptr(), out.data_ptr(), _rows("out", out),
          offsets.data_ptr(), order.data_ptr(), n_pairs, E, N, K, int(top) if first else 0, 0 if first else 1,
          (2 if ungated else 0) if first else 1, _UNGATED_ACT[act] if ungated else _GATE_ACT[act], float(limit), float(alpha),
          _dt(a), _stream())


def moe_combine(pair_out, weights, y, *, top: int, accumulate: bool) -> None:
    """y[t] (+)= sum_k weights[t, k] * pair_out[t * top + k] (32-bit), in the order of k."""
    _cuda("pair_out", pair_out, torch.float32)
    _cuda("weights", weights, torch.float32)
    _cuda("y", y, torch.float32, contiguous=False)
    T, D = y.shape
    if tuple(pair_out.shape) != (T * top, D) or weights.numel() != T * top:
        raise KernelError("moe_combine: shapes do not fit")
    _call("mllm_moe_combine", pair_out.data_ptr(), weights.data_ptr(), y.data_ptr(), _rows("y", y), T, D, int(top),
          int(accumulate), _stream())


REC_WIDE_MAX_ROWS = 128        # rows of a head's state that the kernel for prompt portions takes
recurrence_launches = {}       # "step" / "wide" -> launches so far


def gated_recurrence(a, z, v, f_bias, lower, norm_weight, eps: float, state, ctx, out, *, heads: int, out_scale: float = 1.0,
                     write_state: bool = True, impl: Optional[str] = None) -> None:
    """The gated linear recurrence of csrc/gated_recurrence.cu over the step's tokens, request by request:
    f = lower + (1 - lower) * sigmoid(z + f_bias); S <- diag(f) S + (1 - f) v^T; o = S^T silu(a);
    out = out_scale * rms_norm(o) * norm_weight per head.  a, z [T, heads * ek], v, out [T, heads * ev] (rows
    contiguous; column slices are fine), state [slots, heads, ek, ev] float32, indexed by ctx.state_slots.
    ``impl``: "step" (one CTA per request and head with the norm fused: single tokens) or "wide" (the recurrence
    spread over 32-column CTAs, then the norm kernel: prompt portions); None picks by the step's shape."""
    _cuda("a", a, contiguous=False)
    _cuda("z", z, a.dtype, contiguous=False)
    _cuda("v", v, a.dtype, contiguous=False)
    _cuda("out", out, a.dtype, contiguous=False)
    _cuda("state", state, torch.float32)
    for name, t in (("f_bias", f_bias), ("lower", lower), ("norm_weight", norm_weight)):
        _cuda(name, t, torch.float32)
    T = a.shape[0]
    if state.dim() != 4 or state.shape[1] != heads:
        raise KernelError(f"gated_recurrence: state {tuple(state.shape)} against {heads} heads")
    ek, ev = state.shape[2], state.shape[3]
    if tuple(a.shape) != (T, heads * ek) or tuple(z.shape) != (T, heads * ek) or tuple(v.shape) != (T, heads * ev) \
            or tuple(out.shape) != (T, heads * ev) or f_bias.numel() != heads * ek or lower.numel() != heads * ek \
            or norm_weight.numel() != ev:
        raise KernelError("gated_recurrence: shapes do not fit the state")
    if impl is None:
        impl = "wide" if (T > ctx.S and ek <= REC_WIDE_MAX_ROWS) else "step"
    recurrence_launches[impl] = recurrence_launches.get(impl, 0) + 1
    if impl == "wide":
        # prompt portions: the recurrence spread over many threads, raw outputs in 32-bit, then the per-head norm
        if ek > REC_WIDE_MAX_ROWS:
            raise KernelError(f"gated_recurrence: the wide kernel takes states of up to {REC_WIDE_MAX_ROWS} rows, not {ek}")
        raw = ctx.ws.buf("rec_raw", T, heads * ev, torch.float32)
        _call("mllm_gated_recurrence_wide", a.data_ptr(), _rows("a", a), z.data_ptr(), _rows("z", z), v.data_ptr(),
              _rows("v", v), f_bias.data_ptr(), lower.data_ptr(), state.data_ptr(), ctx.cu_q.data_ptr(),
              ctx.state_slots.data_ptr(), raw.data_ptr(), _rows("raw", raw), ctx.S, heads, ek, ev, int(write_state),
              _dt(a), _stream())
        rmsnorm(raw, norm_weight, eps, out, unit_offset=False, heads=heads, scale=out_scale)
        return
    if impl != "step":
        raise KernelError(f"gated_recurrence: unknown implementation {impl!r}")
    _call("mllm_gated_recurrence", a.data_ptr(), _rows("a", a), z.data_ptr(), _rows("z", z), v.data_ptr(), _rows("v", v),
          f_bias.data_ptr(), lower.data_ptr(), norm_weight.data_ptr(), state.data_ptr(), ctx.cu_q.data_ptr(),
          ctx.state_slots.data_ptr(), out.data_ptr(), _rows("out", out), ctx.S, heads, ek, ev, float(eps), float(out_scale),
          int(write_state), _dt(a), _stream())


attention_launches = {}     # attention kernel name -> launches so far (tests check which kernel a step took)
use_tcgen05_attention = True    # False: prompt portions stay on the mma.sync kernel (for comparisons and profiles)


def _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim == 64 and 8 <= ps <= 128 and ps & (ps - 1) == 0
            and getattr(ctx, "n_tiles_wide", 0) > 0 and ldq % 8 == 0 and q.data_ptr() % 16 == 0 and ldo % 8 == 0
            and out.data_ptr() % 16 == 0 and k_pages.is_contiguous() and k_pages.data_ptr() % 16 == 0)


_TILED_WIDE_HEAD_DIMS = (16, 32, 48, 64)


def _tiled_wide_ok(q, head_dim, ctx, ldq) -> bool:
    """Long prompt portions (128-row tiles mostly full) with heads up to 64, where no tensor-core kernel applies."""
    nw = getattr(ctx, "n_tiles_wide", 0)
    return (head_dim in _TILED_WIDE_HEAD_DIMS and nw > 0 and ctx.T >= 256 and ctx.T >= 80 * nw
            and ldq % (16 // q.element_size()) == 0 and q.data_ptr() % 16 == 0)


def paged_attention(q, k_pages, v_pages, block_table, ctx, out, *, num_heads, num_kv_heads, head_dim, scale,
                    window=None, impl: Optional[str] = None) -> None:
    """Causal attention of the step's tokens over the cache.

    q [T, heads*head_dim] (rows contiguous), pages [num_pages, kv_heads, page_size,
    head_dim], block_table [S, max_pages] int32, ctx.token_seq / ctx.positions [T].
    """
    _cuda("q", q, contiguous=False)
    _cuda("k_pages", k_pages, q.dtype)
    _cuda("v_pages", v_pages, q.dtype)
    _cuda("out", out, q.dtype, contiguous=False)
    _cuda("block_table", block_table, torch.int32, contiguous=False)
    ldq = _rows("q", q)
    ldo = _rows("out", out)
    T = q.shape[0]
    _, Hkv, ps, dh = k_pages.shape
    if Hkv != num_kv_heads or dh != head_dim or q.shape[1] != num_heads * head_dim:
        raise KernelError("paged_attention: head counts or sizes do not fit the pages")
    if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
        raise KernelError(f"paged_attention: head size {head_dim} is not a multiple of 16 in 16..256")
    bt_stride = _rows("block_table", block_table)
    if impl is None:
        impl = "simt"
        if getattr(ctx, "decode_only", False) and head_dim in _DECODE_HEAD_DIMS[q.dtype] and ldq % 8 == 0 \
                and q.data_ptr() % 16 == 0:
            impl = "decode"
        elif use_tcgen05_attention and _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo) and ctx.T >= 256 \
                and ctx.T >= 80 * ctx.n_tiles_wide:
            impl = "flash_tc"       # long prompt portions (tiles of 128 rows mostly full): the tensor-memory kernel
        elif q.dtype == torch.bfloat16 and head_dim in _FLASH_HEAD_DIMS and getattr(ctx, "n_tiles", 0) > 0 \
                and ldq % 8 == 0 and q.data_ptr() % 16 == 0 and ldo % 2 == 0:
            impl = "flash"
        elif _tiled_wide_ok(q, head_dim, ctx, ldq):
            impl = "tiled_wide"     # float32 (or a head size of 48) and long portions: 128 x 128 tiles on CUDA cores
        elif getattr(ctx, "n_tiles", 0) > 0:
            impl = "tiled"          # float32, or a head size the tensor-core kernel does not take
    attention_launches[impl] = attention_launches.get(impl, 0) + 1
    if impl == "tiled_wide":
        if head_dim not in _TILED_WIDE_HEAD_DIMS or getattr(ctx, "n_tiles_wide", 0) <= 0 or ldq % (16 // q.element_size()):
            raise KernelError("paged_attention: the 128 x 128 CUDA-core kernel takes head sizes "
                              f"{_TILED_WIDE_HEAD_DIMS}, 16-byte aligned rows and a list of 128-row tiles")
        _call("mllm_attention_tiled_wide", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles_wide.data_ptr(), int(ctx.n_tiles_wide),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _dt(q), _stream())
        return
    if impl == "tiled":
        _call("mllm_attention_tiled", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles.data_ptr(), int(ctx.n_tiles),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _dt(q), _stream())
        return
    if impl == "flash_tc":
        if not _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo):
            raise KernelError("paged_attention: the tcgen05 kernel takes bfloat16, head size 64, pages of 8..128 "
                              "tokens (a power of two), 16-byte aligned rows and a list of 128-row tiles")
        _call("mllm_attention_tcgen05", q.data_ptr(), ldq, T, k_pages.data_ptr(), v_pages.data_ptr(),
              int(k_pages.shape[0]), block_table.data_ptr(), bt_stride, ctx.attn_tiles_wide.data_ptr(),
              int(ctx.n_tiles_wide), ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim,
              ps, float(scale), int(window or 0), _stream())
        return
    if impl == "flash":
        if q.dtype != torch.bfloat16 or head_dim not in _FLASH_HEAD_DIMS:
            raise KernelError(f"paged_attention: the tensor-core kernel takes bfloat16 and head sizes "
                              f"{_FLASH_HEAD_DIMS}, not {q.dtype} / {head_dim}")
        _call("mllm_attention_flash", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles.data_ptr(), int(ctx.n_tiles),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _stream())
        return
    if impl in ("decode", "decode_scratch"):        # "decode_scratch": splits meet in global scratch, not in a cluster
        if head_dim not in _DECODE_HEAD_DIMS[q.dtype]:
            raise KernelError(f"paged_attention: the split-key kernel takes head sizes {_DECODE_HEAD_DIMS[q.dtype]} "
                              f"for {q.dtype}, not {head_dim}")
        # splits cover the longest context of the step, rounded up so that captured graphs keep their grid
        max_splits = decode_splits(ctx.max_ctx_len)
        # Up to DECODE_CLUSTER_SPLITS splits meet in a thread-block cluster and touch no scratch; only beyond that
        # (contexts over 1,024 tokens) or on request do the partial results go through global memory.  Asking for
        # the buffers only then keeps a growing context from ever replacing a buffer under the captured graphs.
        if impl == "decode_scratch" or max_splits > DECODE_CLUSTER_SPLITS:
            part_o = ctx.ws.buf("attn_part_o", T * num_heads * max_splits, head_dim, torch.float32).data_ptr()
            part_ml = ctx.ws.buf("attn_part_ml", T * num_heads * max_splits, 2, torch.float32).data_ptr()
            counters = ctx.ws.zeroed("attn_counters", T * num_heads).data_ptr()     # the kernel leaves them zero
        else:
            part_o = part_ml = counters = None
        _call("mllm_attention_decode", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(),
              ldo, part_o, part_ml, counters, T, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), max_splits, _dt(q), int(impl == "decode_scratch"), _stream())
        return
    if impl != "simt":
        raise KernelError(f"paged_attention: unknown implementation {impl!r}")
    _call("mllm_attention_simt", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
          bt_stride, ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), ldo, T, num_heads,
          num_kv_heads, head_dim, ps, float(scale), int(window or 0), _dt(q), _stream())


# --------------------------------------------------------------------------- sampling
_argmax_scratch = {}


def argmax(logits, out) -> None:
    """out[r] = index of the largest value of row r, the lowest index among equals."""
    _cuda("logits", logits, torch.float32, contiguous=False)
    _cuda("out", out, torch.int32)
    ld = _rows("logits", logits)
    R, V = logits.shape
    if out.numel() != R:
        raise KernelError("argmax: one output per row")
    slices = 1
    if R * 4 < 592 and V >= 8192:            # few long rows: cut them so that the SMs have work
        slices = min(64, max(2, 592 // max(R, 1)), V // 1024)
    if slices == 1:
        _call("mllm_argmax", logits.data_ptr(), ld, R, V, out.data_ptr(), _stream())
        return
    dev = logits.device
    sc = _argmax_scratch.get(dev)
    if sc is None or sc[0].numel() < R * slices or sc[2].numel() < R:
        n = max(R * slices, 4096)
        sc = (torch.empty(n, dtype=torch.float32, device=dev), torch.empty(n, dtype=torch.int32, device=dev),
              torch.zeros(max(R, 1024), dtype=torch.int32, device=dev))
        _argmax_scratch[dev] = sc
    _call("mllm_argmax_sliced", logits.data_ptr(), ld, R, V, out.data_ptr(), sc[0].data_ptr(), sc[1].data_ptr(),
          sc[2].data_ptr(), slices, _stream())


def sample(logits, temperature, uniform, out) -> None:
    """Per row: argmax if temperature == 0, else an inverse-CDF draw with uniform[r]."""
    _cuda("logits", logits, torch.float32, contiguous=False)
    _cuda("temperature", temperature, torch.float32)
    _cuda("uniform", uniform, torch.float32)
    _cuda("out", out, torch.int32)
    ld = _rows("logits", logits)
    R, V = logits.shape
    if temperature.numel() != R or uniform.numel() != R or out.numel() != R:
        raise KernelError("sample: per-row arguments differ in length")
    _call("mllm_sample", logits.data_ptr(), ld, R, V, temperature.data_ptr(), uniform.data_ptr(), out.data_ptr(),
          _stream())
