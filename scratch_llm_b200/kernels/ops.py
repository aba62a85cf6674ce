"""Python bindings of the engine's CUDA kernels: one function per launcher of ``csrc/``.

Each function checks devices, dtypes and layouts, passes raw pointers and the current CUDA
stream through ctypes, and raises :class:`KernelError` on a non-zero return code.  There is no
other implementation behind these functions: if a library cannot be compiled or loaded, the
call fails.

The reference reaches its compiled kernels through one pybind module (csrc/pybind.cpp:89-127)
and a lazy dispatch table (src/scratch_llm/kernels/attention/dispatch.py:68-90).
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Sequence

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


# library name -> (sources, defines)
CORE_LIBRARIES: dict[str, tuple[tuple[str, ...], tuple[str, ...]]] = {
    "sllm_elementwise": (("elementwise.cu",), ()),
    "sllm_rope_cache": (("rope_cache.cu",), ()),
    "sllm_gemm_simt": (("gemm_simt.cu",), ()),
    "sllm_sampling": (("sampling.cu",), ()),
    "sllm_gemv_mma": (("gemv_mma.cu",), ()),
    "sllm_gemm_tcgen05": (("gemm_tcgen05.cu",), ()),
    "sllm_gemv_tma": (("gemv_tma.cu",), ()),
}
#: libraries that only some architectures need: compiled at the first call that reaches them
EXTRA_LIBRARIES: dict[str, tuple[tuple[str, ...], tuple[str, ...]]] = {
    "sllm_stream_ops": (("stream_ops.cu",), ()),
    "sllm_qk_norm_cache": (("qk_norm_cache.cu",), ()),
    "sllm_recurrent_ops": (("recurrent_ops.cu",), ()),
    "sllm_tanh_norm": (("tanh_norm.cu",), ()),
    "sllm_moe": (("moe.cu",), ()),
    "sllm_moe_tc": (("moe_tc.cu",), ()),
    "sllm_latent_attention": (("latent_attention.cu",), ()),
    "sllm_layer_norm": (("layer_norm.cu",), ()),
    "sllm_norm_rope_cache": (("norm_rope_cache.cu",), ()),
}


def attention_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_simt_hd{head_dim}", ("attention_simt.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def attention_mma_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_mma_hd{head_dim}", ("attention_mma.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def attention_tc_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_tc_hd{head_dim}", ("attention_tc.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def delta_rule_library(key_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_delta_rule_hd{key_dim}", ("delta_rule.cu",), (f"SLLM_HEAD_DIM={key_dim}",))


def general_delta_library(key_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_general_delta_hd{key_dim}", ("general_delta.cu",),
            (f"SLLM_HEAD_DIM={key_dim}",))


#: the generalized delta rule spreads a column of its state over up to 32 lanes of 16 elements
GENERAL_DELTA_MAX_KEY_DIM = 512

#: the delta-rule kernel stages a chunk of keys and queries in shared memory: key sizes up to this
DELTA_MAX_KEY_DIM = 256


def attention_tc_supports(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                          window: int | None, biased: bool = False) -> bool:
    """Whether the tcgen05 attention kernel takes this shape (else attention_mma serves it).
    ``biased``: the caller uses the entry with a window, slopes and sinks."""
    if head_dim % 64 or not 64 <= head_dim <= 256 or (window and not biased):
        return False
    gs = n_heads // n_kv_heads
    return n_heads % n_kv_heads == 0 and 128 % gs == 0 and page_size > 0 and 128 % page_size == 0


#: the tensor-core attention kernels take head sizes up to this; larger ones use the CUDA cores
MMA_MAX_HEAD_DIM = 256
#: the CUDA-core attention kernel takes head sizes up to this (its tiles fill shared memory)
SIMT_MAX_HEAD_DIM = 640

_loaded: dict[str, ctypes.CDLL] = {}


def _load(name: str, sources: Sequence[str], defines: Sequence[str]) -> ctypes.CDLL:
    lib = _loaded.get(name)
    if lib is None:
        path = build.compile_library(name, sources, defines)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None
        _loaded[name] = lib
    return lib


def _core(name: str) -> ctypes.CDLL:
    return _load(name, *(CORE_LIBRARIES.get(name) or EXTRA_LIBRARIES[name]))


def prepare(head_dims: Sequence[int] = (), verbose: bool = True) -> None:
    """Compile (in parallel) and load everything a model with these head sizes needs."""
    jobs = [(n, s, d) for n, (s, d) in CORE_LIBRARIES.items()]
    jobs += [attention_library(hd) for hd in sorted(set(head_dims))]
    jobs += [attention_mma_library(hd) for hd in sorted(set(head_dims)) if hd <= MMA_MAX_HEAD_DIM]
    jobs += [attention_tc_library(hd) for hd in sorted(set(head_dims))
             if hd % 64 == 0 and hd <= 256]
    build.compile_many(jobs, verbose=verbose)
    for n, s, d in jobs:
        _load(n, s, d)


def prepare_jobs(jobs: Sequence[tuple[str, Sequence[str], Sequence[str]]],
                 verbose: bool = True) -> None:
    """Compile (in parallel) and load exactly the listed libraries: what a model whose parts
    state their needs asks for (:meth:`scratch_llm_b200.engine.model.DecoderModel.kernel_jobs`).
    Anything else a step reaches is compiled at that call."""
    seen, unique = set(), []
    for job in jobs:
        if job[0] not in seen:
            seen.add(job[0])
            unique.append((job[0], tuple(job[1]), tuple(job[2])))
    build.compile_many(unique, verbose=verbose)
    for n, s, d in unique:
        _load(n, s, d)


def core_job(name: str) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    sources, defines = CORE_LIBRARIES.get(name) or EXTRA_LIBRARIES[name]
    return (name, sources, defines)


#: kernels of this package launched so far in this process (one per successful op call)
launch_count = 0
#: the same per op name ("gemv_tma", "attention_tc", ...): which kernels a workload reached.
#: Calls recorded into a CUDA graph count once, at the capture; replays are counted by the runner.
launch_counts: dict[str, int] = {}


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    launch_counts[what] = launch_counts.get(what, 0) + 1
    if code != 0:
        raise KernelError(f"{what} failed with CUDA error {code} "
                          f"({'invalid value: a size this kernel does not take' if code == 1 else 'see cudaError_t'})")


# the current stream's handle without building a torch.cuda.Stream object (3 us a call, which
# is a third of a launch's host cost in steps that run outside a captured graph)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    if _raw_stream is not None and _current_device is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}: kernels take float32 and bfloat16") from None


# ------------------------------------------------------------------------------ elementwise

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          pending: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """out[n] = table[ids[n]] widened to 32-bit, times ``scale`` (an architecture's embedding
    multiplier).  ids int32 [N]; table [V, d]; out f32 [N, d].
    An id ``-1 - j`` stands for ``pending[j]`` (int32, on the device): a token that an earlier
    kernel of the stream chose and the host has not read yet."""
    _need(ids, torch.int32, "ids")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _need(table, None, "table")
    _need(out, torch.float32, "out")
    n, d = ids.numel(), table.shape[1]
    if out.shape != (n, d):
        raise KernelError(f"out must be [{n}, {d}], got {list(out.shape)}")
    _check(_core("sllm_elementwise").sllm_embed(
        _ptr(ids), _ptr(pending) if pending is not None else c_void_p(0), _ptr(table), _ptr(out),
        c_int(n), c_int(d), c_int(_code(table.dtype)), c_float(scale), _stream()), "embed")
    return out


def embed_prepare(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                  pending: torch.Tensor | None, scale: float, gain: torch.Tensor,
                  x_out: torch.Tensor, shares: torch.Tensor) -> None:
    """:func:`embed` for up to 8 tokens of a bfloat16 table, with the norm after it prepared for
    the product that follows: ``x_out`` [N, d] = bfloat16(out * gain), ``shares`` [d / 8, 8] the
    tokens' sums of squares in groups of 8 features (see scratch_llm_b200.parts.stream)."""
    _need(ids, torch.int32, "ids")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _need(table, torch.bfloat16, "table")
    _need(out, torch.float32, "out")
    _need(gain, torch.float32, "gain")
    _need(x_out, torch.bfloat16, "x_out", contiguous=False)
    _need(shares, torch.float32, "shares")
    n, d = ids.numel(), table.shape[1]
    if n > 8 or d % 8 or out.shape != (n, d) or x_out.shape != (n, d) or gain.numel() != d \
            or shares.shape != (d // 8, 8) or x_out.stride(1) != 1:
        raise KernelError("embed_prepare shapes")
    _check(_core("sllm_elementwise").sllm_embed_prepare(
        _ptr(ids), _ptr(pending) if pending is not None else c_void_p(0), _ptr(table), _ptr(out),
        c_int(n), c_int(d), c_float(scale), _ptr(gain), _ptr(x_out), c_int64(x_out.stride(0)),
        _ptr(shares), _stream()), "embed_prepare")


def logit_cap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on 32-bit logits: ``cap * tanh(logits * scale / cap)``, or ``logits * scale``
    when ``cap`` is 0."""
    _need(logits, torch.float32, "logits")
    if not logits.is_contiguous():
        raise KernelError("logits must be contiguous")
    if cap < 0:
        raise KernelError(f"cap must not be negative, got {cap}")
    _check(_core("sllm_elementwise").sllm_logit_cap(
        _ptr(logits), c_int64(logits.numel()), c_float(scale), c_float(cap), _stream()),
        "logit_cap")
    return logits


def add_rmsnorm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                eps: float, out: torch.Tensor, index: torch.Tensor | None = None) -> torch.Tensor:
    """resid += delta (if given), out = rmsnorm(resid) * weight.  With ``index`` only the rows
    ``index`` are normed into out[0..len(index)) and resid is left as it was."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(out, None, "out")
    d = resid.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape != resid.shape:
            raise KernelError("delta and resid differ in shape")
    if weight.numel() != d or out.shape[-1] != d:
        raise KernelError("norm width mismatch")
    if index is not None:
        _need(index, torch.int32, "index")
        n_out = index.numel()
    else:
        n_out = resid.shape[0]
    if out.shape[0] != n_out:
        raise KernelError("out has the wrong number of rows")
    _check(_core("sllm_elementwise").sllm_add_rmsnorm(
        _ptr(resid), _ptr(delta), _ptr(index), _ptr(weight), c_float(eps), _ptr(out),
        c_int(n_out), c_int(d), c_int(_code(out.dtype)), _stream()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, f] = silu(gate_up[n, f]) * gate_up[n, F + f]."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2):
        raise KernelError("swiglu shapes")
    _check(_core("sllm_elementwise").sllm_swiglu(
        _ptr(gate_up), _ptr(out), c_int(n), c_int(two_f // 2), c_int(_code(out.dtype)),
        _stream()), "swiglu")
    return out


# ------------------------------------------------------------------------------------ gemm

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T with 32-bit fused multiply-adds on the CUDA cores."""
    _need(x, None, "x", contiguous=False)
    _need(w, x.dtype, "w", contiguous=False)
    _need(out, None, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemm shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    _check(_core("sllm_gemm_simt").sllm_gemm_simt(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(_code(x.dtype)),
        c_int(_code(out.dtype)), _stream()), "gemm_simt")
    return out


#: the streaming small-batch product takes up to this many tokens
GEMV_MAX_TOKENS = 64


def _gate_code(swiglu: bool, activation) -> int:
    """What the fused gate/up kernels take: 0 = a plain product, 1 = silu(gate) * up, 2 = the
    tanh form of gelu on the gate, 3 = the clamped form ``("clamped", limit, slope)``."""
    if not swiglu:
        return 0
    if isinstance(activation, tuple):
        activation = activation[0]
    try:
        return {"silu": 1, "gelu_tanh": 2, "clamped": 3}[activation]
    except KeyError:
        raise KernelError(f"unknown gate activation {activation!r}") from None


def _gate_params(activation) -> tuple:
    """The two numbers of an activation that has some: ``("clamped", limit, slope)`` is, with
    g = min(gate, limit) and u = clamp(up, -limit, limit), g * sigmoid(slope * g) * (u + 1)."""
    if isinstance(activation, tuple):
        return c_float(activation[1]), c_float(activation[2])
    return c_float(0.0), c_float(0.0)


def gemv_mma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False,
             activation: str = "silu") -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 tokens (bfloat16 operands, tensor cores,
    32-bit accumulation), streaming w once.  ``swiglu``: w = [gate rows; up rows] and
    out[M, N/2] = silu(x gate^T) * (x up^T).  ``out`` is bfloat16 or float32."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(out, None, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if k != k2 or out.shape != (m, n_out) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemv shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    if m > GEMV_MAX_TOKENS or k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemv_mma takes up to {GEMV_MAX_TOKENS} tokens and rows that are "
                          f"multiples of 8 elements; got M={m}, K={k}")
    _check(_core("sllm_gemv_mma").sllm_gemv_mma(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(_gate_code(swiglu, activation)),
        c_int(_code(out.dtype)), *_gate_params(activation), _stream()), "gemv_mma")
    return out


#: workspaces of the persistent small-batch product, per device: the words through which the
#: ranges of K exchange partial sums (zero between launches).  A
#: workspace that has been handed to a launch is never freed (a captured CUDA graph may hold its
#: address), so a larger one is made beside it when a wider matrix comes.
_gemv_workspaces: dict[int, list[torch.Tensor]] = {}
_sm_counts: dict[int, int] = {}


def _sm_count(device: torch.device | int | None = None) -> int:
    index = device.index if isinstance(device, torch.device) else device
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def sm_count(device: torch.device | int | None = None) -> int:
    """SMs of ``device`` (the current one by default)."""
    return _sm_count(device)


def gemv_tma_supports(m: int, n: int, k: int, swiglu: bool = False) -> bool:
    """Whether :func:`gemv_tma` takes a product of these sizes (on the current device)."""
    return bool(_core("sllm_gemv_tma").sllm_gemv_tma_supports(
        c_int(m), c_int(n), c_int(k), c_int(int(swiglu)), c_int(_sm_count())))


def gemv_tma_reserve(n: int, k: int, swiglu: bool, device: torch.device) -> torch.Tensor:
    """A zeroed workspace on ``device`` that is large enough for a weight [n, k].  Called when a
    model is built, so that no step allocates it."""
    lib = _core("sllm_gemv_tma")
    lib.sllm_gemv_tma_workspace_bytes.restype = ctypes.c_int64
    need = int(lib.sllm_gemv_tma_workspace_bytes(c_int(n), c_int(k), c_int(int(swiglu)),
                                                 c_int(_sm_count(device))))
    index = device.index if device.index is not None else torch.cuda.current_device()
    held = _gemv_workspaces.setdefault(index, [])
    if not held or held[-1].numel() < need:
        held.append(torch.zeros(need, dtype=torch.uint8, device=device))
    return held[-1]


def gemv_tma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None, swiglu: bool = False,
             scale: tuple[torch.Tensor, int, float] | None = None,
             sink: tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
             activation: str = "silu") -> torch.Tensor | None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 8 tokens by the persistent kernel that streams w
    through shared memory with bulk copies (one CTA per SM, four ranges of K whose partial sums
    the last CTA of a row tile adds in a fixed order).  ``swiglu`` as in :func:`gemv_mma`.
    Launches share one workspace per device and must be ordered by their stream.

    ``scale = (shares, dim, eps)``: x is a stream times a norm's gain whose RMS norm is not
    finished; every output of token t is multiplied by ``rsqrt(shares[:, t].sum() / dim + eps)``
    (``shares`` float32 [parts, 8]).  ``sink = (resid, gain, x_out, shares_out)`` (not with
    ``swiglu``): the output is added into the 32-bit stream ``resid`` [M, N] instead of being
    stored (``out`` may be None), ``x_out`` [M, N] bfloat16 gets ``resid * gain`` and
    ``shares_out`` float32 [ceil(N / 8), 8] the tokens' sums of squares over each 8 features."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if out is not None:
        _need(out, None, "out", contiguous=False)
        if out.shape != (m, n_out) or out.stride(1) != 1:
            raise KernelError(f"gemv out must be [{m}, {n_out}] with contiguous rows")
    elif sink is None:
        raise KernelError("gemv_tma needs an output or a sink")
    if k != k2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemv shapes/strides: x {list(x.shape)}, w {list(w.shape)}")
    if not gemv_tma_supports(m, n, k, swiglu) or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemv_tma takes 1 to 8 tokens, K a multiple of 256 and at least 1024, "
                          f"and rows that are multiples of 8 elements; got M={m}, N={n}, K={k}")
    ss_in, ss_parts, ss_dim, ss_eps = None, 0, 1, 0.0
    if scale is not None:
        ss_in, ss_dim, ss_eps = scale
        _need(ss_in, torch.float32, "scale shares")
        if ss_in.dim() != 2 or ss_in.shape[1] != 8 or ss_dim < 1:
            raise KernelError("scale shares must be float32 [parts, 8]")
        ss_parts = ss_in.shape[0]
    resid = gain = x_out = ss_out = None
    if sink is not None:
        if swiglu:
            raise KernelError("a sink cannot follow the fused activation")
        resid, gain, x_out, ss_out = sink
        _need(resid, torch.float32, "resid", contiguous=False)
        _need(gain, torch.float32, "gain")
        _need(x_out, torch.bfloat16, "x_out", contiguous=False)
        _need(ss_out, torch.float32, "shares_out")
        if resid.shape != (m, n) or x_out.shape != (m, n) or gain.numel() != n \
                or resid.stride(1) != 1 or x_out.stride(1) != 1 \
                or ss_out.numel() < -(-n // 8) * 8:
            raise KernelError("sink shapes: resid and x_out [M, N], gain [N], shares [ceil(N/8), 8]")
    workspace = gemv_tma_reserve(n, k, swiglu, x.device)
    _check(_core("sllm_gemv_tma").sllm_gemv_tma(
        _ptr(x), _ptr(w), _ptr(out), _ptr(workspace), c_int(m), c_int(n), c_int(k),
        c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0) if out is not None else 0),
        c_int(_gate_code(swiglu, activation)), c_int(_code(out.dtype) if out is not None else 1),
        c_int(_sm_count(x.device)), _ptr(ss_in), c_int(ss_parts), c_int(ss_dim), c_float(ss_eps),
        _ptr(resid), c_int64(resid.stride(0) if resid is not None else 0), _ptr(gain), _ptr(x_out),
        c_int64(x_out.stride(0) if x_out is not None else 0), _ptr(ss_out),
        *_gate_params(activation), _stream()), "gemv_tma")
    if sink is not None:    # (counted beside "gemv_tma": which steps handed a norm over)
        launch_counts["gemv_tma_sink"] = launch_counts.get("gemv_tma_sink", 0) + 1
    return out


def gemv_tma_error() -> int:
    """The first error a gemv_tma kernel recorded since the last call (0 = none)."""
    return int(_core("sllm_gemv_tma").sllm_gemv_tma_error())


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False,
            activation: str = "silu") -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T in bfloat16 on tcgen05 tensor cores (TMA-fed, accumulator
    in tensor memory).  ``swiglu``: w = [gate rows; up rows], out[M, N/2] = silu(gate) * up."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(out, torch.bfloat16, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if k != k2 or out.shape != (m, n_out) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemm shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    if k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError("gemm_tc needs rows that are multiples of 8 elements (16 bytes)")
    _check(_core("sllm_gemm_tcgen05").sllm_gemm_tc(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(_gate_code(swiglu, activation)),
        *_gate_params(activation), _stream()), "gemm_tc")
    return out


def gemm_tc_set_pairs(on: bool) -> None:
    """Choose the tcgen05 GEMM kernel: pairs of SMs with 256 x 256 tiles (the default) or single
    SMs with 128 x 256 tiles."""
    _core("sllm_gemm_tcgen05").sllm_gemm_tc_set_pairs(c_int(int(on)))


def gemm_tc_set_tile(features: int | None) -> None:
    """Features per tile of the pair kernel's fused gate/up product: None lets the launcher
    choose (the width whose tiles fill the SM pairs' rounds best), else a multiple of 16 from 16
    to 128."""
    _core("sllm_gemm_tcgen05").sllm_gemm_tc_set_tile(c_int(int(features or 0)))


def gemm_tc_swiglu_tile(m: int, half: int, pairs: int) -> int:
    """The tile width the pair kernel uses for gate/up + SwiGLU of ``m`` tokens and ``half``
    features on ``pairs`` SM pairs."""
    return int(_core("sllm_gemm_tcgen05").sllm_gemm_tc_swiglu_tile(c_int(m), c_int(half),
                                                                   c_int(pairs)))


def gemm_tc_error() -> int:
    """The first error a bounded wait inside gemm_tc recorded since the last call (0 = none).
    Synchronises the device."""
    return int(_core("sllm_gemm_tcgen05").sllm_gemm_tc_error())


# --------------------------------------------------------------------------- rope and cache

def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                  cos: torch.Tensor | None, sin: torch.Tensor | None, pages: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, n_heads: int, n_kv_heads: int,
                  head_dim: int, interleaved: bool, write: bool,
                  bias: torch.Tensor | None = None) -> None:
    """Rotate q (in place) and k by their positions' angles; store k and v into the pages.
    ``cos``/``sin`` None stores k as it is (the position encoding was applied before).  Tables
    of fewer than ``head_dim / 2`` columns rotate only the first ``2 * columns`` entries of each
    head.  ``bias`` (float32 [(H + 2 G) * head_dim]) is added to q, k and v first."""
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    _need(token_row, torch.int32, "token_row")
    _need(pages, qkv.dtype, "pages")
    _need(block_table, torch.int32, "block_table", contiguous=False)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("qkv width does not match the head counts")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    rotate = cos is not None
    if rotate:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if cos.shape[1] > head_dim // 2 or cos.shape[1] < 1 or sin.shape != cos.shape:
            raise KernelError("rotary table width")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("bias must have one entry per column of qkv")
    if block_table.stride(1) != 1:
        raise KernelError("block_table rows must be contiguous")
    _check(_core("sllm_rope_cache").sllm_rope_kv_write(
        _ptr(qkv), _ptr(positions), _ptr(token_row), _ptr(cos), _ptr(sin), _ptr(pages),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), c_int(n),
        c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(int(rotate)),
        c_int(int(interleaved)), c_int(int(write)), c_int(_code(qkv.dtype)), _ptr(bias),
        c_int(2 * cos.shape[1] if rotate else 0), _stream()),
        "rope_kv_write")


# -------------------------------------------------------------------------------- attention

def _page_planes(pages: torch.Tensor, n_kv_heads: int, page_size: int, head_dim: int) -> int:
    """Pages are [n_pages, planes, kv heads, page size, head size]: two planes hold keys, then
    values; one plane holds one vector per token that is its key and, by its leading entries,
    its value (a cache of latents).  Returns the number of planes."""
    if pages.dim() != 5 or pages.shape[1] not in (1, 2) \
            or pages.shape[2:] != (n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 1 or 2, {n_kv_heads}, {page_size}, "
                          f"{head_dim}], got {list(pages.shape)}")
    return int(pages.shape[1])


def _head_vectors(slopes: torch.Tensor | None, sinks: torch.Tensor | None, n_heads: int) -> None:
    for t, name in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n_heads:
                raise KernelError(f"{name} must have one entry per query head")


def attention_simt(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                   page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                   out: torch.Tensor, n_rows: int, max_new: int, n_heads: int, n_kv_heads: int,
                   head_dim: int, scale: float, window: int | None,
                   slopes: torch.Tensor | None = None,
                   sinks: torch.Tensor | None = None, softcap: float = 0.0,
                   chunk: int | None = None) -> torch.Tensor:
    """Causal attention of the packed batch over the paged cache (CUDA cores, 32-bit math).
    ``softcap`` > 0: the scaled score s becomes ``softcap * tanh(s / softcap)``; ``chunk``: the
    query at position p sees only keys from ``p // chunk * chunk`` on.
    ``q`` may be a column slice of a wider buffer (the fused qkv).  ``slopes`` (float32 [H]):
    ``slopes[h] * (query position - key position)`` is taken off head h's scaled scores;
    ``sinks`` (float32 [H]): ``exp(sinks[h])`` joins head h's softmax denominator once, with no
    value behind it."""
    _head_vectors(slopes, sinks, n_heads)
    _need(q, None, "q", contiguous=False)
    _need(pages, q.dtype, "pages")
    _need(out, q.dtype, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    planes = _page_planes(pages, n_kv_heads, page_size, head_dim)
    if not 1 <= head_dim <= SIMT_MAX_HEAD_DIM:
        raise KernelError(f"head size {head_dim}: the CUDA-core attention kernel takes 1 to "
                          f"{SIMT_MAX_HEAD_DIM}")
    lib = _load(*attention_library(head_dim))
    _check(lib.sllm_attn_simt(
        _ptr(q), c_int64(q.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(out), c_int64(out.stride(0)), c_int(n_rows), c_int(max_new), c_int(n_heads),
        c_int(n_kv_heads), c_float(scale), c_int(window or 0), _ptr(slopes), _ptr(sinks),
        c_int(planes), c_float(softcap), c_int(chunk or 0), c_int(_code(q.dtype)), _stream()),
        "attention_simt")
    return out


def attention_mma(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                  page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                  out: torch.Tensor, row_list: torch.Tensor | None, n_list: int, max_new: int,
                  n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                  window: int | None, split: bool, n_splits: int = 1,
                  scratch: torch.Tensor | None = None, slopes: torch.Tensor | None = None,
                  sinks: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                  merge_inside: bool = False, softcap: float = 0.0,
                  chunk: int | None = None) -> torch.Tensor:
    """Causal attention of the listed rows over the paged cache on the tensor cores
    (bfloat16).  ``softcap`` / ``chunk`` as in :func:`attention_simt`.  ``split`` False: the wide kernel for rows with many new tokens; True: the
    split kernel for decode rows, ``n_splits`` CTAs along the keys, partial results in
    ``scratch`` (32-bit, :func:`attention_mma_scratch_floats` entries) when ``n_splits`` > 1.
    ``slopes`` / ``sinks`` as in :func:`attention_simt`.  ``gate`` [N, H * hd] (may be a column
    slice): every output is multiplied by ``sigmoid(gate)`` before it is stored.
    ``merge_inside`` (split rows of one token, head sizes that are multiples of 64): the CTA that
    finishes last for a row, kv head and tile of 16 query heads merges the splits, no merge kernel follows (launches
    share the counters per device and must be ordered by their stream)."""
    _head_vectors(slopes, sinks, n_heads)
    gate_per_head = False
    if gate is not None:
        _need(gate, torch.bfloat16, "gate", contiguous=False)
        gate_per_head = gate.shape == (q.shape[0], n_heads) and head_dim != 1
        if (gate.shape != q.shape and not gate_per_head) or gate.stride(1) != 1:
            raise KernelError("gate must have the queries' shape, or one column per head, and "
                              "contiguous rows")
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    planes = _page_planes(pages, n_kv_heads, page_size, head_dim)
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        raise KernelError(f"head size {head_dim}: the tensor-core attention kernels take "
                          f"multiples of 16 up to {MMA_MAX_HEAD_DIM}")
    n_tokens = q.shape[0]
    if split and n_splits > 1:
        need = attention_mma_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None:
            raise KernelError("the split kernel needs scratch memory for its partial results")
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"scratch holds {scratch.numel()} floats, {need} are needed")
    counters = None
    if merge_inside and split and n_splits > 1 and max_new == 1 and head_dim % 64 == 0:
        counters = _merge_counter(q.device,
                                  n_list * n_kv_heads * -(-(n_heads // n_kv_heads) // 16))
    lib = _load(*attention_mma_library(head_dim))
    _check(lib.sllm_attn_mma(
        _ptr(q), c_int64(q.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(row_list), c_int(n_list), c_int(max_new), _ptr(out), c_int64(out.stride(0)),
        c_int(n_heads), c_int(n_kv_heads), c_float(scale), c_int(window or 0),
        c_int(int(split)), c_int(n_splits), _ptr(scratch), c_int64(n_tokens), _ptr(slopes),
        _ptr(sinks), _ptr(gate), c_int64(gate.stride(0) if gate is not None else 0),
        _ptr(counters), c_int(planes), c_float(softcap), c_int(chunk or 0),
        c_int(int(gate_per_head)), _stream()), "attention_mma")
    return out


_decode_slots: dict[tuple[int, int], int] = {}


def attention_decode_slots(head_dim: int) -> int:
    """CTAs of the split decode attention kernel that the current device holds at once (SMs x
    resident CTAs per SM, asked of the occupancy calculator once per device and head size)."""
    key = (torch.cuda.current_device(), head_dim)
    if key not in _decode_slots:
        n = int(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode_slots())
        if n <= 0:
            raise KernelError("the occupancy of the decode attention kernel could not be read")
        _decode_slots[key] = n
    return _decode_slots[key]


def attention_decode_fused_supported(head_dim: int) -> bool:
    """Whether this head size has the decode attention kernel that rotates q and the new key and
    stores the new key and value itself (head sizes that are multiples of 64)."""
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        return False
    return bool(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode_fused_supported())


#: counters of the decode attention's in-kernel merge, per device (zero between launches; a
#: buffer that has been handed to a launch is never freed: a captured graph may hold its address)
_merge_counters: dict[int, list[torch.Tensor]] = {}


def _merge_counter(device: torch.device, n: int) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    held = _merge_counters.setdefault(index, [])
    if not held or held[-1].numel() < n:
        held.append(torch.zeros(max(n, 4096), dtype=torch.int32, device=device))
    return held[-1]


def attention_mma_decode(qkv: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                         page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                         out: torch.Tensor, row_list: torch.Tensor | None, n_list: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int | None, cos: torch.Tensor, sin: torch.Tensor,
                         interleaved: bool, write: bool, n_splits: int = 1,
                         scratch: torch.Tensor | None = None,
                         merge_inside: bool = True,
                         bias: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention (rows of one new token) over the paged cache on the tensor cores, for
    head sizes that are multiples of 64, straight from the step's fused projection ``qkv``
    [tokens, (H + 2 G) * hd] as the product left it: the kernel rotates q and the new key itself
    (``cos``/``sin`` tables, adjacent pairs if ``interleaved``) and, if ``write``, stores the new
    key and value into ``pages``: no separate rotate-and-store kernel runs.  ``scratch`` as in
    :func:`attention_mma` for several splits; with ``merge_inside`` the CTA that finishes last for
    a row and kv head merges the splits itself (same arithmetic, no merge kernel, nobody waits),
    else a merge kernel follows.  Launches share the merge's counters per device and must be
    ordered by their stream.  Tables of fewer than ``head_dim / 2`` columns turn only the first
    ``2 * columns`` entries of a head; ``bias`` (float32 [(H + 2 G) * head_dim]) is added to q, k
    and v before the rotation."""
    _need(qkv, torch.bfloat16, "qkv", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if qkv.stride(1) != 1 or out.stride(1) != 1 \
            or qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim \
            or out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention qkv/out layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    if not attention_decode_fused_supported(head_dim) or n_heads % n_kv_heads \
            or n_heads // n_kv_heads > 16:
        raise KernelError(f"attention_mma_decode takes head sizes that are multiples of 64 and "
                          f"groups of up to 16 query heads; got {head_dim}, {n_heads}/{n_kv_heads}")
    if not 1 <= cos.shape[1] <= head_dim // 2 or sin.shape != cos.shape:
        raise KernelError("rotary table width")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("bias must have one entry per column of qkv")
    n_tokens = qkv.shape[0]
    if n_splits > 1:
        need = attention_mma_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None:
            raise KernelError("several splits need scratch memory for their partial results")
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} floats, {need} needed")
    if block_table.stride(1) != 1:
        raise KernelError("block_table rows must be contiguous")
    counters = _merge_counter(qkv.device, n_list * n_kv_heads) \
        if merge_inside and n_splits > 1 else None
    _check(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode_biased(
        _ptr(qkv), c_int64(qkv.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(row_list), c_int(n_list), _ptr(out), c_int64(out.stride(0)), c_int(n_heads),
        c_int(n_kv_heads), c_float(scale), c_int(window or 0), c_int(n_splits), _ptr(scratch),
        c_int64(n_tokens), _ptr(cos), _ptr(sin), c_int(int(interleaved)), c_int(int(write)),
        _ptr(counters), _ptr(bias), c_int(2 * cos.shape[1]), _stream()), "attention_mma_decode")
    return out


def attention_tc(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, page_size: int,
                 row_start: torch.Tensor, row_pos0: torch.Tensor, out: torch.Tensor,
                 row_list: torch.Tensor | None, n_list: int, max_new: int, n_heads: int,
                 n_kv_heads: int, head_dim: int, scale: float, window: int | None = None,
                 slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                 biased: bool = False, softcap: float = 0.0,
                 chunk: int | None = None) -> torch.Tensor:
    """Causal attention of the listed rows (prompt portions) over the paged cache on tcgen05
    tensor cores with S, P and O in tensor memory.  What the cache holds in places beyond a
    row's context never reaches a result (NaN included).  With ``biased`` (or any of ``window``,
    ``slopes``, ``sinks``, as in :func:`attention_simt`) the kernel with one query tile per CTA
    runs, which skips key tiles behind the window and never reads pages the row gave back; it
    also takes ``softcap`` and ``chunk`` (as in :func:`attention_simt`)."""
    biased = biased or bool(window) or slopes is not None or sinks is not None \
        or softcap > 0 or bool(chunk)
    _head_vectors(slopes, sinks, n_heads)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if not attention_tc_supports(n_heads, n_kv_heads, head_dim, page_size, window, biased):
        raise KernelError("attention_tc does not take this shape")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    planes = _page_planes(pages, n_kv_heads, page_size, head_dim)
    lib = _load(*attention_tc_library(head_dim))
    common = (_ptr(q), c_int64(q.stride(0)), c_int64(q.shape[0]), _ptr(pages),
              c_int64(pages.shape[0]), _ptr(block_table), c_int(block_table.stride(0)),
              c_int(page_size), _ptr(row_start), _ptr(row_pos0), _ptr(row_list), c_int(n_list),
              c_int(max_new), _ptr(out), c_int64(out.stride(0)), c_int(n_heads), c_int(n_kv_heads),
              c_float(scale))
    if biased:
        if planes != 2:
            raise KernelError("the biased tcgen05 attention takes pages of keys and values")
        _check(lib.sllm_attn_tc_biased(*common, c_int(window or 0), _ptr(slopes), _ptr(sinks),
                                       c_float(softcap), c_int(chunk or 0), _stream()),
               "attention_tc")
    else:
        _check(lib.sllm_attn_tc(*common, c_int(planes), _stream()), "attention_tc")
    return out


def attention_tc_set_two_tiles(head_dim: int, mode: int | bool | None) -> None:
    """Choose the tcgen05 attention kernel for head sizes up to 128.  None (the default):
    two query tiles per CTA, which share every key/value tile, when the launch has at least as
    many such CTAs as the device has SMs, else one; True: always two; False: always one."""
    code = 1 if mode is None else (2 if mode else 0)
    _load(*attention_tc_library(head_dim)).sllm_attn_tc_set_two_tiles(c_int(code))


def attention_tc_error(head_dim: int) -> int:
    return int(_load(*attention_tc_library(head_dim)).sllm_attn_tc_error())


def check_kernel_errors() -> None:
    """Raise if a kernel of a loaded library gave up a bounded wait since the last check (the
    kernels that use mbarriers or flags record a code instead of hanging).  Synchronises the
    device: call it where the host waits anyway (the end of a request batch, of a trace)."""
    found = []
    for name, lib in list(_loaded.items()):
        for symbol in ("sllm_gemm_tc_error", "sllm_gemv_tma_error", "sllm_attn_tc_error"):
            if hasattr(lib, symbol):
                code = int(getattr(lib, symbol)())
                if code:
                    found.append(f"{name}: code {code}")
    if found:
        raise KernelError("a kernel gave up waiting (its results are not valid): " +
                          "; ".join(found))


def attention_mma_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_tokens * n_heads * n_splits * (head_dim + 1) if n_splits > 1 else 0


# --------------------------------------------------------------------------------- sampling

def argmax_scratch_bytes(n_rows: int) -> int:
    lib = _core("sllm_sampling")
    lib.sllm_argmax_scratch_bytes.restype = c_int64
    return int(lib.sllm_argmax_scratch_bytes(c_int(n_rows)))


def argmax(logits: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, rows_capacity: int
           ) -> torch.Tensor:
    """out[r] = first maximum of logits[r] (32-bit, [n, V]), many blocks per row.  ``scratch``:
    uint8 of ``argmax_scratch_bytes(rows_capacity)``, zero-filled once; its layout depends on
    ``rows_capacity``, which must be the same on every call with this scratch."""
    _need(logits, torch.float32, "logits", contiguous=False)
    _need(out, torch.int32, "out")
    _need(scratch, torch.uint8, "scratch")
    n, v = logits.shape
    if logits.stride(1) != 1 or out.numel() != n or n != rows_capacity \
            or scratch.numel() < argmax_scratch_bytes(rows_capacity):
        raise KernelError("argmax shapes")
    _check(_core("sllm_sampling").sllm_argmax(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(scratch), _ptr(out),
        _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seed: torch.Tensor | None = None,
           counter: torch.Tensor | None = None, logprob_out: torch.Tensor | None = None,
           probs_out: torch.Tensor | None = None) -> torch.Tensor:
    """Choose one token per row of ``logits`` [n, V] (32-bit).  Rows whose temperature is 0
    (or all rows when ``temperature`` is None) take the argmax.  seed/counter: int64 [n]."""
    _need(logits, torch.float32, "logits", contiguous=False)
    _need(out, torch.int32, "out")
    n, v = logits.shape
    if logits.stride(1) != 1 or out.numel() != n:
        raise KernelError("sample shapes")
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                        (seed, torch.int64, "seed"), (counter, torch.int64, "counter"),
                        (logprob_out, torch.float32, "logprob_out")):
        if t is not None:
            _need(t, dt, name)
            if t.numel() != n:
                raise KernelError(f"{name} must have one entry per row")
    if probs_out is not None:
        _need(probs_out, torch.float32, "probs_out")
        if probs_out.shape != (n, v):
            raise KernelError("probs_out shape")
    _check(_core("sllm_sampling").sllm_sample(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(temperature),
        _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out), _ptr(logprob_out), _ptr(probs_out),
        _stream()), "sample")
    return out


def log_softmax(logits: torch.Tensor, rows_out: torch.Tensor | None = None,
                taken: torch.Tensor | None = None, taken_out: torch.Tensor | None = None) -> None:
    """log_softmax of each row of ``logits`` [n, V] (32-bit).  ``rows_out`` [n, V] gets the whole
    rows; ``taken`` (int32 [n]) and ``taken_out`` (float32 [n]) the log-probability of one given
    token per row."""
    _need(logits, torch.float32, "logits", contiguous=False)
    n, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("log_softmax: rows must be contiguous")
    if rows_out is not None:
        _need(rows_out, torch.float32, "rows_out")
        if rows_out.shape != (n, v):
            raise KernelError("rows_out shape")
    if (taken is None) != (taken_out is None):
        raise KernelError("taken and taken_out come together")
    if taken is not None:
        _need(taken, torch.int32, "taken")
        _need(taken_out, torch.float32, "taken_out")
        if taken.numel() != n or taken_out.numel() != n:
            raise KernelError("taken / taken_out must have one entry per row")
    _check(_core("sllm_sampling").sllm_log_softmax(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(rows_out), _ptr(taken),
        _ptr(taken_out), _stream()), "log_softmax")


# ------------------------------------------------- layers that norm a branch's output

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def embed_positional(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
                     out: torch.Tensor, cast_out: torch.Tensor | None = None,
                     pending: torch.Tensor | None = None, scale: float = 1.0,
                     inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    """out[n] = table[ids[n]] * scale (32-bit) plus, with ``inv_freq`` (float32 [ceil(d / 2)]),
    the sinusoidal vector of ``positions[n]``: entry 2i gets sin(p * inv_freq[i]), entry 2i + 1
    the cosine, angles in 32-bit.  ``cast_out`` [N, d] in the table's dtype gets the same rows
    rounded.  Ids ``-1 - j`` stand for ``pending[j]`` as in :func:`embed`."""
    _need(ids, torch.int32, "ids")
    _need(positions, torch.int32, "positions")
    _need(table, None, "table")
    _need(out, torch.float32, "out")
    n, d = ids.numel(), table.shape[1]
    if out.shape != (n, d) or positions.numel() != n:
        raise KernelError(f"out must be [{n}, {d}] and positions [{n}]")
    if cast_out is not None:
        _need(cast_out, table.dtype, "cast_out")
        if cast_out.shape != (n, d):
            raise KernelError("cast_out shape")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() != (d + 1) // 2:
            raise KernelError("inv_freq must have one entry per pair of features")
    _check(_core("sllm_stream_ops").sllm_embed_positional(
        _ptr(ids), _ptr(pending), _ptr(positions), _ptr(table), _ptr(out), _ptr(cast_out),
        c_int(n), c_int(d), c_int(_code(table.dtype)), c_float(scale), _ptr(inv_freq), _stream()),
        "embed_positional")
    return out


def add_normed(resid: torch.Tensor, delta: torch.Tensor, gain: torch.Tensor, eps: float,
               cast_out: torch.Tensor | None = None,
               then: tuple[torch.Tensor, float, torch.Tensor] | None = None) -> None:
    """resid += delta / sqrt(mean(delta^2) + eps) * gain, row by row, in 32-bit; ``cast_out``
    (the dtype of ``delta``) gets the updated rows rounded.  ``then = (gain2, eps2, out2)``:
    ``out2`` (the dtype of ``delta``) gets the RMS norm of the updated rows with ``gain2``, the
    norm in front of the next branch, from the same pass."""
    _need(resid, torch.float32, "resid")
    _need(delta, None, "delta")
    _need(gain, torch.float32, "gain")
    n, d = resid.shape
    if delta.shape != (n, d) or gain.numel() != d:
        raise KernelError("add_normed shapes")
    if cast_out is not None:
        _need(cast_out, delta.dtype, "cast_out")
        if cast_out.shape != (n, d):
            raise KernelError("cast_out shape")
    gain2, eps2, out2 = then if then is not None else (None, 0.0, None)
    if then is not None:
        _need(gain2, torch.float32, "gain2")
        _need(out2, delta.dtype, "out2")
        if gain2.numel() != d or out2.shape != (n, d):
            raise KernelError("add_normed: the next norm's shapes")
    _check(_core("sllm_stream_ops").sllm_add_normed(
        _ptr(resid), _ptr(delta), _ptr(gain), c_float(eps), _ptr(cast_out), _ptr(gain2),
        c_float(eps2), _ptr(out2), c_int(n), c_int(d), c_int(_code(delta.dtype)), _stream()),
        "add_normed")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """out[n, f] = act(gate_up[n, f]) * gate_up[n, F + f]; ``activation``: a key of ACTIVATIONS."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2):
        raise KernelError("gated_act shapes")
    _check(_core("sllm_stream_ops").sllm_gated_act(
        _ptr(gate_up), _ptr(out), c_int(n), c_int(two_f // 2), c_int(ACTIVATIONS[activation]),
        c_int(_code(out.dtype)), _stream()), "gated_act")
    return out


def clamped_gate(gate_up: torch.Tensor, out: torch.Tensor, limit: float,
                 slope: float) -> torch.Tensor:
    """With g = min(gate_up[n, f], limit) and u = clamp(gate_up[n, F + f], -limit, limit):
    out[n, f] = g * sigmoid(slope * g) * (u + 1).  ``out`` may be a column slice."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out", contiguous=False)
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2) or out.stride(1) != 1:
        raise KernelError("clamped_gate shapes")
    _check(_core("sllm_stream_ops").sllm_clamped_gate(
        _ptr(gate_up), _ptr(out), c_int64(out.stride(0)), c_int(n), c_int(two_f // 2),
        c_float(limit), c_float(slope), c_int(_code(out.dtype)), _stream()), "clamped_gate")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x *= sigmoid(gate) in place; both [N, C], rows may be slices of wider buffers."""
    _need(x, None, "x", contiguous=False)
    _need(gate, x.dtype, "gate", contiguous=False)
    if x.shape != gate.shape or x.dim() != 2 or x.stride(1) != 1 or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate shapes")
    _check(_core("sllm_stream_ops").sllm_sigmoid_gate(
        _ptr(x), c_int64(x.stride(0)), _ptr(gate), c_int64(gate.stride(0)), c_int(x.shape[0]),
        c_int(x.shape[1]), c_int(_code(x.dtype)), _stream()), "sigmoid_gate")
    return x


def side_gate(a: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, col0: int,
              out: torch.Tensor, activation: str, pending: torch.Tensor | None = None
              ) -> torch.Tensor:
    """out[n, j] = act(a[n, j]) * table[ids[n], col0 + j]: a per-token vector gathered from the
    columns [col0, col0 + dim) of ``table`` [V, columns], gated by the activations ``a``."""
    _need(a, None, "a")
    _need(ids, torch.int32, "ids")
    _need(table, a.dtype, "table")
    _need(out, a.dtype, "out")
    n, dim = a.shape
    if out.shape != (n, dim) or ids.numel() != n or col0 < 0 or col0 + dim > table.shape[1]:
        raise KernelError("side_gate shapes")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _check(_core("sllm_stream_ops").sllm_side_gate(
        _ptr(a), _ptr(ids), _ptr(pending), _ptr(table), c_int64(table.stride(0)), c_int(col0),
        c_int(dim), c_int(ACTIVATIONS[activation]), _ptr(out), c_int(n), c_int(_code(a.dtype)),
        _stream()), "side_gate")
    return out


def qk_norm_kv_write(x: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                     q_gain: torch.Tensor | None, k_gain: torch.Tensor | None, eps: float,
                     temp_coef: float, temp_every: float, v_col0: int | None,
                     pages: torch.Tensor, block_table: torch.Tensor, page_size: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, write: bool) -> None:
    """Per-head RMS norm of the queries (in place, times ``1 + temp_coef * ln(floor((p + 1) /
    temp_every) + 1)`` at position p when ``temp_coef`` is not 0) and of the keys of ``x``
    [N, >= (H + G) * hd]; the normed keys go into the K pages, and into the V pages go the value
    heads at column ``v_col0`` of ``x``, or, with ``v_col0`` None, the keys as projected."""
    _need(x, None, "x", contiguous=False)
    _need(positions, torch.int32, "positions")
    _need(token_row, torch.int32, "token_row")
    _need(pages, x.dtype, "pages")
    _need(block_table, torch.int32, "block_table", contiguous=False)
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _need(g, torch.float32, name)
            if g.numel() != head_dim:
                raise KernelError(f"{name} must have head_dim entries")
    if x.stride(1) != 1 or x.shape[1] < (n_heads + n_kv_heads) * head_dim:
        raise KernelError("qk_norm_kv_write: x layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    if block_table.stride(1) != 1:
        raise KernelError("block_table rows must be contiguous")
    _check(_core("sllm_qk_norm_cache").sllm_qk_norm_kv_write(
        _ptr(x), c_int64(x.stride(0)), _ptr(positions), _ptr(token_row), _ptr(q_gain),
        _ptr(k_gain), c_float(eps), c_float(temp_coef), c_float(temp_every),
        c_int(-1 if v_col0 is None else v_col0), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), c_int(x.shape[0]), c_int(n_heads),
        c_int(n_kv_heads), c_int(head_dim), c_int(int(write)), c_int(_code(x.dtype)), _stream()),
        "qk_norm_kv_write")


# ---------------------------------------------------------------------- recurrent mixers

def conv_silu(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor | None,
              token_row: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor,
              out: torch.Tensor, taps_t: torch.Tensor | None = None) -> torch.Tensor:
    """Short causal convolution over time and silu on the first C columns of ``x`` [N, >= C]:
    ``taps`` float32 [C, K] (the last tap is the current token's), ``state`` [slots, K - 1, C]
    the inputs carried from earlier steps (None when K is 1), ``out`` [N, C].  ``taps_t``: the
    taps' transpose [K, C] (contiguous), which lets bfloat16 rows of whole 16 bytes take the
    kernel with 16-byte accesses."""
    _need(x, None, "x", contiguous=False)
    _need(taps, torch.float32, "taps")
    _need(out, x.dtype, "out")
    for t, name in ((token_row, "token_row"), (row_start, "row_start"), (row_slot, "row_slot")):
        _need(t, torch.int32, name)
    c, k = taps.shape
    if x.stride(1) != 1 or x.shape[1] < c or out.shape != (x.shape[0], c):
        raise KernelError("conv_silu shapes")
    if k > 1:
        if state is None:
            raise KernelError("a convolution of several taps needs its carried inputs")
        _need(state, x.dtype, "state")
        if state.shape[1:] != (k - 1, c):
            raise KernelError(f"conv state must be [slots, {k - 1}, {c}]")
    if taps_t is not None:
        _need(taps_t, torch.float32, "taps_t")
        if taps_t.shape != (k, c):
            raise KernelError("taps_t must be the transpose of taps")
    _check(_core("sllm_recurrent_ops").sllm_conv_silu(
        _ptr(x), c_int64(x.stride(0)), _ptr(taps), _ptr(taps_t), c_int(k),
        _ptr(state if k > 1 else None),
        _ptr(token_row), _ptr(row_start), _ptr(row_slot), _ptr(out), c_int(c),
        c_int(x.shape[0]), c_int(_code(x.dtype)), _stream()), "conv_silu")
    return out


def conv_state_update(x: torch.Tensor, n_taps: int, state: torch.Tensor, row_start: torch.Tensor,
                      row_slot: torch.Tensor, n_rows: int) -> None:
    """The carried inputs of :func:`conv_silu` after this step's tokens (rows without tokens keep
    theirs)."""
    if n_taps <= 1:
        return
    _need(x, None, "x", contiguous=False)
    _need(state, x.dtype, "state")
    _need(row_start, torch.int32, "row_start")
    _need(row_slot, torch.int32, "row_slot")
    c = state.shape[2]
    if state.shape[1] != n_taps - 1 or x.shape[1] < c or x.stride(1) != 1:
        raise KernelError("conv_state_update shapes")
    _check(_core("sllm_recurrent_ops").sllm_conv_state_update(
        _ptr(x), c_int64(x.stride(0)), c_int(n_taps), _ptr(state), _ptr(row_start),
        _ptr(row_slot), c_int(c), c_int(n_rows), c_int(_code(x.dtype)), _stream()),
        "conv_state_update")


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, eps: float,
                   out: torch.Tensor, n_heads: int, gate_activation: str = "silu") -> torch.Tensor:
    """out[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * gain * act(gate[n, h, :]);
    ``o`` float32 [N, H * V], ``gate`` [N, H * V] (may be a column slice), ``gain`` float32 [V]
    (the same for every head) or [H * V]; ``gate_activation``: "silu" or "sigmoid".  ``out`` may
    be a column slice of a wider buffer."""
    _need(o, torch.float32, "o")
    _need(gate, out.dtype, "gate", contiguous=False)
    _need(gain, torch.float32, "gain")
    _need(out, None, "out", contiguous=False)
    n, hv = o.shape
    if hv % n_heads or gain.numel() not in (hv, hv // n_heads):
        raise KernelError("head_norm_gate: the gain has one entry per channel of a head, or of all")
    v = hv // n_heads
    per_head = gain.numel() == hv and n_heads > 1
    if gate.shape != (n, hv) or out.shape != (n, hv) or gate.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_norm_gate shapes")
    try:
        act = {"silu": 0, "sigmoid": 1}[gate_activation]
    except KeyError:
        raise KernelError(f"unknown gate activation {gate_activation!r}") from None
    _check(_core("sllm_recurrent_ops").sllm_head_norm_gate(
        _ptr(o), _ptr(gate), c_int64(gate.stride(0)), _ptr(gain), c_float(eps), _ptr(out),
        c_int64(out.stride(0)), c_int(n), c_int(n_heads), c_int(v), c_int(int(per_head)), c_int(act),
        c_int(_code(out.dtype)), _stream()), "head_norm_gate")
    return out


def lowrank_decay(pre: torch.Tensor, w2t: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor,
                  decay_scale: float, out: torch.Tensor) -> torch.Tensor:
    """Decays and removal rates of a delta-rule mixer (csrc/recurrent_ops.cu): ``pre`` float32
    [N, C + R] holds the removal rates' inputs and the low-rank hidden values, ``w2t`` float32
    [R, C]; ``out`` float32 [N, 2 C] gets ``exp(-decay_scale * sigmoid(w0 + tanh(hidden) w2t))``
    and ``sigmoid(pre[:, :C] + a_bias)``."""
    for t, name in ((pre, "pre"), (w2t, "w2t"), (w0, "w0"), (a_bias, "a_bias"), (out, "out")):
        _need(t, torch.float32, name, contiguous=name != "pre")
    r, c = w2t.shape
    n = pre.shape[0]
    if pre.stride(1) != 1 or pre.shape[1] != c + r or w0.numel() != c or a_bias.numel() != c \
            or out.shape != (n, 2 * c):
        raise KernelError("lowrank_decay shapes")
    _check(_core("sllm_recurrent_ops").sllm_lowrank_decay(
        _ptr(pre), c_int64(pre.stride(0)), _ptr(w2t), _ptr(w0), _ptr(a_bias),
        c_float(decay_scale), _ptr(out), c_int(n), c_int(c), c_int(r), _stream()), "lowrank_decay")
    return out


def general_delta_padded_dim(key_dim: int) -> int:
    """The key size as the generalized delta rule's state stores it (padded to whole lanes)."""
    return int(_load(*general_delta_library(key_dim)).sllm_general_delta_padded_dim())


def general_delta(rkv: torch.Tensor, cols: tuple[int, int, int], wa: torch.Tensor,
                  state: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor,
                  out: torch.Tensor, n_rows: int, n_heads: int, key_dim: int, value_dim: int,
                  unit_eps: float) -> torch.Tensor:
    """The generalized delta rule over the packed batch (csrc/general_delta.cu): ``rkv`` [N, >=]
    holds the heads' receptances, keys and values from the columns ``cols`` on; ``wa`` float32
    [N, 2 H D] the decays and removal rates; ``state`` float32 [slots, H, V, padded D] is read
    and written at the rows' slots; ``out`` float32 [N, H * V]."""
    _need(rkv, None, "rkv", contiguous=False)
    _need(wa, torch.float32, "wa")
    _need(state, torch.float32, "state")
    _need(row_start, torch.int32, "row_start")
    _need(row_slot, torch.int32, "row_slot")
    _need(out, torch.float32, "out")
    n = rkv.shape[0]
    r0, k0, v0 = cols
    hd, hv = n_heads * key_dim, n_heads * value_dim
    if rkv.stride(1) != 1 or max(r0 + hd, k0 + hd, v0 + hv) > rkv.shape[1] or min(cols) < 0 \
            or wa.shape != (n, 2 * hd) or out.shape != (n, hv) \
            or state.shape[1:] != (n_heads, value_dim, general_delta_padded_dim(key_dim)):
        raise KernelError("general_delta shapes")
    _check(_load(*general_delta_library(key_dim)).sllm_general_delta(
        _ptr(rkv), c_int64(rkv.stride(0)), c_int(r0), c_int(k0), c_int(v0), _ptr(wa),
        c_int64(wa.stride(0)), _ptr(state), _ptr(row_start), _ptr(row_slot), _ptr(out),
        c_int(n_rows), c_int(n_heads), c_int(value_dim), c_float(unit_eps),
        c_int(_code(rkv.dtype)), _stream()), "general_delta")
    return out


# ------------------------------------------------------------- a tanh in the place of a norm

def dyt_norm(resid: torch.Tensor, alpha: float, w: torch.Tensor, b: torch.Tensor,
             out: torch.Tensor, index: torch.Tensor | None = None,
             shift: tuple | None = None) -> torch.Tensor:
    """out = tanh(alpha * resid) * w + b (32-bit arithmetic, one rounding), for every row or for
    the rows ``index``.  ``shift = (mu, state, token_row, row_start, row_slot, write)``: every
    token's result h_t becomes ``h_t + (h_{t-1} - h_t) * mu``, where a row's first token takes
    h_{t-1} from ``state`` [slots, d] (float32) at the row's slot; with ``write`` rows of one
    token store their h there (rows of more: :func:`dyt_state_update`)."""
    _need(resid, torch.float32, "resid")
    _need(w, torch.float32, "w")
    _need(b, torch.float32, "b")
    _need(out, None, "out")
    d = resid.shape[1]
    n_out = resid.shape[0] if index is None else index.numel()
    if w.numel() != d or b.numel() != d or out.shape != (n_out, d):
        raise KernelError("dyt_norm shapes")
    if index is not None:
        _need(index, torch.int32, "index")
    mu = state = token_row = row_start = row_slot = None
    write = False
    if shift is not None:
        if index is not None:
            raise KernelError("gathered rows have no neighbours to mix with")
        mu, state, token_row, row_start, row_slot, write = shift
        _need(mu, torch.float32, "mu")
        _need(state, torch.float32, "state")
        for t, name in ((token_row, "token_row"), (row_start, "row_start"), (row_slot, "row_slot")):
            _need(t, torch.int32, name)
        if mu.numel() != d or state.dim() != 2 or state.shape[1] != d:
            raise KernelError("dyt_norm: mu [d], state [slots, d]")
    _check(_core("sllm_tanh_norm").sllm_dyt_norm(
        _ptr(resid), _ptr(index), c_int(n_out), c_int(d), c_float(alpha), _ptr(w), _ptr(b),
        _ptr(mu), _ptr(state), _ptr(token_row), _ptr(row_start), _ptr(row_slot), _ptr(out),
        c_int(int(write)), c_int(_code(out.dtype)), _stream()), "dyt_norm")
    return out


def dyt_state_update(resid: torch.Tensor, alpha: float, w: torch.Tensor, b: torch.Tensor,
                     state: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor,
                     n_rows: int, dtype: torch.dtype = torch.float32) -> None:
    """Rows of two tokens or more store ``tanh(alpha * resid) * w + b`` of their last token in
    ``state`` at their slot.  ``dtype``: the output dtype of the :func:`dyt_norm` calls this goes
    with (the serving path forms its tanh another way, and the carried value must be the one a
    token inside a step would meet)."""
    _need(resid, torch.float32, "resid")
    _need(state, torch.float32, "state")
    _need(row_start, torch.int32, "row_start")
    _need(row_slot, torch.int32, "row_slot")
    d = resid.shape[1]
    if w.numel() != d or b.numel() != d or state.shape[1] != d:
        raise KernelError("dyt_state_update shapes")
    _check(_core("sllm_tanh_norm").sllm_dyt_state_update(
        _ptr(resid), c_int(d), c_float(alpha), _ptr(w), _ptr(b), _ptr(state), _ptr(row_start),
        _ptr(row_slot), c_int(n_rows), c_int(_code(dtype)), _stream()), "dyt_state_update")


def dyt_add(resid: torch.Tensor, delta: torch.Tensor, alpha: float, w: torch.Tensor,
            b: torch.Tensor, then: tuple | None = None, out: torch.Tensor | None = None) -> None:
    """resid += tanh(alpha * delta) * w + b in 32-bit; with ``then = (alpha2, w2, b2)`` also
    ``out = tanh(alpha2 * resid) * w2 + b2`` (the dtype of ``delta``) from the updated rows."""
    _need(resid, torch.float32, "resid")
    _need(delta, None, "delta")
    _need(w, torch.float32, "w")
    _need(b, torch.float32, "b")
    n, d = resid.shape
    if delta.shape != (n, d) or w.numel() != d or b.numel() != d:
        raise KernelError("dyt_add shapes")
    a2, w2, b2 = 0.0, None, None
    if then is not None:
        a2, w2, b2 = then
        _need(w2, torch.float32, "w2")
        _need(b2, torch.float32, "b2")
        if out is None or out.shape != (n, d) or out.dtype != delta.dtype or w2.numel() != d \
                or b2.numel() != d:
            raise KernelError("dyt_add: the second norm needs an output of delta's dtype")
        _need(out, delta.dtype, "out")
    _check(_core("sllm_tanh_norm").sllm_dyt_add(
        _ptr(resid), _ptr(delta), c_int(n), c_int(d), c_float(alpha), _ptr(w), _ptr(b),
        c_float(a2), _ptr(w2), _ptr(b2), _ptr(out if then is not None else None),
        c_int(_code(delta.dtype)), _stream()), "dyt_add")


PARAM_ACTIVATIONS = {"xielu": 0}


def param_act(x: torch.Tensor, out: torch.Tensor, activation: str, p0: float, p1: float
              ) -> torch.Tensor:
    """out = act(x; p0, p1) element by element.  "xielu": ``p0 x^2 + x / 2`` for x > 0 and
    ``p1 (exp(x) - 1 - x) + x / 2`` for x <= 0."""
    _need(x, None, "x")
    _need(out, x.dtype, "out")
    if out.shape != x.shape:
        raise KernelError("param_act shapes")
    _check(_core("sllm_stream_ops").sllm_param_act(
        _ptr(x), _ptr(out), c_int64(x.numel()), c_int(PARAM_ACTIVATIONS[activation]), c_float(p0),
        c_float(p1), c_int(_code(x.dtype)), _stream()), "param_act")
    return out


# --------------------------------------------------------------------- routed feed-forward

def moe_tile_rows() -> int:
    return int(_core("sllm_moe").sllm_moe_tile_rows())


#: rows of a tile of the grouped product on tcgen05 (csrc/moe_tc.cu)
MOE_TC_TILE_ROWS = 128


def moe_max_tiles(n_tokens: int, top: int, n_real: int, tile_rows: int) -> int:
    """An upper bound of the row tiles of the grouped products: every expert may end with a
    tile that is not full."""
    pairs = n_tokens * top
    return -(-pairs // tile_rows) + min(n_real, pairs)


#: steps of up to this many (token, choice) pairs are routed, planned, scattered and gathered by
#: one CTA in one launch (decode steps)
MOE_SMALL_PAIRS = 64


#: router variants (bits of ``flags`` in :func:`moe_route`)
MOE_SIGMOID, MOE_GROUP_TOP2, MOE_RAW_WEIGHTS = 1, 2, 4
#: what a grouped product does with its rows (``gated`` in :func:`moe_product`)
MOE_PLAIN, MOE_GATED, MOE_SQRELU = 0, 1, 2


def moe_route(logits: torch.Tensor, correction: torch.Tensor, token_row: torch.Tensor | None,
              n_real: int, n_groups: int, keep: int, top: int, tile_rows: int | None = None,
              gather_from: torch.Tensor | None = None, flags: int = 0):
    """Route every token of ``logits`` (float32 [N, outputs]) and sort the (token, choice) pairs
    by expert (csrc/moe.cu).  Returns ``(ids [N, top], weights [N, top], pair_token [N * top],
    pair_place [N * top], meta, max_tiles, rows)``; ``meta`` is the tile list of the grouped
    products, in tiles of ``tile_rows`` rows (default: what :func:`moe_product` takes).
    ``gather_from`` (bfloat16 [N, K], K % 8 == 0): the caller wants the tokens' rows in the
    sorted order; ``rows`` is that copy where the router made it on its way (steps of few tokens,
    where one CTA does everything in one launch), else None (:func:`moe_gather_rows` makes it).
    ``flags``: ``MOE_SIGMOID`` scores are ``sigmoid(z)`` instead of a softmax over the outputs;
    ``MOE_GROUP_TOP2`` a group's score is the sum of its two largest choice scores instead of its
    largest; ``MOE_RAW_WEIGHTS`` the weights are the chosen scores, not divided by their sum."""
    _need(logits, torch.float32, "logits")
    _need(correction, torch.float32, "correction")
    n, n_total = logits.shape
    if correction.numel() != n_total:
        raise KernelError("correction must have one entry per router output")
    if token_row is not None:
        _need(token_row, torch.int32, "token_row")
    dev = logits.device
    tile_rows = tile_rows or moe_tile_rows()
    max_tiles = moe_max_tiles(n, top, n_real, tile_rows)
    ids = torch.empty((n, top), dtype=torch.int32, device=dev)
    weights = torch.empty((n, top), dtype=torch.float32, device=dev)
    pair_place = torch.empty(n * top, dtype=torch.int32, device=dev)
    lib = _core("sllm_moe")
    if n_real > 0 and n * top <= MOE_SMALL_PAIRS and \
            int(lib.sllm_moe_route_small_smem(c_int(n_total), c_int(n_real), c_int(n_groups))) \
            <= 48 * 1024:
        pair_token = torch.empty(n * top, dtype=torch.int32, device=dev)
        meta = torch.empty(1 + 3 * max_tiles, dtype=torch.int32, device=dev)
        rows = None
        if gather_from is not None:
            _need(gather_from, torch.bfloat16, "gather_from", contiguous=False)
            if gather_from.shape[0] != n or gather_from.stride(1) != 1 \
                    or gather_from.shape[1] % 8 or gather_from.stride(0) % 8:
                raise KernelError("gather_from must be bfloat16 [N, K] with rows of whole 16 bytes")
            rows = torch.empty((n * top, gather_from.shape[1]), dtype=torch.bfloat16, device=dev)
        _check(lib.sllm_moe_route_small(
            _ptr(logits), _ptr(correction), _ptr(token_row), c_int(n), c_int(n_total),
            c_int(n_real), c_int(n_groups), c_int(keep), c_int(top), _ptr(ids), _ptr(weights),
            _ptr(meta), c_int(max_tiles), c_int(tile_rows), _ptr(pair_token), _ptr(pair_place),
            _ptr(gather_from), c_int64(gather_from.stride(0) if gather_from is not None else 0),
            c_int(gather_from.shape[1] if gather_from is not None else 0), _ptr(rows),
            c_int(flags), _stream()), "moe_route_small")
        return ids, weights, pair_token, pair_place, meta, max_tiles, rows
    # one zero fill: the experts' counters (with the offsets, cursors and tile list behind them)
    # and the places' tokens (places that no pair takes name token 0)
    n_scratch = 3 * n_real + 2 + 3 * max_tiles
    zeros = torch.zeros(n_scratch + n * top, dtype=torch.int32, device=dev)
    work, pair_token = zeros[:n_scratch], zeros[n_scratch:]
    _check(lib.sllm_moe_route(
        _ptr(logits), _ptr(correction), _ptr(token_row), c_int(n), c_int(n_total), c_int(n_real),
        c_int(n_groups), c_int(keep), c_int(top), _ptr(ids), _ptr(weights), _ptr(work),
        c_int(max_tiles), c_int(tile_rows), _ptr(pair_token), _ptr(pair_place), c_int(flags),
        _stream()), "moe_route")
    meta = work[3 * n_real + 1:]
    return ids, weights, pair_token, pair_place, meta, max_tiles, None


def moe_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, meta: torch.Tensor,
                pair_token: torch.Tensor, max_tiles: int, gated: bool | int) -> torch.Tensor:
    """The grouped product of a routed feed-forward over the places of ``meta``.  ``gated``
    True (``MOE_GATED``): ``w`` [E, 2 F, K], ``out[place] = silu(x[token] gate^T) * (x[token]
    up^T)`` (the dtype of ``x``); ``MOE_SQRELU``: ``w`` [E, F, K], ``out[place] =
    relu(x[token] w^T)^2`` (the dtype of ``x``); False: ``w`` [E, F, K], ``out[place] = x[place]
    w^T`` in float32."""
    gated = int(gated)
    _need(x, None, "x", contiguous=False)
    _need(w, x.dtype, "w")
    _need(out, x.dtype if gated else torch.float32, "out")
    _need(meta, torch.int32, "meta")
    _need(pair_token, torch.int32, "pair_token")
    f = w.shape[1] // 2 if gated == MOE_GATED else w.shape[1]
    k = w.shape[2]
    if x.stride(1) != 1 or x.shape[1] != k or out.shape[1] != f \
            or out.shape[0] < pair_token.numel():
        raise KernelError("moe_product shapes")
    _check(_core("sllm_moe").sllm_moe_product(
        _ptr(x), c_int64(x.stride(0)), _ptr(w), _ptr(out), c_int64(out.stride(0)), _ptr(meta),
        _ptr(pair_token), c_int(f), c_int(k), c_int(max_tiles), c_int(gated),
        c_int(_code(x.dtype)), _stream()), "moe_product")
    return out


def moe_tc_supports(k: int, f: int) -> bool:
    """Whether the grouped products on tcgen05 take a routed feed-forward of width ``k`` and
    expert size ``f`` (rows of whole 16 bytes for the tensor copies)."""
    return k % 8 == 0 and f % 8 == 0


def moe_gather_rows(x: torch.Tensor, pair_token: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[place] = x[pair_token[place]] (bfloat16 rows of whole 16 bytes)."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, torch.bfloat16, "out")
    _need(pair_token, torch.int32, "pair_token")
    if x.stride(1) != 1 or out.shape != (pair_token.numel(), x.shape[1]):
        raise KernelError("moe_gather_rows shapes")
    _check(_core("sllm_moe_tc").sllm_moe_gather_rows(
        _ptr(x), c_int64(x.stride(0)), _ptr(pair_token), c_int(pair_token.numel()),
        c_int(x.shape[1]), _ptr(out), _stream()), "moe_gather_rows")
    return out


def moe_tc_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, meta: torch.Tensor,
                   max_tiles: int, gated: bool | int) -> torch.Tensor:
    """The grouped product on tcgen05 (csrc/moe_tc.cu) over the rows of ``x`` [places, K]
    (bfloat16, in the sorted order) with tiles of 128 rows in ``meta``.  ``gated`` True
    (``MOE_GATED``): ``w`` [E, 2 F, K], ``out`` bfloat16 [places, F] = silu(gate) * up;
    ``MOE_SQRELU``: ``w`` [E, F, K], ``out`` bfloat16 [places, F] = relu(x w^T)^2; False: ``w``
    [E, F, K] and ``out`` float32 [places, F]."""
    gated = int(gated)
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16 if gated else torch.float32, "out")
    _need(meta, torch.int32, "meta")
    e, rows, k = w.shape
    f = rows // 2 if gated == MOE_GATED else rows
    if x.shape[1] != k or out.shape != (x.shape[0], f) or k % 8:
        raise KernelError("moe_tc_product shapes")
    _check(_core("sllm_moe_tc").sllm_moe_tc_product(
        _ptr(x), c_int64(x.shape[0]), _ptr(w), c_int(e), _ptr(out), _ptr(meta), c_int(f),
        c_int(k), c_int(max_tiles), c_int(gated), _stream()), "moe_tc_product")
    return out


def moe_combine(y: torch.Tensor, x: torch.Tensor, shared: torch.Tensor | None, ids: torch.Tensor,
                weights: torch.Tensor, pair_place: torch.Tensor, n_real: int, out: torch.Tensor
                ) -> torch.Tensor:
    """out[token] = sum of weight * (the chosen expert's row of ``y``, or ``x[token]`` for an
    identity expert) in the order of the choices, plus ``shared[token]``."""
    _need(y, torch.float32, "y")
    _need(x, None, "x")
    _need(out, x.dtype, "out")
    if shared is not None:
        _need(shared, x.dtype, "shared")
        if shared.shape != x.shape:
            raise KernelError("the shared expert's output must have the input's shape")
    n, d = x.shape
    top = ids.shape[1]
    if out.shape != (n, d) or y.shape[1] != d or ids.shape[0] != n:
        raise KernelError("moe_combine shapes")
    _check(_core("sllm_moe").sllm_moe_combine(
        _ptr(y), _ptr(x), _ptr(shared), _ptr(ids), _ptr(weights), _ptr(pair_place), c_int(n),
        c_int(top), c_int(n_real), c_int(d), _ptr(out), c_int(_code(x.dtype)), _stream()),
        "moe_combine")
    return out


def delta_rule(act: torch.Tensor, ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               state: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor,
               out: torch.Tensor, n_rows: int, n_heads: int, n_kv_heads: int, key_dim: int,
               value_dim: int, max_new: int = 0, log_decay: torch.Tensor | None = None,
               b_col: int | None = None, longest: int = 0) -> torch.Tensor:
    """The gated delta rule over the packed batch (csrc/delta_rule.cu): ``act`` [N, 2 G D + H V]
    holds query heads, key heads and value heads after the convolution; ``ab`` float32
    [N, 2 H] the decay and step inputs; ``state`` float32 [slots, H, V, D] is read and written
    at the rows' slots; ``out`` float32 [N, H * V].  ``max_new``: the most tokens a row brings,
    if known (1 selects the kernel for decode steps; 0: not known).

    ``log_decay`` (float32 [N, H * D], at most 0): a decay per key CHANNEL, given as its
    logarithm; ``a_log`` and ``dt_bias`` are then not read (may be None), and head h's step input
    is column ``b_col + h`` of ``ab`` (any width).  ``longest``: the most tokens any row brings,
    if known and above 1: the chunks' tables of weights are then all formed at once by a kernel
    of their own before the scan (0: every CTA of the scan forms its own)."""
    _need(act, None, "act", contiguous=False)
    _need(ab, torch.float32, "ab", contiguous=False)
    if log_decay is not None:
        return _delta_rule_channels(act, ab, state, row_start, row_slot, out, n_rows, n_heads,
                                    n_kv_heads, key_dim, value_dim, max_new, log_decay,
                                    n_heads if b_col is None else b_col, longest)
    _need(a_log, torch.float32, "A_log")
    _need(dt_bias, torch.float32, "dt_bias")
    _need(state, torch.float32, "state")
    _need(row_start, torch.int32, "row_start")
    _need(row_slot, torch.int32, "row_slot")
    _need(out, torch.float32, "out")
    n = act.shape[0]
    if act.stride(1) != 1 or ab.stride(1) != 1 or ab.shape != (n, 2 * n_heads) \
            or act.shape[1] < 2 * n_kv_heads * key_dim + n_heads * value_dim \
            or out.shape != (n, n_heads * value_dim) \
            or state.shape[1:] != (n_heads, value_dim, key_dim) \
            or a_log.numel() != n_heads or dt_bias.numel() != n_heads:
        raise KernelError("delta_rule shapes")
    if not 1 <= key_dim <= DELTA_MAX_KEY_DIM:
        raise KernelError(f"delta_rule takes key sizes up to {DELTA_MAX_KEY_DIM}, got {key_dim}")
    _check(_load(*delta_rule_library(key_dim)).sllm_delta_rule(
        _ptr(act), c_int64(act.stride(0)), _ptr(ab), c_int64(ab.stride(0)), _ptr(a_log),
        _ptr(dt_bias), _ptr(state), _ptr(row_start), _ptr(row_slot), _ptr(out), c_int(n_rows),
        c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(value_dim), c_void_p(0),
        c_int64(0), c_int(n_heads), c_void_p(0), c_int(0), c_int(_code(act.dtype)), _stream()),
        "delta_rule")
    return out


#: with a decay per channel the delta-rule kernel stages a third table: key sizes up to this
DELTA_CHANNEL_MAX_KEY_DIM = 192


#: tokens per chunk of the delta-rule kernel (a table of weights per chunk and head)
DELTA_CHUNK = 16


def _delta_rule_channels(act, ab, state, row_start, row_slot, out, n_rows, n_heads, n_kv_heads,
                         key_dim, value_dim, max_new, log_decay, b_col, longest) -> torch.Tensor:
    _need(log_decay, torch.float32, "log_decay", contiguous=False)
    _need(state, torch.float32, "state")
    _need(row_start, torch.int32, "row_start")
    _need(row_slot, torch.int32, "row_slot")
    _need(out, torch.float32, "out")
    n = act.shape[0]
    if act.stride(1) != 1 or ab.stride(1) != 1 or ab.shape[0] != n \
            or not 0 <= b_col <= ab.shape[1] - n_heads \
            or act.shape[1] < 2 * n_kv_heads * key_dim + n_heads * value_dim \
            or out.shape != (n, n_heads * value_dim) \
            or state.shape[1:] != (n_heads, value_dim, key_dim) \
            or log_decay.shape != (n, n_heads * key_dim) or log_decay.stride(1) != 1:
        raise KernelError("delta_rule shapes")
    if not 1 <= key_dim <= DELTA_CHANNEL_MAX_KEY_DIM:
        raise KernelError(f"delta_rule with a decay per channel takes key sizes up to "
                          f"{DELTA_CHANNEL_MAX_KEY_DIM}, got {key_dim}")
    tables = None
    if longest > 1 and max_new != 1:
        slots = n // DELTA_CHUNK + n_rows + 1
        tables = torch.empty((slots, n_heads, 2 * DELTA_CHUNK, DELTA_CHUNK), dtype=torch.float32,
                             device=act.device)
    _check(_load(*delta_rule_library(key_dim)).sllm_delta_rule(
        _ptr(act), c_int64(act.stride(0)), _ptr(ab), c_int64(ab.stride(0)), c_void_p(0),
        c_void_p(0), _ptr(state), _ptr(row_start), _ptr(row_slot), _ptr(out), c_int(n_rows),
        c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(value_dim), _ptr(log_decay),
        c_int64(log_decay.stride(0)), c_int(b_col), _ptr(tables), c_int(longest),
        c_int(_code(act.dtype)), _stream()),
        "delta_rule")
    return out


def lowrank_expand(pre: torch.Tensor, col0: int, w2t: torch.Tensor, out: torch.Tensor,
                   bias: torch.Tensor | None = None, rate_log: torch.Tensor | None = None,
                   per_rate: int = 0, also: tuple | None = None) -> torch.Tensor:
    """The second product of a low-rank pair in 32-bit (csrc/recurrent_ops.cu): ``pre`` float32
    [N, *] holds the hidden values in columns ``[col0, col0 + R)``, ``w2t`` float32 [R, C];
    ``out`` [N, C] (float32 or bfloat16) gets ``bias + hidden w2t``, or, with ``rate_log``
    (float32 [C / per_rate]), ``-exp(rate_log[c // per_rate]) * softplus(bias + hidden w2t)``:
    the logarithm of a decay per channel.  ``also = (col0, w2t, out)``: a second plain product of
    the same ``pre`` in the same launch."""
    _need(pre, torch.float32, "pre", contiguous=False)
    n = pre.shape[0]
    if pre.stride(1) != 1:
        raise KernelError("lowrank_expand shapes")
    jobs = [(col0, w2t, out, bias, rate_log, per_rate)]
    if also is not None:
        jobs.append((also[0], also[1], also[2], None, None, 0))
    for c0, w, o, b, rl, per in jobs:
        _need(w, torch.float32, "w2t")
        _need(o, None, "out")
        r, c = w.shape
        if c0 < 0 or pre.shape[1] < c0 + r or o.shape != (n, c):
            raise KernelError("lowrank_expand shapes")
        if b is not None:
            _need(b, torch.float32, "bias")
            if b.numel() != c:
                raise KernelError("lowrank_expand: one bias per output channel")
        if rl is not None:
            _need(rl, torch.float32, "rate_log")
            if per < 1 or c % per or rl.numel() != c // per:
                raise KernelError("lowrank_expand: one rate per `per_rate` channels")
    k = len(jobs)
    ints = lambda vals: (c_int * k)(*vals)  # noqa: E731
    ptrs = lambda ts: (c_void_p * k)(*[None if t is None else t.data_ptr() for t in ts])  # noqa: E731
    _check(_core("sllm_recurrent_ops").sllm_lowrank_expand(
        _ptr(pre), c_int64(pre.stride(0)), c_int(k), ints([j[0] for j in jobs]),
        ptrs([j[1] for j in jobs]), ptrs([j[3] for j in jobs]), ptrs([j[4] for j in jobs]),
        ints([j[5] for j in jobs]), ints([int(j[4] is not None) for j in jobs]),
        ptrs([j[2] for j in jobs]), ints([_code(j[2].dtype) for j in jobs]),
        ints([j[1].shape[1] for j in jobs]), ints([j[1].shape[0] for j in jobs]), c_int(n),
        _stream()), "lowrank_expand")
    return out


# ------------------------------------------------------------------------ latent attention

def latent_prep(a: torch.Tensor, q_rank: int, kv_col: int, kv_rank: int, rot_dim: int,
                q_gain: torch.Tensor, kv_gain: torch.Tensor, eps: float, positions: torch.Tensor,
                token_row: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, cq: torch.Tensor,
                pages: torch.Tensor, block_table: torch.Tensor, page_size: int,
                write: bool) -> torch.Tensor:
    """What a latent attention does with its down projections ``a`` [N, ...] (csrc/
    latent_attention.cu): ``cq`` [N, q_rank] gets the RMS-normed query latent (columns 0 ..
    q_rank of ``a``, times ``q_gain``); the page place of every token gets the RMS-normed
    key/value latent (columns kv_col .. kv_col + kv_rank, times ``kv_gain``), behind it the
    shared key part (the next ``rot_dim`` columns) with its first ``2 * cos.shape[1]`` entries
    rotated by the token's position (entry i pairs with entry i + half), then zeros up to the
    pages' vector size.  ``pages``: [n_pages, 1, 1, page_size, Dp]."""
    _need(a, None, "a", contiguous=False)
    _need(cq, a.dtype, "cq")
    _need(pages, a.dtype, "pages")
    _need(q_gain, torch.float32, "q_gain")
    _need(kv_gain, torch.float32, "kv_gain")
    _need(positions, torch.int32, "positions")
    _need(token_row, torch.int32, "token_row")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    _need(block_table, torch.int32, "block_table", contiguous=False)
    n = a.shape[0]
    rot_dims = 2 * cos.shape[1]
    if a.stride(1) != 1 or a.shape[1] < max(q_rank, kv_col + kv_rank + rot_dim) \
            or cq.shape != (n, q_rank) or q_gain.numel() != q_rank or kv_gain.numel() != kv_rank \
            or sin.shape != cos.shape or rot_dims > rot_dim or block_table.stride(1) != 1:
        raise KernelError("latent_prep shapes")
    if pages.dim() != 5 or pages.shape[1:4] != (1, 1, page_size) \
            or pages.shape[4] < kv_rank + rot_dim:
        raise KernelError(f"pages must be [n_pages, 1, 1, {page_size}, at least "
                          f"{kv_rank + rot_dim}], got {list(pages.shape)}")
    _check(_core("sllm_latent_attention").sllm_latent_prep(
        _ptr(a), c_int64(a.stride(0)), c_int(q_rank), c_int(kv_col), c_int(kv_rank),
        c_int(rot_dim), _ptr(q_gain), _ptr(kv_gain), c_float(eps), _ptr(positions),
        _ptr(token_row), _ptr(cos), _ptr(sin), c_int(rot_dims), _ptr(cq), _ptr(pages),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size),
        c_int(pages.shape[4]), c_int(int(write)), c_int(n), c_int(_code(a.dtype)), _stream()),
        "latent_prep")
    return cq


def latent_q_rot(q: torch.Tensor, n_heads: int, dim: int, rot_dim: int, positions: torch.Tensor,
                 cos: torch.Tensor, sin: torch.Tensor, out: torch.Tensor, kv_rank: int) -> torch.Tensor:
    """``q`` [N, H * (dim + rot_dim)]: every head's last ``rot_dim`` entries, rotated like the
    shared key part in :func:`latent_prep`, go to ``out`` [N, H * Dp] at columns ``h * Dp +
    kv_rank`` on, zeros behind them up to Dp."""
    _need(q, None, "q", contiguous=False)
    _need(out, q.dtype, "out")
    _need(positions, torch.int32, "positions")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    n = q.shape[0]
    if q.stride(1) != 1 or q.shape[1] != n_heads * (dim + rot_dim) or out.shape[0] != n \
            or out.shape[1] % n_heads or out.shape[1] // n_heads < kv_rank + rot_dim \
            or 2 * cos.shape[1] > rot_dim or sin.shape != cos.shape:
        raise KernelError("latent_q_rot shapes")
    _check(_core("sllm_latent_attention").sllm_latent_q_rot(
        _ptr(q), c_int64(q.stride(0)), c_int(n_heads), c_int(dim), c_int(rot_dim),
        _ptr(positions), _ptr(cos), _ptr(sin), c_int(2 * cos.shape[1]), _ptr(out),
        c_int64(out.stride(0)), c_int(kv_rank), c_int(out.shape[1] // n_heads), c_int(n),
        c_int(_code(q.dtype)), _stream()), "latent_q_rot")
    return out


def head_product(x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor,
                 out_head_stride: int) -> torch.Tensor:
    """A product per head on the CUDA cores: ``out[n, h * out_head_stride + j] = sum_k x[n, h *
    x_head_stride + k] * w[h, j, k]`` for ``w`` [H, J, K]; one fixed-order chain of fused
    multiply-adds per output."""
    _need(x, None, "x", contiguous=False)
    _need(w, x.dtype, "w")
    _need(out, x.dtype, "out", contiguous=False)
    h, j, k = w.shape
    n = x.shape[0]
    if x.stride(1) != 1 or out.stride(1) != 1 or out.shape[0] != n \
            or (h - 1) * x_head_stride + k > x.shape[1] \
            or (h - 1) * out_head_stride + j > out.shape[1]:
        raise KernelError("head_product shapes")
    _check(_core("sllm_latent_attention").sllm_head_product(
        _ptr(x), c_int64(x.stride(0)), c_int64(x_head_stride), _ptr(w), _ptr(out),
        c_int64(out.stride(0)), c_int64(out_head_stride), c_int(n), c_int(h), c_int(j), c_int(k),
        c_int(_code(x.dtype)), _stream()), "head_product")
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor, n_heads: int) -> torch.Tensor:
    """``x`` [N, H * V] in place: head h of token n is multiplied by ``sigmoid(gate[n, h])``;
    ``gate`` [N, H] may be a column slice of a wider buffer."""
    _need(x, None, "x", contiguous=False)
    _need(gate, x.dtype, "gate", contiguous=False)
    n = x.shape[0]
    if x.stride(1) != 1 or gate.stride(1) != 1 or gate.shape != (n, n_heads) \
            or x.shape[1] % n_heads:
        raise KernelError("head_gate shapes")
    _check(_core("sllm_latent_attention").sllm_head_gate(
        _ptr(x), c_int64(x.stride(0)), _ptr(gate), c_int64(gate.stride(0)), c_int(n_heads),
        c_int(x.shape[1] // n_heads), c_int(n), c_int(_code(x.dtype)), _stream()), "head_gate")
    return x


#: steps of up to this many tokens take :func:`latent_small` for a latent attention's products
#: per head (beyond it the library's batched product wins)
LATENT_SMALL_MAX_TOKENS = 64


def latent_small_supports(k: int, j: int) -> bool:
    """Whether :func:`latent_small` takes a reduction of ``k`` and ``j`` outputs per head (its
    tile of tokens and its partial sums fit the default shared memory)."""
    return k >= 1 and 1 <= j <= 32 * 65535 and 4 * (8 * k + 8 * 8 * 32) <= 48 * 1024


def latent_small(x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor,
                 out_head_stride: int, gate: torch.Tensor | None = None,
                 rot: tuple[int, torch.Tensor, torch.Tensor, torch.Tensor] | None = None
                 ) -> torch.Tensor:
    """A product per head for steps of few tokens, in one launch with what follows it:
    ``out[n, h * out_head_stride + j] = f * sum_k x[n, h * x_head_stride + k] * w[h, k, j]`` for
    ``w`` [H, K, J] (the output index last).  ``gate`` [N, H] (may be a column slice): ``f =
    sigmoid(gate[n, h])``.  ``rot = (rot_dim, positions, cos, sin)``: the head's next ``rot_dim``
    entries of ``x`` go behind the J outputs, the first ``2 * cos.shape[1]`` of them rotated by
    the token's position (as :func:`latent_q_rot` does), zeros behind them up to
    ``out_head_stride``."""
    _need(x, None, "x", contiguous=False)
    _need(w, x.dtype, "w")
    _need(out, x.dtype, "out", contiguous=False)
    h, k, j = w.shape
    n = x.shape[0]
    r = tail = rot_dims = 0
    positions = cos = sin = None
    if rot is not None:
        r, positions, cos, sin = rot
        _need(positions, torch.int32, "positions")
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        tail, rot_dims = out_head_stride - j, 2 * cos.shape[1]
        if tail < r or rot_dims > r or sin.shape != cos.shape or x_head_stride < k + r:
            raise KernelError("latent_small: the rotated part's shapes")
    if gate is not None:
        _need(gate, x.dtype, "gate", contiguous=False)
        if gate.shape != (n, h) or gate.stride(1) != 1:
            raise KernelError("latent_small: gate must be [tokens, heads]")
    if x.stride(1) != 1 or out.stride(1) != 1 or out.shape[0] != n \
            or (h - 1) * x_head_stride + k + r > x.shape[1] \
            or (h - 1) * out_head_stride + j + tail > out.shape[1] \
            or not latent_small_supports(k, j):
        raise KernelError("latent_small shapes")
    _check(_core("sllm_latent_attention").sllm_latent_small(
        _ptr(x), c_int64(x.stride(0)), c_int64(x_head_stride), _ptr(w), _ptr(out),
        c_int64(out.stride(0)), c_int64(out_head_stride), c_int(n), c_int(h), c_int(k), c_int(j),
        _ptr(gate), c_int64(gate.stride(0) if gate is not None else 0), c_int(r), c_int(tail),
        _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot_dims), c_int(_code(x.dtype)), _stream()),
        "latent_small")
    return out


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[n] = [a[n]; b[n]]`` rounded to the dtype of ``out``, for float32 ``a`` and ``b``
    [N, d] and ``out`` [N, 2 d]."""
    _need(a, torch.float32, "a")
    _need(b, torch.float32, "b")
    _need(out, None, "out")
    n, d = a.shape
    if b.shape != (n, d) or out.shape != (n, 2 * d):
        raise KernelError("concat_cast shapes")
    _check(_core("sllm_stream_ops").sllm_concat_cast(
        _ptr(a), _ptr(b), _ptr(out), c_int(n), c_int(d), c_int(_code(out.dtype)), _stream()),
        "concat_cast")
    return out


# ------------------------------------------------------------------------------- layer norm

LAYERNORM_MAX_TERMS = 4


def add_layernorm(resid: torch.Tensor, terms: Sequence[tuple[torch.Tensor, float]],
                  weight: torch.Tensor, bias: torch.Tensor, eps: float, out: torch.Tensor,
                  out_rows: torch.Tensor | None = None) -> torch.Tensor:
    """``x = resid + sum(coef * term)`` in 32-bit, then ``out = (x - mean) / sqrt(var + eps) *
    weight + bias`` (csrc/layer_norm.cu).  Without ``out_rows`` the stream ``resid`` is updated
    in place and every token is normed; with ``out_rows`` (int32) only those tokens are, and the
    stream is not written.  ``out`` float32 or bfloat16; it may be ``resid`` itself when there
    are no terms (the stream normed in place)."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(bias, torch.float32, "bias")
    _need(out, None, "out")
    n, d = resid.shape
    if len(terms) > LAYERNORM_MAX_TERMS:
        raise KernelError(f"add_layernorm takes up to {LAYERNORM_MAX_TERMS} terms")
    term_dtype = out.dtype
    for i, (t, _) in enumerate(terms):
        _need(t, None, "term")
        if t.shape != (n, d):
            raise KernelError("add_layernorm: a term must have the stream's shape")
        if i and t.dtype != term_dtype:
            raise KernelError("add_layernorm: the terms must share a dtype")
        term_dtype = t.dtype
    if out is resid and terms:
        raise KernelError("add_layernorm: the stream is normed in place only without terms")
    n_out = n if out_rows is None else out_rows.numel()
    if out_rows is not None:
        _need(out_rows, torch.int32, "out_rows")
    if weight.numel() != d or bias.numel() != d or out.shape != (n_out, d):
        raise KernelError("add_layernorm shapes")
    ptrs = (c_void_p * LAYERNORM_MAX_TERMS)(*[t.data_ptr() for t, _ in terms])
    coefs = (c_float * LAYERNORM_MAX_TERMS)(*[float(c) for _, c in terms])
    _check(_core("sllm_layer_norm").sllm_add_layernorm(
        _ptr(resid), ptrs, coefs, c_int(len(terms)), c_int(_code(term_dtype)), _ptr(weight),
        _ptr(bias), c_float(eps), _ptr(out), c_int(_code(out.dtype)), _ptr(out_rows),
        c_int(n_out), c_int(d), _stream()), "add_layernorm")
    return out


def norm_rope_kv_write(x: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                       pages: torch.Tensor, block_table: torch.Tensor, page_size: int,
                       n_heads: int, n_kv_heads: int, head_dim: int, qk_dim: int, eps: float,
                       has_kv: bool, write: bool, bias: torch.Tensor | None = None,
                       q_gain: torch.Tensor | None = None, k_gain: torch.Tensor | None = None,
                       unit_after: bool = False, cos: torch.Tensor | None = None,
                       sin: torch.Tensor | None = None, interleaved: bool = True) -> None:
    """Between an attention mixer's fused projection and its attention kernel
    (csrc/norm_rope_cache.cu): biases, an RMS norm over all of q (and over all of k) with gains
    per column, the rotation by the tables' angles, an RMS norm per head without gains
    (``unit_after``), q back in place and the new keys and values into the pages.  ``x``
    [N, >= (H + 2 G) * head_dim] (only the H query heads without ``has_kv``); ``qk_dim``: the
    heads' true size where they are padded up to ``head_dim``."""
    _need(x, None, "x")
    _need(positions, torch.int32, "positions")
    _need(token_row, torch.int32, "token_row")
    _need(pages, x.dtype, "pages")
    _need(block_table, torch.int32, "block_table", contiguous=False)
    cols = (n_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    if x.shape[1] < cols or block_table.stride(1) != 1:
        raise KernelError("norm_rope_kv_write layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    for t, name, size in ((bias, "bias", cols), (q_gain, "q_gain", n_heads * head_dim),
                          (k_gain, "k_gain", n_kv_heads * head_dim)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != size:
                raise KernelError(f"{name} must have {size} entries")
    rot = 0
    if cos is not None:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        rot = 2 * cos.shape[1]
        if sin.shape != cos.shape or not 2 <= rot <= qk_dim:
            raise KernelError("rotary table width")
    _check(_core("sllm_norm_rope_cache").sllm_norm_rope_kv_write(
        _ptr(x), c_int64(x.stride(0)), _ptr(positions), _ptr(token_row), _ptr(bias),
        _ptr(q_gain), _ptr(k_gain), c_int(int(unit_after)), c_float(eps), c_int(qk_dim),
        _ptr(cos), _ptr(sin), c_int(rot), c_int(int(interleaved)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), c_int(x.shape[0]), c_int(n_heads),
        c_int(n_kv_heads), c_int(head_dim), c_int(int(has_kv)), c_int(int(write)),
        c_int(_code(x.dtype)), _stream()), "norm_rope_kv_write")
