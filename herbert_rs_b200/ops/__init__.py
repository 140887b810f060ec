"""Python faces of the kernels: one function per launcher of the kernel library.

Each function takes CUDA tensors, checks what only the host can check cheaply (device,
dtype, contiguity of the innermost axis) and launches on the current CUDA stream.  A launcher
that refuses its input raises `BackendError` with the launcher's own message.  Nothing here
computes on the CPU and nothing falls back to a library model or attention routine.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from ..errors import BackendError
from . import lib as _libmod
from .options import KernelOptions

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_ROWS = 64
# The one place where a choice between kernels can be changed (by a measurement script or a test
# that assigns its fields); nothing reads the environment.
options = KernelOptions()

_SIGS = {
    "hb_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_rmsnorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "hb_swiglu": [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "hb_add_residual": [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_qk_norm_rope_cache": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                              c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_simt": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_skinny_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_skinny_norm_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                 c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "hb_finish_norm": [c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_gemm_tcgen05_norm_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    "hb_gemm_tcgen05_norm_parts": [c_int, c_int],
    "hb_gemm_tcgen05_qkv_ok": [c_int, c_int],
    "hb_gemm_tcgen05_qkv_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
    "hb_gemm_tcgen05_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "hb_gemm_stream_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                            ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p],
    "hb_attention_simt": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_attention_decode_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_attention_decode_fused_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_attention_prefill_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_attention_prefill_tc_bf16": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                     c_void_p],
    "hb_argmax": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p],
    "hb_gemm_skinny_norm_parts": [c_int, c_int],
    "hb_sample": [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "hb_rng_normal": [c_int, c_void_p, ctypes.c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p],
    "hb_fill": [c_int, c_void_p, ctypes.c_longlong, c_float, c_void_p],
    "hb_cast": [c_int, c_void_p, c_int, c_void_p, ctypes.c_longlong, c_int, c_void_p],
}
_fns: dict = {}


def _fn(name: str):
    f = _fns.get(name)
    if f is None:
        lib = _libmod.load()
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise BackendError(f"kernel library has no entry point {name}") from None
        f.argtypes = _SIGS[name]
        f.restype = c_int
        _fns[name] = f
    return f


# kernels each launcher starts (for honest launch counts)
_KERNELS_PER_CALL = {"hb_attention_decode_bf16": 2, "hb_argmax": 2, "hb_sample": 2}
_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (launches recorded into a graph count once)."""
    return _launches


_timeline = None     # while a `timed()` block is open: [(launcher name, start event, end event)]


def _run(name: str, *args) -> None:
    global _launches
    _launches += _KERNELS_PER_CALL.get(name, 1)
    if _timeline is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = _fn(name)(*args)
        e1.record()
        _timeline.append((name, e0, e1))
    else:
        rc = _fn(name)(*args)
    if rc != 0:
        raise BackendError(f"{name}: {_libmod.last_error()}")


class timed:
    """Where a step's time goes, by launcher: CUDA events around every launch made inside the block
    (eager steps only: a replayed graph makes no launches here).  The reference returns per-layer
    times on request in the same spirit (crates/core/src/backend.rs:97-102, profiler.rs:17-60).

        with ops.timed() as t:
            engine.step(...)
        t.by_kernel()     # {launcher: (launches, milliseconds)}, and "(between launches)"
    """

    def __enter__(self):
        global _timeline
        self._saved, _timeline = _timeline, []
        self._rows = _timeline
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = self._saved
        torch.cuda.synchronize()
        return False

    def by_kernel(self) -> dict:
        out: dict = {}
        for name, e0, e1 in self._rows:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1))
        if self._rows:
            whole = self._rows[0][1].elapsed_time(self._rows[-1][2])
            out["(between launches)"] = (len(self._rows) - 1, whole - sum(ms for _, ms in out.values()))
        return out


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current CUDA stream's handle (also the capturing stream while a graph is recorded).  Asked
    of torch's C layer directly where that entry exists: a step makes some two hundred launches, and
    `torch.cuda.current_stream()` costs several microseconds each time."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise BackendError(f"unsupported activation dtype {dtype}: float32 or bfloat16")


_device_keys: dict = {}


def device_key(device) -> str:
    """One name per CUDA device ("cuda:0"), whether it was given with or without its index."""
    key = _device_keys.get(device)
    if key is None:
        d = torch.device(device)
        if d.index is None:      # depends on the current device: not remembered
            return f"cuda:{torch.cuda.current_device()}"
        key = _device_keys[device] = f"cuda:{d.index}"
    return key


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise BackendError(f"{name} must be a CUDA tensor: there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise BackendError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() > 0 and t.stride(-1) != 1:
        raise BackendError(f"{name} must be contiguous along its last axis")


_pdl_mode = None


def set_pdl(mode: int) -> None:
    """Programmatic dependent launch: 0 off, 1 every kernel, 2 only the launches that ask for it.
    The engine switches it on for eager steps (prompts: the next kernel's CTAs start while the last
    ones of the kernel before drain, 1-3 % of a prefill) and off for steps it records as CUDA graphs
    (inside a replayed graph it measured slower); see `options.pdl_eager`."""
    global _pdl_mode
    if _pdl_mode != int(mode):
        _libmod.load().hb_set_pdl(int(mode))
        _pdl_mode = int(mode)


def set_gemm_pairs(on: bool) -> None:
    """Whether the prefill product runs as pairs of CTAs (cta_group::2) where that applies (default on)."""
    _libmod.load().hb_gemm_tcgen05_set_pairs(1 if on else 0)


def set_gemm_ksplit(on: bool) -> None:
    """Whether products of at most 128 rows cut K over a cluster of CTAs where that applies (default on)."""
    _libmod.load().hb_gemm_tcgen05_set_ksplit(1 if on else 0)


def is_available() -> bool:
    """True when a CUDA device is present (the kernels still have to build and load)."""
    return torch.cuda.is_available()


# ---------------------------------------------------------------------------------------------
def rng_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * normal(key, i): the same bits as `weights.counter_rng.normal`."""
    _check(out, None, "out")
    if not out.is_contiguous():
        raise BackendError("rng_normal: out must be contiguous")
    _run("hb_rng_normal", dtype_code(out.dtype), out.data_ptr(), out.numel(), int(key) & ((1 << 64) - 1),
         float(mean), float(std), _stream())


def fill(out: torch.Tensor, value: float) -> None:
    """Every element of a contiguous float32, bfloat16 or int32 tensor becomes `value`."""
    _check(out, None, "out")
    if not out.is_contiguous():
        raise BackendError("fill: out must be contiguous")
    code = 2 if out.dtype == torch.int32 else dtype_code(out.dtype)
    _run("hb_fill", code, out.data_ptr(), out.numel(), float(value), _stream())


_CAST_SRC = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def cast(src: torch.Tensor, dtype: torch.dtype, round_bf16: bool = False) -> torch.Tensor:
    """`src` (float32, bfloat16 or float16, contiguous, on the device) as a new tensor of `dtype`
    (float32 or bfloat16; float32 -> bfloat16 rounds to nearest even).  With `round_bf16` the
    values pass through bfloat16 whatever `dtype` is.  Returns `src` itself when nothing changes."""
    _check(src, None, "src")
    if src.dtype not in _CAST_SRC:
        raise BackendError(f"cast: cannot read {src.dtype}")
    if src.dtype == dtype and (not round_bf16 or dtype == torch.bfloat16):
        return src
    if not src.is_contiguous():
        raise BackendError("cast: src must be contiguous")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _run("hb_cast", _CAST_SRC[src.dtype], src.data_ptr(), dtype_code(dtype), out.data_ptr(), src.numel(),
         1 if round_bf16 else 0, _stream())
    return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = float(table[ids[t], :]); out is the float residual stream [T, H]."""
    _check(table, None, "table"); _check(ids, torch.int32, "ids"); _check(out, torch.float32, "out")
    _run("hb_embed", dtype_code(table.dtype), table.data_ptr(), ids.data_ptr(), out.data_ptr(),
         ids.numel(), table.shape[1], table.shape[0], _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * w; x and w float, out in the activation dtype."""
    _check(x, torch.float32, "x"); _check(w, torch.float32, "w"); _check(out, None, "out")
    n = out.shape[0]
    _run("hb_rmsnorm", dtype_code(out.dtype), x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(rows),
         n, x.shape[-1], float(eps), _stream())


def swiglu(gu: torch.Tensor, out: torch.Tensor, interleave: int) -> None:
    """out[t, i] = silu(gate) * up from gu [T, 2I] (see the kernel for the column layout)."""
    _check(gu, None, "gu"); _check(out, gu.dtype, "out")
    _run("hb_swiglu", dtype_code(gu.dtype), gu.data_ptr(), gu.stride(0), out.data_ptr(), out.stride(0),
         gu.shape[0], out.shape[1], int(interleave), _stream())


def add_residual(residual: torch.Tensor, y: torch.Tensor) -> None:
    """residual += y (float sum)."""
    _check(residual, torch.float32, "residual"); _check(y, None, "y")
    _run("hb_add_residual", dtype_code(y.dtype), residual.data_ptr(), y.data_ptr(), y.stride(0),
         y.shape[0], y.shape[1], _stream())


def qk_norm_rope_cache(qkv, q_weight, k_weight, eps, cos, sin, rotary_dim, tok_seq, tok_pos, seq_pages,
                       k_cache, v_cache, num_heads, num_kv_heads, head_dim, page_size, write_cache=True) -> None:
    """Head norm + rotation of q (in place) and k (into the cache), v copied into the cache."""
    _check(qkv, None, "qkv")
    _run("hb_qk_norm_rope_cache", dtype_code(qkv.dtype), qkv.data_ptr(), qkv.stride(0), _ptr(q_weight),
         _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), int(rotary_dim),
         0 if cos is None else cos.shape[0], tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), qkv.shape[0], num_heads,
         num_kv_heads, head_dim, page_size, 1 if write_cache else 0, _stream())


def gemm_simt(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T on the CUDA cores, any sizes."""
    _check(a, None, "a"); _check(w, a.dtype, "w"); _check(c, None, "c")
    _run("hb_gemm_simt", dtype_code(a.dtype), a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0),
         c.data_ptr(), c.stride(0), a.shape[0], w.shape[0], a.shape[1], epilogue, _stream())


def attention_simt(q, ldq, out, k_cache, v_cache, tok_seq, tok_pos, seq_pages, num_heads, num_kv_heads,
                   head_dim, page_size, scale, window) -> None:
    _run("hb_attention_simt", dtype_code(out.dtype), q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), out.shape[0], num_heads, num_kv_heads, head_dim, page_size, float(scale),
         int(window or 0), _stream())


_argmax_scratch: dict = {}
ARGMAX_SCRATCH_ROWS = 4096


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of row r."""
    _check(logits, torch.float32, "logits"); _check(out, torch.int32, "out")
    key = device_key(logits.device)
    if key not in _argmax_scratch:
        _argmax_scratch[key] = torch.empty(2 * 64 * ARGMAX_SCRATCH_ROWS, dtype=torch.int32, device=logits.device)
    sc = _argmax_scratch[key]
    _run("hb_argmax", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(),
         sc.data_ptr(), sc.numel(), _stream())


_sample_flags: dict = {}


def sample(logits, temperature, top_k, top_p, uniforms, out) -> None:
    """One token per row under temperature / top-k / top-p with the row's uniform.  A small top_k
    against a large vocabulary takes a kernel that reads the row twice and works on a list of
    candidates in shared memory; rows it cannot hold fall to the general kernel in the same call."""
    _check(logits, torch.float32, "logits"); _check(uniforms, torch.float32, "uniforms"); _check(out, torch.int32, "out")
    key = device_key(logits.device)
    if key not in _sample_flags or _sample_flags[key].numel() < logits.shape[0]:
        _sample_flags[key] = torch.zeros(max(1024, logits.shape[0]), dtype=torch.int32, device=logits.device)
    _run("hb_sample", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], float(temperature),
         int(top_k), float(top_p), uniforms.data_ptr(), out.data_ptr(), _sample_flags[key].data_ptr(), _stream())


def gemm_skinny(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T for at most 64 rows of a (bfloat16), streaming w once; EPI_SWIGLU: w holds
    gate/up rows in groups of 8 and c is [M, N/2]."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    _run("hb_gemm_skinny_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, _stream())


SHARED_NORM_MAX_ROWS = 16


class PendingNorm:
    """An RMSNorm that the product before it has begun and the product after it will finish.

    `xw` [T, D] is x * w in bfloat16; `sumsq` [parts, stride] holds partial sums of x^2 per row, so
    that y = xw / sqrt(sum(sumsq[:, row]) / D + eps).  A product kernel that takes it multiplies its
    results by that row factor; `finish_norm` makes the plain y for anyone else."""

    __slots__ = ("xw", "sumsq", "parts", "eps")

    def __init__(self, xw, sumsq, parts, eps):
        self.xw, self.sumsq, self.parts, self.eps = xw, sumsq, parts, eps

    stride = property(lambda self: self.sumsq.stride(0))

    shape = property(lambda self: self.xw.shape)
    dtype = property(lambda self: self.xw.dtype)


def shared_norm_ok(n_rows: int, dtype, dim: int) -> bool:
    """Whether products of `n_rows` activation rows can carry a norm over `dim` between them: the
    mma.sync kernel can for at most 16 rows, the tensor-memory kernel for any number; between 17
    and 64 rows a product that goes through another kernel leaves the norm to a kernel of its own."""
    return options.shared_norm and dtype == torch.bfloat16 and dim % 8 == 0


def finish_norm(p: PendingNorm, out: torch.Tensor) -> None:
    _check(out, torch.bfloat16, "out")
    _run("hb_finish_norm", p.xw.data_ptr(), p.xw.stride(0), p.sumsq.data_ptr(), p.parts, p.stride, float(p.eps),
         out.data_ptr(), out.stride(0), p.xw.shape[0], p.xw.shape[1], _stream())


def gemm_skinny_norm(a, w, c, epilogue=EPI_STORE, next_norm=None, scratch=None):
    """gemm_skinny with a norm shared on either side (at most 16 rows).  `a` may be a PendingNorm.
    next_norm = (weight [N] float, eps) with EPI_RESIDUAL: returns the PendingNorm of the updated c,
    its buffers taken from `scratch(shape, dtype)`."""
    pend = a if isinstance(a, PendingNorm) else None
    x = pend.xw if pend is not None else a
    _check(x, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    M, N, K = x.shape[0], w.shape[0], x.shape[1]
    out = None
    if next_norm is not None:
        nw, eps = next_norm
        _check(nw, torch.float32, "next norm weight")
        if epilogue != EPI_RESIDUAL or nw.numel() != N:
            raise BackendError("gemm_skinny_norm: the next norm needs the residual epilogue and a weight per output column")
        parts = int(_fn("hb_gemm_skinny_norm_parts")(M, N))
        out = PendingNorm(scratch((M, N), torch.bfloat16), scratch((parts, 16), torch.float32), parts, eps)
    _run("hb_gemm_skinny_norm_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         M, N, K, epilogue,
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         float(pend.eps) if pend is not None else 0.0,
         nw.data_ptr() if out is not None else None,
         out.xw.data_ptr() if out is not None else None, out.xw.stride(0) if out is not None else 0,
         out.sumsq.data_ptr() if out is not None else None, _stream())
    return out


_error_flags: dict = {}


def _error_flag(device) -> torch.Tensor:
    """One int per device that kernels with bounded waits set when a wait runs out."""
    key = device_key(device)
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_kernel_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check (reads one int per device,
    which waits for the device)."""
    for key, flag in _error_flags.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            # a kernel that gave up may have left arrival counters mid-count: start them afresh
            for table in (_decode_counters, _work_counters):
                if key in table:
                    table[key].zero_()
            if _tcgen05_ws.get(key) is not None:
                _tcgen05_ws[key][1].zero_()
            if key in _stream_bufs:
                _stream_bufs[key][1].zero_()
            raise BackendError(f"a kernel on {key} gave up waiting on a barrier (code {code}); its output is not valid")


_tcgen05_ws: dict = {}


def _tcgen05_workspace(device) -> None:
    """Once per device: hand the prefill product the workspace in which CTAs that share an output
    tile leave their pieces (about 39 MB on 148 SMs)."""
    key = device_key(device)
    if key in _tcgen05_ws:
        return
    if not options.prefill_split_tiles:
        _tcgen05_ws[key] = None
        return
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    lib = _libmod.load()
    lib.hb_gemm_tcgen05_workspace_floats.restype = ctypes.c_longlong
    lib.hb_gemm_tcgen05_workspace_floats.argtypes = [c_int]
    n = int(lib.hb_gemm_tcgen05_workspace_floats(sms))
    floats = torch.empty(n, dtype=torch.float32, device=device)
    counters = torch.zeros(sms, dtype=torch.int32, device=device)
    lib.hb_gemm_tcgen05_set_workspace.argtypes = [c_void_p, c_void_p, c_int]
    lib.hb_gemm_tcgen05_set_workspace.restype = c_int
    lib.hb_gemm_tcgen05_set_workspace(floats.data_ptr(), counters.data_ptr(), sms)
    _tcgen05_ws[key] = (floats, counters)


def gemm_tcgen05(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T on tcgen05 tensor cores with TMA-fed tiles (bfloat16, K a multiple of 8)."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    _tcgen05_workspace(c.device)
    _run("hb_gemm_tcgen05_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, _error_flag(a.device).data_ptr(), _stream())


_stream_bufs: dict = {}
STREAM_COUNTERS = 8192


def gemm_tcgen05_norm(a, w, c, epilogue=EPI_STORE, next_norm=None, scratch=None):
    """gemm_tcgen05 with a norm shared on either side (see gemm_skinny_norm): `a` may be a
    PendingNorm; next_norm = (weight, eps) with EPI_RESIDUAL returns the PendingNorm of the updated c."""
    pend = a if isinstance(a, PendingNorm) else None
    x = pend.xw if pend is not None else a
    _check(x, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    M, N, K = x.shape[0], w.shape[0], x.shape[1]
    out, nw = None, None
    if next_norm is not None:
        nw, eps = next_norm
        _check(nw, torch.float32, "next norm weight")
        if epilogue != EPI_RESIDUAL or nw.numel() != N:
            raise BackendError("gemm_tcgen05_norm: the next norm needs the residual epilogue and a weight per output column")
        parts = int(_fn("hb_gemm_tcgen05_norm_parts")(M, N))
        out = PendingNorm(scratch((M, N), torch.bfloat16), scratch((parts, (M + 3) // 4 * 4), torch.float32), parts, eps)
    _tcgen05_workspace(c.device)
    _run("hb_gemm_tcgen05_norm_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         M, N, K, epilogue,
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         pend.stride if pend is not None else 0, float(pend.eps) if pend is not None else 0.0,
         nw.data_ptr() if out is not None else None, out.xw.data_ptr() if out is not None else None,
         out.xw.stride(0) if out is not None else 0, out.sumsq.data_ptr() if out is not None else None,
         out.stride if out is not None else 0, _error_flag(c.device).data_ptr(), _stream())
    return out


def gemm_qkv_fused_ok(x, wqkv, qkv_out, head_dim, rotary_dim, position) -> bool:
    """Whether the q/k/v product of this step can also do the per-head norm, the rotation and the
    cache write in its epilogue: bfloat16, heads of 128 rotated whole, a step of 512 rows and more."""
    a = x.xw if isinstance(x, PendingNorm) else x
    return (options.qkv_epilogue and a.dtype == torch.bfloat16 and qkv_out.dtype == torch.bfloat16 and head_dim == 128
            and rotary_dim == 128 and position is not None and _tcgen05_ok(a, wqkv) and qkv_out.stride(0) % 8 == 0
            and qkv_out.data_ptr() % 16 == 0 and bool(_fn("hb_gemm_tcgen05_qkv_ok")(a.shape[0], wqkv.shape[0])))


def gemm_qkv_fused(x, wqkv, qkv_out, q_weight, k_weight, eps, cos, sin, tok_seq, tok_pos, seq_pages, k_cache, v_cache,
                   num_heads, num_kv_heads, page_size, write_cache, scratch) -> None:
    """qkv_out[:, :num_heads*128] = rotated (and normed) q of x @ wqkv.T; k (normed, rotated) and v go
    into the paged cache.  `x` may be a PendingNorm (its norm is finished inside)."""
    pend = x if isinstance(x, PendingNorm) else None
    a = pend.xw if pend is not None else x
    _tcgen05_workspace(qkv_out.device)
    _run("hb_gemm_tcgen05_qkv_bf16", a.data_ptr(), a.stride(0), wqkv.data_ptr(), wqkv.stride(0), qkv_out.data_ptr(), qkv_out.stride(0),
         a.shape[0], wqkv.shape[0], a.shape[1],
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         pend.stride if pend is not None else 0, float(pend.eps) if pend is not None else 0.0,
         _ptr(q_weight), _ptr(k_weight), float(eps), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
         tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         num_heads, num_kv_heads, page_size, 1 if write_cache else 0, _error_flag(qkv_out.device).data_ptr(), _stream())


def _stream_buffers(device):
    """Per device: scratch for the K slices' partial tiles and the tiles' arrival counters (zero
    between launches).  Fixed addresses, so captured graphs can use them."""
    key = device_key(device)
    if key not in _stream_bufs:
        # K is cut into slices only while (tiles x slices) fits two CTAs per SM: that many partial tiles of 64 x 128 floats
        _stream_bufs[key] = (torch.empty(2 * sm_count(device) * 64 * 128, dtype=torch.float32, device=device),
                             torch.zeros(STREAM_COUNTERS, dtype=torch.int32, device=device))
    return _stream_bufs[key]


def gemm_stream(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T for at most 64 rows of a (bfloat16): weights streamed once through TMA into
    tcgen05 tensor cores, K cut into slices that the last-arriving CTA of a tile sums in order."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    scratch, counters = _stream_buffers(a.device)
    if w.shape[0] > STREAM_COUNTERS * 128:
        raise BackendError(f"gemm_stream: {w.shape[0]} weight rows exceed the {STREAM_COUNTERS * 128} the counters cover")
    _run("hb_gemm_stream_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, scratch.data_ptr(), scratch.numel(), counters.data_ptr(),
         counters.numel(), _error_flag(a.device).data_ptr(), _stream())


def _tcgen05_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _decode_gemm(a, w):
    """Which kernel multiplies at most 64 activation rows.  Measured (microseconds at 17 / 32 / 64
    rows; mma.sync kernel, streaming tcgen05 kernel, prefill kernel) at Qwen3-8B shapes: q/k/v
    19 / 21 / 31, 23 / 23 / 28, 14 / 15 / 16; o 12 / 12 / 18, 27 / 30 / 42, 13 / 14 / 14; gate/up
    58 / 65 / 93, 46 / 49 / 57, 41 / 41 / 42; down 28 / 29 / 42, 53 / 59 / 76, 26 / 26 / 26; at 32B shapes
    the prefill kernel wins all four from 32 rows on, at 0.6B shapes (at most 6 M elements) the
    mma.sync kernel wins all four.
    Up to 16 rows the mma.sync kernel streams the weights at the memory's rate; beyond that every CTA
    of 16 weight rows reads the whole activation matrix again, and the prefill kernel (K cut over a
    cluster of CTAs where the matrix has few tiles) wins wherever the matrix is large enough to pay
    for its start and end.  The streaming kernel keeps the head."""
    if options.decode_gemm == "stream":
        return gemm_stream
    M, N, K = a.shape[0], w.shape[0], a.shape[1]
    if options.decode_gemm == "auto" and M > 16:
        elements = N * K
        if N >= 65536:
            return gemm_stream
        if _tcgen05_ok(a, w) and elements >= 16 * 1024 * 1024 and (M > 32 or N >= 6144 or elements >= 48 * 1024 * 1024):
            return gemm_tcgen05
    return gemm_skinny


def _skinny_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# ---------------------------------------------------------------------------------------------
def _plain_input(a, scratch):
    if isinstance(a, PendingNorm):
        h = scratch(a.xw.shape, torch.bfloat16)
        finish_norm(a, h)
        return h
    return a


def gemm(a, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPI_STORE, next_norm=None, scratch=None):
    """c (op)= a @ w.T with the kernel that fits dtype and sizes.

    a [M, K] and w [N, K] share a dtype (float32: the true 32-bit product on the CUDA cores;
    bfloat16: tensor-core kernels where their size rules hold, else the any-shape kernel).
    `a` may be a PendingNorm; next_norm = (weight, eps) asks for the PendingNorm of the updated c
    (EPI_RESIDUAL), which is returned where the kernel can make it and None otherwise.
    """
    x = a.xw if isinstance(a, PendingNorm) else a
    if (isinstance(a, PendingNorm) or next_norm is not None) and scratch is not None \
            and shared_norm_ok(x.shape[0], x.dtype, w.shape[0] if next_norm is not None else 8):
        if x.shape[0] <= SHARED_NORM_MAX_ROWS and _skinny_ok(x, w):
            return gemm_skinny_norm(a, w, c, epilogue, next_norm, scratch)
        if (x.shape[0] > SKINNY_MAX_ROWS or (_skinny_ok(x, w) and _decode_gemm(x, w) is gemm_tcgen05)) \
                and _tcgen05_ok(x, w) and (next_norm is None or next_norm[0].data_ptr() % 16 == 0):
            return gemm_tcgen05_norm(a, w, c, epilogue, next_norm, scratch)
    a = _plain_input(a, scratch)
    if _skinny_ok(a, w):
        _decode_gemm(a, w)(a, w, c, epilogue)
    elif _tcgen05_ok(a, w):
        gemm_tcgen05(a, w, c, epilogue)
    else:
        gemm_simt(a, w, c, epilogue)


def gemm_swiglu(a, wgu: torch.Tensor, out: torch.Tensor, interleave: int, scratch) -> None:
    """out = silu(gate) * up with [gate | up] = a @ wgu.T.  Fused into the product where a kernel can;
    otherwise the product goes to `scratch(shape, dtype)` and the SwiGLU kernel follows."""
    if isinstance(a, PendingNorm):
        if interleave == 8 and _skinny_ok(a.xw, wgu) and a.xw.shape[0] <= SHARED_NORM_MAX_ROWS:
            gemm_skinny_norm(a, wgu, out, EPI_SWIGLU)
            return
        if interleave == 8 and _tcgen05_ok(a.xw, wgu) and \
                (a.xw.shape[0] > SKINNY_MAX_ROWS or (_skinny_ok(a.xw, wgu) and _decode_gemm(a.xw, wgu) is gemm_tcgen05)):
            gemm_tcgen05_norm(a, wgu, out, EPI_SWIGLU)
            return
        a = _plain_input(a, scratch)
    if interleave == 8 and _skinny_ok(a, wgu):
        _decode_gemm(a, wgu)(a, wgu, out, EPI_SWIGLU)
        return
    if interleave == 8 and _tcgen05_ok(a, wgu):
        gemm_tcgen05(a, wgu, out, EPI_SWIGLU)
        return
    gu = scratch((a.shape[0], wgu.shape[0]), a.dtype)
    gemm(a, wgu, gu)
    swiglu(gu, out, interleave)


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = device_key(dev)
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _sm_counts[key]


def attention_decode_scratch_floats(n_seqs, num_heads, head_dim, nsplit) -> int:
    return n_seqs * num_heads * nsplit * (head_dim + 2)


def decode_splits(n_seqs: int, num_kv_heads: int, max_tiles: int, device=None) -> int:
    """How many key ranges each (sequence, kv head) is cut into, so that the grid fills the GPU:
    `options.decode_ctas_per_sm` CTAs on every SM, one wave."""
    target = options.decode_ctas_per_sm * sm_count(device)
    want = target // max(1, n_seqs * num_kv_heads)      # rounded down: all CTAs resident at once
    # at most 16: beyond that the partial results and their combination cost more than the shorter key
    # ranges save (one sequence of 2,050 keys, 8 kv heads: 11.4 us with 16 splits, 14.8 with 37)
    return max(1, min(want, max_tiles, options.decode_max_splits))


def attention_decode(q, ldq, out, k_cache, v_cache, seq_len, seq_pages, scratch, num_heads, num_kv_heads,
                     head_dim, page_size, nsplit, scale, window) -> None:
    """One query per sequence (row b of q) over the cache; scratch holds the splits' partial results."""
    _check(out, torch.bfloat16, "out"); _check(scratch, torch.float32, "scratch")
    n = out.shape[0]
    if scratch.numel() < attention_decode_scratch_floats(n, num_heads, head_dim, nsplit):
        raise BackendError("attention_decode: scratch is too small")
    _run("hb_attention_decode_bf16", q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0), k_cache.data_ptr(),
         v_cache.data_ptr(), seq_len.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0), scratch.data_ptr(),
         n, num_heads, num_kv_heads, head_dim, page_size, int(nsplit), float(scale), int(window or 0), _stream())


_DECODE_COUNTERS = 65536
_decode_counters: dict = {}


def attention_decode_fused_ok(qkv, out, num_heads, num_kv_heads, head_dim, page_size, rotary_dim, n_seqs) -> bool:
    """Whether one launch can do norm, rotation, cache write, attention and combine for this step."""
    return (options.decode_fused and out.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
            and head_dim == 128 and rotary_dim == head_dim and num_heads // num_kv_heads <= 16 and page_size % 64 == 0
            and qkv.stride(0) % 4 == 0 and qkv.data_ptr() % 8 == 0 and n_seqs * num_kv_heads <= _DECODE_COUNTERS)


def attention_decode_fused(qkv, out, k_cache, v_cache, q_weight, k_weight, eps, cos, sin, write_cache, seq_len,
                           seq_pages, scratch, num_heads, num_kv_heads, page_size, nsplit, scale, window) -> None:
    """Head size 128: the new token's q and k get their per-head norm and rotation, k and v go into
    the cache, every query attends its sequence's keys, and the key splits are combined: one kernel."""
    _check(out, torch.bfloat16, "out"); _check(scratch, torch.float32, "scratch"); _check(qkv, torch.bfloat16, "qkv")
    n = out.shape[0]
    if scratch.numel() < attention_decode_scratch_floats(n, num_heads, 128, nsplit):
        raise BackendError("attention_decode_fused: scratch is too small")
    key = device_key(out.device)
    if key not in _decode_counters:
        _decode_counters[key] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=out.device)
    _run("hb_attention_decode_fused_bf16", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), _ptr(q_weight), _ptr(k_weight), float(eps), cos.data_ptr(), sin.data_ptr(),
         cos.shape[0], 1 if write_cache else 0, seq_len.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
         scratch.data_ptr(), _decode_counters[key].data_ptr(), n, num_heads, num_kv_heads, page_size, int(nsplit),
         float(scale), int(window or 0), _stream())


def attention_prefill(q, ldq, out, k_cache, v_cache, seq_start, seq_pos0, seq_pages, n_seqs, max_q_len,
                      num_heads, num_kv_heads, head_dim, page_size, scale, window) -> None:
    """Causal attention of packed query rows (seq_start marks the sequences) over the cache."""
    _check(out, torch.bfloat16, "out")
    _run("hb_attention_prefill_bf16", q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0), k_cache.data_ptr(),
         v_cache.data_ptr(), seq_start.data_ptr(), seq_pos0.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
         int(n_seqs), int(max_q_len), num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
         _stream())


def attention_prefill_tc(q, ldq, out, k_cache, v_cache, seq_start, seq_pos0, seq_pages, n_seqs, max_q_len,
                         num_heads, num_kv_heads, head_dim, page_size, scale, window) -> None:
    """The same on tcgen05 tensor cores (head sizes 64 and 128): S and O in tensor memory."""
    _check(out, torch.bfloat16, "out")
    _run("hb_attention_prefill_tc_bf16", q.data_ptr(), int(ldq), q.shape[0], out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0], seq_start.data_ptr(), seq_pos0.data_ptr(),
         seq_pages.data_ptr(), seq_pages.stride(0), int(n_seqs), int(max_q_len), num_heads, num_kv_heads, head_dim,
         page_size, float(scale), int(window or 0), _error_flag(out.device).data_ptr(),
         _work_counter(out.device).data_ptr(), _stream())


_work_counters: dict = {}


def _work_counter(device) -> torch.Tensor:
    """One int per device from which the CTAs of a persistent kernel take their next item of work;
    zero between launches (the CTA that fetches last puts it back)."""
    key = device_key(device)
    if key not in _work_counters:
        _work_counters[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _work_counters[key]


def _prefill_tc_ok(q, ldq, out, head_dim, page_size) -> bool:
    return (options.prefill_attention == "tcgen05" and out.dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 64 == 0
            and ldq % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def _prefill_kernel_ok(out, head_dim, page_size) -> bool:
    return out.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and page_size % 64 == 0


def _decode_kernel_ok(out, num_heads, num_kv_heads, head_dim, page_size) -> bool:
    return (out.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and num_heads // num_kv_heads <= 16 and page_size % 64 == 0)


def attention(q, ldq, out, k_cache, v_cache, batch, num_heads, num_kv_heads, head_dim, page_size,
              scale, window, seq_pages, scratch=None) -> None:
    """Attention of every token of the step over its sequence's cached keys and values.

    bfloat16 steps of one token per sequence take the split-key tensor-core kernel, other bfloat16
    steps the flash kernel; head sizes or pages those cannot serve, and the float32 path, take
    the any-shape kernel."""
    if batch.is_decode and scratch is not None and _decode_kernel_ok(out, num_heads, num_kv_heads, head_dim, page_size):
        tiles = seq_pages.shape[1] * (page_size // 64)
        nsplit = decode_splits(batch.n_seqs, num_kv_heads, tiles)
        buf = scratch((attention_decode_scratch_floats(batch.n_seqs, num_heads, head_dim, nsplit),), torch.float32)
        attention_decode(q, ldq, out, k_cache, v_cache, batch.seq_len, seq_pages, buf, num_heads, num_kv_heads,
                         head_dim, page_size, nsplit, scale, window)
        return
    if _prefill_tc_ok(q, ldq, out, head_dim, page_size):
        attention_prefill_tc(q, ldq, out, k_cache, v_cache, batch.seq_start, batch.seq_pos0, seq_pages, batch.n_seqs,
                             batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size, scale, window)
        return
    if _prefill_kernel_ok(out, head_dim, page_size):
        attention_prefill(q, ldq, out, k_cache, v_cache, batch.seq_start, batch.seq_pos0, seq_pages, batch.n_seqs,
                          batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size, scale, window)
        return
    attention_simt(q, ldq, out, k_cache, v_cache, batch.tok_seq, batch.tok_pos, seq_pages, num_heads,
                   num_kv_heads, head_dim, page_size, scale, window)
