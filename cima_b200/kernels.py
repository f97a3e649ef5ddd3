"""The kernel library as Python calls: one method per entry point of ``csrc``.

Arguments are torch tensors on the GPU; the methods check dtypes, shapes and contiguity, pass raw
pointers and the current CUDA stream to the C entry points, and turn a refusal into an exception
with the library's own sentence.  There is no CPU path and no substitute: if the library cannot be
built or loaded, ``Kernels()`` raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import BuildError, library_path

F32, BF16 = 0, 1
ABI_VERSION = 20
SPLIT_BLOCKS = 296          # blocks of the decode attention that one wave holds (two per SM, 148 SMs)
TC_ATTENTION_MIN_LEN = 256  # prompts from this length on take the tcgen05 attention (head_dim 64 or 128)
SPLIT_FEW_BLOCKS = 148      # below this many blocks at 8 splits, more splits are taken
SHORT_CONTEXT_BYTES = 96 * 1024   # up to this many bytes of keys and values (one kv head) a sequence's context is one block's
                                  # work in the decode attention: no split, no merge kernel.  Measured at the 7B shape
                                  # (head_dim 128: 192 positions), batch 1 and 8: up to ~190 positions 4.4 to 6.1 us against
                                  # 6.1 to 6.6 with splits, from ~280 on 7.7 to 10 against 5.7 to 7.4; at head_dim 64 the
                                  # same bytes are 384 positions (Qwen2.5-0.5B, batch 1, contexts 137 to 265: 0.526 ms a
                                  # step without splits, 0.567 with)


def short_context(head_dim: int) -> int:
    """Positions (whole pages of 64) up to which the decode attention of this head size runs without splits."""
    return SHORT_CONTEXT_BYTES // (4 * head_dim) // 64 * 64


# epilogues of the skinny product
SK_STORE, SK_ACCUM, SK_SWIGLU, SK_STORE_F32 = 0, 1, 2, 3
# activations of a gated feed-forward's gate (CIMA_ACT_* of csrc/common.cuh), by the names config files use
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu_new": 1, "gelu": 2, "relu": 3}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt is torch.float32:
        return F32
    if dt is torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is neither float32 nor bfloat16")


_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "cima_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp, _vp, _vp, _vp],
    "cima_rmsnorm": [_vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "cima_swiglu": [_vp, _vp, _i, _i, _i, _i, _vp],
    "cima_add_residual": [_vp, _vp, _i, _sz, _vp],
    "cima_gather_rows": [_vp, _vp, _vp, _i, _i, _vp],
    "cima_add_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "cima_decode_advance": [_vp, _vp, _vp, _vp, _i, _vp],
    "cima_linear_plain": [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_linear_skinny": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "cima_linear_skinny_norm": [_vp, _vp, _i, _f, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_qkv_rope_skinny": [_vp, _vp, _i, _f, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                             _i, _i, _i, _i, _vp],
    "cima_rope_append": [_vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_attention_plain": [_vp, _i, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                             _f, _i, _i, _vp],
    "cima_attention_decode": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp],
    "cima_attention_prefill": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "cima_attention_extend": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "cima_attention_extend_tc": [_vp, _i, _vp, _vp, _vp, _vp, ctypes.c_longlong, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                 _f, _i, _vp, _vp],
    "cima_attention_prefill_tc": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp],
    "cima_gemm_tcgen05_pair": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "cima_argmax": [_vp, _i, _i, _i, _vp, _vp],
    "cima_sample": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cima_sample_general": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda dev: torch.cuda.current_stream(dev).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Kernels:
    """Loads (building first if needed) the CUDA library; fails loudly when it cannot."""

    def __init__(self, verbose: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this library runs on the GPU only")
        try:
            path = library_path(build=True, verbose=verbose)
        except BuildError as e:
            raise KernelError(f"the CUDA kernel library is missing and could not be built: {e}") from e
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from e
        self.path = path
        self.lib.cima_last_error.restype = ctypes.c_char_p
        self.lib.cima_abi_version.restype = ctypes.c_int
        if self.lib.cima_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} has ABI {self.lib.cima_abi_version()}, this package wants {ABI_VERSION}")
        for name, sig in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = sig
            fn.restype = ctypes.c_int
        self.launches = 0
        self.library_launches = 0   # matrix products handed to the library (not counted in ``launches``)
        self._scratch_bufs = {}
        self._retired = []          # replaced scratch buffers, kept alive for the graphs recorded with them
        self._error_flag = None
        self.profile = None         # a StepProfile while a step's launches are being counted and timed

    # ------------------------------------------------------------------ plumbing
    def _admit(self, name: str, nbytes: float = 0, flops: float = 0) -> bool:
        """Asked before every launch.  Without a profile it says yes.  With one (``self.profile``, see
        ``cima_b200.engine.profile``) the launch is noted with the bytes it has to move and the operations it has
        to do, and launches beyond the profile's limit are left out: a step cut after its n-th launch, timed
        against the step cut after launch n - 1, gives launch n's time inside the step."""
        p = self.profile
        return True if p is None else p.admit(name, nbytes, flops)

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            raise KernelError(f"{what}: {self.lib.cima_last_error().decode()} (code {code})")

    @staticmethod
    def _stream() -> int:
        """The current stream's handle (the capture stream while a graph is recorded).  Asked of torch's C layer
        directly: the Python wrapper costs 15 us a call, and a prompt's step makes some 150 of them."""
        return _raw_stream(torch.cuda.current_device())

    @staticmethod
    def _need(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} is on {t.device}; the kernels take GPU tensors only")
        if dtype is not None and t.dtype is not dtype:
            raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")
        if not t.is_contiguous():
            raise KernelError(f"{name} is not contiguous")

    # ------------------------------------------------------------------ elementwise
    def embed(self, ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0,
              ssq: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
              xw: Optional[torch.Tensor] = None) -> None:
        """x[t] = scale * table[ids[t]]; ``ssq`` [T, 1] (optional) receives each row's sum of squares, ``xw``
        [T, H] bf16 (optional) the rows times ``w_next`` (the weight of the norm that follows)."""
        self._need(ids, "ids", torch.int32, 1); self._need(table, "table", None, 2); self._need(x, "x", torch.float32, 2)
        T, (V, H) = ids.numel(), table.shape
        if tuple(x.shape) != (T, H):
            raise KernelError(f"embed: x is {tuple(x.shape)}, expected {(T, H)}")
        if ssq is not None:
            self._need(ssq, "ssq", torch.float32, 2)
            if tuple(ssq.shape) != (T, 1):
                raise KernelError(f"embed: ssq is {tuple(ssq.shape)}, expected {(T, 1)}")
        if xw is not None:
            self._need(xw, "xw", torch.bfloat16, 2); self._need(w_next, "w_next", torch.float32, 1)
            if tuple(xw.shape) != (T, H) or w_next.numel() != H:
                raise KernelError(f"embed: xw {tuple(xw.shape)} / w_next {tuple(w_next.shape)} do not fit {(T, H)}")
        if not self._admit("embed", T * H * (table.element_size() + 4)): return
        self._check(self.lib.cima_embed(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), x.data_ptr(),
                                        T, H, V, scale, _ptr(ssq), _ptr(w_next) if xw is not None else None, _ptr(xw),
                                        self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        self._need(x, "x", torch.float32, 2); self._need(w, "w", torch.float32, 1); self._need(out, "out", None, 2)
        T, H = x.shape
        if w.numel() != H or tuple(out.shape) != (T, H):
            raise KernelError(f"rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if not self._admit("rmsnorm", T * H * (4 + out.element_size())): return
        self._check(self.lib.cima_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                          T, H, eps, self._stream()), "rmsnorm")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor, act: int = 0) -> None:
        """out = act(gate) * up of ``gate_up`` = [gate | up]; ``act`` one of ``ACTIVATIONS``' codes."""
        self._need(gate_up, "gate_up", None, 2); self._need(out, "out", gate_up.dtype, 2)
        T, I2 = gate_up.shape
        if I2 % 2 or tuple(out.shape) != (T, I2 // 2):
            raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} and out {tuple(out.shape)} do not agree")
        if not self._admit("swiglu", T * (I2 + I2 // 2) * out.element_size()): return
        self._check(self.lib.cima_swiglu(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), T, I2 // 2, act,
                                         self._stream()), "swiglu")

    def add_residual(self, x: torch.Tensor, delta: torch.Tensor) -> None:
        self._need(x, "x", torch.float32); self._need(delta, "delta")
        if x.shape != delta.shape:
            raise KernelError(f"add_residual: x {tuple(x.shape)} and delta {tuple(delta.shape)} differ")
        if not self._admit("add_residual", x.numel() * (8 + delta.element_size())): return
        self._check(self.lib.cima_add_residual(x.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype),
                                               x.numel(), self._stream()), "add_residual")

    def add_rmsnorm(self, x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """x += delta (float32 sum), then out = RMSNorm(x; w, eps): the two kernels' results in one pass."""
        self._need(x, "x", torch.float32, 2); self._need(delta, "delta", None, 2); self._need(w, "w", torch.float32, 1)
        self._need(out, "out", delta.dtype, 2)
        T, H = x.shape
        if delta.shape != x.shape or out.shape != x.shape or w.numel() != H:
            raise KernelError(f"add_rmsnorm: x {tuple(x.shape)}, delta {tuple(delta.shape)}, out {tuple(out.shape)}, "
                              f"w {tuple(w.shape)} do not agree")
        if not self._admit("add_rmsnorm", T * H * (8 + 2 * delta.element_size())): return
        self._check(self.lib.cima_add_rmsnorm(x.data_ptr(), delta.data_ptr(), w.data_ptr(), out.data_ptr(),
                                              dtype_code(delta.dtype), T, H, eps, self._stream()), "add_rmsnorm")

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        self._need(x, "x", torch.float32, 2); self._need(rows, "rows", torch.int32, 1); self._need(out, "out", torch.float32, 2)
        if tuple(out.shape) != (rows.numel(), x.shape[1]):
            raise KernelError(f"gather_rows: out is {tuple(out.shape)}, expected {(rows.numel(), x.shape[1])}")
        if not self._admit("gather_rows", rows.numel() * x.shape[1] * 8): return
        self._check(self.lib.cima_gather_rows(x.data_ptr(), rows.data_ptr(), out.data_ptr(), rows.numel(),
                                              x.shape[1], self._stream()), "gather_rows")

    def decode_advance(self, chosen: torch.Tensor, tokens: torch.Tensor, row_pos: torch.Tensor, seq_len: torch.Tensor) -> None:
        """tokens = chosen; every row's position and every sequence's length + 1 (one token per sequence)."""
        B = tokens.numel()
        for n, t in (("chosen", chosen), ("tokens", tokens), ("row_pos", row_pos), ("seq_len", seq_len)):
            self._need(t, n, torch.int32, 1)
            if t.numel() != B:
                raise KernelError(f"decode_advance: {n} has {t.numel()} entries, expected {B}")
        if not self._admit("decode_advance", 16 * B): return
        self._check(self.lib.cima_decode_advance(chosen.data_ptr(), tokens.data_ptr(), row_pos.data_ptr(),
                                                 seq_len.data_ptr(), B, self._stream()), "decode_advance")

    # ------------------------------------------------------------------ matrix products
    def linear_plain(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     accumulate: bool = False) -> None:
        """out = a @ w.T (+ bias), or out += ... when ``accumulate`` (out float32)."""
        self._need(a, "a", None, 2); self._need(w, "w", None, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear_plain: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError(f"linear_plain: bias has {bias.numel()} entries, expected {N}")
        if not self._admit("linear_plain", w.numel() * w.element_size() + (M * K + M * N) * 4, 2.0 * M * N * K): return
        # one launch takes up to 65535 * 64 rows; cut above that
        step = 65535 * 64
        for m0 in range(0, M, step):
            m1 = min(M, m0 + step)
            self._check(self.lib.cima_linear_plain(a[m0:m1].data_ptr(), dtype_code(a.dtype), w.data_ptr(),
                                                   dtype_code(w.dtype), _ptr(bias), out[m0:m1].data_ptr(),
                                                   dtype_code(out.dtype), 1 if accumulate else 0, m1 - m0, N, K,
                                                   K, N, self._stream()), "linear_plain")

    def linear_skinny(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                      mode: int, ssq_out: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
                      xw_out: Optional[torch.Tensor] = None, act: int = 0) -> None:
        """Few rows (<= 8), bf16 operands; ``mode`` is one of SK_*.  For SK_SWIGLU ``w`` is [2N, K].
        With SK_ACCUM, ``ssq_out`` [M, ceil(N / 16)] receives partial sums of squares of the updated rows and
        ``xw_out`` [M, N] bf16 the updated rows times ``w_next`` (the weight of the norm that follows)."""
        self._need(a, "a", torch.bfloat16, 2); self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode in (SK_ACCUM, SK_STORE_F32) else torch.bfloat16
        if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"linear_skinny(mode {mode}): a {tuple(a.shape)}, w {tuple(w.shape)}, "
                              f"out {tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError(f"linear_skinny: bias has {bias.numel()} entries, expected {N}")
        if ssq_out is not None:
            self._need(ssq_out, "ssq_out", torch.float32, 2)
            if mode != SK_ACCUM or tuple(ssq_out.shape) != (M, -(-N // 16)):
                raise KernelError(f"linear_skinny: ssq_out {tuple(ssq_out.shape)} goes with the accumulating mode and "
                                  f"must be {(M, -(-N // 16))}")
        if xw_out is not None:
            self._need(xw_out, "xw_out", torch.bfloat16, 2); self._need(w_next, "w_next", torch.float32, 1)
            if ssq_out is None or tuple(xw_out.shape) != (M, N) or w_next.numel() != N:
                raise KernelError("linear_skinny: xw_out goes with ssq_out and must be [rows, N], w_next [N]")
        if not self._admit(f"linear_skinny[{mode}]", w.numel() * 2 + M * K * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_linear_skinny(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode,
                                                M, N, K, K, N, _ptr(ssq_out), _ptr(w_next) if xw_out is not None else None,
                                                _ptr(xw_out), act, self._stream()), "linear_skinny")

    def linear_skinny_norm(self, xw: torch.Tensor, ssq: torch.Tensor, eps: float, w: torch.Tensor,
                           bias: Optional[torch.Tensor], out: torch.Tensor, mode: int, act: int = 0) -> None:
        """``linear_skinny`` of RMSNorm(x) for at most 8 rows: ``xw`` [M, K] bf16 = bf16(x * norm weight) and
        ``ssq`` [M, parts], the partial sums of squares of the rows x, as ``embed`` or an accumulating
        ``linear_skinny`` left them."""
        self._need(xw, "xw", torch.bfloat16, 2); self._need(ssq, "ssq", torch.float32, 2)
        self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = xw.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode == SK_STORE_F32 else torch.bfloat16
        if w.shape[1] != K or ssq.shape[0] != M or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"linear_skinny_norm(mode {mode}): xw {tuple(xw.shape)}, w {tuple(w.shape)}, ssq "
                              f"{tuple(ssq.shape)}, out {tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        if not self._admit(f"linear_skinny_norm[{mode}]", w.numel() * 2 + M * K * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_linear_skinny_norm(xw.data_ptr(), ssq.data_ptr(), ssq.shape[1], eps, w.data_ptr(),
                                                     _ptr(bias), out.data_ptr(), mode, M, N, K, K, N, act, self._stream()),
                    "linear_skinny_norm")

    def qkv_rope(self, a, w: torch.Tensor, bias: Optional[torch.Tensor], qkv: torch.Tensor, inv_freq: torch.Tensor,
                 row_pos, row_seq, seq_slot, kv, n_heads: int, n_kv_heads: int, head_dim: int, norm=None) -> None:
        """The q/k/v projection of a decode step (at most 8 rows) with rotation and cache append in its
        epilogue: the rotated q lands in ``qkv`` [rows, (heads + 2 kv_heads) * head_dim], k and v in the layer's
        pages.  ``a``: bf16 activations, or with ``norm = (ssq, eps)`` the rows bf16(x * norm weight) and
        the partial sums of squares of x: the RMSNorm is folded in."""
        self._need(w, "w", torch.bfloat16, 2); self._need(qkv, "qkv", torch.bfloat16, 2)
        self._need(inv_freq, "inv_freq", torch.float32, 1)
        M, K = a.shape
        N = (n_heads + 2 * n_kv_heads) * head_dim
        if tuple(w.shape) != (N, K) or tuple(qkv.shape) != (M, N) or inv_freq.numel() != head_dim // 2:
            raise KernelError(f"qkv_rope: a {tuple(a.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}, inv_freq "
                              f"{tuple(inv_freq.shape)} do not agree with {n_heads}+2x{n_kv_heads} heads of {head_dim}")
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        if tuple(kv.storage.shape[1:]) != (2, n_kv_heads, kv.page_size, head_dim):
            raise KernelError(f"qkv_rope: cache pages are {tuple(kv.storage.shape)}")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        self._need(a, "a", torch.bfloat16, 2)
        if norm is None:
            head = (a.data_ptr(), None, 0, 0.0)
        else:
            ssq, eps = norm
            self._need(ssq, "ssq", torch.float32, 2)
            if ssq.shape[0] != M:
                raise KernelError(f"qkv_rope: ssq {tuple(ssq.shape)} does not fit {M} rows")
            head = (a.data_ptr(), ssq.data_ptr(), ssq.shape[1], eps)
        if not self._admit("qkv_rope_skinny", w.numel() * 2 + M * K * 2 + M * N * 2, 2.0 * M * N * K): return
        self._check(self.lib.cima_qkv_rope_skinny(*head, w.data_ptr(), _ptr(bias), qkv.data_ptr(), M, K, K, N,
                                                  inv_freq.data_ptr(), row_pos.data_ptr(), row_seq.data_ptr(),
                                                  seq_slot.data_ptr(), kv.storage.data_ptr(), kv.block_table.data_ptr(),
                                                  kv.block_table.shape[1], kv.ring_pages, kv.page_size, n_heads,
                                                  n_kv_heads, head_dim, self._stream()), "qkv_rope_skinny")

    def gemm_tc_pair(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     mode: int, act: int = 0) -> None:
        """out = epilogue(a @ w.T) on the tcgen05 tensor cores, for many rows: bf16 operands by TMA, float32
        accumulation in tensor memory, pairs of SMs on tiles of 256 x 256 (cta_group::2; each SM of a pair stages
        only half of the weight tile).  ``mode`` as for ``linear_skinny`` (SK_*); for SK_SWIGLU ``w`` is [2N, K]."""
        self._need(a, "a", torch.bfloat16, 2); self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode in (SK_ACCUM, SK_STORE_F32) else torch.bfloat16
        if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"gemm_tc_pair(mode {mode}): a {tuple(a.shape)}, w {tuple(w.shape)}, out "
                              f"{tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=a.device)
        if not self._admit(f"gemm_tcgen05_pair[{mode}]", (w.numel() + M * K) * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_gemm_tcgen05_pair(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, M,
                                                    w.shape[0], K, N, N if mode == SK_SWIGLU else 0, act,
                                                    self._error_flag.data_ptr(), self._stream()), "gemm_tcgen05_pair")

    def error_flag(self, device) -> torch.Tensor:
        """The int32 word that kernels with bounded waits set when a wait runs out (``device_errors`` reads it)."""
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        return self._error_flag

    def device_errors(self) -> int:
        """The error flag that a bounded wait inside a kernel sets when it runs out (synchronises).  Reading it
        clears it: a later, sound step is not blamed for an earlier one."""
        if self._error_flag is None:
            return 0
        v = int(self._error_flag.item())
        if v:
            self._error_flag.zero_()
        return v

    # ------------------------------------------------------------------ attention
    def rope_append(self, qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, row_pos, row_seq, seq_slot,
                    seq_len, kv, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        """Rotate q and k of ``qkv`` in place and append k, v to the layer's pages (``kv`` a LayerKV or None)."""
        self._need(qkv, "qkv", None, 2); self._need(inv_freq, "inv_freq", torch.float32, 1)
        for n, t in (("row_pos", row_pos), ("row_seq", row_seq), ("seq_slot", seq_slot), ("seq_len", seq_len)):
            self._need(t, n, torch.int32, 1)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError(f"rope_append: inv_freq has {inv_freq.numel()} entries, expected {rotary_dim // 2}")
        T = qkv.shape[0]
        if row_pos.numel() < T or row_seq.numel() < T:
            raise KernelError("rope_append: the rows' positions do not cover the rows")
        if kv is not None:
            self._need(kv.storage, "cache", qkv.dtype, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
            if tuple(kv.storage.shape[1:]) != (2, n_kv_heads, kv.page_size, head_dim):
                raise KernelError(f"rope_append: cache pages are {tuple(kv.storage.shape)}, expected "
                                  f"[*, 2, {n_kv_heads}, {kv.page_size}, {head_dim}]")
            args = (kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.ring_pages, kv.page_size)
        else:
            args = (None, None, 0, 0, 0)
        if not self._admit("rope_append", 2 * qkv.numel() * qkv.element_size()): return
        self._check(self.lib.cima_rope_append(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[1], inv_freq.data_ptr(),
                                              rotary_dim, row_pos.data_ptr(), row_seq.data_ptr(), seq_slot.data_ptr(),
                                              seq_len.data_ptr(), *args, T, n_heads, n_kv_heads, head_dim, self._stream()), "rope_append")

    def attention_plain(self, qkv: torch.Tensor, kv, row_pos, row_seq, seq_slot, seq_first_row, out: torch.Tensor,
                        n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int,
                        from_cache: bool) -> None:
        self._need(qkv, "qkv", None, 2); self._need(out, "out", qkv.dtype, 2)
        T = qkv.shape[0]
        if tuple(out.shape) != (T, n_heads * head_dim):
            raise KernelError(f"attention: out is {tuple(out.shape)}, expected {(T, n_heads * head_dim)}")
        if from_cache:
            if kv is None:
                raise KernelError("attention: decoding needs the layer's cache")
            self._need(kv.storage, "cache", qkv.dtype, 5)
            args = (kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.ring_pages, kv.page_size)
        else:
            args = (None, None, 0, 0, 1)
        if not self._admit("attention_plain", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        self._check(self.lib.cima_attention_plain(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[1], *args,
                                                  row_pos.data_ptr(), row_seq.data_ptr(), seq_slot.data_ptr(),
                                                  seq_first_row.data_ptr(), out.data_ptr(), out.shape[1], T,
                                                  n_heads, n_kv_heads, head_dim, scale, window,
                                                  1 if from_cache else 0, self._stream()), "attention_plain")

    def _attention_work(self, qkv, n_heads, n_kv_heads, head_dim):
        """(bytes, operations) of an attention launch while a step is profiled: the keys and values of the step's
        sequences (``profile.kv_tokens``: positions that the step's rows read, each once) and the products over the
        (query, key) pairs (``profile.qk_pairs``); the step's maker states both."""
        p = self.profile
        if p is None:
            return 0, 0
        elt = qkv.element_size()
        return (2.0 * p.kv_tokens * n_kv_heads * head_dim * elt + 2.0 * qkv.shape[0] * n_heads * head_dim * elt,
                4.0 * p.qk_pairs * n_heads * head_dim)

    def library_mm(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """out = a @ w.T (+ bias) by the library's matrix product (cuBLAS through torch), where the reference calls
        its library too; ``out`` may be float32 for bfloat16 operands (the head).  Counted apart from this
        library's own launches."""
        if not self._admit("library_mm", (w.numel() + a.numel()) * a.element_size() + out.numel() * out.element_size(),
                           2.0 * a.shape[0] * w.shape[0] * w.shape[1]):
            return
        self.library_launches += 1
        if out.dtype is not a.dtype:
            torch.mm(a, w.t(), out_dtype=out.dtype, out=out)
            if bias is not None:
                out += bias
        elif bias is not None:
            torch.addmm(bias, a, w.t(), out=out)
        else:
            torch.mm(a, w.t(), out=out)

    def attention(self, qkv: torch.Tensor, kv, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                  head_dim: int, scale: float, window: int, from_cache: bool, after_append: bool = False) -> None:
        """Attention of a step's rows: over the step's own keys (a prompt from position 0) or over the
        cache.  Chooses the kernel; every choice computes the same function.  ``after_append``: the kernel
        launched just before wrote nothing but ``qkv`` and the newest position of each sequence in the cache."""
        if (from_cache and qkv.dtype is torch.bfloat16 and kv.page_size == 64 and head_dim % 16 == 0
                and head_dim <= 128 and batch.n_rows == batch.n_seqs):
            return self.attention_decode(qkv, kv, batch.seq_slot, batch.seq_len, out, n_heads, n_kv_heads, head_dim,
                                         scale, window, batch.max_len, early=after_append)
        many = (qkv.dtype is torch.bfloat16 and head_dim in (64, 128) and qkv.shape[1] % 8 == 0
                and getattr(batch, "n_q_tiles_tc", 0) > 0 and getattr(batch, "max_rows", 0) >= TC_ATTENTION_MIN_LEN)
        if from_cache and many and kv.page_size == 64 and kv.storage.numel() // head_dim < 2 ** 31:
            return self.attention_prefill_tc(qkv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, kv=kv)
        if (from_cache and qkv.dtype is torch.bfloat16 and kv.page_size == 64 and head_dim % 16 == 0
                and head_dim <= 128 and qkv.shape[1] % 8 == 0 and getattr(batch, "n_q_tiles", 0) > 0):
            return self.attention_extend(qkv, kv, batch, out, n_heads, n_kv_heads, head_dim, scale, window)
        if not from_cache and many:
            return self.attention_prefill_tc(qkv, batch, out, n_heads, n_kv_heads, head_dim, scale, window)
        if (not from_cache and qkv.dtype is torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128
                and qkv.shape[1] % 8 == 0 and getattr(batch, "n_q_tiles", 0) > 0):
            return self.attention_prefill(qkv, batch.q_tile_seq, batch.q_tile_row0, batch.seq_first_row, out,
                                          n_heads, n_kv_heads, head_dim, scale, window)
        self.attention_plain(qkv, kv, batch.row_pos, batch.row_seq, batch.seq_slot, batch.seq_first_row, out,
                             n_heads, n_kv_heads, head_dim, scale, window, from_cache)

    def attention_prefill(self, qkv: torch.Tensor, tile_seq, tile_row0, seq_first_row, out: torch.Tensor,
                          n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int) -> None:
        """Flash attention of ragged prompts that start at position 0 (bf16, head_dim <= 128);
        ``tile_seq``/``tile_row0`` list the blocks of 64 query rows."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        for n, t in (("tile_seq", tile_seq), ("tile_row0", tile_row0), ("seq_first_row", seq_first_row)):
            self._need(t, n, torch.int32, 1)
        T = qkv.shape[0]
        if tuple(out.shape) != (T, n_heads * head_dim) or tile_seq.numel() != tile_row0.numel():
            raise KernelError(f"attention_prefill: out {tuple(out.shape)} or the block list do not fit")
        if not self._admit("attention_prefill", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        self._check(self.lib.cima_attention_prefill(qkv.data_ptr(), qkv.shape[1], tile_seq.data_ptr(), tile_row0.data_ptr(),
                                                    seq_first_row.data_ptr(), out.data_ptr(), out.shape[1], T,
                                                    tile_seq.numel(), n_heads, n_kv_heads, head_dim, scale, window,
                                                    self._stream()), "attention_prefill")

    def attention_extend(self, qkv: torch.Tensor, kv, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int) -> None:
        """Flash attention of sequences that bring several rows to a cache that already holds keys (bf16, pages of
        64, head_dim <= 128): the rows of sequence s stand at positions seq_len[s] - rows .. seq_len[s] - 1, and all
        keys, the step's own included, are read from the layer's pages.  ``batch`` brings the blocks of 64 rows."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        T = qkv.shape[0]
        if tuple(out.shape) != (T, n_heads * head_dim) or batch.q_tile_seq.numel() != batch.q_tile_row0.numel():
            raise KernelError(f"attention_extend: out {tuple(out.shape)} or the block list do not fit")
        if not self._admit("attention_extend", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        self._check(self.lib.cima_attention_extend(
            qkv.data_ptr(), qkv.shape[1], batch.q_tile_seq.data_ptr(), batch.q_tile_row0.data_ptr(),
            batch.seq_first_row.data_ptr(), kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
            kv.ring_pages, kv.page_size, batch.seq_slot.data_ptr(), batch.seq_len.data_ptr(), out.data_ptr(), out.shape[1],
            T, batch.q_tile_seq.numel(), n_heads, n_kv_heads, head_dim, scale, window, self._stream()), "attention_extend")

    def attention_prefill_tc(self, qkv: torch.Tensor, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                             head_dim: int, scale: float, window: int, kv=None) -> None:
        """Flash attention of ragged prompts on the tcgen05 tensor cores (bf16, head_dim 64 or 128): blocks of 128
        query rows, both products with their results in tensor memory.  ``batch`` brings the blocks
        (``q_tile_tc_*``).  Without ``kv`` the sequences start at position 0 and the keys are the step's own rows;
        with ``kv`` (a layer's pages, to which the step has appended) the rows of sequence s stand at positions
        seq_len[s] - rows .. seq_len[s] - 1 and all keys come from the pages."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        T = qkv.shape[0]
        if tuple(out.shape) != (T, n_heads * head_dim) or batch.n_q_tiles_tc <= 0:
            raise KernelError(f"attention_prefill_tc: out {tuple(out.shape)} or the block list do not fit")
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=qkv.device)
        if not self._admit("attention_prefill_tc", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        if kv is not None:
            self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
            self._check(self.lib.cima_attention_extend_tc(
                qkv.data_ptr(), qkv.shape[1], batch.q_tile_tc_seq.data_ptr(), batch.q_tile_tc_row0.data_ptr(),
                batch.seq_first_row.data_ptr(), kv.storage.data_ptr(), kv.storage.shape[0], kv.block_table.data_ptr(),
                kv.block_table.shape[1], kv.ring_pages, kv.page_size, batch.seq_slot.data_ptr(), batch.seq_len.data_ptr(),
                out.data_ptr(), out.shape[1], T, batch.n_q_tiles_tc, n_heads, n_kv_heads, head_dim, scale, window,
                self._error_flag.data_ptr(), self._stream()), "attention_extend_tc")
            return
        self._check(self.lib.cima_attention_prefill_tc(
            qkv.data_ptr(), qkv.shape[1], batch.q_tile_tc_seq.data_ptr(), batch.q_tile_tc_row0.data_ptr(),
            batch.seq_first_row.data_ptr(), out.data_ptr(),
            out.shape[1], T, batch.n_q_tiles_tc, n_heads, n_kv_heads, head_dim, scale, window,
            self._error_flag.data_ptr(), self._stream()), "attention_prefill_tc")

    def attention_decode(self, qkv: torch.Tensor, kv, seq_slot, seq_len, out: torch.Tensor, n_heads: int,
                         n_kv_heads: int, head_dim: int, scale: float, window: int, max_len: int = 0,
                         n_splits: Optional[int] = None, early: bool = False) -> None:
        """One query per sequence over the paged cache (bf16, pages of 64, head_dim <= 128), keys split
        over ``n_splits`` blocks per (sequence, kv head).  ``max_len`` (0 = unknown) only bounds the
        number of splits chosen here.  ``early``: the kernel launched just before this one wrote neither
        ``seq_slot``, ``seq_len``, the block table nor a page before the one of a sequence's newest position,
        so the first pages may be fetched while it finishes."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        B = qkv.shape[0]
        if tuple(out.shape) != (B, n_heads * head_dim) or seq_slot.numel() < B or seq_len.numel() < B:
            raise KernelError(f"attention_decode: out {tuple(out.shape)} / sequences do not fit {B} rows")
        if n_splits is None:
            mtiles = -(-(n_heads // n_kv_heads) // 16)
            # one wave of blocks (two of them fit an SM): never a second, nearly empty wave; beyond 8 splits
            # only while the GPU would otherwise stay mostly idle.  The splits are merged by a second kernel: merging
            # inside a thread-block cluster (clusters of 8 blocks with 100 KB of shared memory each are slow to
            # place) and merging in the last block to finish (a fence and a ticket per block) were both measured
            # slower inside the decode step
            base = B * n_kv_heads * mtiles
            # 32 splits at most, 64 where even 32 leave SMs without a block (one sequence of 4 kv heads: measured at
            # the 7B shape 19 to 25 us against 28 to 31 at 30,000 positions, 15 against 19 at 16,384, the same up to
            # 6,000; with two sequences 32 are the best again)
            n_splits = max(1, min(64 if base * 32 < SPLIT_FEW_BLOCKS else 32, SPLIT_BLOCKS // base))
            if n_splits > 8 and base * 8 >= SPLIT_FEW_BLOCKS:
                n_splits = 8
            if max_len > 0:
                n_splits = min(n_splits, -(-max_len // 64))
                # a short context is a few pages: one block reads them in less time than the merge of splits takes
                if max_len <= short_context(head_dim):
                    n_splits = 1
        if not self._admit(f"attention_decode[{n_splits} splits]", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        part_o = part_ml = None
        if n_splits > 1:
            part_o = self._scratch("attn_o", B * n_heads * n_splits * head_dim, qkv.device)
            part_ml = self._scratch("attn_ml", B * n_heads * n_splits * 2, qkv.device)
        self._check(self.lib.cima_attention_decode(
            qkv.data_ptr(), qkv.shape[1], kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
            kv.ring_pages, kv.page_size, seq_slot.data_ptr(), seq_len.data_ptr(), _ptr(part_o), _ptr(part_ml),
            out.data_ptr(), out.shape[1], B, n_heads, n_kv_heads, head_dim, scale, window, n_splits, int(early),
            self._stream()), "attention_decode")
        if n_splits > 1:
            self.launches += 1

    def _scratch(self, name: str, numel: int, device) -> torch.Tensor:
        """Float32 scratch that lives as long as this object (grown on demand, outside graph capture:
        a captured step always follows an eager one of the same sizes).  A buffer that a larger one replaces is
        kept, not freed: a captured step holds the address it was recorded with and goes on writing there."""
        t = self._scratch_bufs.get(name)
        if t is None or t.numel() < numel or t.device != torch.device(device):
            if t is not None:
                self._retired.append(t)
            t = self._scratch_bufs[name] = torch.empty(numel, dtype=torch.float32, device=device)
        return t

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits: torch.Tensor, tokens: torch.Tensor) -> None:
        self._need(logits, "logits", torch.float32, 2); self._need(tokens, "tokens", torch.int32, 1)
        n, V = logits.shape
        if tokens.numel() < n:
            raise KernelError(f"argmax: {tokens.numel()} token places for {n} rows")
        if not self._admit("argmax", n * V * 4): return
        self._check(self.lib.cima_argmax(logits.data_ptr(), V, n, V, tokens.data_ptr(), self._stream()), "argmax")

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, params: torch.Tensor, rng: torch.Tensor,
               ring: torch.Tensor, count: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor,
               all_greedy: bool = False, general: bool = False) -> None:
        """The whole sampling chain per row; per-slot state (rng, ring, count) is read and advanced.
        ``all_greedy`` (no row penalises or draws) takes the argmax kernel and leaves the state alone.
        ``general``: the one-block-per-row kernel whatever the size (it otherwise serves only vocabularies too long
        for the fast kernel's shared memory)."""
        self._need(logits, "logits", torch.float32, 2); self._need(tokens, "tokens", torch.int32, 1)
        n, V = logits.shape
        if tokens.numel() < n:
            raise KernelError(f"sample: {tokens.numel()} token places for {n} rows")
        if not self._admit("argmax" if all_greedy else "sample", n * V * 4): return
        if all_greedy:
            self._check(self.lib.cima_argmax(logits.data_ptr(), V, n, V, tokens.data_ptr(), self._stream()), "argmax")
            return
        self._need(row_slot, "row_slot", torch.int32, 1); self._need(params, "params", torch.float32, 2)
        self._need(rng, "rng", torch.int64); self._need(ring, "ring", torch.int32, 2); self._need(count, "count", torch.int32)
        self._need(work, "work", torch.float32, 2)
        if params.shape != (n, 4) or ring.shape[1] != 64 or work.shape[0] < n or work.shape[1] != V:
            raise KernelError("sample: params must be [rows, 4], the ring [slots, 64], the scratch [>= rows, vocab]")
        fn = self.lib.cima_sample_general if general else self.lib.cima_sample
        self._check(fn(logits.data_ptr(), V, n, V, row_slot.data_ptr(), params.data_ptr(), rng.data_ptr(),
                       ring.data_ptr(), count.data_ptr(), work.data_ptr(), tokens.data_ptr(), self._stream()), "sample")
