"""y = a W^T (+ bias): the one place that chooses how a matrix product runs.

* 32-bit path, or a weight that is stored in 32-bit: the plain FFMA kernel (``linear_plain``).
* bfloat16, at most ``SKINNY_ROWS`` rows, K a multiple of 8: the hand-written skinny kernel with its
  fused epilogues (bias, residual accumulate, gated activation, float32 store).
* bfloat16, more rows: the library matrix product (cuBLAS through ``torch.mm``), where the reference
  also calls its library (``cublasGemmEx`` for rows > 1, src/models/transformer.rs:1068-1084,
  src/cuda.rs:2484-2541), followed by the bias / residual kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import SK_ACCUM, SK_STORE, SK_STORE_F32, SK_SWIGLU

FOLDED_NORM_ROWS = 8     # most rows of the skinny kernel's folded RMSNorm (the kernel takes at most 8 rows)
TCGEN05_ROWS = 256       # rows of a tile of the tcgen05 kernel, and the fewest rows for which the gated product runs on it
# Measured on B200 inside a recorded decode step of the 7B shape: for 12 and 16 rows the skinny kernel with two
# 8-row tiles took 77 us for gate|up, 43 us for down and 224 us for the head, the library product with its activation
# and norm kernels 47 + 3, 29 + 3 and 181 us; the skinny kernel therefore serves 8 rows at most.
SKINNY_ROWS = 8


class Linear:
    def __init__(self, weight, bias: Optional[torch.Tensor], rt):
        """``weight``: a matrix [N, K], or a list of matrices of one width that are stacked by rows."""
        self.rt = rt
        self.weight = rt.matrix_rows(weight) if isinstance(weight, (list, tuple)) else rt.matrix(weight)    # [N, K]
        self.bias = rt.vector(bias) if bias is not None else None
        self.N, self.K = self.weight.shape
        self._bias_act = None

    # ------------------------------------------------------------------ choices
    def _plain(self) -> bool:
        return self.rt.full_precision or self.weight.dtype is torch.float32

    def _skinny(self, rows: int) -> bool:
        return (not self._plain()) and rows <= SKINNY_ROWS and self.K % 8 == 0

    def nbytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        return n + (self.bias.numel() * 4 if self.bias is not None else 0)

    # ------------------------------------------------------------------ products
    def _folds(self, a, rows: int) -> bool:
        """Whether ``a`` is a pending RMSNorm that the skinny kernel can fold in."""
        return (hasattr(a, "tensor") and a.ssq is not None and a.xw is not None and self._skinny(rows)
                and rows <= FOLDED_NORM_ROWS and a.norm.spec.kind == "rmsnorm")

    def store(self, a, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a W^T + bias in the activation dtype (``a``: activations, or a pending norm)."""
        K_ = self.rt.kernels
        M = a.shape[0]
        if out is None:
            out = self.rt.empty(M, self.N)
        if M == 0:
            return out
        if self._folds(a, M):
            K_.linear_skinny_norm(a.xw, a.ssq, a.norm.spec.eps, self.weight, self.bias, out, SK_STORE)
            return out
        if hasattr(a, "tensor"):
            a = a.tensor()
        if self._plain():
            K_.linear_plain(a, self.weight, self.bias, out)
        elif self._skinny(M):
            K_.linear_skinny(a, self.weight, self.bias, out, SK_STORE)
        else:
            if self.bias is not None and self._bias_act is None:
                self._bias_act = self.bias.to(self.rt.dtype)
            K_.library_mm(a, self.weight, out, self._bias_act)
        return out

    def accumulate(self, a: torch.Tensor, x: torch.Tensor, next_norm=None):
        """x += a W^T (+ bias), x being the float32 residual stream.  Returns a ``RowsInfo`` about the updated
        rows when the kernels left something behind that saves the next norm a pass: partial sums of squares
        (skinny product), or the rows already normalised with ``next_norm`` (library product: the residual add
        and the norm run as one kernel)."""
        from .norm import RowsInfo
        K_ = self.rt.kernels
        M = a.shape[0]
        if M == 0:
            return None
        if self._plain():
            K_.linear_plain(a, self.weight, self.bias, x, accumulate=True)
        elif self._skinny(M):
            if M > FOLDED_NORM_ROWS:
                K_.linear_skinny(a, self.weight, self.bias, x, SK_ACCUM)
                return None
            ssq = self.rt.empty(M, -(-self.N // 16), dtype=torch.float32)
            if (next_norm is not None and getattr(next_norm, "weight", None) is not None
                    and next_norm.spec.kind == "rmsnorm" and next_norm.spec.size == self.N):
                # the rows also leave multiplied by the next norm's weight: the product after that norm then
                # reads plain bf16 activations and applies the rows' factors at its end
                xw = self.rt.empty(M, self.N)
                K_.linear_skinny(a, self.weight, self.bias, x, SK_ACCUM, ssq, next_norm.weight, xw)
                return RowsInfo(ssq=ssq, xw=xw, xw_norm=next_norm)
            K_.linear_skinny(a, self.weight, self.bias, x, SK_ACCUM, ssq)
            return RowsInfo(ssq=ssq)
        elif (next_norm is not None and getattr(next_norm, "weight", None) is not None
              and next_norm.spec.kind == "rmsnorm" and next_norm.spec.size == self.N and hasattr(K_, "add_rmsnorm")):
            h = self.rt.empty(M, self.N)
            K_.add_rmsnorm(x, self.store(a), next_norm.weight, next_norm.spec.eps, h)
            return RowsInfo(norm=next_norm, h=h)
        else:
            K_.add_residual(x, self.store(a))
        return None

    def logits(self, a) -> torch.Tensor:
        """a W^T + bias in float32 whatever the path (the head)."""
        K_ = self.rt.kernels
        M = a.shape[0]
        out = self.rt.empty(M, self.N, dtype=torch.float32)
        if M == 0:
            return out
        if self._folds(a, M):
            K_.linear_skinny_norm(a.xw, a.ssq, a.norm.spec.eps, self.weight, self.bias, out, SK_STORE_F32)
            return out
        if hasattr(a, "tensor"):
            a = a.tensor()
        if self._plain() or self.K % 8:
            K_.linear_plain(a, self.weight, self.bias, out)
        elif self._skinny(M):
            K_.linear_skinny(a, self.weight, self.bias, out, SK_STORE_F32)
        else:
            # more rows than the skinny kernel streams well (it takes 600 us for 64 rows of a 152,064-wide head,
            # the library 180 us): the library product with a float32 result, the bias added to that
            K_.library_mm(a, self.weight, out, self.bias)
        return out


class GatedLinearPair:
    """gate and up projections kept as one [2I, K] matrix (gate rows first), so that one product
    gives both and the skinny kernel can apply act(gate) * up before anything is stored
    (the reference fuses the same way at load, src/models/transformer.rs:864-873, and in its
    decode GEMV mode 2, src/kernels.cu:533-537)."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, rt, activation: str = "silu"):
        from ..kernels import ACTIVATIONS
        if activation not in ACTIVATIONS:
            raise ValueError(f"gated activation '{activation}' is not one of {sorted(ACTIVATIONS)}")
        self.act = ACTIVATIONS[activation]
        self.lin = Linear([gate, up], None, rt)
        self.rt = rt
        self.I = gate.shape[0]

    def nbytes(self) -> int:
        return self.lin.nbytes()

    def _gated_on_tcgen05(self, rows: int) -> bool:
        """Whether the tcgen05 product with the fused activation beats the library product plus the activation
        kernel.  With a short sum the tile's epilogue (256 x 256 accumulators through the activation) outlasts
        its main loop: measured at 2,048 rows, K 896 / 1,536 / 2,048 / 3,584: 55 / 93 / 136 / 366 us against
        41 / 96 / 147 / 385; at 512 rows 31 / 36 / 54 / 101 against 17 / 32 / 52 / 105.  And the kernel works in
        tiles of 256 rows, a last tile that is mostly padding costing a whole one, where the library's time follows
        the rows: inside a prompt step of the 7B shape (K 3,584) 300 rows took 115 us against 65 + 11 for the
        library and the activation, 600: 163 against 103 + 16, 1,000: 209 against 167 + 25; with full tiles the two
        are within 5 % (256: 72 / 80, 1,024: 194 / 192, 2,048: 375 / 379, 4,096: 749 / 772, 8,192: 1,576 / 1,586).
        So the kernel takes the product when at most 2 % of its tiles' rows are padding."""
        K = self.lin.K
        if K % 8 or K < 1536 or rows < (TCGEN05_ROWS if K >= 3072 else 1024):
            return False
        return rows >= 0.98 * TCGEN05_ROWS * -(-rows // TCGEN05_ROWS)

    def activated(self, a) -> torch.Tensor:
        """act(a Wg^T) * (a Wu^T) in the activation dtype, [M, I]."""
        K_ = self.rt.kernels
        M = a.shape[0]
        out = self.rt.empty(M, self.I)
        if M == 0:
            return out
        if self.lin._folds(a, M):
            K_.linear_skinny_norm(a.xw, a.ssq, a.norm.spec.eps, self.lin.weight, None, out, SK_SWIGLU, act=self.act)
            return out
        if hasattr(a, "tensor"):
            a = a.tensor()
        if self.lin._skinny(M):
            K_.linear_skinny(a, self.lin.weight, None, out, SK_SWIGLU, act=self.act)
        elif (not self.lin._plain()) and self._gated_on_tcgen05(M) and hasattr(K_, "gemm_tc_pair"):
            # many rows: the tcgen05 product with the activation in its epilogue (measured 366 us against 385 us
            # for the library product followed by the activation kernel at 2,048 x 37,888 x 3,584, and without the
            # [rows, 2I] intermediate)
            K_.gemm_tc_pair(a, self.lin.weight, None, out, SK_SWIGLU, act=self.act)              # pairs of SMs, 256 x 256 tiles
        else:
            K_.swiglu(self.lin.store(a), out, self.act)
        return out
