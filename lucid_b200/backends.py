"""Engine switch for the quantized modules (lucid/backends/__init__.py:57-96).

The reference's values are ``"auto" | "mlx_group" | "reference"``; this build
adds ``"b200_i8"`` (the integer tcgen05 path) and makes ``"auto"`` select it.
``"reference"`` keeps its meaning -- dequantize the weight, run the float
contraction, fake-quantize the result -- evaluated on the GPU with this
package's streaming kernels around a library float GEMM.  ``"mlx_group"`` keeps
the reference's meaning too: ``convert`` / ``quantize_dynamic`` route the Linear
family to the weight-only group-wise layer (``QuantizedLinearMLX``, here on this
library's CUDA kernels), everything else takes the dequantize-to-float route.
Unlike the reference, ``"auto"`` does not pick that route: it selects the integer
W8A8 path.
"""

from __future__ import annotations

from . import _lib

_VALID = ("auto", "b200_i8", "mlx_group", "reference")


class _QuantizedBackend:
    _engine: str = "auto"

    @property
    def available(self) -> bool:
        """True if the B200 kernels are built and a CUDA device is visible."""
        return _lib.is_available()

    @property
    def engine(self) -> str:
        return self._engine

    @engine.setter
    def engine(self, value: str) -> None:
        if value not in _VALID:
            raise ValueError(
                "quantized.engine must be 'auto'/'b200_i8'/'mlx_group'/'reference', "
                f"got {value!r}")
        self._engine = value

    def use_int8(self) -> bool:
        """Whether modules run the integer GEMM given the current mode."""
        return self._engine in ("auto", "b200_i8")

    def use_mlx(self) -> bool:
        """Whether ``convert`` / ``quantize_dynamic`` route Linear layers to the group-wise
        weight-only kernel (lucid/backends/__init__.py:90-96)."""
        return self._engine == "mlx_group"


quantized = _QuantizedBackend()

__all__ = ["quantized"]
