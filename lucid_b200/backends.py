"""Engine switch for the quantized modules (lucid/backends/__init__.py:57-96).

The reference's values are ``"auto" | "mlx_group" | "reference"``; this build
adds ``"b200_i8"`` (the integer tcgen05 path) and makes ``"auto"`` select it.
``"reference"`` keeps its meaning -- dequantize the weight, run the float
contraction, fake-quantize the result -- evaluated on the GPU with this
package's streaming kernels around a library float GEMM.  ``"mlx_group"`` names
a Metal kernel that does not exist on this platform and is rejected when used.
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
        if self._engine == "reference":
            return False
        if self._engine == "mlx_group":
            raise _lib.EngineUnavailable("the MLX group-wise kernel is unavailable on this platform")
        return True

    # name kept for callers written against the reference
    def use_mlx(self) -> bool:
        return False


quantized = _QuantizedBackend()

__all__ = ["quantized"]
