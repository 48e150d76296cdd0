"""One prepared sample and its input contract.

Retained reference surface: the class name, its five fields in this order, the ``shape`` property and
the wording of every rejection are what the reference's callers, tests and stored samples rely on
(``python/adangel/trace/schema.py:8-47``), so they are kept as they are; the checking code is this
build's own.  The contract -- INT8 ``A[M,K]`` with an FP32 scale per row, packed E2M1 ``W[N,K/2]`` with a
UE8M0 code per K32 block, K a multiple of 64, no scale code 255 -- is what every ops entry point
enforces before it touches the GPU (the native side repeats it, ``csrc/runtime.cu: check_shape``).
"""

from __future__ import annotations

from dataclasses import dataclass

FORMAL_SHAPE = (4096, 4096, 4096)
FORBIDDEN_SCALE_CODE = 255  # UE8M0 NaN


@dataclass(frozen=True)
class PreparedInputs:
    sample_id: str
    A_int8: object
    A_scale: object
    W_mxfp4: object
    W_scale: object

    @property
    def shape(self) -> tuple[int, int, int]:
        """(M, N, K) of ``Y[M,N] = A[M,K] @ W[N,K].T``."""
        rows_a, k = self.A_int8.shape
        rows_w = self.W_mxfp4.shape[0]
        return int(rows_a), int(rows_w), int(k)


def _field_contract(m: int, n: int, k: int):
    """Field name -> (shape, torch dtype name) for a problem of M x N x K."""
    return (
        ("A_int8", (m, k), "int8"),
        ("A_scale", (m,), "float32"),
        ("W_mxfp4", (n, k // 2), "uint8"),
        ("W_scale", (n, k // 32), "uint8"),
    )


def validate_prepared(inputs: PreparedInputs, formal: bool = False) -> None:
    """Raises ``TypeError`` / ``ValueError`` with the reference's messages when ``inputs`` breaks the
    contract; ``formal=True`` additionally pins the canonical 4096^3 shape."""
    import torch

    fields = {name: getattr(inputs, name) for name, _, _ in _field_contract(1, 1, 64)}
    if any(not isinstance(value, torch.Tensor) for value in fields.values()):
        raise TypeError("prepared fields must be torch.Tensor instances")
    m, n, k = inputs.shape
    if formal and (m, n, k) != FORMAL_SHAPE:
        raise ValueError(f"formal experiment requires 4096^3, got {(m, n, k)}")
    if k % 64 != 0:
        raise ValueError("K must be divisible by 64 for the O2 MMA")
    for name, shape, dtype_name in _field_contract(m, n, k):
        tensor, dtype = fields[name], getattr(torch, dtype_name)
        if tuple(tensor.shape) != shape or tensor.dtype != dtype:
            raise ValueError(f"{name}: expected {shape}/{dtype}, got {tuple(tensor.shape)}/{tensor.dtype}")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if bool((fields["W_scale"] == FORBIDDEN_SCALE_CODE).any()):
        raise ValueError("UE8M0 NaN scale code 255 is forbidden")
