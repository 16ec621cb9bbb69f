"""Error kinds, named after the variants of deers' ``Error`` enum (src/error.rs:8-42)."""


class DeersError(Exception):
    pass


class LayoutMismatch(DeersError):
    """Shapes or strides do not fit the op (src/error.rs:13-18)."""


class DTypeMismatch(DeersError):
    """Operand dtypes differ or are unsupported (src/error.rs:19-22)."""


class DeviceMismatch(DeersError):
    """Operands live on different devices (src/error.rs:23-26)."""


class CudaError(DeersError):
    """A backend failure, carrying the library's status text (src/error.rs:40-41)."""

    def __init__(self, status: int, text: str):
        super().__init__(f"deers_b200 status {status}: {text}")
        self.status = status
