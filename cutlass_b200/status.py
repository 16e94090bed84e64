"""Status object returned by support checks (same contract as the reference's
``operators/cutlass/operators/status.py:35``): truthy on success, carries the
exception otherwise."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Status:
    error: Exception | None = None

    def __bool__(self) -> bool:
        return self.error is None

    @classmethod
    def success(cls) -> "Status":
        return cls()

    @classmethod
    def fail(cls, error: str | Exception) -> "Status":
        if isinstance(error, str):
            error = ValueError(error)
        return cls(error=error)

    def raise_on_error(self) -> None:
        if self.error is not None:
            raise self.error
