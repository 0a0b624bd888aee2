"""Errors of the kernel language, tied to the line of the Python source they come from
(zse-compiler/zse_compiler/errors.py:13-92)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SourceLocation:
    """A place in the Python source of a kernel (zse-compiler/zse_compiler/errors.py:13-26); ``KernelError`` carries the
    same facts as ``filename`` / ``lineno`` / ``source_line`` and returns them in this form from ``location``."""
    file: str
    line: int
    col: int = 0
    text: str = ""

    def __str__(self) -> str:
        return f"{self.file}:{self.line}" + (f"\n  {self.text.strip()}" if self.text else "")


class KernelError(Exception):
    """Base class; ``str()`` gives ``file:line: message`` and the offending source line when they are known."""

    def __init__(self, message: str, filename: Optional[str] = None, lineno: Optional[int] = None,
                 source_line: Optional[str] = None):
        self.message, self.filename, self.lineno, self.source_line = message, filename, lineno, source_line
        where = f"{filename or '<kernel>'}:{lineno}: " if lineno is not None else ""
        text = where + message
        if source_line:
            text += "\n    " + source_line.strip()
        super().__init__(text)

    @property
    def location(self) -> Optional[SourceLocation]:
        if self.lineno is None:
            return None
        return SourceLocation(self.filename or "<kernel>", int(self.lineno), 0, self.source_line or "")


class KernelSyntaxError(KernelError):
    """The function uses Python that the kernel language does not have."""


class KernelTypeError(KernelError):
    """Types that cannot be combined, or an argument that does not fit its parameter."""


class KernelCompileError(KernelError):
    """nvcc rejected the generated source; ``log`` holds its output and ``source`` the CUDA text."""

    def __init__(self, message: str, log: str = "", source: str = ""):
        super().__init__(message + ("\n" + log if log else ""))
        self.log, self.source = log, source


class KernelLaunchError(KernelError):
    """A launch configuration outside the device's limits, or a driver call that failed."""
