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


def get_kernel_source_lines(func) -> list:
    """The dedented source lines of a kernel function; an empty list when the source cannot be read
    (zse-compiler/zse_compiler/errors.py:69-75)."""
    import inspect
    import textwrap
    func = getattr(func, "_func", func)               # a decorated kernel or the plain function
    try:
        return textwrap.dedent(inspect.getsource(func)).split("\n")
    except (OSError, TypeError):
        return []


def format_parse_error(func, node_line: int, message: str, context: int = 2) -> str:
    """A message with the offending line of the kernel (1-based, relative to the function) and ``context`` lines on
    either side, for tools that report several problems at once; ``KernelError`` itself carries file and line
    (zse-compiler/zse_compiler/errors.py:78-92)."""
    name = getattr(func, "__name__", getattr(func, "name", "kernel"))
    lines = get_kernel_source_lines(func)
    if not lines or node_line <= 0 or node_line > len(lines):
        return f"Parse error in '{name}': {message}"
    out = [f"Parse error in '{name}', line {node_line}:"]
    for i in range(max(0, node_line - 1 - context), min(len(lines), node_line + context)):
        out.append(f"  {'>>' if i == node_line - 1 else '  '} {i + 1:3d}| {lines[i]}")
    out.append(f"  Error: {message}")
    return "\n".join(out)
