"""``python -m zse_b200.dsl.report FILE.py [FILE.py ...]``: compiles every ``@kernel`` function found at the top level of
the given Python files for sm_100a and prints what ptxas reports for each (registers, spills, shared memory).  Needs
nvcc, not a GPU."""
from __future__ import annotations

import importlib.util
import os
import sys

from .kernel import KernelFunction


def kernels_of(path: str):
    name = "_zse_report_" + os.path.splitext(os.path.basename(path))[0]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    sys.path.insert(0, os.path.dirname(os.path.abspath(path)))
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.path.pop(0)
    return [(n, v) for n, v in vars(mod).items() if isinstance(v, KernelFunction)]


def main(argv=None) -> int:
    files = list(argv if argv is not None else sys.argv[1:])
    if not files:
        print(__doc__)
        return 2
    print("| kernel | registers | spill bytes (st/ld) | stack | static shared | barriers |")
    print("|---|---|---|---|---|---|")
    for path in files:
        for name, k in kernels_of(path):
            r = k.resources()
            print(f"| `{k.name}` | {r['registers']} | {r['spill_stores']}/{r['spill_loads']} | {r['stack_frame']} | "
                  f"{r['shared_bytes']} | {r['barriers']} |")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
