"""``python -m zse_b200.format <hf_dir> <out.zse> --quant int4|int8|fp16 --group-size 128 --arch X --no-tokenizer -q``
(zse-engine/zse_engine/format/__main__.py:39-123)."""
import argparse
import sys
import time

from .convert import convert_hf_to_zse
from .spec import QuantMethod


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="zse-convert", description="Convert a HuggingFace model directory to .zse")
    ap.add_argument("model_dir")
    ap.add_argument("output")
    ap.add_argument("--quant", default="int4", choices=["int4", "int8", "fp16"])
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--arch", default=None)
    ap.add_argument("--no-tokenizer", action="store_true")
    ap.add_argument("-q", "--quiet", action="store_true")
    a = ap.parse_args(argv)
    method = {"int4": QuantMethod.INT4_ASYM, "int8": QuantMethod.INT8_SYM, "fp16": QuantMethod.NONE}[a.quant]
    t0 = time.time()
    last = [0.0]

    def progress(name, i, n):
        if not a.quiet and time.time() - last[0] > 0.5:
            last[0] = time.time()
            print(f"\r[{i}/{n}] {name[:60]:60s}", end="", file=sys.stderr, flush=True)

    try:
        convert_hf_to_zse(a.model_dir, a.output, progress, int(method), None, a.group_size, a.arch, a.no_tokenizer,
                          quiet=a.quiet)
    except (FileNotFoundError, ValueError) as exc:
        print(f"\nerror: {exc}", file=sys.stderr)
        return 1
    if not a.quiet:
        print(f"\ndone in {time.time() - t0:.1f}s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
