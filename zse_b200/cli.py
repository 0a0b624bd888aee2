"""``zse`` command line: ``serve | convert | info | version | warm | keys | synth | bench-kernels``.

Same verbs and flags as zse-engine/zse_engine/cli.py:213-285 (``serve [model] --port --host --admin-key --db-path
--model-name -q --tp N``; ``convert <hf_dir> <out.zse> --quant int4|int8|fp16 --group-size --arch --no-tokenizer -q``;
``info``; ``version``; ``warm <model>``; ``keys create|list|revoke``), plus the engine knobs the reference cannot reach
from its CLI (chunk size, speculative depth, graphs, comm back end) and two helpers: ``synth`` writes a random model of
a named shape, ``bench-kernels`` runs the per-kernel microbenchmarks.
"""
from __future__ import annotations

import argparse
import asyncio
import os
import secrets
import signal
import sys
import time


def _cmd_serve(a) -> int:
    if a.model and not os.path.exists(a.model):
        print(f"error: model file not found: {a.model}", file=sys.stderr)
        return 1
    if not a.admin_key:
        a.admin_key = f"sk-zse-admin-{secrets.token_hex(16)}"
        if not a.quiet:
            print(f"  admin key: {a.admin_key}\n  (shown once - save it)\n")
    from .config import EngineConfig
    from .server.app import ZSEServer
    cfg = EngineConfig.from_env(tp_size=a.tp_size, max_seq_len=a.max_seq_len or None,
                                max_batch_seqs=a.max_batch_seqs, prefill_chunk_size=a.prefill_chunk_size,
                                speculative_k=a.speculative_k, speculative_mode=a.speculative_mode,
                                use_cuda_graphs=not a.no_graphs, comm_backend=a.comm, quiet=a.quiet,
                                device="cpu" if a.cpu else None)
    server = ZSEServer(a.model, a.host, a.port, a.admin_key, a.db_path, a.model_name, a.quiet, a.tp_size,
                       engine_config=cfg, require_auth=a.require_auth)
    loop = asyncio.new_event_loop()

    def shutdown(*_):
        loop.call_soon_threadsafe(loop.stop)

    rc = [0]

    def watch_engine():
        # a device fault ends the CUDA context of this process for good: leave with a non-zero code, so that whatever
        # supervises the server (systemd, a container runtime) starts a fresh one, instead of answering 503 for ever
        fatal = getattr(server.engine, "fatal_error", None) if server.engine is not None else None
        if fatal:
            print(f"[zse] device fault, shutting down: {fatal}", file=sys.stderr)
            rc[0] = 3
            loop.stop()
            return
        loop.call_later(1.0, watch_engine)

    signal.signal(signal.SIGINT, shutdown)
    signal.signal(signal.SIGTERM, shutdown)
    try:
        loop.run_until_complete(server.start())
        loop.call_later(1.0, watch_engine)
        loop.run_forever()
    finally:
        server.close()
        loop.close()
    return rc[0]


def _cmd_convert(a) -> int:
    from .format.__main__ import main as convert_main
    argv = [a.model_dir, a.output, "--quant", a.quant, "--group-size", str(a.group_size)]
    if a.arch:
        argv += ["--arch", a.arch]
    if a.no_tokenizer:
        argv.append("--no-tokenizer")
    if a.quiet:
        argv.append("--quiet")
    return convert_main(argv)


def _cmd_convert_lora(a) -> int:
    from .format.lora_convert import convert_peft_to_zse_lora
    try:
        info = convert_peft_to_zse_lora(a.adapter_dir, a.output, a.modules.split(",") if a.modules else None)
    except (OSError, ValueError, KeyError) as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    print(f"wrote {a.output}: rank {info['rank']}, alpha {info['alpha']:g}, {info['num_layers']} layers, targets "
          f"{', '.join(info['targets'])}" + (f"; {len(info['skipped'])} tensors skipped" if info["skipped"] else ""))
    return 0


def _cmd_info(a) -> int:
    from .runtime.device import describe_devices
    print("zse_b200 device info")
    print("=" * 50)
    for line in describe_devices():
        print(line)
    if a.model:
        from .format.loader import ZSELoader
        with ZSELoader(a.model) as l:
            print()
            print(l.summary())
    if getattr(a, "env", False):
        from .utils import env
        print()
        print("environment switches")
        for line in env.describe():
            print(line)
    return 0


def _cmd_version(a) -> int:
    import torch

    from . import __version__
    print(f"zse_b200 {__version__}")
    print(f"  python  {sys.version.split()[0]} on {sys.platform}")
    print(f"  torch   {torch.__version__} (CUDA {torch.version.cuda})")
    try:
        from .ops import native
        print(f"  native  {native.build_info()}")
    except Exception as exc:
        print(f"  native  not built ({exc})")
    return 0


def _cmd_warm(a) -> int:
    """Reads the model file once so its pages sit in the OS page cache before ``serve``
    (zse-engine/zse_engine/cli.py:132-164)."""
    if not os.path.exists(a.model):
        print(f"error: model file not found: {a.model}", file=sys.stderr)
        return 1
    size, done, t0 = os.path.getsize(a.model), 0, time.time()
    fd = os.open(a.model, os.O_RDONLY)
    try:
        if hasattr(os, "posix_fadvise"):
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_WILLNEED)
        buf = bytearray(16 << 20)
        while True:
            n = os.readv(fd, [buf])
            if n <= 0:
                break
            done += n
    finally:
        os.close(fd)
    dt = max(time.time() - t0, 1e-6)
    print(f"warmed {done / 2**30:.2f} GiB of {size / 2**30:.2f} GiB in {dt:.1f}s ({done / 2**30 / dt:.2f} GiB/s)")
    return 0


def _cmd_keys(a) -> int:
    from .server.database import ServerDatabase
    db = ServerDatabase(getattr(a, "db_path_after", None) or a.db_path)
    if a.keys_cmd == "revoke":
        a.id = a.id if a.id is not None else a.id_flag
        if a.id is None:
            print("revoke needs a key id or prefix")
            return 2
        a.id = str(a.id)
    if a.keys_cmd == "create":
        key, info = db.create_key(a.name, a.rpm, a.tpm, a.models)
        print(f"created key {info.id} ({info.name or 'unnamed'}):\n  {key}\n  (shown once - save it)")
    elif a.keys_cmd == "list":
        for k in db.list_keys():
            print(f"{k.id:4d}  {k.key_prefix}...  {'active ' if k.is_active else 'revoked'}  rpm={k.rate_limit_rpm} "
                  f"tpm={k.rate_limit_tpm} models={k.allowed_models} requests={k.total_requests} "
                  f"tokens={k.total_tokens}  {k.name}")
    elif a.keys_cmd == "revoke":
        ok = db.revoke_key(int(a.id)) if a.id.isdigit() else db.revoke_key_by_prefix(a.id)
        print("revoked" if ok else "no such active key")
        return 0 if ok else 1
    return 0


def _cmd_synth(a) -> int:
    from .format import synth
    cfg = synth.shape_config(a.shape, quant=a.quant)
    t0 = time.time()
    synth.write_random_model(a.output, cfg, seed=a.seed, fast=a.fast)
    print(f"wrote {a.output} ({os.path.getsize(a.output) / 2**30:.2f} GiB) in {time.time() - t0:.1f}s")
    return 0


def _cmd_bench_kernels(a) -> int:
    from .runtime import microbench
    sys.argv = ["microbench", "--shape", a.shape, "--tokens", str(a.tokens), "--tp", str(a.tp)]
    microbench.main()
    return 0


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="zse", description="Blackwell-native LLM inference engine for .zse models")
    sub = p.add_subparsers(dest="cmd")
    s = sub.add_parser("serve", help="serve a .zse model over the OpenAI-compatible HTTP API")
    s.add_argument("model", nargs="?", default=None)
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--host", default="0.0.0.0")
    s.add_argument("--admin-key", default=None)
    s.add_argument("--db-path", default="~/.zse/server.db")
    s.add_argument("--model-name", default="zse-model")
    s.add_argument("-q", "--quiet", action="store_true")
    s.add_argument("--tp", "--tensor-parallel", dest="tp_size", type=int, default=1, help="tensor-parallel GPUs")
    s.add_argument("--max-seq-len", type=int, default=0)
    s.add_argument("--max-batch-seqs", type=int, default=64)
    s.add_argument("--prefill-chunk-size", type=int, default=2048)
    s.add_argument("--speculative-k", type=int, default=0)
    s.add_argument("--speculative-mode", default="ngram", choices=["ngram", "self"])
    s.add_argument("--no-graphs", action="store_true")
    s.add_argument("--comm", default="fused", choices=["fused", "nccl", "nccl-sp"],
                   help="tensor-parallel collectives: fused in-kernel exchange, NCCL all-reduce, or NCCL with "
                        "sequence-parallel prefill (reduce-scatter / all-gather, residual split by rows)")
    s.add_argument("--require-auth", action="store_true")
    s.add_argument("--cpu", action="store_true", help="run on the CPU reference path")
    s.set_defaults(fn=_cmd_serve)
    c = sub.add_parser("convert", help="convert a HuggingFace directory to .zse")
    c.add_argument("model_dir")
    c.add_argument("output")
    c.add_argument("--quant", default="int4", choices=["int4", "int8", "fp16"])
    c.add_argument("--group-size", type=int, default=128)
    c.add_argument("--arch", default=None)
    c.add_argument("--no-tokenizer", action="store_true")
    c.add_argument("-q", "--quiet", action="store_true")
    c.set_defaults(fn=_cmd_convert)
    cl = sub.add_parser("convert-lora", help="convert a HuggingFace PEFT LoRA adapter directory to .zse-lora")
    cl.add_argument("adapter_dir")
    cl.add_argument("output")
    cl.add_argument("--modules", default="", help="comma separated projections to keep (default: all present)")
    cl.set_defaults(fn=_cmd_convert_lora)
    i = sub.add_parser("info", help="GPUs and, optionally, a model file summary")
    i.add_argument("model", nargs="?", default=None)
    i.add_argument("--env", action="store_true", help="also list the ZSE_* environment switches and their values")
    i.set_defaults(fn=_cmd_info)
    sub.add_parser("version").set_defaults(fn=_cmd_version)
    w = sub.add_parser("warm", help="pull a model file into the page cache")
    w.add_argument("model")
    w.set_defaults(fn=_cmd_warm)
    k = sub.add_parser("keys", help="manage API keys")
    k.add_argument("--db-path", default="~/.zse/server.db")
    ks = k.add_subparsers(dest="keys_cmd", required=True)
    # ``--db-path`` is accepted before or after the action (the reference's CLI takes it after)
    kc = ks.add_parser("create")
    kc.add_argument("--name", default="")
    kc.add_argument("--rpm", "--rate-limit-rpm", dest="rpm", type=int, default=60)
    kc.add_argument("--tpm", "--rate-limit-tpm", dest="tpm", type=int, default=100000)
    kc.add_argument("--models", default="*")
    kl = ks.add_parser("list")
    kr = ks.add_parser("revoke")
    kr.add_argument("id", nargs="?", default=None, help="key id or key prefix")
    kr.add_argument("--id", dest="id_flag", default=None, help="key id (the reference's spelling)")
    for sp in (kc, kl, kr):
        sp.add_argument("--db-path", dest="db_path_after", default=None)
    k.set_defaults(fn=_cmd_keys)
    y = sub.add_parser("synth", help="write a random-weight model of a named shape")
    y.add_argument("shape")
    y.add_argument("output")
    y.add_argument("--quant", default="int4", choices=["int4", "int8", "fp16"])
    y.add_argument("--seed", type=int, default=0)
    y.add_argument("--fast", action="store_true")
    y.set_defaults(fn=_cmd_synth)
    b = sub.add_parser("bench-kernels", help="per-kernel microbenchmarks with roofline fractions")
    b.add_argument("--shape", default="qwen2.5-14b")
    b.add_argument("--tokens", type=int, default=64)
    b.add_argument("--tp", type=int, default=1)
    b.set_defaults(fn=_cmd_bench_kernels)
    return p


def main(argv=None) -> int:
    p = build_parser()
    a = p.parse_args(argv)
    if not getattr(a, "fn", None):
        p.print_help()
        return 0
    return int(a.fn(a) or 0)


if __name__ == "__main__":
    sys.exit(main())
