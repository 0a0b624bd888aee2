"""HuggingFace safetensors -> ``.zse`` conversion.

Pipeline of zse-engine/zse_engine/format/convert.py:148-331: read ``config.json``, pick the architecture
adapter, index every ``*.safetensors`` shard (8-byte little-endian header length + JSON header), embed the
tokenizer, then convert tensor by tensor in name order, checkpointing after each tensor into
``<out>.progress`` (written atomically) so that an interrupted run resumes by truncating the output to the
recorded position.  Tensor bytes go from a memory map of the shard straight through the vectorised (or
native) quantiser; INT4 payloads are written row-major.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from .arch import detect_architecture, get_adapter
from .config import ModelConfig
from .header import SectionEntry
from .quantize import quantize_int4_arrays, quantize_int8_arrays
from .spec import QuantMethod, SectionType
from .tokenizer import BPETokenizer
from .weight_index import WeightEntry, WeightIndex
from .writer import ZSEWriter

_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64,
              "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}


def read_safetensors_metadata(path: str) -> Tuple[dict, int]:
    """Returns ``(header dict, absolute offset of the data area)``."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n).decode("utf-8"))
    return meta, 8 + n


def read_safetensors_tensor_raw(path: str, info: dict, data_base: int):
    a, b = info["data_offsets"]
    with open(path, "rb") as f:
        f.seek(data_base + a)
        return f.read(b - a), info["dtype"], tuple(info["shape"])


def _to_f32(raw, dtype: str) -> np.ndarray:
    np_dt = _ST_DTYPES.get(dtype)
    if np_dt is None:
        raise ValueError(f"unsupported safetensors dtype {dtype}")
    arr = np.frombuffer(raw, dtype=np_dt)
    if dtype == "BF16":
        return (arr.astype(np.uint32) << 16).view(np.float32)
    return arr.astype(np.float32)


def read_safetensors_tensor(path: str, info: dict, data_base: int):
    raw, dtype, shape = read_safetensors_tensor_raw(path, info, data_base)
    return _to_f32(raw, dtype), shape


def find_safetensor_files(model_dir: str) -> List[str]:
    files = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {model_dir}")
    return files


def build_tensor_map(files: List[str]) -> Dict[str, Tuple[str, dict, int]]:
    out = {}
    for path in files:
        meta, base = read_safetensors_metadata(path)
        for name, info in meta.items():
            if name != "__metadata__":
                out[name] = (path, info, base)
    return out


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], bf16: bool = False) -> None:
    """Minimal safetensors writer (tests and synthetic checkpoints).  ``bf16=True`` stores float arrays
    as truncated bfloat16."""
    header, blobs, at = {}, [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        if bf16 and arr.dtype.kind == "f":
            raw, tag = (arr.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes(), "BF16"
        else:
            tag = {v: k for k, v in _ST_DTYPES.items() if k != "BF16"}[arr.dtype.type]
            raw = arr.tobytes()
        header[name] = {"dtype": tag, "shape": list(arr.shape), "data_offsets": [at, at + len(raw)]}
        at += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class _Shards:
    """Keeps one memory map per shard so tensors are sliced, not read()."""

    def __init__(self):
        self._maps = {}

    def view(self, path: str, info: dict, base: int) -> memoryview:
        mm = self._maps.get(path)
        if mm is None:
            with open(path, "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = mm
        a, b = info["data_offsets"]
        return memoryview(mm)[base + a: base + b]

    def close(self):
        for mm in self._maps.values():
            try:
                mm.close()
            except BufferError:
                pass
        self._maps.clear()


def _save_progress(path: str, model_dir: str, quant_method: int, group_size: int, done: int, w: ZSEWriter) -> None:
    state = {"model_dir": os.path.abspath(model_dir), "quant_method": int(quant_method), "group_size": group_size,
             "completed_tensors": done, "file_position": w._fp.tell(), "weight_data_start": w._weight_data_start,
             "weight_offset": w._current_weight_offset,
             "weight_entries": [e.to_dict() for e in w._weight_index],
             "sections": [{"type": int(s.type), "offset": s.offset, "size": s.size, "crc32": s.crc32}
                          for s in w._sections]}
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(state, f)
    os.replace(tmp, path)


def _resume_writer(output_path: str, state: dict, cfg: ModelConfig, tok: Optional[bytes]) -> ZSEWriter:
    w = ZSEWriter.__new__(ZSEWriter)
    w._path = output_path
    w._fp = open(output_path, "r+b")
    w._fp.truncate(state["file_position"])
    w._fp.seek(state["file_position"])
    w._config, w._tokenizer_bytes = cfg, tok
    w._weight_index = WeightIndex()
    for d in state.get("weight_entries", []):
        w._weight_index.add(WeightEntry.from_dict(d))
    w._sections = [SectionEntry(SectionType(s["type"]), s["offset"], s["size"], s["crc32"])
                   for s in state.get("sections", [])]
    w._finalized = False
    w._has_tokenizer = tok is not None
    w._num_sections = 3 + int(tok is not None)
    w._weight_data_start = state["weight_data_start"]
    w._current_weight_offset = state["weight_offset"]
    return w


def _quantize(values: np.ndarray, method: int, group_size: int, native) -> tuple:
    if native is not None:
        return native(values, method, group_size)
    if method == QuantMethod.INT8_SYM:
        return quantize_int8_arrays(values, group_size)
    return quantize_int4_arrays(values, group_size)


def convert_hf_to_zse(model_dir: str, output_path: str,
                      progress_callback: Optional[Callable[[str, int, int], None]] = None,
                      quant_method: Optional[int] = None, quant_bits: Optional[int] = None,
                      group_size: Optional[int] = None, arch_override: Optional[str] = None,
                      skip_tokenizer: bool = False, quiet: bool = True,
                      stop_after: Optional[int] = None) -> None:
    """``quant_method``: ``QuantMethod.INT4_ASYM`` (default), ``INT8_SYM`` or ``NONE`` (fp16).
    ``stop_after=n`` interrupts after n tensors (used to test the resume path)."""
    quant_method = int(QuantMethod.INT4_ASYM if quant_method is None else quant_method)
    group_size = 128 if group_size is None else int(group_size)
    quant_bits = {QuantMethod.INT4_ASYM: 4, QuantMethod.INT8_SYM: 8, QuantMethod.NONE: 16}.get(
        QuantMethod(quant_method), 4) if quant_bits is None else quant_bits
    with open(os.path.join(model_dir, "config.json"), "r") as f:
        hf = json.load(f)
    adapter = get_adapter(arch_override or detect_architecture(hf))
    cfg = adapter.config_from_hf(hf)
    cfg.quant.method, cfg.quant.bits, cfg.quant.group_size = quant_method, quant_bits, group_size
    for warning in adapter.validate_config(cfg):
        if not quiet:
            print(f"WARNING: {warning}")
    tensor_map = build_tensor_map(find_safetensor_files(model_dir))
    tok_bytes = None
    if not skip_tokenizer and os.path.exists(os.path.join(model_dir, "tokenizer.json")):
        tok_bytes = BPETokenizer.from_hf_dir(model_dir).serialize()

    progress_path, resume_from, writer = output_path + ".progress", 0, None
    if os.path.exists(progress_path) and os.path.exists(output_path):
        try:
            with open(progress_path, "r") as f:
                st = json.load(f)
            if (st.get("model_dir") == os.path.abspath(model_dir) and st.get("quant_method") == quant_method
                    and st.get("group_size") == group_size and st.get("completed_tensors", 0) > 0):
                writer = _resume_writer(output_path, st, cfg, tok_bytes)
                resume_from = st["completed_tensors"]
        except (ValueError, KeyError, OSError):
            writer, resume_from = None, 0
    if writer is None:
        writer = ZSEWriter(output_path)
        writer.set_config(cfg)
        if tok_bytes:
            writer.set_tokenizer(tok_bytes)
        writer.begin_weights()
    else:
        writer.set_config(cfg)

    try:
        from ..ops import host_native
        native = host_native.quantize if host_native.available() else None
    except Exception:
        native = None

    names = adapter.tensor_load_order(list(tensor_map))
    shards = _Shards()
    try:
        for i, hf_name in enumerate(names):
            if i < resume_from:
                continue
            if stop_after is not None and i >= stop_after:
                raise KeyboardInterrupt("conversion interrupted on request")
            name = adapter.map_tensor_name(hf_name)
            if progress_callback:
                progress_callback(name, i + 1, len(names))
            path, info, base = tensor_map[hf_name]
            shape = tuple(info["shape"])
            values = _to_f32(shards.view(path, info, base), info["dtype"])
            floating = info["dtype"] in ("F64", "F32", "F16", "BF16")
            if floating and quant_method != QuantMethod.NONE and adapter.should_quantize(name):
                res = _quantize(values, quant_method, group_size, native)
                if quant_method == QuantMethod.INT8_SYM:
                    writer.add_weight_raw_int8(name, shape, res[0], res[1], group_size)
                else:
                    writer.add_weight_raw(name, shape, res[0], res[1], res[2], group_size)
            else:
                writer.add_weight_raw_fp16(name, shape, values.astype(np.float16))
            del values
            _save_progress(progress_path, model_dir, quant_method, group_size, i + 1, writer)
        writer.finalize()
        if os.path.exists(progress_path):
            os.unlink(progress_path)
    except BaseException:
        writer.abort()
        raise
    finally:
        shards.close()
    if not quiet:
        print(f"wrote {output_path} ({os.path.getsize(output_path):,} bytes): {cfg.arch}, {cfg.num_layers} layers, "
              f"hidden {cfg.hidden_size}, {len(names)} tensors")
