"""Weight files: writer and loader for the safetensors layout that sb_model_load_file reads.

The reference keeps its model as a bundle directory (src/models.rs:5-8: `parakeet-v2/encoder.mlmodelc`,
`decoder.mlmodelc`, `joint-decision.mlmodelc`, `vocab.txt`); here the three networks are one weight file
`parakeet-v2/model.safetensors` beside the same `parakeet-v2/vocab.txt`.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct

import numpy as np

from . import _lib
from ._lib import ScriptrsError, check

MODEL_FILE = os.path.join("parakeet-v2", "model.safetensors")
VOCAB_FILE = os.path.join("parakeet-v2", "vocab.txt")
VAD_FILE = os.path.join("vad", "silero-vad.safetensors")  # stands where the reference has vad/silero-vad.mlmodelc (src/models.rs:10)


def _to_bf16_bytes(a: np.ndarray) -> bytes:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16  # round to nearest even
    return rounded.astype("<u2").tobytes()


def save_safetensors(path: str, tensors: dict, dtype: str = "F32", metadata: dict | None = None) -> None:
    """Writes named arrays as a safetensors file.  dtype: "F32", "F16" or "BF16" for every tensor."""
    header, blobs, pos = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, a in tensors.items():
        a = np.asarray(a)
        if dtype == "F32":
            b = np.ascontiguousarray(a, "<f4").tobytes()
        elif dtype == "F16":
            b = np.ascontiguousarray(a, "<f2").tobytes()
        elif dtype == "BF16":
            b = _to_bf16_bytes(a)
        else:
            raise ValueError(dtype)
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [pos, pos + len(b)]}
        blobs.append(b)
        pos += len(b)
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * (-len(h) % 8)  # the data section starts 8-byte aligned
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def list_weights_file(path: str):
    """[(name, dtype, shape)] of a weight file; host only."""
    L = _lib.lib()
    n = L.sb_weights_file_list(os.fsencode(path), None, 0)
    if n < 0:
        check(int(-n))
    buf = C.create_string_buffer(int(n) + 1)
    L.sb_weights_file_list(os.fsencode(path), buf, len(buf))
    out = []
    for line in buf.value.decode("utf-8").splitlines():
        name, dt, shp = line.rsplit(" ", 2)
        out.append((name, dt, () if shp == "scalar" else tuple(int(x) for x in shp.split("x"))))
    return out


def load_model_file(ctx, path: str, encoder_layers: int = -1, scale_input: bool = False, has_encoder: bool = True,
                    has_decoder: bool = True, fp8_weights: bool = False, prefix: str | None = None) -> None:
    """sb_model_load_file: uploads the tensors of a weight file (encoder_layers < 0: as many blocks as it holds)."""
    desc = _lib.ModelDescC(encoder_layers, int(scale_input), int(has_encoder), int(has_decoder), int(fp8_weights))
    check(_lib.lib().sb_model_load_file(ctx.handle, C.byref(desc), os.fsencode(path),
                                        prefix.encode() if prefix else None))


def validate_bundle(models_dir: str):
    """ModelBundle::from_dir + validate_base (src/models.rs:36-66): the paths of the weight file and the
    vocabulary under `models_dir`; a missing one raises MissingModelAsset with its path."""
    model, vocab = os.path.join(models_dir, MODEL_FILE), os.path.join(models_dir, VOCAB_FILE)
    for p in (model, vocab):
        if not os.path.exists(p):
            raise ScriptrsError(3, f"missing model asset: {p}")
    return model, vocab


def vad_path(models_dir: str) -> str:
    """ModelBundle::vad_dir (src/models.rs:96-99)."""
    return os.path.join(models_dir, VAD_FILE)


def validate_with_vad(models_dir: str):
    """ModelBundle::validate_with_vad (src/models.rs:68-78): the base bundle plus the VAD network file."""
    model, vocab = validate_bundle(models_dir)
    vad = vad_path(models_dir)
    if not os.path.exists(vad):
        raise ScriptrsError(3, f"missing model asset: {vad}")
    return model, vocab, vad
