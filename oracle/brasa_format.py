"""`.brasa` container for the oracle side: reader and writer.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Layout (tools/convert_brasa.py:92-170, crates/quant/src/brasa_file.rs:64-131): ``"BRSA"``, u32
version 1, u64 JSON length, compact JSON header, then each tensor at an absolute offset that is a
multiple of the 16 KiB page; tensors sorted by name; per-tensor sha256 and ``data_sha256`` = sha256
of the concatenated hex digests.
"""

from __future__ import annotations

import hashlib
import json
import pathlib
import struct

import numpy as np

import oracle

PAGE = 16384
MAGIC = b"BRSA"
VERSION = 1


def align(n: int) -> int:
    return (n + PAGE - 1) // PAGE * PAGE


def dtype_for(name: str, ndim: int) -> str:
    """tools/convert_brasa.py:33-38: norms f32, the embedding table q6_0, every other matrix q4_0."""
    if ndim == 1:
        return "f32"
    if name == "model.embed_tokens.weight":
        return "q6_0"
    return "q4_0"


def header_bytes(meta: dict) -> bytes:
    js = json.dumps(meta, ensure_ascii=False, separators=(",", ":")).encode()
    return MAGIC + struct.pack("<IQ", VERSION, len(js)) + js


class BrasaFile:
    def __init__(self, path):
        self.path = pathlib.Path(path)
        self.map = np.memmap(self.path, dtype=np.uint8, mode="r")
        if self.map.size < 16 or bytes(self.map[:4]) != MAGIC:
            raise ValueError("not a .brasa file")
        version, n = struct.unpack("<IQ", bytes(self.map[4:16]))
        if version != VERSION:
            raise ValueError(f"unsupported version {version}")
        self.meta = json.loads(bytes(self.map[16:16 + n]))
        self.tensors = {t["name"]: t for t in self.meta["tensors"]}

    def config(self) -> dict:
        return self.meta["model"]["config"]

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.asarray(self.map[t["offset"]:t["offset"] + t["nbytes"]])

    def get_f32(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        n = int(np.prod(t["shape"]))
        return oracle.dequantize(oracle.QTYPE[t["dtype"]], self.raw(name), n).reshape(t["shape"])

    def verify(self) -> None:
        hexes = []
        for t in self.meta["tensors"]:
            h = hashlib.sha256(self.raw(t["name"]).tobytes()).hexdigest()
            if h != t["sha256"]:
                raise ValueError(f"{t['name']}: sha256 mismatch")
            hexes.append(h)
        if hashlib.sha256("".join(hexes).encode()).hexdigest() != self.meta["data_sha256"]:
            raise ValueError("data_sha256 mismatch")


def write_brasa(path, config: dict, weights: dict[str, np.ndarray], dtypes: dict[str, str] | None = None,
                source_repo: str = "synthetic", source_commit: str = "0") -> dict:
    """Quantises f32 `weights` (HF tensor names) with the oracle quantisers and writes a `.brasa`."""
    names = sorted(weights)
    tensors, blobs = [], {}
    for name in names:
        w = np.ascontiguousarray(weights[name], dtype=np.float32)
        dt = (dtypes or {}).get(name) or dtype_for(name, w.ndim)
        data = w.astype("<f4").tobytes() if dt == "f32" else oracle.quantize(oracle.QTYPE[dt], w).tobytes()
        blobs[name] = data
        tensors.append({"name": name, "dtype": dt, "shape": list(w.shape), "nbytes": len(data),
                        "offset": 0, "sha256": hashlib.sha256(data).hexdigest()})
    meta = {
        "format": "brasa", "version": VERSION, "converter": "oracle/brasa_format.py",
        "model": {"family": "qwen3", "source_repo": source_repo, "source_commit": source_commit, "config": config},
        "quant": {"block": 32, "scheme": "q4_0 linears, q6_0 embeddings/lm_head, f32 norms"},
        "page": PAGE, "tensors": tensors,
        "data_sha256": hashlib.sha256("".join(t["sha256"] for t in tensors).encode()).hexdigest(),
    }
    data_start = PAGE
    while True:
        off = data_start
        for t in tensors:
            t["offset"] = off
            off = align(off + t["nbytes"])
        if len(header_bytes(meta)) <= data_start:
            break
        data_start += PAGE
    with open(path, "wb") as f:
        f.truncate(off)
        f.write(header_bytes(meta))
        for t in tensors:
            f.seek(t["offset"])
            f.write(blobs[t["name"]])
    return meta


def tiny_config(layers=2, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=512, max_pos=4096) -> dict:
    return {"model_type": "qwen3", "tie_word_embeddings": True, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
            "rms_norm_eps": 1e-6, "rope_theta": 1e6, "hidden_size": hidden, "intermediate_size": ffn,
            "vocab_size": vocab, "max_position_embeddings": max_pos}


def synth_weights(config: dict, seed: int, std: float = 0.02, norm_jitter: float = 0.0) -> dict[str, np.ndarray]:
    """Random-init weights ~ N(0, std); norm vectors 1 (+ optional jitter so they are exercised)."""
    rng = np.random.default_rng(seed)
    H, F, V = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    D = config["head_dim"]
    qd, kvd = config["num_attention_heads"] * D, config["num_key_value_heads"] * D

    def mat(r, c):
        return rng.standard_normal((r, c), dtype=np.float32) * np.float32(std)

    def norm(n):
        return (1.0 + norm_jitter * rng.standard_normal(n)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": norm(H)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_norm.weight"] = norm(D)
        w[p + "self_attn.k_norm.weight"] = norm(D)
        w[p + "self_attn.q_proj.weight"] = mat(qd, H)
        w[p + "self_attn.k_proj.weight"] = mat(kvd, H)
        w[p + "self_attn.v_proj.weight"] = mat(kvd, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, qd)
        w[p + "mlp.gate_proj.weight"] = mat(F, H)
        w[p + "mlp.up_proj.weight"] = mat(F, H)
        w[p + "mlp.down_proj.weight"] = mat(H, F)
    if not config.get("tie_word_embeddings", True):
        w["lm_head.weight"] = mat(V, H)
    return w
