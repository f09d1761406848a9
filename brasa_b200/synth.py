"""Synthetic random-init Qwen3 models in the `.brasa` container, generated and quantised on the GPU.

The benchmark configurations call for weights drawn N(0, 0.02) from a seed with norm vectors at 1 and
the `.brasa` quantisation (linear layers q4_0, embedding table q6_0, norms f32). This module is the
device-side converter for that case: values come from brasa_k_randn, blocks from brasa_k_quantize
(bit-identical to crates/quant/src/convert.rs:70-151), and the container is laid out exactly like
tools/convert_brasa.py:92-170 writes it (sorted names, 16 KiB pages, per-tensor sha256).
"""

from __future__ import annotations

import hashlib
import json
import pathlib
import struct

import numpy as np

from . import Context, Kernels, WeightType

PAGE = 16384
QWEN3_4B = {"model_type": "qwen3", "tie_word_embeddings": True, "num_hidden_layers": 36, "hidden_size": 2560,
            "intermediate_size": 9728, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
            "rms_norm_eps": 1e-6, "rope_theta": 1e6, "vocab_size": 151936, "max_position_embeddings": 40960}
QWEN3_32B = {"model_type": "qwen3", "tie_word_embeddings": False, "num_hidden_layers": 64, "hidden_size": 5120,
             "intermediate_size": 25600, "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128,
             "rms_norm_eps": 1e-6, "rope_theta": 1e6, "vocab_size": 151936, "max_position_embeddings": 40960}
_BLOCK_BYTES = {"q4_0": 18, "q6_0": 26, "q8_0": 34}
_QT = {"q4_0": WeightType.Q4_0, "q6_0": WeightType.Q6_0, "q8_0": WeightType.Q8_0}


def tensor_shapes(cfg: dict) -> dict[str, list[int]]:
    H, F, V, D = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["head_dim"]
    qd, kvd = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    t = {"model.embed_tokens.weight": [V, H], "model.norm.weight": [H]}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t.update({p + "input_layernorm.weight": [H], p + "post_attention_layernorm.weight": [H],
                  p + "self_attn.q_norm.weight": [D], p + "self_attn.k_norm.weight": [D],
                  p + "self_attn.q_proj.weight": [qd, H], p + "self_attn.k_proj.weight": [kvd, H],
                  p + "self_attn.v_proj.weight": [kvd, H], p + "self_attn.o_proj.weight": [H, qd],
                  p + "mlp.gate_proj.weight": [F, H], p + "mlp.up_proj.weight": [F, H], p + "mlp.down_proj.weight": [H, F]})
    if not cfg.get("tie_word_embeddings", True):
        t["lm_head.weight"] = [cfg.get("tp_head_rows", V), H]  # a tensor-parallel shard holds its rows of the vocabulary
    return t


def dtype_for(name: str, ndim: int) -> str:
    if ndim == 1:
        return "f32"
    return "q6_0" if name == "model.embed_tokens.weight" else "q4_0"


def _nbytes(dtype: str, shape) -> int:
    n = int(np.prod(shape))
    return 4 * n if dtype == "f32" else n // 32 * _BLOCK_BYTES[dtype]


def _header(meta: dict) -> bytes:
    js = json.dumps(meta, ensure_ascii=False, separators=(",", ":")).encode()
    return b"BRSA" + struct.pack("<IQ", 1, len(js)) + js


def write_synthetic_model(ctx: Context, path, cfg: dict, seed: int = 0, std: float = 0.02) -> dict:
    """Writes `path` (model.brasa) with seeded N(0, std) matrices and norm vectors of ones."""
    path = pathlib.Path(path)
    K = Kernels(ctx)
    shapes = tensor_shapes(cfg)
    tensors = []
    for name in sorted(shapes):
        dt = dtype_for(name, len(shapes[name]))
        tensors.append({"name": name, "dtype": dt, "shape": shapes[name], "nbytes": _nbytes(dt, shapes[name]), "offset": 0,
                        "sha256": "0" * 64})
    meta = {"format": "brasa", "version": 1, "converter": "brasa_b200.synth",
            "model": {"family": "qwen3", "source_repo": "synthetic", "source_commit": f"seed-{seed}", "config": cfg},
            "quant": {"block": 32, "scheme": "q4_0 linears, q6_0 embeddings/lm_head, f32 norms"},
            "page": PAGE, "tensors": tensors, "data_sha256": "0" * 64}
    data_start = PAGE
    while True:
        off = data_start
        for t in tensors:
            t["offset"] = off
            off = (off + t["nbytes"] + PAGE - 1) // PAGE * PAGE
        if len(_header(meta)) <= data_start:
            break
        data_start += PAGE
    total, provisional = off, len(_header(meta))
    biggest = max(int(np.prod(t["shape"])) for t in tensors if t["dtype"] != "f32")
    f32buf = ctx.buffer(biggest * 4)
    qbuf = ctx.buffer(max(t["nbytes"] for t in tensors))
    stream_off = 0
    # a tensor-parallel shard (brasa_b200.tp.shard_config): the replicated embedding table comes from the shared seed,
    # everything else from a seed of the rank's own
    own_seed = seed + 1000003 * (cfg["tp_rank"] + 1) if "tp_rank" in cfg else seed
    with open(path, "wb") as f:
        f.truncate(total)
        for t in tensors:
            n = int(np.prod(t["shape"]))
            if t["dtype"] == "f32":
                data = np.ones(n, dtype="<f4").tobytes()
            else:
                cmd = ctx.command()
                shared = "tp_rank" in cfg and t["name"] == "model.embed_tokens.weight"
                K.randn(cmd, f32buf, n, seed if shared else own_seed, 0 if shared else stream_off, std)
                K.quantize(cmd, _QT[t["dtype"]], f32buf, qbuf, n)
                cmd.wait()
                data = qbuf.download(np.uint8, t["nbytes"]).tobytes()
                stream_off += 0 if shared else (n + 1) // 2
            t["sha256"] = hashlib.sha256(data).hexdigest()
            f.seek(t["offset"])
            f.write(data)
        meta["data_sha256"] = hashlib.sha256("".join(t["sha256"] for t in tensors).encode()).hexdigest()
        header = _header(meta)
        assert len(header) == provisional
        f.seek(0)
        f.write(header)
    f32buf.free()
    qbuf.free()
    return meta


def weight_bytes_per_token(cfg: dict) -> int:
    """Bytes of weights one decode token reads: every quantised matrix once, norm vectors, one embedding row."""
    total = 0
    for name, shape in tensor_shapes(cfg).items():
        dt = dtype_for(name, len(shape))
        if name == "model.embed_tokens.weight" and not cfg.get("tie_word_embeddings", True):
            continue
        total += _nbytes(dt, shape)
    total += cfg["hidden_size"] // 32 * 26  # the embedding row of the input token
    return total


def kv_bytes_per_position(cfg: dict, kv: str = "f16") -> int:
    rows = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"]
    return rows * {"f32": 512, "f16": 256, "q8_0": 136}[kv]
