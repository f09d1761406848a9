"""Tensor parallelism inside one node: shard files, the peer-memory exchange and its set-up across processes.

The reference runs one device. A model split Megatron-style keeps q/k/v and gate/up whole in their input and split
by output rows (attention heads, FFN rows), o_proj and down_proj split by input columns, an untied lm_head split by
vocabulary rows; every rank then holds an ordinary `.brasa` file whose config names its share, and the two residual
adds of a layer (crates/models/src/qwen3.rs:763-831) become sums over ranks.
"""

from __future__ import annotations

import ctypes as C
import hashlib
import json
import pathlib
import struct

import numpy as np

from . import Context, lib
from .synth import PAGE, _BLOCK_BYTES, _header, _nbytes

HANDLE_BYTES = 64
FFN_UNIT = 256  # columns of down_proj move in units the tiled weight layout accepts


def _share(total: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of `total` units for `rank`: the first total % world ranks hold one unit more."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_ranges(cfg: dict, rank: int, world: int) -> dict:
    """Which heads, KV heads, FFN rows and vocabulary rows rank `rank` of `world` holds."""
    hq, hkv, F, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    if hkv % world or F % FFN_UNIT or F // FFN_UNIT < world:
        raise ValueError(f"cannot split {hkv} KV heads / {F} FFN rows over {world} ranks")
    if cfg.get("tie_word_embeddings", True) and world > 1:
        raise ValueError("a tied lm_head is not sharded: tensor parallelism needs an untied lm_head")
    kv0, kv1 = _share(hkv, rank, world)
    g = hq // hkv
    f0, f1 = _share(F // FFN_UNIT, rank, world)
    v0, v1 = _share(V, rank, world)
    return {"heads": (kv0 * g, kv1 * g), "kv_heads": (kv0, kv1), "ffn": (f0 * FFN_UNIT, f1 * FFN_UNIT), "vocab": (v0, v1)}


def shard_config(cfg: dict, rank: int, world: int) -> dict:
    r = shard_ranges(cfg, rank, world)
    out = dict(cfg)
    out.update({"num_attention_heads": r["heads"][1] - r["heads"][0], "num_key_value_heads": r["kv_heads"][1] - r["kv_heads"][0],
                "intermediate_size": r["ffn"][1] - r["ffn"][0], "tp_rank": rank, "tp_world": world,
                "tp_vocab_offset": r["vocab"][0], "tp_head_rows": r["vocab"][1] - r["vocab"][0]})
    return out


def _rows(data: np.ndarray, dtype: str, shape, r0: int, r1: int) -> np.ndarray:
    if dtype == "f32":
        return data.reshape(shape)[r0:r1].reshape(-1)
    per_row = shape[1] // 32 * _BLOCK_BYTES[dtype]
    return data[r0 * per_row:r1 * per_row]


def _cols(data: np.ndarray, dtype: str, shape, c0: int, c1: int) -> np.ndarray:
    bb = _BLOCK_BYTES[dtype]
    return np.ascontiguousarray(data.reshape(shape[0], shape[1] // 32, bb)[:, c0 // 32:c1 // 32, :]).reshape(-1)


def read_container(path) -> tuple[dict, np.memmap]:
    """Header (the JSON of a `.brasa` file) and a byte view of the whole file."""
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    if bytes(raw[:4]) != b"BRSA":
        raise ValueError(f"{path}: not a .brasa file")
    _, n = struct.unpack("<IQ", bytes(raw[4:16]))
    return json.loads(bytes(raw[16:16 + n]).decode()), raw


def write_container(path, meta: dict, blobs: dict[str, np.ndarray]) -> None:
    """Writes a `.brasa` file (tools/convert_brasa.py:92-170 layout: sorted names, 16 KiB pages, per-tensor sha256)."""
    tensors = meta["tensors"]
    data_start = PAGE
    while True:
        off = data_start
        for t in tensors:
            t["offset"] = off
            off = (off + t["nbytes"] + PAGE - 1) // PAGE * PAGE
        if len(_header(meta)) <= data_start:
            break
        data_start += PAGE
    with open(path, "wb") as f:
        f.truncate(off)
        for t in tensors:
            b = np.ascontiguousarray(blobs[t["name"]]).tobytes()
            assert len(b) == t["nbytes"], t["name"]
            t["sha256"] = hashlib.sha256(b).hexdigest()
            f.seek(t["offset"])
            f.write(b)
        meta["data_sha256"] = hashlib.sha256("".join(t["sha256"] for t in tensors).encode()).hexdigest()
        f.seek(0)
        f.write(_header(meta))


def split_model(full_path, out_paths) -> list[dict]:
    """Splits the model in `full_path` (untied lm_head) into len(out_paths) shard files; returns the shard configs."""
    meta, raw = read_container(full_path)
    cfg = meta["model"]["config"]
    world = len(out_paths)
    by_name = {t["name"]: t for t in meta["tensors"]}
    D = cfg["head_dim"]
    configs = []
    for rank, out in enumerate(out_paths):
        r = shard_ranges(cfg, rank, world)
        blobs, tensors = {}, []
        for name in sorted(by_name):
            t = by_name[name]
            data = raw[t["offset"]:t["offset"] + t["nbytes"]]
            dt, shape = t["dtype"], list(t["shape"])
            if dt == "f32":
                data = data.view("<f4")
            if name.endswith("q_proj.weight"):
                sel, shape = _rows(data, dt, shape, r["heads"][0] * D, r["heads"][1] * D), [(r["heads"][1] - r["heads"][0]) * D, shape[1]]
            elif name.endswith(("k_proj.weight", "v_proj.weight")):
                sel, shape = _rows(data, dt, shape, r["kv_heads"][0] * D, r["kv_heads"][1] * D), [(r["kv_heads"][1] - r["kv_heads"][0]) * D, shape[1]]
            elif name.endswith("o_proj.weight"):
                sel, shape = _cols(data, dt, shape, r["heads"][0] * D, r["heads"][1] * D), [shape[0], (r["heads"][1] - r["heads"][0]) * D]
            elif name.endswith(("gate_proj.weight", "up_proj.weight")):
                sel, shape = _rows(data, dt, shape, *r["ffn"]), [r["ffn"][1] - r["ffn"][0], shape[1]]
            elif name.endswith("down_proj.weight"):
                sel, shape = _cols(data, dt, shape, *r["ffn"]), [shape[0], r["ffn"][1] - r["ffn"][0]]
            elif name == "lm_head.weight":
                sel, shape = _rows(data, dt, shape, *r["vocab"]), [r["vocab"][1] - r["vocab"][0], shape[1]]
            else:  # norms and the embedding table are replicated
                sel = data
            sel = np.ascontiguousarray(sel).view(np.uint8).reshape(-1)
            blobs[name] = sel
            tensors.append({"name": name, "dtype": dt, "shape": shape, "nbytes": int(sel.size), "offset": 0, "sha256": "0" * 64})
            assert sel.size == _nbytes(dt, shape), name
        scfg = shard_config(cfg, rank, world)
        smeta = dict(meta)
        smeta["model"] = dict(meta["model"], config=scfg)
        smeta["tensors"] = tensors
        write_container(out, smeta, blobs)
        configs.append(scfg)
    return configs


class TensorParallel:
    """This rank's exchange buffer, connected to its peers' (brasa_tp). `gather` takes this rank's 64-byte handle and
    returns every rank's, by rank: the default uses torch.distributed's all_gather_object."""

    def __init__(self, ctx: Context, rank: int, world: int, max_elems: int, gather=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        self._h = C.c_void_p()
        ctx._check(lib().brasa_tp_create(ctx._h, C.c_uint32(rank), C.c_uint32(world), C.c_uint64(max_elems), C.byref(self._h)))
        if world > 1:
            mine = (C.c_uint8 * HANDLE_BYTES)()
            ctx._check(lib().brasa_tp_handle(self._h, mine))
            if gather is None:
                import torch.distributed as dist

                def gather(h):
                    out = [None] * world
                    dist.all_gather_object(out, h)
                    dist.barrier()
                    return out
            handles = gather(bytes(mine))
            flat = (C.c_uint8 * (HANDLE_BYTES * world)).from_buffer_copy(b"".join(handles))
            ctx._check(lib().brasa_tp_connect(self._h, flat))

    @staticmethod
    def same_process(ctxs, max_elems: int) -> list["TensorParallel"]:
        """One exchange per context of this process (several devices, or several ranks on one device in tests)."""
        tps = []
        for r, ctx in enumerate(ctxs):
            tp = TensorParallel.__new__(TensorParallel)
            tp.ctx, tp.rank, tp.world = ctx, r, len(ctxs)
            tp._h = C.c_void_p()
            ctx._check(lib().brasa_tp_create(ctx._h, C.c_uint32(r), C.c_uint32(len(ctxs)), C.c_uint64(max_elems), C.byref(tp._h)))
            tps.append(tp)
        arr = (C.c_void_p * len(tps))(*[t._h for t in tps])
        ctxs[0]._check(lib().brasa_tp_connect_same_process(arr, C.c_uint32(len(tps))))
        return tps

    def set_poll_limit(self, polls: int):
        """Re-reads of one exchange word before a receive gives up (the call then ends in BrasaError ETIMEOUT)."""
        self.ctx._check(lib().brasa_tp_set_poll_limit(self._h, C.c_uint32(polls)))

    def free(self):
        if self._h and self.ctx._h:
            lib().brasa_tp_free(self._h)
        self._h = C.c_void_p()
