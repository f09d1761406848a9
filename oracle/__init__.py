"""CPU oracle for the Qwen3 token loop: ctypes front end of ``brasa_oracle.c``.

TEST INFRASTRUCTURE ONLY. The product (``brasa_b200``) never imports this package; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``.

The C file restates the reference's CPU arithmetic (crates/quant/src/qtype.rs,
crates/quant/src/convert.rs, crates/kernels/src/reference.rs, crates/kernels/src/testutil.rs,
crates/runtime/src/sampler.rs, tools/qwen3_ref.py); its header says how it is pinned.
"""

from __future__ import annotations

import ctypes as C
import os
import pathlib
import subprocess

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libbrasa_oracle.so"

Q4_0, Q8_0, Q6_0, F32 = 0, 1, 2, 3
QTYPE = {"q4_0": Q4_0, "q8_0": Q8_0, "q6_0": Q6_0, "f32": F32}
QNAME = {v: k for k, v in QTYPE.items()}
KV_F32, KV_F16, KV_Q8 = 0, 1, 2
KVTYPE = {"f32": KV_F32, "f16": KV_F16, "q8_0": KV_Q8}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q6_0: 26}


def build(force: bool = False) -> pathlib.Path:
    """Compiles brasa_oracle.c with gcc (OpenMP) into oracle/_build/."""
    src = HERE / "brasa_oracle.c"
    if not force and LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= src.stat().st_mtime:
        return LIB_PATH
    LIB_PATH.parent.mkdir(exist_ok=True)
    tmp = LIB_PATH.with_suffix(f".{os.getpid()}.tmp.so")
    subprocess.check_call(
        ["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off",
         "-o", str(tmp), str(src), "-lm"]
    )
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        L = _lib
        L.bo_f16_to_f32.restype = C.c_float
        L.bo_f16_to_f32.argtypes = [C.c_uint16]
        L.bo_f32_to_f16.restype = C.c_uint16
        L.bo_f32_to_f16.argtypes = [C.c_float]
        L.bo_nbytes.restype = C.c_size_t
        L.bo_nbytes.argtypes = [C.c_int, C.c_size_t]
        L.bo_argmax.restype = C.c_uint32
        L.bo_sample.restype = C.c_uint32
        L.bo_pcg32_next_u32.restype = C.c_uint32
        L.bo_pcg32_next_f32.restype = C.c_float
        L.bo_rng_next_u64.restype = C.c_uint64
        L.bo_qwen3_forward.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        a = np.frombuffer(a, dtype=np.uint8)
    return np.ascontiguousarray(a, dtype=np.uint8)


# ---- f16 ---------------------------------------------------------------------------------------

def f16_to_f32(h: int) -> float:
    return float(lib().bo_f16_to_f32(int(h)))


def f32_to_f16(f: float) -> int:
    return int(lib().bo_f32_to_f16(C.c_float(f)))


def f32_to_f16_array(x) -> np.ndarray:
    """Bits (uint16) of RNE f32 -> f16, element-wise, through the C restatement."""
    x = _f32(x).ravel()
    out = np.empty(x.size, np.uint16)
    lib().bo_f32_to_f16_array(_p(x), C.c_size_t(x.size), _p(out))
    return out


# ---- block formats -----------------------------------------------------------------------------

def nbytes(q: int, n: int) -> int:
    return int(lib().bo_nbytes(q, n))


def dequantize(q: int, data, n: int) -> np.ndarray:
    data = _u8(data)
    assert data.size == nbytes(q, n), "inconsistent data size"
    out = np.empty(n, np.float32)
    lib().bo_dequantize(C.c_int(q), _p(data), C.c_size_t(n), _p(out))
    return out


def quantize(q: int, w) -> np.ndarray:
    w = _f32(w).ravel()
    assert w.size % 32 == 0
    out = np.empty(nbytes(q, w.size), np.uint8)
    fn = {Q4_0: lib().bo_quant_q4_0, Q6_0: lib().bo_quant_q6_0, Q8_0: lib().bo_quant_q8_0}[q]
    fn(_p(w), C.c_size_t(w.size), _p(out))
    return out


def quantize_kv_q8(x) -> np.ndarray:
    x = _f32(x).ravel()
    assert x.size % 128 == 0
    out = np.empty(x.size // 128 * 136, np.uint8)
    lib().bo_quantize_kv_q8(_p(x), C.c_size_t(x.size), _p(out))
    return out


def dequantize_kv_q8(data) -> np.ndarray:
    data = _u8(data)
    assert data.size % 136 == 0
    n = data.size // 136 * 128
    out = np.empty(n, np.float32)
    lib().bo_dequantize_kv_q8(_p(data), C.c_size_t(n), _p(out))
    return out


def round_kv(kv: int, x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().bo_round_kv(C.c_int(kv), _p(x), C.c_size_t(x.size), _p(out))
    return out


# ---- per-kernel references ---------------------------------------------------------------------

def add(a, b):
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().bo_add(_p(a), _p(b), C.c_size_t(a.size), _p(out))
    return out


def swiglu(g, u):
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().bo_swiglu(_p(g), _p(u), C.c_size_t(g.size), _p(out))
    return out


def rms_norm(x, w, n: int, eps: float):
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().bo_rms_norm(_p(x), _p(w), C.c_size_t(x.size // n), C.c_size_t(n), C.c_float(eps), _p(out))
    return out


def softmax(x, n: int):
    x = _f32(x)
    out = np.empty_like(x)
    lib().bo_softmax(_p(x), C.c_size_t(x.size // n), C.c_size_t(n), _p(out))
    return out


def rope_table(theta: float, dim: int, max_pos: int):
    cos = np.empty(max_pos * dim // 2, np.float32)
    sin = np.empty_like(cos)
    lib().bo_rope_table(C.c_double(theta), C.c_int(dim), C.c_size_t(max_pos), _p(cos), _p(sin))
    return cos, sin


def rope_neox(x, heads: int, dim: int, pos0: int, cos, sin):
    x = _f32(x).copy()
    tokens = x.size // (heads * dim)
    lib().bo_rope_neox(_p(x), C.c_size_t(tokens), C.c_int(heads), C.c_int(dim), C.c_size_t(pos0),
                       _p(_f32(cos)), _p(_f32(sin)))
    return x


def matmul(q: int, w, rows: int, cols: int, x, f16_inputs: bool = False):
    """Returns (y[tokens, rows], abs_sum[tokens, rows])."""
    w, x = _u8(w), _f32(x).ravel()
    tokens = x.size // cols
    assert w.size == nbytes(q, rows * cols)
    y = np.empty((tokens, rows), np.float32)
    a = np.empty((tokens, rows), np.float32)
    lib().bo_matmul(C.c_int(q), _p(w), C.c_size_t(rows), C.c_size_t(cols), _p(x), C.c_size_t(tokens),
                    _p(y), _p(a), C.c_int(int(f16_inputs)))
    return y, a


def embed(q: int, table, h: int, ids):
    table = _u8(table)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.empty((ids.size, h), np.float32)
    lib().bo_embed(C.c_int(q), _p(table), C.c_size_t(h), _p(ids), C.c_size_t(ids.size), _p(out))
    return out


def attention(q, k, v, tokens: int, hq: int, hkv: int, dim: int, pos0: int, q16: bool = False):
    """q: [T, hq, dim]; k, v: [pos0+T, hkv, dim]. Returns (o, vmax)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    o = np.empty(tokens * hq * dim, np.float32)
    vmax = np.empty_like(o)
    lib().bo_attention(_p(q), _p(k), _p(v), C.c_size_t(tokens), C.c_int(hq), C.c_int(hkv), C.c_int(dim),
                       C.c_size_t(pos0), C.c_size_t(hkv * dim), C.c_int(int(q16)), _p(o), _p(vmax))
    return o, vmax


# ---- deterministic test inputs -----------------------------------------------------------------

class Rng:
    """xorshift64* of the reference's kernel tests (crates/kernels/src/testutil.rs:3-28)."""

    def __init__(self, seed: int):
        self.s = C.c_uint64(max(seed, 1))

    def next_u64(self) -> int:
        return int(lib().bo_rng_next_u64(C.byref(self.s)))

    def vec(self, n: int, scale: float) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().bo_rng_vec(C.byref(self.s), C.c_size_t(n), C.c_float(scale), _p(out))
        return out

    def qmatrix(self, q: int, rows: int, cols: int) -> np.ndarray:
        out = np.empty(nbytes(q, rows * cols), np.uint8)
        lib().bo_rng_qmatrix(C.byref(self.s), C.c_int(q), C.c_size_t(rows), C.c_size_t(cols), _p(out))
        return out


# ---- sampler -----------------------------------------------------------------------------------

class _Pcg(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


def argmax(v) -> int:
    v = _f32(v)
    return int(lib().bo_argmax(_p(v), C.c_size_t(v.size)))


class Sampler:
    """crates/runtime/src/sampler.rs: greedy / temperature / top-k / top-p with PCG32."""

    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, seed=0):
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.rng = _Pcg()
        lib().bo_pcg32_new(C.c_uint64(seed), C.byref(self.rng))
        self.last_keep = 0

    def next_u32(self) -> int:
        return int(lib().bo_pcg32_next_u32(C.byref(self.rng)))

    def next_f32(self) -> float:
        return float(lib().bo_pcg32_next_f32(C.byref(self.rng)))

    def sample(self, logits) -> int:
        logits = _f32(logits)
        keep = C.c_size_t(0)
        t = lib().bo_sample(C.byref(self.rng), C.c_float(self.temperature), C.c_size_t(self.top_k),
                            C.c_float(self.top_p), _p(logits), C.c_size_t(logits.size), C.byref(keep))
        self.last_keep = keep.value
        return int(t)


# ---- whole model -------------------------------------------------------------------------------

class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("attn_norm", "q_norm", "k_norm", "ffn_norm", "wq", "wk", "wv", "wo", "gate", "up", "down")]


class _Model(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32), ("eps", C.c_float),
                ("rope_theta", C.c_double), ("layer_qtype", C.c_int32), ("embed_qtype", C.c_int32),
                ("head_qtype", C.c_int32), ("embed", C.c_void_p), ("head", C.c_void_p),
                ("final_norm", C.c_void_p), ("layer", C.POINTER(_Layer))]


class _Cache(C.Structure):
    _fields_ = [("kv_type", C.c_int32), ("ctx", C.c_size_t), ("k", C.c_void_p), ("v", C.c_void_p)]


_LAYER_NAMES = {
    "attn_norm": "input_layernorm.weight", "q_norm": "self_attn.q_norm.weight",
    "k_norm": "self_attn.k_norm.weight", "ffn_norm": "post_attention_layernorm.weight",
    "wq": "self_attn.q_proj.weight", "wk": "self_attn.k_proj.weight", "wv": "self_attn.v_proj.weight",
    "wo": "self_attn.o_proj.weight", "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
    "down": "mlp.down_proj.weight",
}


class Qwen3Oracle:
    """Whole-model forward over the raw tensors of a ``.brasa`` file (see brasa_format.BrasaFile)."""

    def __init__(self, brasa, kv: str = "f32", ctx: int = 256):
        cfg = brasa.config()
        self.cfg = cfg
        self._keep = []

        def raw(name):
            a = np.ascontiguousarray(brasa.raw(name))
            self._keep.append(a)
            return a.ctypes.data

        L = cfg["num_hidden_layers"]
        self._layers = (_Layer * L)()
        for i in range(L):
            for f, n in _LAYER_NAMES.items():
                setattr(self._layers[i], f, raw(f"model.layers.{i}.{n}"))
        tied = "lm_head.weight" not in brasa.tensors
        m = _Model()
        m.hidden, m.layers = cfg["hidden_size"], L
        m.heads, m.kv_heads, m.head_dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        m.ffn, m.vocab = cfg["intermediate_size"], cfg["vocab_size"]
        m.eps, m.rope_theta = cfg.get("rms_norm_eps", 1e-6), cfg.get("rope_theta", 1e6)
        m.layer_qtype = QTYPE[brasa.tensors["model.layers.0.self_attn.q_proj.weight"]["dtype"]]
        m.embed_qtype = QTYPE[brasa.tensors["model.embed_tokens.weight"]["dtype"]]
        m.embed = raw("model.embed_tokens.weight")
        if tied:
            m.head, m.head_qtype = m.embed, m.embed_qtype
        else:
            m.head = raw("lm_head.weight")
            m.head_qtype = QTYPE[brasa.tensors["lm_head.weight"]["dtype"]]
        m.final_norm = raw("model.norm.weight")
        m.layer = C.cast(self._layers, C.POINTER(_Layer))
        self.m = m
        self.kv = KVTYPE[kv] if isinstance(kv, str) else kv
        self.ctx = ctx
        kvd = m.kv_heads * m.head_dim
        self.k = np.zeros((L, ctx, kvd), np.float32)
        self.v = np.zeros((L, ctx, kvd), np.float32)
        self.c = _Cache(self.kv, ctx, self.k.ctypes.data, self.v.ctypes.data)
        self.pos = 0

    def reset(self):
        self.pos = 0

    def forward(self, ids, pos0: int | None = None, logit_rows: int = 1, f16_prefill: bool = False,
                capture_hidden: bool = False):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        pos0 = self.pos if pos0 is None else pos0
        logits = np.empty((logit_rows, self.m.vocab), np.float32)
        hid = np.empty((self.m.layers, ids.size, self.m.hidden), np.float32) if capture_hidden else None
        rc = lib().bo_qwen3_forward(C.byref(self.m), C.byref(self.c), _p(ids), C.c_size_t(ids.size),
                                    C.c_size_t(pos0), C.c_size_t(logit_rows), C.c_int(int(f16_prefill)),
                                    _p(logits), _p(hid) if capture_hidden else None)
        if rc != 0:
            raise ValueError("bo_qwen3_forward: bad arguments")
        self.pos = pos0 + ids.size
        return (logits, hid) if capture_hidden else logits
