"""brasa_b200: Python front end of libbrasa_cuda.so, the CUDA (sm_100a) backend of the Qwen3 token loop.

The classes mirror the reference's Rust interfaces so that tests read like the reference's own:

  Context, Buffer, Command          crates/metal/src/runtime.rs
  Kernels, QMatrix, AttnShape,
  KvType, WeightType, RopeTable     crates/kernels/src/lib.rs
  Qwen3, Limits, Config             crates/models/src/qwen3.rs
  Session, SamplingParams, GenStats crates/runtime/src/{session,sampler}.rs
  planner                           crates/memory/src/planner.rs

Everything computes on the GPU through the C ABI in include/brasa_cuda.h. There is no CPU fallback: if
the shared library is missing or no CUDA device is present, construction fails loudly.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
import enum
import pathlib

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = HERE / "libbrasa_cuda.so"

DECODE_CHUNK = 128
KV_ALIGN = 64
NORM_PREP_TG = 256
KV_Q8_DIM = 128
KV_Q8_ROW = 136


class BrasaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{ERRORS.get(code, code)}] {message}")
        self.code = code


ERRORS = {-1: "EINVAL", -2: "ENOMEM", -3: "ECUDA", -4: "ETIMEOUT", -5: "EIO", -6: "EBUDGET"}
EINVAL, ENOMEM, ECUDA, ETIMEOUT, EIO, EBUDGET = -1, -2, -3, -4, -5, -6


class WeightType(enum.IntEnum):
    Q4_0 = 0
    Q8_0 = 1
    Q6_0 = 2


class KvType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q8_0 = 2

    def block_bytes(self) -> int:
        return {KvType.F32: 128, KvType.F16: 64, KvType.Q8_0: 34}[self]

    def bytes(self, n: int) -> int:
        if self == KvType.Q8_0:
            assert n % KV_Q8_DIM == 0, "KV Q8: rows of 128 values"
            return n // KV_Q8_DIM * KV_Q8_ROW
        return n * self.block_bytes() // 32

    @staticmethod
    def parse(s: str) -> "KvType | None":
        return {"f32": KvType.F32, "f16": KvType.F16, "q8_0": KvType.Q8_0, "q8": KvType.Q8_0}.get(s)


class PrefillPrecision(enum.IntEnum):
    F16 = 0
    F32 = 1


class Layout(enum.IntEnum):
    FILE = 0
    TILED = 1


class _Arg(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("offset", C.c_uint64)]


class _QMatrix(C.Structure):
    _fields_ = [("data", _Arg), ("qtype", C.c_int32), ("layout", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32)]


class _AttnShape(C.Structure):
    _fields_ = [("tokens", C.c_uint32), ("hq", C.c_uint32), ("hkv", C.c_uint32), ("dim", C.c_uint32), ("pos0", C.c_uint32),
                ("kv", C.c_int32)]


class _PagedKv(C.Structure):
    _fields_ = [("kpool", _Arg), ("vpool", _Arg), ("table", _Arg), ("lens", _Arg), ("seqs", C.c_uint32), ("max_pages", C.c_uint32),
                ("num_pages", C.c_uint32), ("kv", C.c_int32)]


class _ModelShape(C.Structure):
    _fields_ = [("weight_bytes", C.c_uint64), ("layers", C.c_uint32), ("hidden", C.c_uint32), ("heads", C.c_uint32),
                ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32)]


class _SessionShape(C.Structure):
    _fields_ = [("ctx", C.c_uint32), ("max_tokens", C.c_uint32), ("max_logit_rows", C.c_uint32), ("kv", C.c_int32)]


class _MemoryPlan(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("weights", "kv", "workspace", "overhead", "total")]


class _BatchShape(C.Structure):
    _fields_ = [("max_seqs", C.c_uint32), ("num_pages", C.c_uint32), ("max_positions", C.c_uint32), ("head_rows", C.c_uint32), ("kv", C.c_int32)]


class _BatchPlan(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("kv_pages", "tables", "logits", "attention_partials", "sampler", "total")]


class _Limits(C.Structure):
    _fields_ = [("ctx", C.c_uint32), ("max_tokens", C.c_uint32), ("max_logit_rows", C.c_uint32), ("kv", C.c_int32)]


class _Config(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("layers", C.c_uint32), ("heads", C.c_uint32), ("kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32), ("max_position", C.c_uint32),
                ("eps", C.c_float), ("rope_theta", C.c_double), ("tied", C.c_int32), ("head_rows", C.c_uint32), ("head_row0", C.c_uint32)]


class _Allocated(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("weights", "kv", "workspace")]


class _SamplingParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("seed", C.c_uint64)]


class _GenStats(C.Structure):
    _fields_ = [("prompt_tokens", C.c_uint32), ("reused_tokens", C.c_uint32), ("generated", C.c_uint32), ("stop", C.c_int32),
                ("prefill_ms", C.c_double), ("ttft_ms", C.c_double), ("decode_ms", C.c_double)]


TOKEN_CB = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint32)

_lib = None


def lib() -> C.CDLL:
    """Loads the in-tree shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: run `python -m brasa_b200.build` (needs nvcc)")
        L = C.CDLL(str(LIB_PATH))
        L.brasa_last_error.restype = C.c_char_p
        L.brasa_last_error.argtypes = [C.c_void_p]
        L.brasa_ctx_stream.restype = C.c_void_p
        L.brasa_buf_ptr.restype = C.c_void_p
        L.brasa_buf_bytes.restype = C.c_uint64
        L.brasa_decode_partials_len.restype = C.c_uint64
        L.brasa_kv_bytes.restype = C.c_uint64
        L.brasa_qtype_nbytes.restype = C.c_uint64
        L.brasa_plan_buffer_bytes.restype = C.c_uint64
        L.brasa_session_model.restype = C.c_void_p
        L.brasa_ctx_launch_count.restype = C.c_uint64
        L.brasa_ctx_destroy.restype = None
        L.brasa_model_free.restype = None
        L.brasa_session_free.restype = None
        L.brasa_graph_free.restype = None
        L.brasa_batch_free.restype = None
        L.brasa_batch_free.argtypes = [C.c_void_p]
        L.brasa_batch_sequences.argtypes = [C.c_void_p]
        L.brasa_batch_pages_in_use.argtypes = [C.c_void_p]
        L.brasa_batch_prefix_cache_stats.argtypes = [C.c_void_p] * 5
        L.brasa_tp_free.restype = None
        L.brasa_tp_free.argtypes = [C.c_void_p]
        L.brasa_tp_rank.argtypes = [C.c_void_p]
        L.brasa_tp_world.argtypes = [C.c_void_p]
        L.brasa_tp_rank.restype = C.c_uint32
        L.brasa_tp_world.restype = C.c_uint32
        for name in ("brasa_ctx_destroy", "brasa_model_free", "brasa_session_free", "brasa_buf_free", "brasa_buf_ptr", "brasa_buf_bytes",
                     "brasa_ctx_stream", "brasa_session_model", "brasa_graph_free"):
            getattr(L, name).argtypes = [C.c_void_p]
        _lib = L
    return _lib


def decode_partials_len(hq: int, lk: int) -> int:
    return int(lib().brasa_decode_partials_len(C.c_uint32(hq), C.c_uint32(lk)))


def norm_partials(n: int) -> int:
    return int(lib().brasa_norm_partials(C.c_uint32(n)))


def gqa_supported(hq: int, hkv: int) -> bool:
    return bool(lib().brasa_gqa_supported(C.c_uint32(hq), C.c_uint32(hkv)))


def qtype_nbytes(q: int, n: int) -> int:
    return int(lib().brasa_qtype_nbytes(C.c_int32(int(q)), C.c_uint64(n)))


def rope_table(theta: float, dim: int, max_pos: int):
    cos = np.empty(max_pos * dim // 2, np.float32)
    sin = np.empty_like(cos)
    rc = lib().brasa_rope_table(C.c_double(theta), C.c_uint32(dim), C.c_uint32(max_pos), cos.ctypes.data_as(C.c_void_p),
                                sin.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise BrasaError(rc, "rope_table")
    return cos, sin


class Context:
    """One CUDA device, one stream (crates/metal/src/runtime.rs:134 Context). Not thread-safe."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        rc = lib().brasa_ctx_create(C.c_int32(device), C.byref(self._h))
        if rc != 0:
            raise BrasaError(rc, f"no usable CUDA device {device}: the CUDA backend has no CPU fallback")
        self.device = device

    def _check(self, rc: int):
        if rc != 0:
            raise BrasaError(rc, lib().brasa_last_error(self._h).decode(errors="replace"))

    def close(self):
        if self._h:
            lib().brasa_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def buffer(self, nbytes: int) -> "Buffer":
        """Zero-filled device buffer of nbytes."""
        return Buffer(self, nbytes)

    def buffer_from(self, array) -> "Buffer":
        a = np.ascontiguousarray(array)
        b = Buffer(self, a.nbytes)
        b.upload(a)
        return b

    def command(self) -> "Command":
        return Command(self)

    def sync(self):
        self._check(lib().brasa_ctx_sync(self._h))

    def capture(self, record) -> "Graph":
        """Records the kernels `record(cmd)` enqueues into a CUDA graph instead of running them."""
        cmd = self.command()
        self._check(lib().brasa_graph_capture_begin(self._h))
        try:
            record(cmd)
        finally:
            g = C.c_void_p()
            rc = lib().brasa_graph_capture_end(self._h, C.byref(g))
        self._check(rc)
        cmd.wait()
        return Graph(self, g)

    def launch_count(self) -> int:
        """Kernels enqueued on this context so far (graph replays count their kernels)."""
        return int(lib().brasa_ctx_launch_count(self._h))

    def mem_info(self) -> tuple[int, int]:
        f, t = C.c_uint64(), C.c_uint64()
        self._check(lib().brasa_ctx_mem_info(self._h, C.byref(f), C.byref(t)))
        return f.value, t.value

    @property
    def stream(self) -> int:
        return int(lib().brasa_ctx_stream(self._h) or 0)


class Buffer:
    """Untyped device bytes (crates/metal/src/runtime.rs:44 Buffer<T>)."""

    def __init__(self, ctx: Context, nbytes: int):
        self.ctx = ctx
        self._h = C.c_void_p()
        ctx._check(lib().brasa_buf_alloc(ctx._h, C.c_uint64(nbytes), C.byref(self._h)))
        self.nbytes = nbytes

    def upload(self, array, offset: int = 0):
        a = np.ascontiguousarray(array)
        self.ctx._check(lib().brasa_buf_upload(self._h, C.c_uint64(offset), a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes)))

    def download(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset) // dt.itemsize
        out = np.empty(count, dt)
        self.ctx._check(lib().brasa_buf_download(self._h, C.c_uint64(offset), out.ctypes.data_as(C.c_void_p), C.c_uint64(out.nbytes)))
        return out

    def fill(self, byte: int, offset: int = 0, n: int | None = None):
        self.ctx._check(lib().brasa_buf_fill(self._h, C.c_uint64(offset), C.c_int32(byte), C.c_uint64(self.nbytes - offset if n is None else n)))

    def at(self, offset: int) -> "Arg":
        return Arg(self, offset)

    @property
    def ptr(self) -> int:
        return int(lib().brasa_buf_ptr(self._h) or 0)

    def free(self):
        if self._h and self.ctx._h:
            lib().brasa_buf_free(self._h)
        self._h = C.c_void_p()


@dataclasses.dataclass
class Arg:
    """A buffer and a byte offset (crates/metal/src/runtime.rs:255 Arg::buf_at)."""
    buf: Buffer | None
    offset: int = 0


def _arg(a) -> _Arg:
    if a is None:
        return _Arg(None, 0)
    if isinstance(a, Buffer):
        return _Arg(a._h, 0)
    return _Arg(a.buf._h if a.buf is not None else None, a.offset)


@dataclasses.dataclass
class QMatrix:
    """Quantised matrix [rows, cols] in a byte buffer (crates/kernels/src/lib.rs:146)."""
    data: Buffer | Arg
    qtype: WeightType
    rows: int
    cols: int
    layout: Layout = Layout.FILE

    def _c(self) -> _QMatrix:
        return _QMatrix(_arg(self.data), int(self.qtype), int(self.layout), self.rows, self.cols)


@dataclasses.dataclass
class AttnShape:
    tokens: int
    hq: int
    hkv: int
    dim: int
    pos0: int
    kv: KvType

    def _c(self) -> _AttnShape:
        return _AttnShape(self.tokens, self.hq, self.hkv, self.dim, self.pos0, int(self.kv))


class Command:
    """Kernels are enqueued on the context's stream between begin and wait
    (crates/metal/src/runtime.rs:306 Command, :411 GpuTiming)."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        self._h = C.c_void_p()
        ctx._check(lib().brasa_cmd_begin(ctx._h, C.byref(self._h)))

    def commit(self) -> "Command":
        self.ctx._check(lib().brasa_cmd_commit(self._h))
        return self

    def wait(self) -> float:
        """Blocks until the work is done; returns its device time in seconds."""
        s = C.c_double()
        h, self._h = self._h, C.c_void_p()
        self.ctx._check(lib().brasa_cmd_wait(h, C.byref(s)))
        return s.value

    commit_and_wait = wait


class Graph:
    """A recorded sequence of kernels, replayed with one submission."""

    def __init__(self, ctx: Context, handle):
        self.ctx, self._h = ctx, handle

    def launch(self, cmd: Command):
        self.ctx._check(lib().brasa_graph_launch(cmd._h, self._h))

    def free(self):
        if self._h:
            lib().brasa_graph_free(self._h)
        self._h = C.c_void_p()


class RopeTable:
    """cos/sin table [max_pos, dim/2] computed in double precision (crates/kernels/src/lib.rs:1369)."""

    def __init__(self, ctx: Context, theta: float, dim: int, max_pos: int):
        cos, sin = rope_table(theta, dim, max_pos)
        self.cos, self.sin = ctx.buffer_from(cos), ctx.buffer_from(sin)
        self.dim, self.max_pos = dim, max_pos


class Kernels:
    """One method per reference `Kernels` method, same argument order (crates/kernels/src/lib.rs:391-1300)."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.L = lib()

    def _k(self, rc):
        self.ctx._check(rc)

    # tensor-parallel exchange
    def tp_allreduce_add(self, cmd, tp, partial, resid, out, n, phase=None):
        if phase is None:
            self._k(self.L.brasa_k_tp_allreduce_add(cmd._h, tp._h, _arg(partial), _arg(resid), _arg(out), C.c_uint64(n)))
        else:  # "push" or "gather": the two halves as separate launches (ranks sharing one device)
            self._k(self.L.brasa_k_tp_allreduce_add_phase(cmd._h, tp._h, _arg(partial), _arg(resid), _arg(out), C.c_uint64(n),
                                                          C.c_int32(int(phase == "gather"))))

    def gemv_allreduce(self, cmd, tp, w: QMatrix, x, resid, out, phase=None):
        """out = resid + sum over ranks of (w x); phase "push" / "gather" runs one half (ranks sharing a device)."""
        if phase is None:
            self._k(self.L.brasa_k_gemv_allreduce(cmd._h, tp._h, w._c(), _arg(x), _arg(resid), _arg(out)))
        else:
            self._k(self.L.brasa_k_gemv_allreduce_phase(cmd._h, tp._h, w._c(), _arg(x), _arg(resid), _arg(out), C.c_int32(1 if phase == "gather" else 0)))

    def tp_argmax(self, cmd, tp, logits, n, row0, out, phase=None):
        if phase is None:
            self._k(self.L.brasa_k_tp_argmax(cmd._h, tp._h, _arg(logits), C.c_uint32(n), C.c_uint32(row0), _arg(out)))
        else:
            self._k(self.L.brasa_k_tp_argmax_phase(cmd._h, tp._h, _arg(logits), C.c_uint32(n), C.c_uint32(row0), _arg(out),
                                                   C.c_int32(int(phase == "gather"))))

    # layout / converter
    def repack(self, cmd, qtype, src, dst, rows, cols):
        self._k(self.L.brasa_k_repack(cmd._h, C.c_int32(int(qtype)), _arg(src), _arg(dst), C.c_uint32(rows), C.c_uint32(cols)))

    def unpack(self, cmd, qtype, src, dst, rows, cols):
        self._k(self.L.brasa_k_unpack(cmd._h, C.c_int32(int(qtype)), _arg(src), _arg(dst), C.c_uint32(rows), C.c_uint32(cols)))

    def quantize(self, cmd, qtype, src, dst, n):
        self._k(self.L.brasa_k_quantize(cmd._h, C.c_int32(int(qtype)), _arg(src), _arg(dst), C.c_uint64(n)))

    def dequantize(self, cmd, qtype, src, dst, n):
        self._k(self.L.brasa_k_dequantize(cmd._h, C.c_int32(int(qtype)), _arg(src), _arg(dst), C.c_uint64(n)))

    def randn(self, cmd, dst, n, seed, offset=0, std=1.0):
        self._k(self.L.brasa_k_randn(cmd._h, _arg(dst), C.c_uint64(n), C.c_uint64(seed), C.c_uint64(offset), C.c_float(std)))

    # element-wise, norms, rope, embed
    def add(self, cmd, a, b, out, n):
        self._k(self.L.brasa_k_add(cmd._h, _arg(a), _arg(b), _arg(out), C.c_uint64(n)))

    def swiglu(self, cmd, gate, up, out, n):
        self._k(self.L.brasa_k_swiglu(cmd._h, _arg(gate), _arg(up), _arg(out), C.c_uint64(n)))

    def swiglu_f16(self, cmd, gate, up, out, n):
        self._k(self.L.brasa_k_swiglu_f16(cmd._h, _arg(gate), _arg(up), _arg(out), C.c_uint64(n)))

    def rms_norm(self, cmd, x, w, out, rows, n, eps):
        self._k(self.L.brasa_k_rms_norm(cmd._h, _arg(x), _arg(w), _arg(out), C.c_uint32(rows), C.c_uint32(n), C.c_float(eps)))

    def rms_norm_f16(self, cmd, x, w, out, rows, n, eps):
        self._k(self.L.brasa_k_rms_norm_f16(cmd._h, _arg(x), _arg(w), _arg(out), C.c_uint32(rows), C.c_uint32(n), C.c_float(eps)))

    def softmax(self, cmd, x, out, rows, n):
        self._k(self.L.brasa_k_softmax(cmd._h, _arg(x), _arg(out), C.c_uint32(rows), C.c_uint32(n)))

    def rope_neox(self, cmd, x, table: RopeTable, tokens, heads, dim, pos0):
        self._k(self.L.brasa_k_rope_neox(cmd._h, _arg(x), _arg(table.cos), _arg(table.sin), C.c_uint32(table.dim), C.c_uint32(table.max_pos),
                                         C.c_uint32(tokens), C.c_uint32(heads), C.c_uint32(dim), C.c_uint32(pos0)))

    def embed(self, cmd, table: QMatrix, ids, out, tokens):
        self._k(self.L.brasa_k_embed(cmd._h, table._c(), _arg(ids), _arg(out), C.c_uint32(tokens)))

    def add_norm_prep(self, cmd, x, h, w, xw, ss, n):
        self._k(self.L.brasa_k_add_norm_prep(cmd._h, _arg(x), _arg(h), _arg(w), _arg(xw), _arg(ss), C.c_uint32(n)))

    # GEMV / GEMM
    def gemv_scaled(self, cmd, w: QMatrix, xw, ss, eps, y):
        self._k(self.L.brasa_k_gemv_scaled(cmd._h, w._c(), _arg(xw), _arg(ss), C.c_float(eps), _arg(y)))

    def gemv_scaled3(self, cmd, w, xw, ss, eps, y):
        ws = (_QMatrix * 3)(*[m._c() for m in w])
        ys = (_Arg * 3)(*[_arg(a) for a in y])
        self._k(self.L.brasa_k_gemv_scaled3(cmd._h, ws, _arg(xw), _arg(ss), C.c_float(eps), ys))

    def gemv_scaled_swiglu(self, cmd, gate: QMatrix, up: QMatrix, xw, ss, eps, y):
        self._k(self.L.brasa_k_gemv_scaled_swiglu(cmd._h, gate._c(), up._c(), _arg(xw), _arg(ss), C.c_float(eps), _arg(y)))

    def gemv(self, cmd, w: QMatrix, x, y, tokens):
        self._k(self.L.brasa_k_gemv(cmd._h, w._c(), _arg(x), _arg(y), C.c_uint32(tokens)))

    def gemv_simple(self, cmd, w: QMatrix, x, y, tokens):
        self._k(self.L.brasa_k_gemv_simple(cmd._h, w._c(), _arg(x), _arg(y), C.c_uint32(tokens)))

    def gemm(self, cmd, w: QMatrix, x, y, tokens):
        self._k(self.L.brasa_k_gemm(cmd._h, w._c(), _arg(x), _arg(y), C.c_uint32(tokens)))

    def gemm_add(self, cmd, w: QMatrix, x, acc, scratch, tokens):
        """acc += W x (f16 inputs): the residual add folded into the GEMM."""
        self._k(self.L.brasa_k_gemm_add(cmd._h, w._c(), _arg(x), _arg(acc), _arg(scratch), C.c_uint32(tokens)))

    def gemm_add_rms_norm_f16(self, cmd, w: QMatrix, x, acc, scratch, norm_w, out, tokens, eps):
        """acc += W x, then out = f16(rms_norm(acc) * norm_w)."""
        self._k(self.L.brasa_k_gemm_add_rms_norm_f16(cmd._h, w._c(), _arg(x), _arg(acc), _arg(scratch), _arg(norm_w), _arg(out), C.c_uint32(tokens),
                                                     C.c_float(eps)))

    def gemm_with(self, cmd, w: QMatrix, x, y, tokens, precision):
        self._k(self.L.brasa_k_gemm_with(cmd._h, w._c(), _arg(x), _arg(y), C.c_uint32(tokens), C.c_int32(int(precision))))

    def gemm_multi(self, cmd, ws, x, ys, tokens, precision):
        n = len(ws)
        cw = (_QMatrix * n)(*[m._c() for m in ws])
        cy = (_Arg * n)(*[_arg(a) for a in ys])
        self._k(self.L.brasa_k_gemm_multi(cmd._h, cw, C.c_uint32(n), _arg(x), cy, C.c_uint32(tokens), C.c_int32(int(precision))))

    def gemm_swiglu(self, cmd, wg: QMatrix, wu: QMatrix, x, gate, up, out, tokens):
        self._k(self.L.brasa_k_gemm_swiglu(cmd._h, wg._c(), wu._c(), _arg(x), _arg(gate), _arg(up), _arg(out), C.c_uint32(tokens)))

    # attention
    def qk_norm_rope_store(self, cmd, kv, qkv, norms, eps, table: RopeTable, dst, shape: AttnShape):
        cq = (_Arg * 3)(*[_arg(a) for a in qkv])
        cn = (_Arg * 2)(*[_arg(a) for a in norms])
        cd = (_Arg * 2)(*[_arg(a) for a in dst])
        self._k(self.L.brasa_k_qk_norm_rope_store(cmd._h, C.c_int32(int(kv)), cq, cn, C.c_float(eps), _arg(table.cos), _arg(table.sin),
                                                  C.c_uint32(table.dim), C.c_uint32(table.max_pos), cd, shape._c()))

    @staticmethod
    def paged_kv(kpool, vpool, table, lens, seqs: int, max_pages: int, num_pages: int, kv) -> _PagedKv:
        """One layer's KV pages, the sequences' page tables (i32 [seqs][max_pages]) and lengths (u32 [seqs]) on the device."""
        return _PagedKv(_arg(kpool), _arg(vpool), _arg(table), _arg(lens), seqs, max_pages, num_pages, int(kv))

    def qk_norm_rope_store_paged(self, cmd, q, k, v, q_norm, k_norm, eps, table: RopeTable, paged: _PagedKv, hq: int, hkv: int):
        self._k(self.L.brasa_k_qk_norm_rope_store_paged(cmd._h, _arg(q), _arg(k), _arg(v), _arg(q_norm), _arg(k_norm), _arg(table.cos), _arg(table.sin),
                                                        C.c_float(eps), paged, C.c_uint32(hq), C.c_uint32(hkv)))

    def decode_attention_paged(self, cmd, q, paged: _PagedKv, partials, o, hq: int, hkv: int):
        self._k(self.L.brasa_k_decode_attention_paged(cmd._h, _arg(q), paged, _arg(partials), C.c_uint64(partials.nbytes // 4), _arg(o),
                                                      C.c_uint32(hq), C.c_uint32(hkv)))

    def store_kv(self, cmd, kv, src, dst, n):
        self._k(self.L.brasa_k_store_kv(cmd._h, C.c_int32(int(kv)), _arg(src), _arg(dst), C.c_uint64(n)))

    def decode_attention(self, cmd, q, k, v, partials: Buffer, o, shape: AttnShape):
        self._k(self.L.brasa_k_decode_attention(cmd._h, _arg(q), _arg(k), _arg(v), _arg(partials), C.c_uint64(partials.nbytes // 4), _arg(o),
                                                shape._c()))

    def decode_attention_lanes(self, cmd, q, k, v, partials: Buffer, o, shape: AttnShape):
        self._k(self.L.brasa_k_decode_attention_lanes(cmd._h, _arg(q), _arg(k), _arg(v), _arg(partials), C.c_uint64(partials.nbytes // 4),
                                                      _arg(o), shape._c()))

    def decode_attention_static(self, cmd, q, k, v, o, shape: AttnShape):
        """decode_attention without a scratch argument, for callers that cannot allocate device memory: the
        chunk partials go to a fixed array inside the library (at most 64 query heads and 8192 keys)."""
        self._k(self.L.brasa_k_decode_attention_static(cmd._h, _arg(q), _arg(k), _arg(v), _arg(o), shape._c()))

    def flash_attention(self, cmd, q, k, v, o, shape: AttnShape):
        self._k(self.L.brasa_k_flash_attention(cmd._h, _arg(q), _arg(k), _arg(v), _arg(o), shape._c()))

    def flash_attention_with(self, cmd, q, k, v, o, shape: AttnShape, precision):
        self._k(self.L.brasa_k_flash_attention_with(cmd._h, _arg(q), _arg(k), _arg(v), _arg(o), shape._c(), C.c_int32(int(precision))))

    def argmax(self, cmd, logits, n, out):
        self._k(self.L.brasa_k_argmax(cmd._h, _arg(logits), C.c_uint32(n), _arg(out)))

    def sample_top_p(self, cmd, logits, n, temperature, top_k, top_p, rng_state, out):
        """Sampler::sample on the device; rng_state is a 16-byte buffer made by pcg32_state(seed)."""
        self._k(self.L.brasa_k_sample_top_p(cmd._h, _arg(logits), C.c_uint32(n), C.c_float(temperature), C.c_uint32(top_k), C.c_float(top_p),
                                            _arg(rng_state), _arg(out)))

    def sample_rows(self, cmd, logits, n, count, temperature, top_k, top_p, rng_states, scratch, out):
        """The same for `count` rows; rng_states holds one pcg32_state per row, scratch count * n * 8 bytes."""
        self._k(self.L.brasa_k_sample_rows(cmd._h, _arg(logits), C.c_uint32(n), C.c_uint32(count), C.c_float(temperature), C.c_uint32(top_k),
                                           C.c_float(top_p), _arg(rng_states), _arg(scratch), _arg(out)))


def pcg32_state(seed: int) -> np.ndarray:
    """Pcg32::new(seed) as the {state, increment} pair the device sampler keeps."""
    out = (C.c_uint64 * 2)()
    lib().brasa_pcg32_seed(C.c_uint64(seed), out)
    return np.array([out[0], out[1]], dtype=np.uint64)


# ---- model / session ---------------------------------------------------------------------------


@dataclasses.dataclass
class Limits:
    """crates/models/src/qwen3.rs:175 Limits."""
    ctx: int
    max_tokens: int = 1024
    max_logit_rows: int = 1
    kv: KvType = KvType.F16

    def _c(self) -> _Limits:
        return _Limits(self.ctx, self.max_tokens, self.max_logit_rows, int(self.kv))


@dataclasses.dataclass
class SamplingParams:
    """crates/runtime/src/sampler.rs:5 SamplingParams; temperature 0 is greedy."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    @staticmethod
    def greedy() -> "SamplingParams":
        return SamplingParams()


@dataclasses.dataclass
class GenStats:
    """crates/runtime/src/session.rs:29 GenStats."""
    prompt_tokens: int
    reused_tokens: int
    prefill_ms: float
    ttft_ms: float
    generated: int
    decode_ms: float
    stop: str

    def prefill_tok_s(self) -> float:
        return (self.prompt_tokens - self.reused_tokens) / (self.prefill_ms / 1e3)

    def decode_tok_s(self) -> float:
        return 0.0 if self.generated < 2 else (self.generated - 1) / (self.decode_ms / 1e3)


def _cfg_dict(c: _Config) -> dict:
    return {n: getattr(c, n) for n, _ in _Config._fields_}


def model_shape(path) -> tuple[_ModelShape, dict]:
    """Memory shape of the model in `path`, reading only the header (crates/models/src/qwen3.rs:79)."""
    shape, cfg = _ModelShape(), _Config()
    err = C.create_string_buffer(512)
    rc = lib().brasa_model_shape_from_file(str(path).encode(), C.byref(shape), C.byref(cfg), err, C.c_uint64(512))
    if rc != 0:
        raise BrasaError(rc, err.value.decode(errors="replace"))
    return shape, _cfg_dict(cfg)


def file_check(path, verify: bool = True) -> None:
    """BrasaFile::open (+ verify): raises BrasaError(EIO) with the reason."""
    err = C.create_string_buffer(512)
    rc = lib().brasa_file_check(str(path).encode(), C.c_int32(int(verify)), err, C.c_uint64(512))
    if rc != 0:
        raise BrasaError(rc, err.value.decode(errors="replace"))


class planner:
    """crates/memory/src/planner.rs: bytes a session needs, before anything is loaded."""

    @staticmethod
    def buffer_bytes(n: int) -> int:
        return int(lib().brasa_plan_buffer_bytes(C.c_uint64(n)))

    @staticmethod
    def plan(shape: _ModelShape, limits: Limits) -> dict:
        p = _MemoryPlan()
        s = _SessionShape(limits.ctx, limits.max_tokens, limits.max_logit_rows, int(limits.kv))
        rc = lib().brasa_plan(C.byref(shape), C.byref(s), C.byref(p))
        if rc != 0:
            raise BrasaError(rc, "plan: bad arguments")
        return {n: getattr(p, n) for n, _ in _MemoryPlan._fields_}

    @staticmethod
    def check(ctx: Context | None, shape: _ModelShape, limits: Limits, budget: int = 0) -> tuple[bool, dict, int]:
        """(fits, plan, largest context that fits)."""
        p, mx = _MemoryPlan(), C.c_uint32()
        s = _SessionShape(limits.ctx, limits.max_tokens, limits.max_logit_rows, int(limits.kv))
        rc = lib().brasa_plan_check(ctx._h if ctx else None, C.byref(shape), C.byref(s), C.c_uint64(budget), C.byref(p), C.byref(mx))
        if rc not in (0, EBUDGET):
            raise BrasaError(rc, "plan_check")
        return rc == 0, {n: getattr(p, n) for n, _ in _MemoryPlan._fields_}, mx.value


    @staticmethod
    def plan_batch(shape: _ModelShape, max_seqs: int, num_pages: int, max_positions: int, kv: KvType, head_rows: int | None = None) -> dict:
        """Bytes of a batch over a paged KV pool, buffer by buffer as brasa_batch_create allocates them."""
        p = _BatchPlan()
        s = _BatchShape(max_seqs, num_pages, max_positions, head_rows if head_rows is not None else shape.vocab, int(kv))
        rc = lib().brasa_plan_batch(C.byref(shape), C.byref(s), C.byref(p))
        if rc != 0:
            raise BrasaError(rc, "plan_batch: bad arguments")
        return {n: getattr(p, n) for n, _ in _BatchPlan._fields_}

    @staticmethod
    def max_batch(ctx: Context | None, shape: _ModelShape, kv: KvType, shared_prefix: int, positions_per_seq: int, budget: int = 0,
                  cap: int = 1 << 20, head_rows: int | None = None) -> tuple[int, int, dict]:
        """(largest number of sequences that fits, pages it needs, its plan); 0 sequences when not even one fits."""
        p, n, pages = _BatchPlan(), C.c_uint32(), C.c_uint32()
        rc = lib().brasa_plan_batch_max_seqs(ctx._h if ctx else None, C.byref(shape), C.c_int32(int(kv)),
                                             C.c_uint32(head_rows if head_rows is not None else shape.vocab), C.c_uint32(shared_prefix),
                                             C.c_uint32(positions_per_seq), C.c_uint32(cap), C.c_uint64(budget), C.byref(n), C.byref(pages), C.byref(p))
        if rc not in (0, EBUDGET):
            raise BrasaError(rc, "plan_batch_max_seqs: bad arguments")
        return n.value, pages.value, {k: getattr(p, k) for k, _ in _BatchPlan._fields_}


class Qwen3:
    """Model on the device with its KV cache and workspace (crates/models/src/qwen3.rs:301 Qwen3)."""

    def __init__(self, ctx: Context, path, limits: Limits, _handle=None):
        self.ctx = ctx
        self._own = _handle is None
        self._h = C.c_void_p(_handle) if _handle is not None else C.c_void_p()
        if _handle is None:
            ctx._check(lib().brasa_model_load(ctx._h, str(path).encode(), limits._c(), C.byref(self._h)))
        c, l = _Config(), _Limits()
        lib().brasa_model_config(self._h, C.byref(c))
        lib().brasa_model_limits(self._h, C.byref(l))
        self.cfg = _cfg_dict(c)
        self.limits = Limits(l.ctx, l.max_tokens, l.max_logit_rows, KvType(l.kv))

    @classmethod
    def load(cls, ctx: Context, path, limits: Limits) -> "Qwen3":
        return cls(ctx, path, limits)

    def free(self):
        if self._own and self._h and self.ctx._h:
            lib().brasa_model_free(self._h)
        self._h = C.c_void_p()

    def set_tp(self, tp) -> None:
        """Attaches a tensor-parallel exchange (brasa_b200.tp.TensorParallel) to this shard, before its first step."""
        self.ctx._check(lib().brasa_model_set_tp(self._h, tp._h))
        self._tp = tp

    def allocated(self) -> dict:
        a = _Allocated()
        self.ctx._check(lib().brasa_model_allocated(self._h, C.byref(a)))
        return {"weights": a.weights, "kv": a.kv, "workspace": a.workspace}

    def set_prefill_precision(self, p: PrefillPrecision):
        self.ctx._check(lib().brasa_model_set_prefill_precision(self._h, C.c_int32(int(p))))

    def forward(self, ids, pos0: int, logit_rows: int = 1, want_logits: bool = True):
        """Returns (logits [logit_rows, vocab] or None, device seconds); a tensor-parallel shard returns its own
        head_rows columns of the vocabulary, starting at head_row0."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        logits = np.empty((logit_rows, self.cfg["head_rows"]), np.float32) if want_logits else None
        secs = C.c_double()
        self.ctx._check(lib().brasa_model_forward(self._h, ids.ctypes.data_as(C.c_void_p), C.c_uint32(ids.size), C.c_uint32(pos0),
                                                  C.c_uint32(logit_rows), logits.ctypes.data_as(C.c_void_p) if want_logits else None,
                                                  C.byref(secs)))
        return logits, secs.value

    def run_layers(self, x, pos0: int, layers: range) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).copy()
        tokens = x.size // self.cfg["hidden"]
        self.ctx._check(lib().brasa_model_run_layers(self._h, x.ctypes.data_as(C.c_void_p), C.c_uint32(tokens), C.c_uint32(pos0),
                                                     C.c_uint32(layers.start), C.c_uint32(layers.stop)))
        return x

    def decode_greedy(self, first: int, pos0: int, steps: int):
        """Device-resident greedy decode: (ids[steps], device seconds)."""
        out = np.empty(steps, np.uint32)
        secs = C.c_double()
        self.ctx._check(lib().brasa_model_decode_greedy(self._h, C.c_uint32(first), C.c_uint32(pos0), C.c_uint32(steps),
                                                        out.ctypes.data_as(C.c_void_p), C.byref(secs)))
        return out, secs.value

    def load_stats(self) -> dict:
        """Seconds the weights took from the file to their device layout, the bytes moved, and the rate."""
        s, n = C.c_double(0.0), C.c_uint64(0)
        self.ctx._check(lib().brasa_model_load_stats(self._h, C.byref(s), C.byref(n)))
        return {"seconds": s.value, "bytes": int(n.value), "gb_per_s": n.value / s.value / 1e9 if s.value > 0 else None}

    def read_kv(self, layer: int, which: str, pos_begin: int, pos_end: int) -> np.ndarray:
        kvd = self.cfg["kv_heads"] * self.cfg["head_dim"]
        n = self.limits.kv.bytes((pos_end - pos_begin) * kvd)
        out = np.empty(n, np.uint8)
        self.ctx._check(lib().brasa_model_read_kv(self._h, C.c_uint32(layer), C.c_int32(1 if which == "v" else 0), C.c_uint32(pos_begin),
                                                  C.c_uint32(pos_end), out.ctypes.data_as(C.c_void_p), C.c_uint64(n)))
        return out


_STOP = {0: "Stop", 1: "MaxTokens", 2: "ContextFull", 3: "Cancelled"}


class Session:
    """Generation session: prefix reuse, chunked prefill, decode loop (crates/runtime/src/session.rs)."""

    def __init__(self, ctx: Context, path, limits: Limits, budget: int = 0):
        self.ctx = ctx
        self._h = C.c_void_p()
        ctx._check(lib().brasa_session_create(ctx._h, str(path).encode(), limits._c(), C.c_uint64(budget), C.byref(self._h)))
        self.model = Qwen3(ctx, path, limits, _handle=lib().brasa_session_model(self._h))

    @classmethod
    def load_with_budget(cls, ctx, path, limits, budget) -> "Session":
        return cls(ctx, path, limits, budget)

    def free(self):
        if self._h and self.ctx._h:
            lib().brasa_session_free(self._h)
        self._h = C.c_void_p()

    def reset(self):
        self.ctx._check(lib().brasa_session_reset(self._h))

    def set_stop_ids(self, ids, ignore_stop: bool = False):
        a = np.ascontiguousarray(ids, dtype=np.uint32)
        self.ctx._check(lib().brasa_session_set_stop_ids(self._h, a.ctypes.data_as(C.c_void_p), C.c_uint32(a.size), C.c_int32(int(ignore_stop))))

    def generate(self, prompt, max_new: int, params: SamplingParams | None = None, on_token=None):
        """Returns (ids of the generated tokens, GenStats)."""
        params = params or SamplingParams.greedy()
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(max(max_new, 1), np.uint32)
        st = _GenStats()
        cb = TOKEN_CB(lambda _u, tok: 1 if on_token(int(tok)) else 0) if on_token else C.cast(None, TOKEN_CB)
        sp = _SamplingParams(params.temperature, params.top_k, params.top_p, params.seed)
        self.ctx._check(lib().brasa_session_generate(self._h, p.ctypes.data_as(C.c_void_p), C.c_uint32(p.size), C.c_uint32(max_new), sp, cb, None,
                                                     out.ctypes.data_as(C.c_void_p), C.byref(st)))
        stats = GenStats(st.prompt_tokens, st.reused_tokens, st.prefill_ms, st.ttft_ms, st.generated, st.decode_ms, _STOP.get(st.stop, "?"))
        return out[:st.generated].copy(), stats


class Batch:
    """Many independent sequences of one model decoded together over a paged KV pool, with a prefix shared by all of
    them computed once (the reference's single cached prefix, crates/runtime/src/session.rs:230-237, for many sequences)."""

    PAGE = 16

    def __init__(self, model: "Qwen3", max_seqs: int, num_pages: int, max_positions: int):
        self.model, self.ctx = model, model.ctx
        self._h = C.c_void_p()
        self.ctx._check(lib().brasa_batch_create(model._h, C.c_uint32(max_seqs), C.c_uint32(num_pages), C.c_uint32(max_positions), C.byref(self._h)))

    def free(self):
        if self._h and self.ctx._h:
            lib().brasa_batch_free(self._h)
        self._h = C.c_void_p()

    def set_prefix(self, ids):
        a = np.ascontiguousarray(ids, dtype=np.uint32)
        self.ctx._check(lib().brasa_batch_set_prefix(self._h, a.ctypes.data_as(C.c_void_p), C.c_uint32(a.size)))

    def add_sequence(self, ids, params: SamplingParams | None = None) -> int:
        params = params or SamplingParams.greedy()
        a = np.ascontiguousarray(ids, dtype=np.uint32)
        seq = C.c_uint32(0)
        sp = _SamplingParams(params.temperature, params.top_k, params.top_p, params.seed)
        self.ctx._check(lib().brasa_batch_add_sequence(self._h, a.ctypes.data_as(C.c_void_p), C.c_uint32(a.size), sp, C.byref(seq)))
        return int(seq.value)

    @property
    def sequences(self) -> int:
        return int(lib().brasa_batch_sequences(self._h))

    @property
    def pages_in_use(self) -> int:
        return int(lib().brasa_batch_pages_in_use(self._h))

    def allocated(self) -> int:
        n = C.c_uint64(0)
        self.ctx._check(lib().brasa_batch_allocated(self._h, C.byref(n)))
        return int(n.value)

    def prefix_cache_stats(self) -> dict:
        """Prompt tokens served from the prefix cache and computed so far, pages the cache knows, pages all sequences share."""
        hit, done, pages, common = C.c_uint64(0), C.c_uint64(0), C.c_uint32(0), C.c_uint32(0)
        self.ctx._check(lib().brasa_batch_prefix_cache_stats(self._h, C.byref(hit), C.byref(done), C.byref(pages), C.byref(common)))
        return {"hit_tokens": int(hit.value), "prefilled_tokens": int(done.value), "cached_pages": int(pages.value), "common_pages": int(common.value)}

    def decode(self, steps: int, params: SamplingParams | None = None):
        """Returns (ids [sequences][steps + 1] with the token drawn at add time first, device seconds)."""
        params = params or SamplingParams.greedy()
        n = self.sequences
        out = np.zeros((n, steps + 1), np.uint32)
        secs = C.c_double(0.0)
        sp = _SamplingParams(params.temperature, params.top_k, params.top_p, params.seed)
        self.ctx._check(lib().brasa_batch_decode(self._h, C.c_uint32(steps), sp, out.ctypes.data_as(C.c_void_p), C.byref(secs)))
        return out, float(secs.value)

    def peek_logits(self) -> np.ndarray:
        n = self.sequences
        out = np.zeros((n, self.model.cfg["head_rows"]), np.float32)
        self.ctx._check(lib().brasa_batch_peek_logits(self._h, out.ctypes.data_as(C.c_void_p)))
        return out
