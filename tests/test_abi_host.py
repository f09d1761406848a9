"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header declares, and its
host-side logic (file reader, planner, helpers) agrees with the oracle. No kernel runs here."""

import ctypes as C
import pathlib
import re

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def B():
    import brasa_b200
    from brasa_b200 import build
    build.build()
    return brasa_b200


def test_library_exports_every_declared_symbol(B):
    header = (ROOT / "include" / "brasa_cuda.h").read_text()
    declared = sorted(set(re.findall(r"\b(brasa_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) > 60
    L = B.lib()
    missing = [n for n in declared if not hasattr(L, n)]
    assert not missing, missing


def test_helpers_match_reference_formulas(B):
    assert B.decode_partials_len(32, 1) == 32 * 130
    assert B.decode_partials_len(32, 129) == 32 * 2 * 130
    assert B.norm_partials(2560) == 10 and B.norm_partials(2561) == 11
    assert [B.gqa_supported(h, 8) for h in (8, 16, 32, 64, 24, 40)] == [True, True, True, True, False, False]
    assert not B.gqa_supported(8, 0)
    assert B.qtype_nbytes(B.WeightType.Q4_0, 64) == 36
    assert B.qtype_nbytes(B.WeightType.Q6_0, 64) == 52
    assert B.qtype_nbytes(B.WeightType.Q8_0, 64) == 68
    assert B.KvType.F16.bytes(256) == 512 and B.KvType.Q8_0.bytes(256) == 272 and B.KvType.F32.bytes(32) == 128
    assert B.KvType.parse("q8") == B.KvType.Q8_0 and B.KvType.parse("nope") is None
    assert (B.DECODE_CHUNK, B.KV_ALIGN, B.NORM_PREP_TG) == (128, 64, 256)


def test_rope_table_is_the_oracles(B):
    cos, sin = B.rope_table(1e6, 128, 300)
    oc, os_ = O.rope_table(1e6, 128, 300)
    assert np.array_equal(cos, oc) and np.array_equal(sin, os_)


def test_file_reader_accepts_the_reference_file_and_detects_damage(B, golden_dir, tmp_path):
    path = golden_dir / "tiny" / "model.brasa"
    B.file_check(path, verify=True)
    shape, cfg = B.model_shape(path)
    assert (cfg["layers"], cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"]) == (2, 256, 4, 2, 128, 512, 512)
    assert cfg["tied"] == 1 and abs(cfg["eps"] - 1e-6) < 1e-12 and cfg["rope_theta"] == 1e6
    f = BF.BrasaFile(path)
    assert shape.weight_bytes == sum(B.planner.buffer_bytes(t["nbytes"]) for t in f.meta["tensors"])
    raw = bytearray(path.read_bytes())
    # a flipped data byte passes the structure check and fails verification
    bad = bytearray(raw)
    bad[f.tensors["model.norm.weight"]["offset"] + 5] ^= 0x40
    (tmp_path / "flip.brasa").write_bytes(bad)
    B.file_check(tmp_path / "flip.brasa", verify=False)
    with pytest.raises(B.BrasaError) as e:
        B.file_check(tmp_path / "flip.brasa", verify=True)
    assert e.value.code == B.EIO and "sha256" in str(e.value)
    # truncation, bad magic, bad version
    (tmp_path / "short.brasa").write_bytes(raw[: len(raw) // 2])
    (tmp_path / "magic.brasa").write_bytes(b"XXXX" + raw[4:])
    (tmp_path / "version.brasa").write_bytes(raw[:4] + (2).to_bytes(4, "little") + raw[8:])
    (tmp_path / "tiny.brasa").write_bytes(raw[:10])
    for name in ("short", "magic", "version", "tiny"):
        with pytest.raises(B.BrasaError) as e:
            B.file_check(tmp_path / f"{name}.brasa", verify=False)
        assert e.value.code == B.EIO
    with pytest.raises(B.BrasaError):
        B.file_check(tmp_path / "does-not-exist.brasa")


def test_hand_built_file_alignment_rules(B, tmp_path):
    cfg = BF.tiny_config(layers=1)
    w = BF.synth_weights(cfg, seed=3)
    meta = BF.write_brasa(tmp_path / "m.brasa", cfg, w)
    B.file_check(tmp_path / "m.brasa", verify=True)
    assert all(t["offset"] % 16384 == 0 for t in meta["tensors"])
    # an offset that is not page aligned is rejected by the structure check (same header length)
    raw = (tmp_path / "m.brasa").read_bytes()
    off = meta["tensors"][0]["offset"]
    old, new = f'"offset":{off}'.encode(), f'"offset":{off + 1}'.encode()
    assert len(old) == len(new) and raw.count(old) >= 1
    (tmp_path / "unaligned.brasa").write_bytes(raw.replace(old, new, 1))
    with pytest.raises(B.BrasaError) as e:
        B.file_check(tmp_path / "unaligned.brasa", verify=False)
    assert "aligned" in str(e.value)


def test_planner_arithmetic(B, golden_dir):
    shape, cfg = B.model_shape(golden_dir / "tiny" / "model.brasa")
    lim = B.Limits(ctx=300, max_tokens=64, max_logit_rows=2, kv=B.KvType.F16)
    p = B.planner.plan(shape, lim)
    bb = B.planner.buffer_bytes
    cap = 320  # ctx rounded up to KV_ALIGN
    assert p["kv"] == 2 * bb(2 * (2 * cap * 2 * 128))
    f = lambda n: bb(4 * n)
    t, h, qd, kvd, ffn = 64, 256, 512, 256, 512
    want_ws = (3 * f(t * h) + 2 * f(t * qd) + 2 * f(t * kvd) + 2 * f(t * ffn) + bb(2 * t * 512) + f(t) + f(1)
               + f(4 * 3 * 130) + f(2 * 512) + 2 * f(300 * 64))
    assert p["workspace"] == want_ws
    assert p["weights"] == shape.weight_bytes and p["overhead"] == 256 << 20
    assert p["total"] == p["weights"] + p["kv"] + p["workspace"] + p["overhead"]
    q8 = B.planner.plan(shape, B.Limits(ctx=300, max_tokens=64, max_logit_rows=2, kv=B.KvType.Q8_0))
    assert q8["kv"] == 2 * bb((2 * cap * 2 * 128) // 128 * 136)
    # budget check without a device: explicit budget
    ok, plan, mx = B.planner.check(None, shape, lim, budget=p["total"])
    assert ok and mx == 300
    ok, plan, mx = B.planner.check(None, shape, lim, budget=p["total"] - 1)
    assert not ok and 0 < mx < 300
    smaller = B.planner.plan(shape, B.Limits(ctx=mx, max_tokens=min(64, mx), max_logit_rows=2, kv=B.KvType.F16))
    assert smaller["total"] <= p["total"] - 1
    ok, _, mx0 = B.planner.check(None, shape, lim, budget=1000)
    assert not ok and mx0 == 0


def test_no_cpu_fallback_without_a_device(B):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(B.BrasaError) as e:
        B.Context(0)
    assert e.value.code == B.ECUDA


def test_batch_planner_arithmetic_and_largest_batch(B):
    """The paged pool's plan (crates/memory/src/planner.rs:57-95 retargeted): every buffer of a batch at the allocation
    granularity, and the largest batch that fits a budget (planner.rs:237-281 for sequences): one more sequence than
    the answer does not fit, the answer does."""
    shape = B._ModelShape(0, 36, 2560, 32, 8, 128, 9728, 151936)  # the Qwen3-4B architecture
    bb = B.planner.buffer_bytes
    p = B.planner.plan_batch(shape, 64, 2048 // 16 + 64 * 97, 3600, B.KvType.F16)
    row = 8 * 128 * 2
    assert p["kv_pages"] == 2 * bb(36 * (128 + 64 * 97) * 16 * row)
    assert p["tables"] == bb(64 * 225 * 4) + 3 * bb(64 * 4) + bb(64 * 16)
    assert p["logits"] == bb(64 * 151936 * 4) and p["sampler"] == bb(64 * 2 * 151936 * 4)
    assert p["attention_partials"] == bb(64 * 32 * ((225 * 16 + 127) // 128) * 130 * 4)
    assert p["total"] == sum(v for k, v in p.items() if k != "total")
    q8 = B.planner.plan_batch(shape, 64, 2048 // 16 + 64 * 97, 3600, B.KvType.Q8_0)
    assert q8["kv_pages"] == 2 * bb(36 * (128 + 64 * 97) * 16 * 8 * 136)
    # 64 sequences of 3 600 positions behind a 2 048-token shared prefix: 13.9 GiB of pages; 31.5 GiB without sharing
    assert abs(p["kv_pages"] / 2**30 - 13.92) < 0.05
    budget = 40 << 30
    n, pages, plan = B.planner.max_batch(None, shape, B.KvType.F16, 2048, 3600, budget=budget)
    assert n > 64 and plan["total"] <= budget and pages == 128 + n * 97
    more = B.planner.plan_batch(shape, n + 1, 128 + (n + 1) * 97, 3600, B.KvType.F16)
    assert more["total"] > budget
    n0, _, _ = B.planner.max_batch(None, shape, B.KvType.F16, 2048, 3600, budget=1 << 20)
    assert n0 == 0
    n_cap, _, _ = B.planner.max_batch(None, shape, B.KvType.F16, 2048, 3600, budget=budget, cap=10)
    assert n_cap == 10
    # a tensor-parallel shard (an eighth of the lm_head's rows): two more full-width logits buffers for the sampled choice
    sh = B.planner.plan_batch(shape, 16, 2048 // 16 + 16 * 97, 3600, B.KvType.F16, head_rows=151936 // 8)
    assert sh["logits"] == bb(16 * (151936 // 8) * 4)
    assert sh["sampler"] == bb(16 * 2 * 151936 * 4) + 2 * bb(16 * 151936 * 4)


def test_few_token_gemm_partition(B):
    """The cut of a few-token GEMM over the SMs (`brasa_gemm_few_tokens_plan`): the runs tile the units exactly, every
    unit's owner is the block whose run holds it, the blocks that share a tile are consecutive and never more than
    `max_parts`, and the scratch holds one 64 x 128 f32 tile per (tile, part). Shapes: the Qwen3-4B layer at 148 SMs
    (qkv, o, gate + up, down), a shard's, tiny ones, and one too large for 32-bit unit arithmetic."""
    L = B.lib()
    L.brasa_gemm_few_tokens_plan.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
    L.brasa_gemm_few_tokens_plan.restype = C.c_int32
    L.brasa_gemm_few_tokens_owner.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    L.brasa_gemm_few_tokens_owner.restype = C.c_uint32
    for sms, tiles, stages in [(148, 48, 40), (148, 20, 64), (148, 152, 40), (148, 20, 152), (148, 1, 4), (148, 3, 4), (148, 1, 1), (132, 25, 38),
                               (148, 200, 4), (7, 5, 9)]:
        blocks, parts, scratch = C.c_uint32(), C.c_uint32(), C.c_uint64()
        assert L.brasa_gemm_few_tokens_plan(sms, tiles, stages, C.byref(blocks), C.byref(parts), C.byref(scratch)) == 0
        nb, units = blocks.value, tiles * stages
        assert 1 <= nb <= min(sms, units) and (nb == sms or nb == max(1, units // 4))
        beg = [b * units // nb for b in range(nb + 1)]
        assert beg[0] == 0 and beg[-1] == units and all(beg[b] < beg[b + 1] for b in range(nb))  # no empty run
        owner = [L.brasa_gemm_few_tokens_owner(units, nb, u) for u in range(units)]
        for u, b in enumerate(owner):
            assert beg[b] <= u < beg[b + 1], (u, b)
        worst = 0
        for t in range(tiles):
            own = owner[t * stages:(t + 1) * stages]
            assert own == sorted(own) and set(own) == set(range(own[0], own[-1] + 1))  # consecutive blocks, in K order
            worst = max(worst, own[-1] - own[0] + 1)
        assert parts.value == worst
        assert scratch.value == tiles * worst * 64 * 128 * 4
    blocks, parts, scratch = C.c_uint32(), C.c_uint32(), C.c_uint64()
    assert L.brasa_gemm_few_tokens_plan(148, 1 << 20, 1 << 6, C.byref(blocks), C.byref(parts), C.byref(scratch)) != 0
    assert L.brasa_gemm_few_tokens_plan(148, 0, 4, C.byref(blocks), C.byref(parts), C.byref(scratch)) != 0
    assert L.brasa_gemm_few_tokens_owner(100, 10, 100) == 0xFFFFFFFF
