"""Parity at the shapes the benchmark runs, not only at the reference's small test shapes:

* the serving batch: GQA group 4, 64 sequences behind a 2 048-token shared prefix (the blocks that take four
  sequences' heads at once over shared K/V tiles), greedy and sampled;
* a 16 384-token prompt in 3 584-token chunks over f16 and q8_0 caches plus decode steps, against golden logits made
  by the reference's own forward (tools/qwen3_ref.py; tests/golden/make_golden_long.py);
* decode attention beyond 8 192 positions with GQA groups 2 and 8 on both decode paths (one kernel per token, one
  kernel per operation);
* the prefill GEMMs at the real matrix sizes and at the token counts that select every block shape and K split.

Bounds are the reference's: crates/models/tests/forward.rs:40-55 for logits (1e-3 f16 cache, 2e-2 q8_0 cache, 2e-3
floor with f16 GEMM inputs), the tie rule of forward.rs:131-138 for tokens, 1e-5 of sum |w x| for GEMMs
(crates/kernels/src/lib.rs:7-15)."""

import os

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF

pytestmark = pytest.mark.gpu

LOGIT_TOL = {"F16": 1e-3, "Q8_0": 2e-2}
F16_PREFILL_FLOOR = 2e-3


@pytest.fixture(scope="module")
def B():
    import brasa_b200
    return brasa_b200


@pytest.fixture(scope="module")
def ctx(B):
    c = B.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def K(B, ctx):
    return B.Kernels(ctx)


def run(ctx, fn):
    cmd = ctx.command()
    fn(cmd)
    return cmd.wait()


def rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


# ---- serving shape -----------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def group4_model(tmp_path_factory):
    """3 layers, hidden 512, 8 query heads over 2 KV heads: the GQA group of Qwen3-4B."""
    d = tmp_path_factory.mktemp("serving")
    cfg = BF.tiny_config(layers=3, hidden=512, heads=8, kv_heads=2, ffn=1536, vocab=1024)
    BF.write_brasa(d / "model.brasa", cfg, BF.synth_weights(cfg, seed=11, std=0.04, norm_jitter=0.1))
    return d / "model.brasa"


NSEQ, PREFIX = 64, 2048


def serving_prompts():
    rng = np.random.default_rng(64)
    prefix = rng.integers(0, 1024, PREFIX).astype(np.uint32)
    suffixes = [rng.integers(0, 1024, int(n)).astype(np.uint32) for n in rng.integers(3, 70, NSEQ)]
    return prefix, suffixes


def test_serving_batch_of_64_sequences_matches_each_sequence_alone(B, ctx, group4_model):
    prefix, suffixes = serving_prompts()
    steps = 16
    m = B.Qwen3.load(ctx, group4_model, B.Limits(ctx=PREFIX + 192, max_tokens=512, max_logit_rows=1, kv=B.KvType.F16))
    try:
        bt = B.Batch(m, max_seqs=NSEQ, num_pages=PREFIX // 16 + NSEQ * 7, max_positions=PREFIX + 96)
        try:
            bt.set_prefix(prefix)
            for sfx in suffixes:
                bt.add_sequence(sfx)
            first = bt.peek_logits()
            ids, _ = bt.decode(steps)
        finally:
            bt.free()
        tol = 5e-3  # projections of a 64-row step are f16-input GEMMs, like a prefill chunk
        flips = 0
        for s, sfx in enumerate(suffixes):
            prompt = np.concatenate([prefix, sfx])
            lg = None
            for off in range(0, prompt.size, 512):
                lg, _ = m.forward(prompt[off:off + 512], off)
            # the token drawn when the sequence was added: the argmax of its prompt's last logits
            scale = np.abs(lg[0]).max()
            top2 = np.sort(lg[0])[-2:]
            assert int(ids[s, 0]) == int(np.argmax(lg[0])) or top2[1] - top2[0] <= 4 * tol * scale, s
            tok = int(ids[s, 0])
            for i in range(steps):  # teacher-forced with the batch's own tokens: every step is compared
                lg, _ = m.forward([tok], prompt.size + i)
                if i == 0:  # the batch's logits for its first decode step, all 64 rows at once
                    assert np.abs(first[s] - lg[0]).max() <= tol * np.abs(lg[0]).max(), s
                got = int(ids[s, i + 1])
                if got != int(np.argmax(lg[0])):
                    top2 = np.sort(lg[0])[-2:]
                    assert lg[0][got] >= top2[1] - 4 * tol * scale, (s, i)  # the tie rule: a flip only inside the tolerance
                    flips += 1
                tok = got
        assert flips <= NSEQ * steps // 50, flips
    finally:
        m.free()


def test_serving_batch_sampled_tokens_follow_the_reference_sampler(B, ctx, group4_model):
    """Temperature 0.7 / top-p 0.95 with one PCG32 stream per sequence: every step's token of every sequence against
    the oracle's Sampler::sample (sampler.rs:60-146) fed the logits the GPU itself produced for that step."""
    prefix, suffixes = serving_prompts()
    steps = 12
    params = B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=100)
    m = B.Qwen3.load(ctx, group4_model, B.Limits(ctx=PREFIX + 192, max_tokens=512, max_logit_rows=1, kv=B.KvType.F16))
    try:
        bt = B.Batch(m, max_seqs=NSEQ, num_pages=PREFIX // 16 + NSEQ * 7, max_positions=PREFIX + 96)
        try:
            bt.set_prefix(prefix)
            for sfx in suffixes:
                bt.add_sequence(sfx, params)
            refs = [O.Sampler(temperature=0.7, top_k=0, top_p=0.95, seed=100 + s) for s in range(NSEQ)]
            for r in refs:
                r.next_f32()  # the draw that chose the sequence's first token when it was added
            agree = total = 0
            for _ in range(steps):
                lg = bt.peek_logits()
                ids, _ = bt.decode(1, params)
                for s in range(NSEQ):
                    want = refs[s].sample(lg[s])
                    total += 1
                    agree += int(ids[s, 1]) == want
        finally:
            bt.free()
        print(f"sampled serving tokens identical to the reference sampler: {agree} of {total}")
        assert agree >= 0.97 * total, (agree, total)
    finally:
        m.free()


# ---- 16k prompt against the reference's own forward -----------------------------------------------------------------

@pytest.fixture(scope="module")
def tiny_long_context(golden_dir, tmp_path_factory):
    """The golden tiny model with `max_position_embeddings` raised to 32 768 in its header: the same tensor bytes (the
    reference's forward, which made the goldens, does not read that field; the loader here enforces it)."""
    from brasa_b200 import tp
    meta, raw = tp.read_container(golden_dir / "tiny" / "model.brasa")
    meta["model"]["config"]["max_position_embeddings"] = 32768
    blobs = {t["name"]: np.array(raw[t["offset"]:t["offset"] + t["nbytes"]]) for t in meta["tensors"]}
    out = tmp_path_factory.mktemp("tiny_long") / "model.brasa"
    tp.write_container(out, meta, blobs)
    return out


@pytest.mark.parametrize("kv", ["F16", "Q8_0"])
def test_16k_prompt_in_bench_chunks_against_reference_goldens(B, ctx, golden_dir, tiny_long_context, kv):
    g = np.load(golden_dir / "tiny" / f"ref_long_{kv.lower()}.npz")
    prompt = g["prompt"].astype(np.uint32)
    n = prompt.size
    assert n == 16384
    tol = max(LOGIT_TOL[kv], F16_PREFILL_FLOOR)
    m = B.Qwen3.load(ctx, tiny_long_context, B.Limits(ctx=n + 64, max_tokens=3584, max_logit_rows=1, kv=B.KvType[kv]))
    try:
        lg = None
        for off in range(0, n, 3584):
            lg, _ = m.forward(prompt[off:off + 3584], off)
        assert rel(lg[0], g["prefill_last_logits"]) <= tol
        scale = np.abs(g["prefill_last_logits"]).max()
        tok = int(g["greedy"][0])
        top2 = np.sort(g["prefill_last_logits"])[-2:]
        assert int(np.argmax(lg[0])) == tok or top2[1] - top2[0] <= 4 * tol * scale
        for i in range(8):  # teacher-forced with the reference's tokens (forward.rs:131-138)
            tok = int(g["greedy"][i])
            lg, _ = m.forward([tok], n + i)
            want = g["decode_logits"][i]
            assert rel(lg[0], want) <= tol, i
            top2 = np.sort(want)[-2:]
            assert int(np.argmax(lg[0])) == int(np.argmax(want)) or top2[1] - top2[0] <= 4 * tol * np.abs(want).max(), i
        # the device-resident greedy loop over the same cache gives the session's tokens
        for off in range(0, n, 3584):
            m.forward(prompt[off:off + 3584], off, want_logits=False)
        dev, _ = m.decode_greedy(int(g["greedy"][0]), n, 7)
        mismatch = [i for i in range(7) if int(dev[i]) != int(g["greedy"][i + 1])]
        if mismatch:  # only a near tie may differ, and then the continuation is another sequence: stop comparing there
            i = mismatch[0]
            top2 = np.sort(g["decode_logits"][i])[-2:]
            assert top2[1] - top2[0] <= 4 * tol * np.abs(g["decode_logits"][i]).max(), i
    finally:
        m.free()


# ---- decode beyond 8 192 positions, both decode paths, GQA groups 2 and 8 -------------------------------------------

@pytest.mark.parametrize("heads,kv_heads", [(4, 2), (8, 1)])
@pytest.mark.parametrize("token_kernel", ["1", "0"])
def test_decode_past_8192_positions_on_both_decode_paths(B, tmp_path, heads, kv_heads, token_kernel):
    """Prefill 8 300 tokens on the GPU, hand the GPU's own f16 cache to the oracle, then compare four decode steps:
    whatever the decode path (BRASA_TOKEN_KERNEL=1: one kernel per token; 0: one kernel per operation with the fused
    attention that merges its 65 chunks of 128 keys), logits must match the oracle's decode over the same cache within
    the reference's bound for an f16 cache."""
    cfg = BF.tiny_config(layers=2, hidden=256, heads=heads, kv_heads=kv_heads, ffn=512, vocab=512, max_pos=16384)
    path = tmp_path / "model.brasa"
    BF.write_brasa(path, cfg, BF.synth_weights(cfg, seed=heads, std=0.05, norm_jitter=0.1))
    n, steps = 8300, 4
    prompt = np.random.default_rng(heads).integers(0, 512, n).astype(np.uint32)
    old = os.environ.get("BRASA_TOKEN_KERNEL")
    os.environ["BRASA_TOKEN_KERNEL"] = token_kernel
    try:
        c = B.Context(0)
    finally:
        if old is None:
            os.environ.pop("BRASA_TOKEN_KERNEL", None)
        else:
            os.environ["BRASA_TOKEN_KERNEL"] = old
    try:
        m = B.Qwen3.load(c, path, B.Limits(ctx=n + 64, max_tokens=2048, max_logit_rows=1, kv=B.KvType.F16))
        lg = None
        for off in range(0, n, 2048):
            lg, _ = m.forward(prompt[off:off + 2048], off)
        first = int(np.argmax(lg[0]))
        orc = O.Qwen3Oracle(BF.BrasaFile(path), kv="f16", ctx=n + steps + 1)
        kvd = kv_heads * 128
        for li in range(2):
            orc.k[li, :n] = m.read_kv(li, "k", 0, n).view(np.float16).astype(np.float32).reshape(n, kvd)
            orc.v[li, :n] = m.read_kv(li, "v", 0, n).view(np.float16).astype(np.float32).reshape(n, kvd)
        orc.pos = n
        dev, _ = m.decode_greedy(first, n, steps - 1)  # the device-resident loop: tokens first .. first + steps - 1
        toks = [first] + [int(t) for t in dev]
        want = [orc.forward([t])[0] for t in toks]
        # same tokens through forward(): the logits of every step
        for off in range(0, n, 2048):
            m.forward(prompt[off:off + 2048], off, want_logits=False)
        for i, t in enumerate(toks):
            got, _ = m.forward([t], n + i)
            assert rel(got[0], want[i]) <= 1e-3, (i, rel(got[0], want[i]))  # forward.rs:40-55: the bound for an f16 cache
            if i + 1 < len(toks):
                top2 = np.sort(want[i])[-2:]
                assert toks[i + 1] == int(np.argmax(want[i])) or top2[1] - top2[0] <= 1e-3 * np.abs(want[i]).max(), i
        m.free()
    finally:
        c.close()


# ---- prefill GEMMs at the real matrix sizes --------------------------------------------------------------------------

def tiled_q4(B, ctx, K, raw, rows, cols):
    src, dst = ctx.buffer_from(raw), ctx.buffer(raw.nbytes)
    run(ctx, lambda c: K.repack(c, 0, src, dst, rows, cols))
    src.free()
    return B.QMatrix(dst, B.WeightType.Q4_0, rows, cols, B.Layout.TILED)


def sampled_rows(rows, per_tile):
    """Row indices that touch every 128-row tile (first, last and spread rows of each)."""
    idx = []
    for t0 in range(0, rows, 128):
        idx += sorted({t0, t0 + 127, *(t0 + 1 + (37 * j) % 126 for j in range(per_tile - 2))})
    return np.array(idx)


def take_rows(raw, rows, cols, idx):
    rb = cols // 32 * 18
    return np.ascontiguousarray(raw.reshape(rows, rb)[idx]).reshape(-1)


@pytest.mark.parametrize("rows,cols", [(9728, 2560), (2560, 9728), (4096, 2560), (2560, 4096)])
def test_prefill_gemm_real_shapes_every_block_shape(B, ctx, K, rows, cols):
    """brasa_k_gemm at the 4B model's matrix sizes for the bench's 3 584-token chunk, a 1 024- and 512-token prompt, a
    ragged count and a 64-token serving step: together they select every (token tiles, weight tiles, K split) form of
    the tcgen05 kernel. Every token of sampled rows of every 128-row tile against the oracle's f16-input matmul."""
    rng = O.Rng(rows + cols)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    w = tiled_q4(B, ctx, K, raw, rows, cols)
    idx = sampled_rows(rows, 3 if rows > 4096 else 4)
    sub = take_rows(raw, rows, cols, idx)
    for tokens in (3584, 1024, 512, 333, 64, 37, 9):
        xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
        gx, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
        run(ctx, lambda c: K.gemm(c, w, gx, gy, tokens))
        got = gy.download(np.float32).reshape(tokens, rows)[:, idx]
        want, s = O.matmul(O.Q4_0, sub, idx.size, cols, xh.astype(np.float32), f16_inputs=True)
        assert np.max(np.abs(got - want) / s) <= 1e-5, tokens
        if cols == 9728 or cols == 4096:  # o_proj and down_proj: the residual add in the epilogue gives the same bits + acc
            acc0 = rng.vec(tokens * rows, 2.0)
            ga, gs = ctx.buffer_from(acc0), ctx.buffer(tokens * rows * 4)
            run(ctx, lambda c: K.gemm_add(c, w, gx, ga, gs, tokens))
            both = ga.download(np.float32).reshape(tokens, rows)
            assert np.array_equal(both, gy.download(np.float32).reshape(tokens, rows) + acc0.reshape(tokens, rows)), tokens
            ga.free()
            gs.free()
        gx.free()
        gy.free()


@pytest.mark.parametrize("tokens", [3584, 512, 200, 64, 23])
def test_prefill_gemm_swiglu_real_shape(B, ctx, K, tokens):
    """gate and up of the 4B model (9 728 x 2 560 each) as the one-launch SwiGLU GEMM: sampled rows of every tile."""
    rows, cols = 9728, 2560
    rng = O.Rng(tokens)
    graw, uraw = rng.qmatrix(O.Q4_0, rows, cols), rng.qmatrix(O.Q4_0, rows, cols)
    g, u = tiled_q4(B, ctx, K, graw, rows, cols), tiled_q4(B, ctx, K, uraw, rows, cols)
    idx = sampled_rows(rows, 3)
    xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
    gx = ctx.buffer_from(xh)
    gg, gu = ctx.buffer(tokens * rows * 4), ctx.buffer(tokens * rows * 4)
    go = ctx.buffer(tokens * rows * 2)
    run(ctx, lambda c: K.gemm_swiglu(c, g, u, gx, gg, gu, go, tokens))
    got = go.download(np.uint16, tokens * rows).view(np.float16).astype(np.float32).reshape(tokens, rows)[:, idx]
    wg, sg = O.matmul(O.Q4_0, take_rows(graw, rows, cols, idx), idx.size, cols, xh.astype(np.float32), f16_inputs=True)
    wu, su = O.matmul(O.Q4_0, take_rows(uraw, rows, cols, idx), idx.size, cols, xh.astype(np.float32), f16_inputs=True)
    want = O.swiglu(wg, wu).reshape(tokens, idx.size)
    bound = 1e-5 * (np.abs(wu) * 1.1 * sg + np.abs(wg) * su) + np.abs(want) * 2.0 ** -10 + 1e-7
    assert np.all(np.abs(got - want) <= bound)


@pytest.mark.parametrize("rows,cols,tokens", [(128, 1792, 16), (256, 2816, 40), (128, 3328, 100), (384, 1792, 64)])
def test_gemm_split_k_with_uneven_stage_counts(B, ctx, K, rows, cols, tokens):
    """Few output tiles: the K stages of a tile (cols / 64: 28, 44, 52) are shared by several blocks, and the split
    (3, 5, 6 ways) does not divide them, so the blocks of one tile run different stage counts. Full comparison with the oracle, and a second launch
    right after (the arrival counters must be back at zero)."""
    rng = O.Rng(cols)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    w = tiled_q4(B, ctx, K, raw, rows, cols)
    xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
    gx, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
    want, s = O.matmul(O.Q4_0, raw, rows, cols, xh.astype(np.float32), f16_inputs=True)
    for _ in range(2):
        gy.fill(0xFF)
        run(ctx, lambda c: K.gemm(c, w, gx, gy, tokens))
        got = gy.download(np.float32).reshape(tokens, rows)
        assert np.max(np.abs(got - want) / s) <= 1e-5
