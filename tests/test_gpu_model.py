"""Model and session on the GPU against the oracle and the reference's golden files, following the
reference's model-level protocol (crates/models/tests/{layers,forward}.rs, crates/runtime/tests/
{session,planner}.rs): hidden states by relative L2, last-position logits by max|delta|/max|ref| with
one bound per KV type, teacher-forced top-1 through both the prefill and the decode path with an
explicit tie rule, greedy continuation, prefix reuse and chunking invariants, plan == allocated."""

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF

pytestmark = pytest.mark.gpu

# crates/models/tests/forward.rs:40-55: logits bound per KV type (f32, f16, q8_0), and the floor
# that applies when the prefill runs with f16 inputs.
LOGIT_TOL = {"F32": 1e-4, "F16": 1e-3, "Q8_0": 2e-2}
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
def mid_model(tmp_path_factory):
    """3 layers, hidden 512, 8 query heads over 2 KV heads (GQA group 4, like Qwen3-4B), written with
    the oracle's quantisers."""
    d = tmp_path_factory.mktemp("mid")
    cfg = BF.tiny_config(layers=3, hidden=512, heads=8, kv_heads=2, ffn=1536, vocab=1024)
    BF.write_brasa(d / "model.brasa", cfg, BF.synth_weights(cfg, seed=11, std=0.04, norm_jitter=0.1))
    return d / "model.brasa"


def rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
def test_tiny_model_against_reference_goldens(B, ctx, golden_dir, kv):
    path = golden_dir / "tiny" / "model.brasa"
    g = np.load(golden_dir / "tiny" / f"ref_{kv.lower()}.npz")
    prompt = g["prompt"]
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=64, max_tokens=32, max_logit_rows=32, kv=B.KvType[kv]))
    try:
        tol = LOGIT_TOL[kv]
        # exact prefill (f32 inputs)
        m.set_prefill_precision(B.PrefillPrecision.F32)
        logits, secs = m.forward(prompt, 0, logit_rows=prompt.size)
        assert secs > 0
        assert rel(logits, g["prefill_logits"]) <= tol
        nxt = int(np.argmax(logits[-1]))
        for step in range(8):
            assert nxt == int(g["greedy"][step])
            lg, _ = m.forward([nxt], prompt.size + step)
            assert rel(lg[0], g["decode_logits"][step]) <= tol
            nxt = int(np.argmax(lg[0]))
        # hot path: f16 GEMM inputs and Q in the attention
        m.set_prefill_precision(B.PrefillPrecision.F16)
        logits16, _ = m.forward(prompt, 0, logit_rows=1)
        assert rel(logits16[0], g["prefill_logits"][-1]) <= max(tol, F16_PREFILL_FLOOR)
        # chunked prefill: 16 + 8
        m.forward(prompt[:16], 0, want_logits=False)
        tail, _ = m.forward(prompt[16:], 16, logit_rows=8)
        assert rel(tail, g["chunked_tail_logits"]) <= max(tol, F16_PREFILL_FLOOR)
    finally:
        m.free()


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
def test_hidden_states_and_kv_cache_against_oracle(B, ctx, mid_model, kv):
    f = BF.BrasaFile(mid_model)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, 1024, size=40).astype(np.uint32)
    orc = O.Qwen3Oracle(f, kv=kv.lower(), ctx=64)
    want_logits, hid = orc.forward(prompt, logit_rows=1, capture_hidden=True)
    emb = O.embed(O.Q6_0, f.raw("model.embed_tokens.weight"), 512, prompt)
    m = B.Qwen3.load(ctx, mid_model, B.Limits(ctx=64, max_tokens=64, max_logit_rows=4, kv=B.KvType[kv]))
    try:
        m.set_prefill_precision(B.PrefillPrecision.F32)
        # crates/models/tests/layers.rs:81-82 bounds (KV f32); a rounded cache moves a few values by one step
        slack = 1.0 if kv == "F32" else 20.0
        x0 = m.run_layers(emb, 0, range(0, 1))
        assert rel_l2(x0, hid[0].ravel()) <= 1e-5 * slack
        xl = m.run_layers(emb, 0, range(0, 3))
        assert rel_l2(xl, hid[2].ravel()) <= 1e-4 * slack
        # the cache written by the GPU holds the same codes as the oracle's, up to rounding flips
        kvd = 2 * 128
        raw = m.read_kv(0, "k", 0, prompt.size)
        if kv == "F32":
            got = raw.view(np.float32)
        elif kv == "F16":
            got = raw.view(np.float16).astype(np.float32)
        else:
            got = O.dequantize_kv_q8(raw)
        want = orc.k[0, :prompt.size].ravel()
        flips = got != want
        assert got.size == prompt.size * kvd
        if kv == "F32":
            assert rel(got, want) <= 1e-5
        else:
            assert flips.mean() <= 0.01 and np.all(np.abs(got - want)[flips] <= np.abs(want[flips]) * 2.0 ** -6 + 1e-6)
        # one decode token through the fused decode path against the oracle's next step
        lg, _ = m.forward(prompt, 0, logit_rows=1)
        assert rel(lg[0], want_logits[0]) <= LOGIT_TOL[kv]
        nxt = int(np.argmax(lg[0]))
        dec, _ = m.forward([nxt], prompt.size)
        want_dec = orc.forward([nxt])
        assert rel(dec[0], want_dec[0]) <= LOGIT_TOL[kv]
        # single-token run_layers takes the fused decode order: same hidden state as the oracle's
        emb1 = O.embed(O.Q6_0, f.raw("model.embed_tokens.weight"), 512, [nxt])
        orc2 = O.Qwen3Oracle(f, kv=kv.lower(), ctx=64)
        orc2.forward(prompt)
        _, hid1 = orc2.forward([nxt], capture_hidden=True)
        m.forward(prompt, 0, want_logits=False)
        x1 = m.run_layers(emb1, prompt.size, range(0, 3))
        assert rel_l2(x1, hid1[2].ravel()) <= (1e-4 if kv == "F32" else 5e-3)
    finally:
        m.free()


def test_f16_prefill_matches_oracle_f16_mode(B, ctx, mid_model):
    f = BF.BrasaFile(mid_model)
    rng = np.random.default_rng(6)
    prompt = rng.integers(0, 1024, size=48).astype(np.uint32)
    orc = O.Qwen3Oracle(f, kv="f16", ctx=64)
    want = orc.forward(prompt, logit_rows=1, f16_prefill=True)
    exact = O.Qwen3Oracle(f, kv="f16", ctx=64).forward(prompt, logit_rows=1)
    m = B.Qwen3.load(ctx, mid_model, B.Limits(ctx=64, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
    try:
        got, _ = m.forward(prompt, 0)
        assert rel(got[0], want[0]) <= 1e-3      # same rounding points, f32 against f64 accumulation
        assert rel(got[0], exact[0]) <= F16_PREFILL_FLOOR + 1e-3
    finally:
        m.free()


@pytest.mark.parametrize("kv", ["F16", "Q8_0"])
def test_teacher_forced_top1_prefill_and_decode(B, ctx, mid_model, kv):
    """Top-1 at every position must equal the oracle's, through the prefill path (all rows at once)
    and through the decode path (one token at a time). Tie rule (crates/models/tests/forward.rs:
    131-138): a mismatch counts only if the oracle's top-1/top-2 gap exceeds twice the logit bound."""
    f = BF.BrasaFile(mid_model)
    rng = np.random.default_rng(8)
    ids = rng.integers(0, 1024, size=48).astype(np.uint32)
    orc = O.Qwen3Oracle(f, kv=kv.lower(), ctx=64)
    want = orc.forward(ids, logit_rows=ids.size)
    m = B.Qwen3.load(ctx, mid_model, B.Limits(ctx=64, max_tokens=64, max_logit_rows=64, kv=B.KvType[kv]))
    try:
        m.set_prefill_precision(B.PrefillPrecision.F32)
        pre, _ = m.forward(ids, 0, logit_rows=ids.size)
        dec = np.stack([m.forward([int(t)], i)[0][0] for i, t in enumerate(ids)])
        bound = LOGIT_TOL[kv] * np.abs(want).max()
        for name, got in (("prefill", pre), ("decode", dec)):
            assert rel(got, want) <= LOGIT_TOL[kv], name
            top = np.argmax(want, axis=1)
            srt = np.sort(want, axis=1)
            gap = srt[:, -1] - srt[:, -2]
            bad = (np.argmax(got, axis=1) != top) & (gap > 2 * bound)
            assert not bad.any(), (name, np.nonzero(bad)[0])
    finally:
        m.free()


def test_session_generate_greedy_reuse_chunking_and_stops(B, ctx, golden_dir):
    path = golden_dir / "tiny" / "model.brasa"
    g = np.load(golden_dir / "tiny" / "ref_f16.npz")
    prompt = g["prompt"]
    s = B.Session(ctx, path, B.Limits(ctx=64, max_tokens=32, max_logit_rows=1, kv=B.KvType.F16))
    try:
        s.model.set_prefill_precision(B.PrefillPrecision.F32)
        ids, st = s.generate(prompt, 8)
        assert list(ids) == list(g["greedy"])
        assert (st.prompt_tokens, st.reused_tokens, st.generated, st.stop) == (24, 0, 8, "MaxTokens")
        assert st.prefill_ms > 0 and st.ttft_ms >= st.prefill_ms and st.decode_ms > 0 and st.decode_tok_s() > 0
        # same prompt again: everything but the last prompt token is reused, output unchanged
        ids2, st2 = s.generate(prompt, 8)
        assert list(ids2) == list(ids) and st2.reused_tokens == 23
        # a prompt that extends the conversation reuses the common prefix
        longer = np.concatenate([prompt, ids[:3]])
        ids3, st3 = s.generate(longer, 5)
        assert st3.reused_tokens == 26 and list(ids3) == list(ids[3:8])
        # diverging prompt: only the common part is reused
        other = prompt.copy()
        other[10] = (other[10] + 1) % 512
        _, st4 = s.generate(other, 2)
        assert st4.reused_tokens == 10
        s.reset()
        _, st5 = s.generate(prompt, 1)
        assert st5.reused_tokens == 0
        # stop ids end the generation and are reported; ignore_stop masks them out of the logits
        s.reset()
        s.set_stop_ids([int(ids[2])])
        ids6, st6 = s.generate(prompt, 8)
        assert st6.stop == "Stop" and list(ids6) == list(ids[:3])
        s.reset()
        s.set_stop_ids([int(ids[2])], ignore_stop=True)
        ids7, st7 = s.generate(prompt, 8)
        assert st7.stop == "MaxTokens" and int(ids[2]) not in ids7 and list(ids7[:2]) == list(ids[:2])
        s.set_stop_ids([])
        # cancellation from the callback
        s.reset()
        seen = []
        ids8, st8 = s.generate(prompt, 8, on_token=lambda t: (seen.append(t), len(seen) < 3)[1])
        assert st8.stop == "Cancelled" and len(ids8) == 3
        # context full
        s.reset()
        _, st9 = s.generate(prompt, 100)
        assert st9.stop == "ContextFull" and st9.generated == 64 - 24 + 1
        # error paths
        with pytest.raises(B.BrasaError):
            s.generate([], 1)
        with pytest.raises(B.BrasaError):
            s.generate(np.zeros(64, np.uint32), 1)
    finally:
        s.free()
    # chunked prefill (8 tokens per forward) produces the same continuation
    s = B.Session(ctx, path, B.Limits(ctx=64, max_tokens=8, max_logit_rows=1, kv=B.KvType.F16))
    try:
        idc, _ = s.generate(prompt, 8)
        assert list(idc) == list(g["greedy"])
    finally:
        s.free()


def test_device_resident_decode_equals_session(B, ctx, mid_model):
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, 1024, size=20).astype(np.uint32)
    s = B.Session(ctx, mid_model, B.Limits(ctx=96, max_tokens=32, max_logit_rows=1, kv=B.KvType.F16))
    try:
        ids, _ = s.generate(prompt, 24)
        # replay: prefill again, then let the device feed itself
        m = s.model
        m.forward(prompt, 0, want_logits=False)
        dev, secs = m.decode_greedy(int(ids[0]), prompt.size, 23)
        assert secs > 0 and list(dev) == list(ids[1:])
    finally:
        s.free()


def test_sampling_session_matches_oracle_sampler(B, ctx, mid_model):
    f = BF.BrasaFile(mid_model)
    rng = np.random.default_rng(10)
    prompt = rng.integers(0, 1024, size=12).astype(np.uint32)
    s = B.Session(ctx, mid_model, B.Limits(ctx=64, max_tokens=32, max_logit_rows=1, kv=B.KvType.F32))
    try:
        s.model.set_prefill_precision(B.PrefillPrecision.F32)
        params = B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=1234)
        a, _ = s.generate(prompt, 10, params)
        s.reset()
        b, _ = s.generate(prompt, 10, params)
        assert list(a) == list(b)
        s.reset()
        c, _ = s.generate(prompt, 10, B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=99))
        assert list(a) != list(c)
        # teacher-forced: with the GPU's own logits, the oracle sampler picks the same tokens
        smp = O.Sampler(temperature=0.7, top_k=0, top_p=0.95, seed=1234)
        m = s.model
        lg, _ = m.forward(prompt, 0)
        pos = prompt.size
        for tok in a:
            assert smp.sample(lg[0]) == int(tok)
            lg, _ = m.forward([int(tok)], pos)
            pos += 1
    finally:
        s.free()


def test_plan_equals_allocated_and_rejection_loads_nothing(B, ctx, mid_model):
    shape, cfg = B.model_shape(mid_model)
    lim = B.Limits(ctx=300, max_tokens=64, max_logit_rows=2, kv=B.KvType.Q8_0)
    plan = B.planner.plan(shape, lim)
    m = B.Qwen3.load(ctx, mid_model, lim)
    try:
        a = m.allocated()
        assert a["weights"] == plan["weights"] and a["kv"] == plan["kv"] and a["workspace"] == plan["workspace"]
    finally:
        m.free()
    ctx.sync()
    free0, _ = ctx.mem_info()
    with pytest.raises(B.BrasaError) as e:
        B.Session.load_with_budget(ctx, mid_model, lim, budget=plan["total"] - 1)
    assert e.value.code == B.EBUDGET and "context that fits" in str(e.value)
    free1, _ = ctx.mem_info()
    assert free1 >= free0
    ok, _, mx = B.planner.check(ctx, shape, lim)   # budget from the device's free memory
    assert ok and mx == 300
    with pytest.raises(B.BrasaError):
        B.Qwen3.load(ctx, mid_model, B.Limits(ctx=10_000, max_tokens=8, max_logit_rows=1))  # beyond max_position
    with pytest.raises(B.BrasaError):
        m2 = B.Qwen3.load(ctx, mid_model, B.Limits(ctx=64, max_tokens=8, max_logit_rows=1))
        try:
            m2.forward(np.arange(9, dtype=np.uint32), 0)
        finally:
            m2.free()


@pytest.mark.gpu
@pytest.mark.parametrize("kv", ["f32", "f16", "q8_0"])
def test_token_kernel_matches_kernel_per_operation_path(kv, monkeypatch, golden_dir):
    """The whole-token decode kernel and the kernel-per-operation decode path give the same logits within the model
    tolerance of crates/models/tests/forward.rs:40-55, and the same greedy tokens up to ties within it, over positions
    that cross the attention chunk boundaries (32 / 64 keys) and need the per-head merge."""
    import brasa_b200 as B
    kvt = {"f32": B.KvType.F32, "f16": B.KvType.F16, "q8_0": B.KvType.Q8_0}[kv]
    tol = {"f32": 1e-4, "f16": 1e-3, "q8_0": 2e-2}[kv]
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, 512, 30)]
    steps = 110
    runs = {}
    # The two paths round the GEMV input differently for f16 and q8_0 caches (22-bit against 16-bit fixed point), so a
    # near tie may send their greedy choices apart. The second path is therefore fed the first one's tokens: every
    # position stays comparable, and where the choices differ the two candidates must be a tie within the tolerance.
    fed = None
    for mode in ("0", "1"):
        monkeypatch.setenv("BRASA_TOKEN_KERNEL", mode)
        ctx = B.Context(0)
        m = B.Qwen3.load(ctx, golden_dir / "tiny" / "model.brasa", B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=kvt))
        lg, _ = m.forward(prompt, 0)
        tok = int(np.argmax(lg[0]))
        logits, toks = [], []
        for i in range(steps):
            lg, _ = m.forward([tok], len(prompt) + i)
            logits.append(lg[0].copy())
            toks.append(int(np.argmax(lg[0])))
            tok = toks[-1] if fed is None else fed[i]
        if fed is None:
            fed = toks
        m.forward(prompt, 0, want_logits=False)
        out, _ = m.decode_greedy(fed[0], len(prompt) + 1, 16)
        runs[mode] = (np.stack(logits), toks, [int(t) for t in out])
    (la, ta, ra), (lb, tb, rb) = runs["0"], runs["1"]
    scale = np.abs(la).max()
    assert np.abs(la - lb).max() <= tol * scale
    for i, (a, b) in enumerate(zip(ta, tb)):
        if a != b:
            assert abs(la[i][a] - la[i][b]) <= 2 * tol * scale, f"token {i}: {a} vs {b}"
    assert len(ra) == len(rb) == 16


@pytest.mark.gpu
def test_token_kernel_long_cache_groups_chunks(monkeypatch, golden_dir):
    """Past (SMs / kv heads) attention chunks a block of the whole-token kernel walks several chunks with a running
    maximum and sum: 2 700 positions of an f32 cache (32-key chunks, 2 kv heads) are well beyond that point. Logits must
    match the kernel-per-operation path within the f32-cache tolerance of crates/models/tests/forward.rs:40-55."""
    import brasa_b200 as B
    n_prompt, steps = 2700, 5
    prompt = np.random.default_rng(8).integers(0, 512, n_prompt).astype(np.uint32)
    runs = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("BRASA_TOKEN_KERNEL", mode)
        ctx = B.Context(0)
        m = B.Qwen3.load(ctx, golden_dir / "tiny" / "model.brasa", B.Limits(ctx=2816, max_tokens=128, max_logit_rows=1, kv=B.KvType.F32))
        m.set_prefill_precision(B.PrefillPrecision.F32)
        lg = None
        for off in range(0, n_prompt, 128):
            lg, _ = m.forward(prompt[off:off + 128], off)
        tok = int(np.argmax(lg[0]))
        logits = []
        for i in range(steps):
            lg, _ = m.forward([tok], n_prompt + i)
            logits.append(lg[0].copy())
            tok = int(np.argmax(lg[0]))
        runs[mode] = np.stack(logits)
        m.free()
    a, b = runs["0"], runs["1"]
    assert np.abs(a - b).max() <= 1e-4 * np.abs(a).max()
