"""Batched decode over the paged KV pool against the single-sequence path: a sequence decoded inside a batch must give
what it gives alone (crates/runtime/tests/session.rs:53-60: prefix reuse never changes the output)."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def B():
    import brasa_b200
    return brasa_b200


def alone(B, ctx, path, kvt, prompt, steps, ctx_len=256):
    """Greedy decode of one sequence through the single-sequence model: (logits per step, tokens)."""
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=ctx_len, max_tokens=64, max_logit_rows=1, kv=kvt))
    try:
        lg = None
        for off in range(0, len(prompt), 64):
            lg, _ = m.forward(prompt[off:off + 64], off)
        tok = int(np.argmax(lg[0]))
        toks, logits = [tok], []
        for i in range(steps):
            lg, _ = m.forward([tok], len(prompt) + i)
            logits.append(lg[0].copy())
            tok = int(np.argmax(lg[0]))
            toks.append(tok)
        return np.stack(logits), toks
    finally:
        m.free()


@pytest.mark.parametrize("kv,nseq", [("f32", 3), ("f16", 3), ("q8_0", 2), ("f16", 12)])
def test_batch_matches_sequences_decoded_alone(B, golden_dir, kv, nseq):
    kvt = {"f32": B.KvType.F32, "f16": B.KvType.F16, "q8_0": B.KvType.Q8_0}[kv]
    path = golden_dir / "tiny" / "model.brasa"
    rng = np.random.default_rng(31)
    prefix = rng.integers(0, 512, 32).astype(np.uint32)
    suffixes = [rng.integers(0, 512, int(n)).astype(np.uint32) for n in rng.integers(1, 40, nseq)]
    steps = 20
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=kvt))
    bt = B.Batch(m, max_seqs=nseq, num_pages=2 + nseq * 8, max_positions=128)
    try:
        bt.set_prefix(prefix)
        for sfx in suffixes:
            bt.add_sequence(sfx)
        assert bt.sequences == nseq and bt.pages_in_use == 2 + nseq * 6
        first = bt.peek_logits()
        ids, secs = bt.decode(steps)
        assert secs > 0 and ids.shape == (nseq, steps + 1)
    finally:
        bt.free()
        m.free()
    # above 8 sequences the projections are f16-input GEMMs, like a prefill chunk: the looser bound of that precision
    tol = {"f32": 1e-4, "f16": 1e-3, "q8_0": 2e-2}[kv] if nseq <= 8 else 5e-3
    for s, sfx in enumerate(suffixes):
        want_logits, want_toks = alone(B, ctx, path, kvt, np.concatenate([prefix, sfx]), steps)
        scale = np.abs(want_logits[0]).max()
        assert ids[s, 0] == want_toks[0]
        assert np.abs(first[s] - want_logits[0]).max() <= tol * scale
        # same tokens as long as the margin between the two best logits is clear of the tolerance
        for i in range(steps):
            if int(ids[s, i + 1]) != want_toks[i + 1]:
                top2 = np.sort(want_logits[i])[-2:]
                assert top2[1] - top2[0] <= 4 * tol * scale, (s, i)
                break


@pytest.mark.parametrize("nseq,prefix_len", [(5, 256), (9, 144)])
def test_batch_with_a_long_shared_prefix(B, golden_dir, nseq, prefix_len):
    """A prefix of several 128-key chunks: those chunks are served by blocks that take the heads of four sequences at
    once (the shared K and V tiles are fetched once per group); an odd sequence count leaves the last group ragged and
    a prefix that is not a multiple of 128 leaves its tail to the per-sequence blocks. Same bounds as above."""
    path = golden_dir / "tiny" / "model.brasa"
    rng = np.random.default_rng(57)
    prefix = rng.integers(0, 512, prefix_len).astype(np.uint32)
    suffixes = [rng.integers(0, 512, int(n)).astype(np.uint32) for n in rng.integers(1, 30, nseq)]
    steps = 12
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=512, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
    bt = B.Batch(m, max_seqs=nseq, num_pages=prefix_len // 16 + nseq * 4, max_positions=prefix_len + 64)
    try:
        bt.set_prefix(prefix)
        for sfx in suffixes:
            bt.add_sequence(sfx)
        first = bt.peek_logits()
        ids, _ = bt.decode(steps)
    finally:
        bt.free()
        m.free()
    tol = 1e-3 if nseq <= 8 else 5e-3
    for s, sfx in enumerate(suffixes):
        want_logits, want_toks = alone(B, ctx, path, B.KvType.F16, np.concatenate([prefix, sfx]), steps, ctx_len=512)
        scale = np.abs(want_logits[0]).max()
        assert ids[s, 0] == want_toks[0]
        assert np.abs(first[s] - want_logits[0]).max() <= tol * scale
        for i in range(steps):
            if int(ids[s, i + 1]) != want_toks[i + 1]:
                top2 = np.sort(want_logits[i])[-2:]
                assert top2[1] - top2[0] <= 4 * tol * scale, (s, i)
                break


def test_batch_sampling_uses_one_stream_per_sequence(B, golden_dir):
    """The first token of sequence i is drawn from its prompt's last logits with Pcg32(seed + i), exactly like the
    oracle's sampler on the same logits."""
    path = golden_dir / "tiny" / "model.brasa"
    rng = np.random.default_rng(5)
    prefix = rng.integers(0, 512, 16).astype(np.uint32)
    suffixes = [rng.integers(0, 512, 9).astype(np.uint32) for _ in range(4)]
    params = B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=100)
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=128, max_tokens=32, max_logit_rows=1, kv=B.KvType.F32))
    m.set_prefill_precision(B.PrefillPrecision.F32)
    bt = B.Batch(m, max_seqs=4, num_pages=40, max_positions=64)
    try:
        bt.set_prefix(prefix)
        for sfx in suffixes:
            bt.add_sequence(sfx, params)
        ids, _ = bt.decode(6, params)
        again = None
    finally:
        bt.free()
    try:
        for i, sfx in enumerate(suffixes):
            lg, _ = m.forward(np.concatenate([prefix, sfx]), 0)
            assert O.Sampler(temperature=0.7, top_k=0, top_p=0.95, seed=100 + i).sample(lg[0]) == int(ids[i, 0])
        assert len({tuple(r) for r in ids.tolist()}) > 1  # different prompts and streams give different continuations
    finally:
        m.free()


def test_batch_rejects_what_does_not_fit(B, golden_dir):
    path = golden_dir / "tiny" / "model.brasa"
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=128, max_tokens=32, max_logit_rows=1, kv=B.KvType.F16))
    try:
        with pytest.raises(B.BrasaError):
            B.Batch(m, max_seqs=33, num_pages=8, max_positions=64)  # more sequences than the workspace holds
        bt = B.Batch(m, max_seqs=2, num_pages=5, max_positions=64)
        with pytest.raises(B.BrasaError):
            bt.set_prefix(np.arange(10, dtype=np.uint32))  # not whole pages
        bt.set_prefix(np.arange(16, dtype=np.uint32))
        bt.add_sequence(np.arange(3, dtype=np.uint32))
        with pytest.raises(B.BrasaError):
            bt.add_sequence(np.arange(3, dtype=np.uint32))  # pages exhausted: 1 shared + 3 own, 5 in all
        with pytest.raises(B.BrasaError):
            bt.decode(64)  # would pass max_positions
        bt.free()
    finally:
        m.free()


def test_prefix_cache_finds_pages_of_earlier_sequences(B, golden_dir):
    """No prefix is declared. Sequences that happen to start alike share the pages an earlier one computed: a whole
    branch (A, then A + B), a fork inside it (A + C), an unrelated prompt, and a prompt given twice (everything but the
    page of its last token is served from the cache). The invariant of crates/runtime/tests/session.rs:53-60: tokens
    and logits are what each sequence gives alone, where nothing is reused."""
    path = golden_dir / "tiny" / "model.brasa"
    rng = np.random.default_rng(77)
    a, b2, c2, other = (rng.integers(0, 512, k).astype(np.uint32) for k in (150, 70, 45, 90))
    prompts = [a, np.concatenate([a, b2]), np.concatenate([a, c2]), other, np.concatenate([a, b2]), np.concatenate([a[:100], c2])]
    # pages of 16 tokens served from the cache: 0; 9 (144 of a); 9; 0; 13 (219 tokens: 13 full pages, the last recomputed); 6 (96 of a[:100])
    want_hits = [0, 144, 144, 0, 208, 96]
    steps = 10
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=512, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
    bt = B.Batch(m, max_seqs=len(prompts), num_pages=len(prompts) * 20, max_positions=320)
    try:
        seen = 0
        for p, w in zip(prompts, want_hits):
            bt.add_sequence(p)
            st = bt.prefix_cache_stats()
            assert st["hit_tokens"] - seen == w, (len(p), st)
            seen = st["hit_tokens"]
        assert st["prefilled_tokens"] == sum(len(p) for p in prompts) - sum(want_hits)
        assert st["common_pages"] == 0  # the unrelated prompt shares nothing with the first
        first = bt.peek_logits()
        ids, _ = bt.decode(steps)
    finally:
        bt.free()
        m.free()
    assert np.array_equal(ids[1], ids[4])  # the same prompt twice: the same continuation, computed or reused
    for s, p in enumerate(prompts):
        want_logits, want_toks = alone(B, ctx, path, B.KvType.F16, p, steps, ctx_len=512)
        scale = np.abs(want_logits[0]).max()
        assert ids[s, 0] == want_toks[0], s
        assert np.abs(first[s] - want_logits[0]).max() <= 1e-3 * scale, s
        for i in range(steps):
            if int(ids[s, i + 1]) != want_toks[i + 1]:
                top2 = np.sort(want_logits[i])[-2:]
                assert top2[1] - top2[0] <= 4e-3 * scale, (s, i)
                break


def test_batch_plan_equals_allocated_and_rejects_what_cannot_fit(B, golden_dir):
    """crates/runtime/tests/planner.rs:59-62 for the paged pool: the plan made before brasa_batch_create equals what it
    allocates; a pool larger than the device is refused with BRASA_EBUDGET before anything is allocated."""
    path = golden_dir / "tiny" / "model.brasa"
    ctx = B.Context(0)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=512, max_tokens=64, max_logit_rows=1, kv=B.KvType.Q8_0))
    try:
        shape, _ = B.model_shape(path)
        bt = B.Batch(m, max_seqs=7, num_pages=150, max_positions=400)
        plan = B.planner.plan_batch(shape, 7, 150, 400, B.KvType.Q8_0)
        assert bt.allocated() == plan["total"]
        bt.free()
        free0, _ = ctx.mem_info()
        with pytest.raises(B.BrasaError) as e:
            B.Batch(m, max_seqs=7, num_pages=2_000_000_000, max_positions=400)
        assert e.value.code == B.EBUDGET
        free1, _ = ctx.mem_info()
        assert abs(free1 - free0) < (64 << 20)
    finally:
        m.free()
