"""CUDA kernels against the CPU oracle, through the C ABI, on the reference's own test shapes, seeds
and tolerances (crates/kernels/tests/{ops,attention,fused,elementwise}.rs; tolerances from
crates/kernels/src/lib.rs:7-15). Integer and byte outputs must match bit for bit."""

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


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


QT = {"q4_0": (O.Q4_0, 0), "q8_0": (O.Q8_0, 1), "q6_0": (O.Q6_0, 2)}  # oracle id, ABI id


def tiled(B, ctx, K, name, raw, rows, cols):
    src = ctx.buffer_from(raw)
    dst = ctx.buffer(raw.nbytes)
    run(ctx, lambda c: K.repack(c, QT[name][1], src, dst, rows, cols))
    return B.QMatrix(dst, B.WeightType(QT[name][1]), rows, cols, B.Layout.TILED), dst


# ---- layout and converter ------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["q4_0", "q6_0"])
def test_repack_is_a_bijection(B, ctx, K, name):
    rows, cols = 100, 512
    raw = O.Rng(5).qmatrix(QT[name][0], rows, cols)
    _, t = tiled(B, ctx, K, name, raw, rows, cols)
    packed = t.download(np.uint8)
    assert packed.size == raw.size and not np.array_equal(packed, raw)
    back = ctx.buffer(raw.nbytes)
    run(ctx, lambda c: K.unpack(c, QT[name][1], t, back, rows, cols))
    assert np.array_equal(back.download(np.uint8), raw)
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.repack(c, QT[name][1], t, back, rows, 100))


@pytest.mark.parametrize("name", ["q4_0", "q6_0", "q8_0"])
def test_quantize_and_dequantize_bit_exact(B, ctx, K, name, golden_dir):
    g = np.load(golden_dir / "quant_cases.npz")
    rng = np.random.default_rng(7)
    w = np.concatenate([g["w"].ravel(), (rng.standard_normal(32 * 4000) * 0.02).astype(np.float32),
                        rng.standard_normal(32 * 500).astype(np.float32) * 50])
    # exact half-way cases for every quantiser
    d = np.float32(0.125)
    w[:32] = (np.arange(32, dtype=np.float32) - 15.5) * d
    src = ctx.buffer_from(w)
    dst = ctx.buffer(O.nbytes(QT[name][0], w.size))
    run(ctx, lambda c: K.quantize(c, QT[name][1], src, dst, w.size))
    got = dst.download(np.uint8)
    want = O.quantize(QT[name][0], w)
    assert np.array_equal(got, want)
    out = ctx.buffer(w.size * 4)
    run(ctx, lambda c: K.dequantize(c, QT[name][1], dst, out, w.size))
    assert np.array_equal(out.download(np.float32).view(np.uint32), O.dequantize(QT[name][0], want, w.size).view(np.uint32))


def test_randn_is_seeded_and_normal(ctx, K):
    n = 1 << 20
    a, b = ctx.buffer(n * 4), ctx.buffer(n * 4)
    run(ctx, lambda c: (K.randn(c, a, n, 42, 0, 0.02), K.randn(c, b, n, 42, 0, 0.02)))
    x, y = a.download(np.float32), b.download(np.float32)
    assert np.array_equal(x, y)
    assert abs(x.mean()) < 1e-4 and abs(x.std() - 0.02) < 2e-4
    run(ctx, lambda c: K.randn(c, b, n, 43, 0, 0.02))
    assert not np.array_equal(x, b.download(np.float32))
    # a later offset continues the same stream
    run(ctx, lambda c: K.randn(c, b, n // 2, 42, n // 4, 0.02))
    assert np.array_equal(b.download(np.float32)[: n // 2], x[n // 2:])


# ---- element-wise --------------------------------------------------------------------------------

def test_add_and_swiglu(B, ctx, K):
    rng = O.Rng(1)
    n = 9728 * 3 + 5
    a, b = rng.vec(n, 4.0), rng.vec(n, 4.0)
    ga, gb, go = ctx.buffer_from(a), ctx.buffer_from(b), ctx.buffer(n * 4)
    run(ctx, lambda c: K.add(c, ga, gb, go, n))
    assert np.array_equal(go.download(np.float32), O.add(a, b))
    run(ctx, lambda c: K.swiglu(c, ga, gb, go, n))
    got, want = go.download(np.float32), O.swiglu(a, b)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) <= 1e-6
    gh = ctx.buffer(n * 2)
    run(ctx, lambda c: K.swiglu_f16(c, ga, gb, gh, n))
    assert np.array_equal(gh.download(np.uint16), O.f32_to_f16_array(got))  # == f16(f32 result), bit for bit
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.add(c, ga, gb, go, n + 1))


@pytest.mark.parametrize("rows,n", [(1, 2560), (37, 2560), (301, 2560), (2048, 128), (3, 100)])
def test_rms_norm(ctx, K, rows, n):
    rng = O.Rng(11)
    x, w = rng.vec(rows * n, 3.0), rng.vec(n, 2.0)
    gx, gw, go, gh = ctx.buffer_from(x), ctx.buffer_from(w), ctx.buffer(rows * n * 4), ctx.buffer(rows * n * 2)
    run(ctx, lambda c: (K.rms_norm(c, gx, gw, go, rows, n, 1e-6), K.rms_norm_f16(c, gx, gw, gh, rows, n, 1e-6)))
    got, want = go.download(np.float32), O.rms_norm(x, w, n, 1e-6)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-6)) <= 1e-5
    assert np.array_equal(gh.download(np.uint16), O.f32_to_f16_array(got))


def test_softmax(ctx, K):
    rng = O.Rng(12)
    for rows, n in [(4, 1000), (32, 129), (1, 16384)]:
        x = rng.vec(rows * n, 8.0)
        gx, go = ctx.buffer_from(x), ctx.buffer(rows * n * 4)
        run(ctx, lambda c: K.softmax(c, gx, go, rows, n))
        got, want = go.download(np.float32), O.softmax(x, n)
        assert np.max(np.abs(got - want) / np.maximum(want, 1e-12)) <= 1e-5


@pytest.mark.parametrize("pos0", [0, 3, 40944])
def test_rope(B, ctx, K, pos0):
    rng = O.Rng(13)
    tokens, heads, dim = 4, 5, 128
    table = B.RopeTable(ctx, 1e6, dim, pos0 + tokens)
    cos, sin = O.rope_table(1e6, dim, pos0 + tokens)
    x = rng.vec(tokens * heads * dim, 2.0)
    gx = ctx.buffer_from(x)
    run(ctx, lambda c: K.rope_neox(c, gx, table, tokens, heads, dim, pos0))
    got, want = gx.download(np.float32), O.rope_neox(x, heads, dim, pos0, cos, sin)
    xv = x.reshape(-1, dim)
    bound = 1e-6 * (np.abs(xv) + np.abs(np.roll(xv, 64, axis=1))).ravel()
    assert np.all(np.abs(got - want) <= bound + 1e-12)
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.rope_neox(c, gx, table, tokens, heads, dim, pos0 + 1))


def test_embed_exact(B, ctx, K):
    rng = O.Rng(14)
    vocab, h = 256, 512
    ids = np.array([0, 255, 17, 17, 128, 64, 63], dtype=np.uint32)
    gi = ctx.buffer_from(ids)
    for name in ("q6_0", "q8_0"):
        raw = rng.qmatrix(QT[name][0], vocab, h)
        want = O.embed(QT[name][0], raw, h, ids)
        out = ctx.buffer(ids.size * h * 4)
        m = B.QMatrix(ctx.buffer_from(raw), B.WeightType(QT[name][1]), vocab, h)
        run(ctx, lambda c: K.embed(c, m, gi, out, ids.size))
        assert np.array_equal(out.download(np.float32).reshape(-1, h), want)
        if name == "q6_0":
            mt, _ = tiled(B, ctx, K, name, raw, vocab, h)
            run(ctx, lambda c: K.embed(c, mt, gi, out, ids.size))
            assert np.array_equal(out.download(np.float32).reshape(-1, h), want)
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.embed(c, B.QMatrix(ctx.buffer(64), B.WeightType.Q4_0, 2, 32), gi, out, 1))


def test_add_norm_prep(B, ctx, K):
    rng = O.Rng(15)
    n = 2560
    x, h, w = rng.vec(n, 3.0), rng.vec(n, 1.0), rng.vec(n, 2.0)
    for add in (False, True):
        gx, gh, gw = ctx.buffer_from(x), ctx.buffer_from(h), ctx.buffer_from(w)
        gxw, gss = ctx.buffer(n * 4), ctx.buffer(B.norm_partials(n) * 4)
        run(ctx, lambda c: K.add_norm_prep(c, gx, gh if add else None, gw, gxw, gss, n))
        xs = (x + h) if add else x
        assert np.array_equal(gx.download(np.float32), xs)
        assert np.array_equal(gxw.download(np.float32), xs * w)
        ss = gss.download(np.float32)
        want = (xs.astype(np.float64) ** 2).reshape(-1, 256).sum(axis=1)
        assert np.max(np.abs(ss - want) / want) <= 1e-6


# ---- GEMV ----------------------------------------------------------------------------------------

GEMV_SHAPES = [(4096, 2560), (9728, 2560), (2560, 9728), (5, 64)]


@pytest.mark.parametrize("name", ["q4_0", "q6_0", "q8_0"])
@pytest.mark.parametrize("rows,cols", GEMV_SHAPES)
def test_gemv_layouts_and_types(B, ctx, K, name, rows, cols):
    rng = O.Rng(16)
    raw = rng.qmatrix(QT[name][0], rows, cols)
    for tokens in (1, 3):
        x = rng.vec(tokens * cols, 1.0)
        want, scale = O.matmul(QT[name][0], raw, rows, cols, x)
        gx, gy = ctx.buffer_from(x), ctx.buffer(tokens * rows * 4)
        m = B.QMatrix(ctx.buffer_from(raw), B.WeightType(QT[name][1]), rows, cols)
        for fn in (K.gemv, K.gemv_simple):
            gy.fill(0xFF)
            run(ctx, lambda c: fn(c, m, gx, gy, tokens))
            got = gy.download(np.float32).reshape(tokens, rows)
            assert np.max(np.abs(got - want) / scale) <= 1e-5, (name, fn.__name__)
        if name != "q8_0" and cols % 256 == 0:
            mt, _ = tiled(B, ctx, K, name, raw, rows, cols)
            gy.fill(0xFF)
            run(ctx, lambda c: K.gemv(c, mt, gx, gy, tokens))
            got = gy.download(np.float32).reshape(tokens, rows)
            assert np.max(np.abs(got - want) / scale) <= 1e-5, (name, "tiled")
            # the split-K reduction has a fixed order: same bits on every run
            run(ctx, lambda c: K.gemv(c, mt, gx, gy, tokens))
            assert np.array_equal(gy.download(np.float32).reshape(tokens, rows), got)


def test_gemv_config1_shape_with_quantised_gaussian_weights(B, ctx, K):
    """[9728 x 2560] weights ~ N(0, 0.02) through the q4_0 quantiser, x ~ N(0, 1) rounded to f16."""
    rng = np.random.default_rng(2024)
    rows, cols = 9728, 2560
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    raw = O.quantize(O.Q4_0, w)
    x = rng.standard_normal(cols).astype(np.float16).astype(np.float32)
    want, scale = O.matmul(O.Q4_0, raw, rows, cols, x)
    mt, _ = tiled(B, ctx, K, "q4_0", raw, rows, cols)
    gx, gy = ctx.buffer_from(x), ctx.buffer(rows * 4)
    run(ctx, lambda c: K.gemv(c, mt, gx, gy, 1))
    got = gy.download(np.float32)
    err = np.abs(got - want[0])
    assert np.max(err / scale[0]) <= 1e-5
    assert np.max(err) <= 1e-2 and np.max(err / np.maximum(np.abs(want[0]), 1e-2)) <= 1e-3
    # against dequantise-then-matvec in numpy f64, as the configuration describes
    ref = O.dequantize(O.Q4_0, raw, rows * cols).reshape(rows, cols).astype(np.float64) @ x.astype(np.float64)
    assert np.max(np.abs(got - ref)) <= 1e-2


def _norm_inputs(B, ctx, K, rng, cols):
    x, w = rng.vec(cols, 3.0), rng.vec(cols, 1.5)
    gx, gw, gxw, gss = ctx.buffer_from(x), ctx.buffer_from(w), ctx.buffer(cols * 4), ctx.buffer(B.norm_partials(cols) * 4)
    run(ctx, lambda c: K.add_norm_prep(c, gx, None, gw, gxw, gss, cols))
    normed = O.rms_norm(x, w, cols, 1e-6)
    return gxw, gss, normed


@pytest.mark.parametrize("layout", ["file", "tiled"])
def test_gemv_scaled_family(B, ctx, K, layout):
    rng = O.Rng(17)
    cols = 2560

    def mat(name, rows):
        raw = rng.qmatrix(QT[name][0], rows, cols)
        if layout == "tiled":
            return tiled(B, ctx, K, name, raw, rows, cols)[0], raw
        return B.QMatrix(ctx.buffer_from(raw), B.WeightType(QT[name][1]), rows, cols), raw

    gxw, gss, normed = _norm_inputs(B, ctx, K, rng, cols)
    # gemv_scaled: q4_0 and q6_0
    for name, rows in (("q4_0", 4096), ("q6_0", 1024)):
        m, raw = mat(name, rows)
        want, scale = O.matmul(QT[name][0], raw, rows, cols, normed)
        gy = ctx.buffer(rows * 4)
        run(ctx, lambda c: K.gemv_scaled(c, m, gxw, gss, 1e-6, gy))
        assert np.max(np.abs(gy.download(np.float32) - want[0]) / scale[0]) <= 2e-5
    # gemv_scaled3 == three gemv_scaled
    ms = [mat("q4_0", r) for r in (4096, 1024, 1024)]
    ys = [ctx.buffer(r * 4) for r in (4096, 1024, 1024)]
    run(ctx, lambda c: K.gemv_scaled3(c, [m for m, _ in ms], gxw, gss, 1e-6, ys))
    for (m, raw), gy in zip(ms, ys):
        want, scale = O.matmul(O.Q4_0, raw, m.rows, cols, normed)
        got = gy.download(np.float32)
        assert np.max(np.abs(got - want[0]) / scale[0]) <= 2e-5
        single = ctx.buffer(m.rows * 4)
        run(ctx, lambda c: K.gemv_scaled(c, m, gxw, gss, 1e-6, single))
        assert np.array_equal(single.download(np.float32), got)  # same bits fused or not
    # gemv_scaled_swiglu
    (g, graw), (u, uraw) = mat("q4_0", 9728), mat("q4_0", 9728)
    gy = ctx.buffer(9728 * 4)
    run(ctx, lambda c: K.gemv_scaled_swiglu(c, g, u, gxw, gss, 1e-6, gy))
    wg, sg = O.matmul(O.Q4_0, graw, 9728, cols, normed)
    wu, su = O.matmul(O.Q4_0, uraw, 9728, cols, normed)
    want = O.swiglu(wg[0], wu[0])
    got = gy.download(np.float32)
    # error of silu(g)*u from errors in g and u: |u| * (|dsilu| <= 1.1) * eg + |silu(g)| * eu
    bound = 2e-5 * (np.abs(wu[0]) * 1.1 * sg[0] + np.abs(wg[0]) * su[0]) + 1e-6 * np.abs(want)
    assert np.all(np.abs(got - want) <= bound + 1e-9)
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.gemv_scaled_swiglu(c, g, ms[0][0], gxw, gss, 1e-6, gy))


# ---- KV store ------------------------------------------------------------------------------------

def test_store_kv_f32_and_f16(B, ctx, K):
    rng = O.Rng(24)
    x = rng.vec(4099, 50.0)
    mid = np.float32((O.f16_to_f32(0x3C01) + O.f16_to_f32(0x3C02)) / 2.0)
    x[:8] = [mid, -mid, 65520.0, 1e-7, 3e-8, 0.0, -0.0, 70000.0]
    src, d32, d16 = ctx.buffer_from(x), ctx.buffer(x.size * 4), ctx.buffer(x.size * 2)
    run(ctx, lambda c: (K.store_kv(c, B.KvType.F32, src, d32, x.size), K.store_kv(c, B.KvType.F16, src, d16, x.size)))
    assert np.array_equal(d32.download(np.float32).view(np.uint32), x.view(np.uint32))
    assert np.array_equal(d16.download(np.uint16), O.f32_to_f16_array(x))


def test_store_kv_q8_bit_exact(B, ctx, K):
    rng = O.Rng(26)
    x = rng.vec(128 * 64, 20.0)
    x[32:64] = 0.0
    d = np.float32(O.f16_to_f32(O.f32_to_f16(1.0 / 127.0)))
    x[128:160] = (np.arange(32, dtype=np.float32) - np.float32(15.5)) * d  # exact ties
    x[128 + 31] = 1.0
    x[256:288] = 3000.0
    src, dst = ctx.buffer_from(x), ctx.buffer(B.KvType.Q8_0.bytes(x.size))
    run(ctx, lambda c: K.store_kv(c, B.KvType.Q8_0, src, dst, x.size))
    assert np.array_equal(dst.download(np.uint8), O.quantize_kv_q8(x))
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.store_kv(c, B.KvType.Q8_0, src, dst, 100))


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
@pytest.mark.parametrize("tokens,pos0", [(1, 0), (1, 777), (7, 3), (64, 448)])
def test_qk_norm_rope_store(B, ctx, K, kv, tokens, pos0):
    kvt = B.KvType[kv]
    rng = O.Rng(27)
    hq, hkv, dim = 32, 8, 128
    q, k, v = rng.vec(tokens * hq * dim, 2.0), rng.vec(tokens * hkv * dim, 2.0), rng.vec(tokens * hkv * dim, 3.0)
    qn, kn = rng.vec(dim, 1.5), rng.vec(dim, 1.5)
    table = B.RopeTable(ctx, 1e6, dim, pos0 + tokens)
    cos, sin = O.rope_table(1e6, dim, pos0 + tokens)
    gq, gk, gv, gqn, gkn = (ctx.buffer_from(a) for a in (q, k, v, qn, kn))
    cap = pos0 + tokens
    kc, vc = ctx.buffer(kvt.bytes(cap * hkv * dim)), ctx.buffer(kvt.bytes(cap * hkv * dim))
    off = kvt.bytes(pos0 * hkv * dim)
    shape = B.AttnShape(tokens, hq, hkv, dim, pos0, kvt)
    run(ctx, lambda c: K.qk_norm_rope_store(c, kvt, [gq, gk, gv], [gqn, gkn], 1e-6, table, [kc.at(off), vc.at(off)], shape))
    want_q = O.rope_neox(O.rms_norm(q, qn, dim, 1e-6), hq, dim, pos0, cos, sin)
    want_k = O.rope_neox(O.rms_norm(k, kn, dim, 1e-6), hkv, dim, pos0, cos, sin)
    got_q, got_k = gq.download(np.float32), gk.download(np.float32)
    assert np.max(np.abs(got_q - want_q)) <= 2e-5 * np.max(np.abs(want_q))
    assert np.max(np.abs(got_k - want_k)) <= 2e-5 * np.max(np.abs(want_k))
    n = tokens * hkv * dim
    kb, vb = kc.download(np.uint8, kvt.bytes(n), off), vc.download(np.uint8, kvt.bytes(n), off)
    # the cache holds exactly the rounding of the values the kernel produced
    if kvt == B.KvType.F32:
        assert np.array_equal(kb.view(np.float32), got_k) and np.array_equal(vb.view(np.float32), v)
    elif kvt == B.KvType.F16:
        assert np.array_equal(kb.view(np.uint16), O.f32_to_f16_array(got_k))
        assert np.array_equal(vb.view(np.uint16), O.f32_to_f16_array(v))
    else:
        assert np.array_equal(kb, O.quantize_kv_q8(got_k)) and np.array_equal(vb, O.quantize_kv_q8(v))
    # nothing before pos0 was touched
    assert not kc.download(np.uint8, off).any()


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
def test_paged_store_and_decode_attention(B, ctx, K, kv):
    """The kernel-level paged operators: three sequences of different lengths whose 16-position pages lie scattered in
    the pool. The new token's K and V land in the right page in the cache type (exact rounding of what the kernel
    produced), q and k come back normalised and rotated at each sequence's own position, and attention over the page
    tables equals the oracle's attention over each sequence's contiguous rows (1e-5 of max |v|, as the reference's test)."""
    kvt = B.KvType[kv]
    rng = O.Rng(61)
    hq, hkv, dim = 8, 2, 128
    lens = np.array([5, 200, 333], np.uint32)
    seqs, max_pages, num_pages = 3, 24, 80
    perm = np.random.default_rng(3).permutation(num_pages)[:seqs * max_pages].astype(np.int32).reshape(seqs, max_pages)
    row = hkv * dim
    kpool_f = np.zeros((num_pages * 16, row), np.float32)
    vpool_f = np.zeros((num_pages * 16, row), np.float32)
    old_k, old_v = [], []
    for s in range(seqs):
        k, v = rng.vec(int(lens[s]) * row, 2.0).reshape(-1, row), rng.vec(int(lens[s]) * row, 3.0).reshape(-1, row)
        old_k.append(k)
        old_v.append(v)
        for pos in range(int(lens[s])):
            slot = perm[s, pos // 16] * 16 + pos % 16
            kpool_f[slot], vpool_f[slot] = k[pos], v[pos]
    gk, gv, kr, vr = make_cache(B, ctx, kvt, kpool_f.reshape(-1), vpool_f.reshape(-1))  # pools in the cache type + the values they hold
    q, kn_, vn_ = rng.vec(seqs * hq * dim, 2.0), rng.vec(seqs * hkv * dim, 2.0), rng.vec(seqs * hkv * dim, 3.0)
    qn, knorm = rng.vec(dim, 1.5), rng.vec(dim, 1.5)
    table = B.RopeTable(ctx, 1e6, dim, max_pages * 16)
    cos, sin = O.rope_table(1e6, dim, max_pages * 16)
    gq, gkn, gvn, gqn, gknorm = (ctx.buffer_from(a) for a in (q, kn_, vn_, qn, knorm))
    gt, gl = ctx.buffer_from(perm.reshape(-1)), ctx.buffer_from(lens)
    paged = K.paged_kv(gk, gv, gt, gl, seqs, max_pages, num_pages, kvt)
    run(ctx, lambda c: K.qk_norm_rope_store_paged(c, gq, gkn, gvn, gqn, gknorm, 1e-6, table, paged, hq, hkv))
    got_q, got_k = gq.download(np.float32).reshape(seqs, hq * dim), gkn.download(np.float32).reshape(seqs, hkv * dim)
    part = ctx.buffer(seqs * hq * ((max_pages * 16 + 127) // 128) * 130 * 4)
    go = ctx.buffer(seqs * hq * dim * 4)
    run(ctx, lambda c: K.decode_attention_paged(c, gq, paged, part, go, hq, hkv))
    out = go.download(np.float32).reshape(seqs, hq * dim)
    kr, vr = kr.reshape(-1, row), vr.reshape(-1, row)
    for s in range(seqs):
        pos = int(lens[s])
        want_q = O.rope_neox(O.rms_norm(q.reshape(seqs, -1)[s], qn, dim, 1e-6), hq, dim, pos, cos, sin)
        want_k = O.rope_neox(O.rms_norm(kn_.reshape(seqs, -1)[s], knorm, dim, 1e-6), hkv, dim, pos, cos, sin)
        assert np.max(np.abs(got_q[s] - want_q)) <= 2e-5 * np.max(np.abs(want_q))
        assert np.max(np.abs(got_k[s] - want_k)) <= 2e-5 * np.max(np.abs(want_k))
        newk, newv = O.round_kv(int(kvt), got_k[s]), O.round_kv(int(kvt), vn_.reshape(seqs, -1)[s])
        slots = [perm[s, p // 16] * 16 + p % 16 for p in range(pos)]
        kseq = np.concatenate([kr[slots].reshape(-1), newk])
        vseq = np.concatenate([vr[slots].reshape(-1), newv])
        want, vmax = O.attention(got_q[s], kseq, vseq, 1, hq, hkv, dim, pos)
        assert np.max(np.abs(out[s] - want) / np.maximum(vmax, 1e-30)) <= 1e-5, s
    with pytest.raises(B.BrasaError):  # a pool smaller than its page count says
        bad = K.paged_kv(gk, gv, gt, gl, seqs, max_pages, num_pages * 2, kvt)
        run(ctx, lambda c: K.decode_attention_paged(c, gq, bad, part, go, hq, hkv))


# ---- attention -----------------------------------------------------------------------------------

def make_cache(B, ctx, kvt, k, v):
    """Device cache in type kvt and the values the kernel will see (crates/kernels/src/testutil.rs:93-154)."""
    if kvt == B.KvType.F32:
        return ctx.buffer_from(k), ctx.buffer_from(v), k, v
    if kvt == B.KvType.F16:
        kh, vh = k.astype(np.float16), v.astype(np.float16)
        return ctx.buffer_from(kh), ctx.buffer_from(vh), kh.astype(np.float32), vh.astype(np.float32)
    kq, vq = O.quantize_kv_q8(k), O.quantize_kv_q8(v)
    return ctx.buffer_from(kq), ctx.buffer_from(vq), O.dequantize_kv_q8(kq), O.dequantize_kv_q8(vq)


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
@pytest.mark.parametrize("hq", [32, 8, 16, 64])
def test_decode_attention(B, ctx, K, kv, hq):
    kvt = B.KvType[kv]
    rng = O.Rng(23)
    hkv, dim = 8, 128
    positions = [0, 1, 255, 256, 700, 4095, 16383] if hq == 32 else [0, 300, 4095]
    worst = 0.0
    for pos0 in positions:
        lk = pos0 + 1
        q = rng.vec(hq * dim, 2.0)
        gk, gv, k, v = make_cache(B, ctx, kvt, rng.vec(lk * hkv * dim, 2.0), rng.vec(lk * hkv * dim, 3.0))
        want, vmax = O.attention(q, k, v, 1, hq, hkv, dim, pos0)
        gq, go = ctx.buffer_from(q), ctx.buffer(hq * dim * 4)
        part = ctx.buffer(B.decode_partials_len(hq, lk) * 4)
        shape = B.AttnShape(1, hq, hkv, dim, pos0, kvt)
        for fn in (K.decode_attention, K.decode_attention_lanes):
            go.fill(0xFF)
            run(ctx, lambda c: fn(c, gq, gk, gv, part, go, shape))
            got = go.download(np.float32)
            worst = max(worst, float(np.max(np.abs(got - want) / np.maximum(vmax, 1e-30))))
        for b in (gk, gv, gq, go, part):
            b.free()
    assert worst <= 1e-5, worst


def test_decode_attention_rejects_bad_arguments(B, ctx, K):
    q, o = ctx.buffer(32 * 128 * 4), ctx.buffer(32 * 128 * 4)
    k = ctx.buffer(8 * 128 * 4 * 10)
    small = ctx.buffer(16)
    big = ctx.buffer(B.decode_partials_len(32, 10) * 4)
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.decode_attention(c, q, k, k, small, o, B.AttnShape(1, 32, 8, 128, 9, B.KvType.F32)))
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.decode_attention(c, q, k, k, big, o, B.AttnShape(2, 32, 8, 128, 8, B.KvType.F32)))
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.decode_attention(c, q, k, k, big, o, B.AttnShape(1, 32, 8, 64, 9, B.KvType.F32)))
    with pytest.raises(B.BrasaError):
        run(ctx, lambda c: K.decode_attention_lanes(c, q, k, k, big, o, B.AttnShape(1, 24, 8, 128, 9, B.KvType.F32)))


@pytest.mark.parametrize("kv", ["F32", "F16", "Q8_0"])
def test_flash_attention_gqa_causal(B, ctx, K, kv):
    kvt = B.KvType[kv]
    rng = O.Rng(22)
    hq, hkv, dim = 32, 8, 128
    w16 = wraw = w32 = 0.0
    for tokens, pos0 in [(9, 0), (5, 11), (1, 0), (1, 1500), (33, 40), (64, 448), (32, 0), (100, 7)]:
        lk = pos0 + tokens
        cap = (lk + 63) // 64 * 64  # capacity rounded to KV_ALIGN with finite garbage past the range
        q = rng.vec(tokens * hq * dim, 2.0)
        gk, gv, k, v = make_cache(B, ctx, kvt, rng.vec(cap * hkv * dim, 2.0), rng.vec(cap * hkv * dim, 3.0))
        want16, vmax = O.attention(q, k, v, tokens, hq, hkv, dim, pos0, q16=True)
        raw, _ = O.attention(q, k, v, tokens, hq, hkv, dim, pos0)
        gq, go, goh = ctx.buffer_from(q), ctx.buffer(q.size * 4), ctx.buffer(q.size * 2)
        shape = B.AttnShape(tokens, hq, hkv, dim, pos0, kvt)
        run(ctx, lambda c: K.flash_attention(c, gq, gk, gv, goh, shape))
        oh = goh.download(np.float16).astype(np.float32)
        # the final rounding of the output to f16 (at most 2^-11 |value|) is discounted
        d = np.maximum(np.abs(oh - want16) - np.abs(want16) * 2.0 ** -11, 0.0)
        w16 = max(w16, float(np.max(d / np.maximum(vmax, 1e-30))))
        wraw = max(wraw, float(np.max(np.abs(oh - raw) / np.maximum(vmax, 1e-30))))
        run(ctx, lambda c: K.flash_attention_with(c, gq, gk, gv, go, shape, B.PrefillPrecision.F32))
        w32 = max(w32, float(np.max(np.abs(go.download(np.float32) - raw) / np.maximum(vmax, 1e-30))))
    assert w16 <= 1e-5 and w32 <= 1e-5 and wraw <= 2e-3, (w16, w32, wraw)


# ---- prefill GEMM --------------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(4096, 2560), (2560, 9728), (192, 256), (100, 96)])
def test_gemm_f16_and_f32(B, ctx, K, rows, cols):
    rng = O.Rng(18)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    mt, _ = tiled(B, ctx, K, "q4_0", raw, rows, cols) if cols % 256 == 0 else (None, None)
    mf = B.QMatrix(ctx.buffer_from(raw), B.WeightType.Q4_0, rows, cols)
    for tokens in (9, 33, 64, 100, 150):
        x = rng.vec(tokens * cols, 1.0)
        xh = x.astype(np.float16)
        want16, s16 = O.matmul(O.Q4_0, raw, rows, cols, x, f16_inputs=True)
        want32, s32 = O.matmul(O.Q4_0, raw, rows, cols, x)
        gx, gxh, gy = ctx.buffer_from(x), ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
        for m in filter(None, (mf, mt)):
            run(ctx, lambda c: K.gemm(c, m, gxh, gy, tokens))
            got = gy.download(np.float32).reshape(tokens, rows)
            assert np.max(np.abs(got - want16) / s16) <= 1e-5
            assert np.max(np.abs(got - want32) / s32) <= 2.0 ** -10  # f16 inputs against the unrounded product
            run(ctx, lambda c: K.gemm_with(c, m, gx, gy, tokens, B.PrefillPrecision.F32))
            got = gy.download(np.float32).reshape(tokens, rows)
            assert np.max(np.abs(got - want32) / s32) <= 1e-5
        if rows == 4096:
            break  # one token count is enough for the large shapes


@pytest.mark.parametrize("tokens", [40, 70, 300])
def test_gemm_swiglu_equals_unfused(B, ctx, K, tokens):
    """From 128 tokens on gate and up run as one tensor-core launch whose epilogue forms silu(gate) * up; up to 64 tokens
    as one few-token launch whose partial-tile sum forms it; in between, as two GEMMs and the element-wise kernel. All
    must give the bits of the unfused sequence."""
    rng = O.Rng(19)
    rows, cols = 1024, 512
    graw, uraw = rng.qmatrix(O.Q4_0, rows, cols), rng.qmatrix(O.Q4_0, rows, cols)
    g, _ = tiled(B, ctx, K, "q4_0", graw, rows, cols)
    u, _ = tiled(B, ctx, K, "q4_0", uraw, rows, cols)
    xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
    gx = ctx.buffer_from(xh)
    gg, gu, go, go2 = (ctx.buffer(tokens * rows * 4) for _ in range(4))
    run(ctx, lambda c: K.gemm_swiglu(c, g, u, gx, gg, gu, go, tokens))
    fused = go.download(np.uint16, tokens * rows)
    run(ctx, lambda c: (K.gemm_multi(c, [g, u], gx, [gg, gu], tokens, B.PrefillPrecision.F16), K.swiglu_f16(c, gg, gu, go2, tokens * rows)))
    assert np.array_equal(fused, go2.download(np.uint16, tokens * rows))
    wg, sg = O.matmul(O.Q4_0, graw, rows, cols, xh.astype(np.float32), f16_inputs=True)
    wu, su = O.matmul(O.Q4_0, uraw, rows, cols, xh.astype(np.float32), f16_inputs=True)
    want = O.swiglu(wg, wu).ravel()
    got = fused.view(np.float16).astype(np.float32)
    # f32 accumulation error of gate and up carried through silu(g) * u, plus the final f16 rounding
    bound = 1e-5 * (np.abs(wu) * 1.1 * sg + np.abs(wg) * su).ravel() + np.abs(want) * 2.0 ** -10 + 1e-7
    assert np.all(np.abs(got - want) <= bound)


@pytest.mark.parametrize("rows,cols,tokens", [(256, 4096, 16), (256, 4096, 300), (1024, 512, 300), (100, 96, 20)])
def test_gemm_add_equals_gemm_then_add(B, ctx, K, rows, cols, tokens):
    """acc += W x with the add in the GEMM's epilogue (split K, plain tensor-core and generic paths) gives the very
    bits of the GEMM followed by the element-wise add."""
    rng = O.Rng(83)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    m = tiled(B, ctx, K, "q4_0", raw, rows, cols)[0] if cols % 256 == 0 else B.QMatrix(ctx.buffer_from(raw), B.WeightType.Q4_0, rows, cols)
    xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
    acc0 = rng.vec(tokens * rows, 2.0)
    gx, gy, gs = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4), ctx.buffer(tokens * rows * 4)
    ga, gb = ctx.buffer_from(acc0), ctx.buffer_from(acc0)
    run(ctx, lambda c: (K.gemm(c, m, gx, gy, tokens), K.add(c, gb, gy, gb, tokens * rows)))
    run(ctx, lambda c: K.gemm_add(c, m, gx, ga, gs, tokens))
    assert np.array_equal(ga.download(np.float32), gb.download(np.float32))


@pytest.mark.parametrize("rows,cols", [((1024, 256, 256), 2560), ((25600,), 256), ((2560,), 9728), ((6400, 6400), 512)])
def test_gemm_few_tokens_persistent(B, ctx, K, rows, cols):
    """Up to 64 tokens the tiled q4_0 GEMM is one persistent launch whose blocks take equal runs of (row tile, K stage)
    pairs: runs that end inside a tile (partial tiles added up by the last block to arrive), runs that hold several whole
    tiles, one to three matrices per launch, with and without the residual. Same bound as every GEMM; the residual form
    gives the very bits of GEMM then add; a second launch gives the bits of the first (the sum's order is fixed)."""
    rng = O.Rng(91)
    raws = [rng.qmatrix(O.Q4_0, r, cols) for r in rows]
    ms = [tiled(B, ctx, K, "q4_0", raw, r, cols)[0] for raw, r in zip(raws, rows)]
    for tokens in (9, 40, 64):
        x = rng.vec(tokens * cols, 1.0)
        xh = x.astype(np.float16)
        gxh = ctx.buffer_from(xh)
        gys = [ctx.buffer(tokens * r * 4) for r in rows]
        run(ctx, lambda c: K.gemm_multi(c, ms, gxh, gys, tokens, B.PrefillPrecision.F16))
        first = [gy.download(np.float32) for gy in gys]
        for raw, r, got in zip(raws, rows, first):
            want16, s16 = O.matmul(O.Q4_0, raw, r, cols, x, f16_inputs=True)
            assert np.max(np.abs(got.reshape(tokens, r) - want16) / s16) <= 1e-5, (tokens, r)
        run(ctx, lambda c: K.gemm_multi(c, ms, gxh, gys, tokens, B.PrefillPrecision.F16))
        for gy, got in zip(gys, first):
            assert np.array_equal(gy.download(np.float32), got)
        if len(rows) == 1:
            acc0 = rng.vec(tokens * rows[0], 2.0)
            ga, gs = ctx.buffer_from(acc0), ctx.buffer(tokens * rows[0] * 4)
            run(ctx, lambda c: K.gemm_add(c, ms[0], gxh, ga, gs, tokens))
            assert np.array_equal(ga.download(np.float32), acc0 + first[0])


@pytest.mark.parametrize("rows,cols,tokens", [(2560, 4096, 40), (2560, 9728, 64), (5120, 512, 9), (1024, 512, 33), (2560, 4096, 100)])
def test_gemm_add_rms_norm_equals_the_two_calls(B, ctx, K, rows, cols, tokens):
    """acc += W x followed by the RMS norm of acc, as one call: behind the few-token GEMM one kernel adds the blocks' partial
    tiles and the residual and forms the norm; shapes it does not take fall back to the two calls. Same bits either way."""
    rng = O.Rng(59)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    m = tiled(B, ctx, K, "q4_0", raw, rows, cols)[0]
    xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
    acc0, wn = rng.vec(tokens * rows, 2.0), rng.vec(rows, 1.0)
    gx, gs, gw = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4), ctx.buffer_from(wn)
    ga, gb = ctx.buffer_from(acc0), ctx.buffer_from(acc0)
    oa, ob = ctx.buffer(tokens * rows * 2), ctx.buffer(tokens * rows * 2)
    run(ctx, lambda c: (K.gemm_add(c, m, gx, ga, gs, tokens), K.rms_norm_f16(c, ga, gw, oa, tokens, rows, 1e-6)))
    run(ctx, lambda c: K.gemm_add_rms_norm_f16(c, m, gx, gb, gs, gw, ob, tokens, 1e-6))
    assert np.array_equal(ga.download(np.float32), gb.download(np.float32))
    assert np.array_equal(oa.download(np.uint16, tokens * rows), ob.download(np.uint16, tokens * rows))
    # and in place: the norm written over the GEMM's input, as the layer loop does
    if cols == rows:
        return
    gb2 = ctx.buffer_from(acc0)
    gx2 = ctx.buffer(max(tokens * cols, tokens * rows) * 2)
    gx2.upload(xh)
    run(ctx, lambda c: K.gemm_add_rms_norm_f16(c, m, gx2, gb2, gs, gw, gx2, tokens, 1e-6))
    assert np.array_equal(gx2.download(np.uint16, tokens * rows), oa.download(np.uint16, tokens * rows))


@pytest.mark.parametrize("tokens", [16, 200])
def test_gemm_tiled_q6_tensor_core(B, ctx, K, tokens):
    """A tiled q6_0 matrix whose rows are a multiple of 128 (the tied lm_head of a batch step) runs on the tcgen05 GEMM:
    codes rebuilt from the nibbles and the high-bit words, same bound as every GEMM."""
    rows, cols = 1280, 2560
    rng = O.Rng(47)
    raw = rng.qmatrix(O.Q6_0, rows, cols)
    m = tiled(B, ctx, K, "q6_0", raw, rows, cols)[0]
    x = rng.vec(tokens * cols, 1.0)
    xh = x.astype(np.float16)
    want16, s16 = O.matmul(O.Q6_0, raw, rows, cols, x, f16_inputs=True)
    gxh, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
    run(ctx, lambda c: K.gemm(c, m, gxh, gy, tokens))
    got = gy.download(np.float32).reshape(tokens, rows)
    assert np.max(np.abs(got - want16) / s16) <= 1e-5


# ---- argmax --------------------------------------------------------------------------------------

def test_argmax_edge_cases(ctx, K):
    inf, nan = float("-inf"), float("nan")
    cases = [[inf, inf], [nan, inf, nan], [nan, 1.0, nan, 1.0], [-3.0, -1.0, -1.0, -2.0],
             [float((i * 7919) % 1000) for i in range(151_936)], [float((i * 13) % 5 - 2) for i in range(37)], [5.0]]
    out = ctx.buffer(4)
    for v in cases:
        a = np.array(v, dtype=np.float32)
        g = ctx.buffer_from(a)
        run(ctx, lambda c: K.argmax(c, g, a.size, out))
        assert int(out.download(np.uint32)[0]) == O.argmax(a), v[:8]
    rng = O.Rng(31)
    a = rng.vec(151_936, 5.0)
    a[[77, 90_000, 151_935]] = 9.0  # ties: the first one wins
    g = ctx.buffer_from(a)
    run(ctx, lambda c: K.argmax(c, g, a.size, out))
    assert int(out.download(np.uint32)[0]) == 77


@pytest.mark.parametrize("rows,cols", [(1024, 512), (128, 256), (256, 4096)])
def test_gemm_tensor_core_token_counts(B, ctx, K, rows, cols):
    """The tcgen05 prefill GEMM (tiled q4_0, rows a multiple of 128) over token counts that exercise 1, 2 and 4
    token tiles per block, ragged last tiles and every pipeline depth; same bound as the reference's GEMM test
    (1e-5 of sum |w x| against the f16-rounded product)."""
    rng = O.Rng(77)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    mt, _ = tiled(B, ctx, K, "q4_0", raw, rows, cols)
    for tokens in (16, 127, 128, 129, 300, 512, 700):
        x = rng.vec(tokens * cols, 1.0)
        xh = x.astype(np.float16)
        want16, s16 = O.matmul(O.Q4_0, raw, rows, cols, x, f16_inputs=True)
        gxh, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
        run(ctx, lambda c: K.gemm(c, mt, gxh, gy, tokens))
        got = gy.download(np.float32).reshape(tokens, rows)
        assert np.max(np.abs(got - want16) / s16) <= 1e-5, tokens


@pytest.mark.parametrize("kv", ["F16", "Q8_0"])
@pytest.mark.parametrize("tokens,pos0", [(512, 0), (300, 77), (129, 255), (200, 1500)])
def test_flash_attention_tensor_core_many_query_tiles(B, ctx, K, tokens, pos0, kv):
    """The tcgen05 prefill attention (F16 precision over an f16 cache, and over a q8_0 cache expanded to hi + lo f16
    tiles) with several 128-query tiles, ragged last tiles, key ranges that start before the queries and rows whose
    reference value moves while O is being accumulated; bound of the reference's attention test."""
    rng = O.Rng(23)
    hq, hkv, dim = 8, 2, 128
    lk = pos0 + tokens
    cap = (lk + 63) // 64 * 64
    q = rng.vec(tokens * hq * dim, 2.0)
    kvt = getattr(B.KvType, kv)
    kraw = rng.vec(cap * hkv * dim, 2.0)
    kraw[(lk - 40) * hkv * dim:] *= 4.0  # late keys with much larger scores: the rows' references move after many tiles
    gk, gv, k, v = make_cache(B, ctx, kvt, kraw, rng.vec(cap * hkv * dim, 3.0))
    want16, vmax = O.attention(q, k, v, tokens, hq, hkv, dim, pos0, q16=True)
    gq, goh = ctx.buffer_from(q), ctx.buffer(q.size * 2)
    shape = B.AttnShape(tokens, hq, hkv, dim, pos0, kvt)
    run(ctx, lambda c: K.flash_attention(c, gq, gk, gv, goh, shape))
    oh = goh.download(np.float16).astype(np.float32)
    d = np.maximum(np.abs(oh - want16) - np.abs(want16) * 2.0 ** -11, 0.0)  # the output's own f16 rounding is discounted
    assert float(np.max(d / np.maximum(vmax, 1e-30))) <= 1e-5


# ---- sampling ------------------------------------------------------------------------------------

@pytest.mark.parametrize("n", [50, 5000, 151_936])
def test_device_sampler_follows_the_reference_sampler(B, ctx, K, n):
    """brasa_k_sample_top_p against the oracle's restatement of Sampler::sample (sampler.rs:60-146) with the same
    PCG32 stream. The device sums in a tree where the reference adds 150 000 f32 terms one after another, so both
    carry rounding in the cumulative mass: every device pick must be a candidate the reference keeps and must sit
    within 1e-3 of the total mass of the reference's pick in the sorted order; for vocabularies where f32 addition
    order matters little (n <= 5000) at least 97 % of the draws must be the very same token."""
    rng = np.random.default_rng(n)
    out = ctx.buffer(4)
    agree = total = 0
    for temperature, top_k, top_p, seed in [(0.7, 0, 0.95, 11), (1.0, 40, 0.9, 5), (1.3, 0, 1.0, 7), (0.6, 20, 0.95, 3), (1.0, 3, 1.0, 1)]:
        ref = O.Sampler(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
        state = ctx.buffer_from(B.pcg32_state(seed))
        for _ in range(12):
            logits = (rng.standard_normal(n) * 3.0).astype(np.float32)
            if n > 100:
                logits[rng.integers(0, n, 5)] = logits.max()  # equal logits: ascending id order
            want = ref.sample(logits)
            g = ctx.buffer_from(logits)
            run(ctx, lambda c: K.sample_top_p(c, g, n, temperature, top_k, top_p, state, out))
            got = int(out.download(np.uint32, 1)[0])
            total += 1
            agree += got == want
            order = np.lexsort((np.arange(n), -logits.astype(np.float64)))
            rank = {int(t): i for i, t in enumerate(order[:ref.last_keep + 1])}
            assert got in rank, (temperature, top_k, top_p, ref.last_keep)
            w = np.exp((logits[order].astype(np.float64) - float(logits.max())) / temperature)
            cum = np.cumsum(w[:ref.last_keep + 1])
            assert abs(cum[rank[got]] - cum[rank[want]]) <= 1e-3 * cum[-1] + max(w[rank[got]], w[rank[want]]), (got, want)
    if n <= 5000:
        assert agree >= 0.97 * total, (agree, total)


@pytest.mark.parametrize("n", [5000, 151_936])
def test_sampler_for_many_rows_follows_the_reference_sampler(B, ctx, K, n):
    """brasa_k_sample_rows: every row spread over several blocks, masses in 64-bit fixed point. Same bounds as the
    one-row sampler against the oracle's Sampler::sample restatement (sampler.rs:60-146), each row with its own PCG32
    stream over several consecutive draws; and a row's tokens do not depend on how many rows share the launch."""
    rows, draws = 6, 5
    rng = np.random.default_rng(n + 1)
    for temperature, top_p in [(0.7, 0.95), (1.0, 1.0), (1.2, 0.5)]:
        refs = [O.Sampler(temperature=temperature, top_k=0, top_p=top_p, seed=40 + r) for r in range(rows)]
        states = ctx.buffer_from(np.concatenate([B.pcg32_state(40 + r) for r in range(rows)]))
        alone = ctx.buffer_from(np.concatenate([B.pcg32_state(40 + r) for r in range(2)]))
        scratch, out, out2 = ctx.buffer(rows * n * 8), ctx.buffer(rows * 4), ctx.buffer(2 * 4)
        agree = total = 0
        for _ in range(draws):
            logits = (rng.standard_normal((rows, n)) * 3.0).astype(np.float32)
            for r in range(rows):
                logits[r, rng.integers(0, n, 5)] = logits[r].max()  # equal logits: ascending id order
            g = ctx.buffer_from(logits)
            run(ctx, lambda c: K.sample_rows(c, g, n, rows, temperature, 0, top_p, states, scratch, out))
            run(ctx, lambda c: K.sample_rows(c, g, n, 2, temperature, 0, top_p, alone, scratch, out2))
            got = out.download(np.uint32, rows)
            assert list(out2.download(np.uint32, 2)) == list(got[:2])
            for r in range(rows):
                want = refs[r].sample(logits[r])
                total += 1
                agree += int(got[r]) == want
                order = np.lexsort((np.arange(n), -logits[r].astype(np.float64)))
                rank = {int(t): i for i, t in enumerate(order[:refs[r].last_keep + 1])}
                w = np.exp((logits[r][order].astype(np.float64) - float(logits[r].max())) / temperature)
                cum = np.cumsum(w[:refs[r].last_keep + 1])
                # the device's cut may sit one rounding step past the reference's: allow the next candidate
                nxt = int(order[refs[r].last_keep + 1]) if refs[r].last_keep + 1 < n else -1
                assert int(got[r]) in rank or int(got[r]) == nxt, (temperature, top_p, r)
                if int(got[r]) in rank:
                    assert abs(cum[rank[int(got[r])]] - cum[rank[want]]) <= 1e-3 * cum[-1] + max(w[rank[int(got[r])]], w[rank[want]])
        if n <= 5000:
            assert agree >= 0.97 * total, (agree, total)


def test_device_sampler_frequency_and_greedy(B, ctx, K):
    """The reference's frequency check (sampler.rs:252-267): logits (0, ln 3) at temperature 1 pick token 1 three
    times out of four; temperature 0 is the greedy argmax."""
    out = ctx.buffer(4)
    g = ctx.buffer_from(np.array([0.0, np.log(3.0)], dtype=np.float32))
    state = ctx.buffer_from(B.pcg32_state(3))
    ones = 0
    draws = 2000
    for _ in range(draws):
        run(ctx, lambda c: K.sample_top_p(c, g, 2, 1.0, 0, 1.0, state, out))
        ones += int(out.download(np.uint32, 1)[0])
    assert abs(ones / draws - 0.75) < 0.03
    g2 = ctx.buffer_from(np.array([0.1, 3.0, -1.0, 2.9], dtype=np.float32))
    run(ctx, lambda c: K.sample_top_p(c, g2, 4, 0.0, 0, 1.0, state, out))
    assert int(out.download(np.uint32, 1)[0]) == 1


@pytest.mark.parametrize("name", ["q6_0", "q8_0"])
@pytest.mark.parametrize("layout", ["file", "tiled"])
def test_gemm_other_weight_types(B, ctx, K, name, layout):
    """The warp-MMA prefill GEMM over q6_0 (both layouts: the lm_head of a batch) and q8_0 weights."""
    if name == "q8_0" and layout == "tiled":
        pytest.skip("q8_0 has no tiled layout")
    rows, cols, tokens = 512, 256, 19
    rng = O.Rng(41)
    raw = rng.qmatrix(QT[name][0], rows, cols)
    m = tiled(B, ctx, K, name, raw, rows, cols)[0] if layout == "tiled" else B.QMatrix(ctx.buffer_from(raw), B.WeightType(QT[name][1]), rows, cols)
    x = rng.vec(tokens * cols, 1.0)
    xh = x.astype(np.float16)
    want16, s16 = O.matmul(QT[name][0], raw, rows, cols, x, f16_inputs=True)
    gxh, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
    run(ctx, lambda c: K.gemm(c, m, gxh, gy, tokens))
    got = gy.download(np.float32).reshape(tokens, rows)
    assert np.max(np.abs(got - want16) / s16) <= 1e-5
