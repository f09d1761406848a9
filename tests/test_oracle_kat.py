"""Known-answer tests of the reference's own unit tests, re-expressed against the oracle.

Vectors are those of crates/quant/src/qtype.rs:186-303, crates/quant/src/convert.rs:361-390 and
crates/runtime/src/sampler.rs:177-267.
"""

import math

import numpy as np

import oracle as O


def test_f16_known_values():
    assert O.f16_to_f32(0x3C00) == 1.0
    assert O.f16_to_f32(0xC000) == -2.0
    assert O.f16_to_f32(0x3555) == float(np.float32(0.33325195))
    assert O.f16_to_f32(0x0001) == float(np.float32(5.9604645e-8))
    assert O.f16_to_f32(0x7BFF) == 65504.0
    assert math.isinf(O.f16_to_f32(0x7C00))
    for h in range(0, 0x7C00, 7):
        f = O.f16_to_f32(h)
        assert math.isfinite(f) and f >= 0.0


def test_f16_agrees_with_numpy_everywhere():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(h)) for h in bits], dtype=np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok].view(np.uint32), want[ok].view(np.uint32))
    assert np.isnan(got[~ok]).all()


def test_f32_to_f16_round_trip_and_ties_to_even():
    bits = np.arange(65536, dtype=np.uint16)
    vals = bits.view(np.float16).astype(np.float32)
    back = O.f32_to_f16_array(vals)
    ok = ~np.isnan(vals)
    assert np.array_equal(back[ok], bits[ok])
    # midpoints between consecutive f16 go to the even one; one f32 ulp either side goes to nearest
    h = np.arange(0, 0x7BFF, dtype=np.uint16)
    a, b = h.view(np.float16).astype(np.float32), (h + 1).astype(np.uint16).view(np.float16).astype(np.float32)
    mid = ((a.astype(np.float64) + b.astype(np.float64)) / 2).astype(np.float32)
    even = np.where(h % 2 == 0, h, h + 1).astype(np.uint16)
    assert np.array_equal(O.f32_to_f16_array(mid), even)
    assert np.array_equal(O.f32_to_f16_array((mid.view(np.uint32) + 1).view(np.float32)), h + 1)
    assert np.array_equal(O.f32_to_f16_array((mid.view(np.uint32) - 1).view(np.float32)), h)
    assert np.array_equal(O.f32_to_f16_array(-mid), even | 0x8000)
    assert O.f32_to_f16(65520.0) == 0x7C00
    assert O.f32_to_f16(1e10) == 0x7C00
    assert O.f32_to_f16(2.0 ** -25) == 0
    assert O.f32_to_f16(float(np.float32(2.0 ** -25) * np.float32(1.0001))) == 1
    assert math.isnan(O.f16_to_f32(O.f32_to_f16(float("nan"))))


def test_f32_to_f16_matches_numpy_on_random_bits():
    rng = np.random.default_rng(1)
    x = rng.integers(0, 2 ** 32, size=200_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    x = x[~np.isnan(x)]
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.f32_to_f16_array(x), want)


def test_q4_0_hand_block():
    b = bytes([0x00, 0x38] + [j | ((15 - j) << 4) for j in range(16)])
    out = O.dequantize(O.Q4_0, b, 32)
    for j in range(16):
        assert out[j] == 0.5 * (j - 8.0)
        assert out[j + 16] == 0.5 * (7.0 - j)


def test_q6_0_hand_block():
    q = [2 * j for j in range(32)]
    b = [0x00, 0x3C]
    b += [(q[j] & 15) | ((q[j + 16] & 15) << 4) for j in range(16)]
    b += [(q[j] >> 4) | ((q[j + 8] >> 4) << 2) | ((q[j + 16] >> 4) << 4) | ((q[j + 24] >> 4) << 6) for j in range(8)]
    out = O.dequantize(O.Q6_0, bytes(b), 32)
    assert np.array_equal(out, 2.0 * np.arange(32, dtype=np.float32) - 32.0)


def test_q8_0_hand_block():
    b = bytes([0x00, 0x3C] + [(j - 16) & 0xFF for j in range(32)])
    assert np.array_equal(O.dequantize(O.Q8_0, b, 32), np.arange(32, dtype=np.float32) - 16.0)


def test_quantise_dequantise_identity_on_integer_blocks():
    v4 = (np.arange(32) % 16).astype(np.float32) - 8.0
    assert np.array_equal(O.dequantize(O.Q4_0, O.quantize(O.Q4_0, v4), 32), v4)
    v6 = 2.0 * np.arange(32, dtype=np.float32) - 32.0
    assert np.array_equal(O.dequantize(O.Q6_0, O.quantize(O.Q6_0, v6), 32), v6)
    z = np.zeros(32, np.float32)
    assert np.array_equal(O.dequantize(O.Q6_0, O.quantize(O.Q6_0, z), 32), z)
    assert np.array_equal(O.dequantize(O.Q4_0, O.quantize(O.Q4_0, z), 32), z)
    v8 = np.arange(32, dtype=np.float32) - 16.0
    v8[0] = 127.0
    assert np.array_equal(O.dequantize(O.Q8_0, O.quantize(O.Q8_0, v8), 32), v8)
    assert O.nbytes(O.Q4_0, 64) == 36 and O.nbytes(O.Q6_0, 64) == 52 and O.nbytes(O.Q8_0, 64) == 68


def test_kv_q8_round_trip_bounds():
    x = np.array([((i * 37 % 101) - 50.0) * 0.173 for i in range(128)], dtype=np.float32)
    x[32:64] = 0.0
    q = O.quantize_kv_q8(x)
    assert q.size == 136
    y = O.dequantize_kv_q8(q)
    for b in range(4):
        blk = x[b * 32:(b + 1) * 32]
        amax = np.abs(blk).max()
        assert np.all(np.abs(blk - y[b * 32:(b + 1) * 32]) <= amax / 127.0 * 0.5 * (1 + 1e-3) + 1e-12)
        if amax > 0:
            assert (np.abs(q[b * 32:(b + 1) * 32].view(np.int8).astype(np.int32)) == 127).any()
    assert np.all(y[32:64] == 0.0)


def test_argmax_edge_cases():
    inf, nan = float("-inf"), float("nan")

    def scalar(v):
        best = (0, inf)
        for i, x in enumerate(v):
            if x > best[1]:
                best = (i, x)
        return best[0]

    cases = [[], [inf, inf], [nan, inf, nan], [nan, 1.0, nan, 1.0], [-3.0, -1.0, -1.0, -2.0],
             [float((i * 7919) % 1000) for i in range(151_936)], [float((i * 13) % 5 - 2) for i in range(37)]]
    for v in cases:
        assert O.argmax(np.array(v, dtype=np.float32)) == scalar(v)


def test_pcg32_is_the_published_generator():
    # PCG32 (O'Neill) with the reference's seeding: state 0, fixed increment, advance, add seed, advance.
    def ref(seed, n):
        M = (1 << 64) - 1
        state, inc = 0, ((0xDA3E39CB94B95BDB << 1) | 1) & M
        out = []

        def nxt():
            nonlocal state
            old = state
            state = (old * 6364136223846793005 + inc) & M
            x = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
            rot = old >> 59
            return ((x >> rot) | (x << ((32 - rot) & 31))) & 0xFFFFFFFF

        nxt()
        state = (state + seed) & M
        nxt()
        for _ in range(n):
            out.append(nxt())
        return out

    for seed in (0, 1, 7, 2 ** 63 + 5):
        s = O.Sampler(temperature=1.0, seed=seed)
        assert [s.next_u32() for _ in range(16)] == ref(seed, 16)
    s = O.Sampler(temperature=1.0, seed=3)
    u = ref(3, 4)
    assert [s.next_f32() for _ in range(4)] == [float(np.float32(v >> 8) / np.float32(1 << 24)) for v in u]


def test_sampler_greedy_seed_topk_topp_frequency():
    assert O.Sampler().sample([0.1, 3.0, -1.0, 2.9]) == 1
    logits = np.array([((i * 37) % 101) / 10.0 for i in range(1000)], dtype=np.float32)

    def run(seed):
        s = O.Sampler(temperature=0.6, top_k=20, top_p=0.95, seed=seed)
        return [s.sample(logits) for _ in range(50)]

    assert run(7) == run(7)
    assert run(7) != run(8)
    logits = 10.0 - np.arange(100, dtype=np.float32)
    s = O.Sampler(temperature=1.0, top_k=3, top_p=1.0, seed=1)
    assert all(s.sample(logits) < 3 for _ in range(500))
    s = O.Sampler(temperature=1.0, top_k=0, top_p=0.5, seed=1)
    assert all(s.sample(logits) == 0 for _ in range(200))
    s = O.Sampler(temperature=1.0, seed=3)
    two = np.array([math.log(3.0), 0.0], dtype=np.float32)
    n = 20_000
    f = sum(s.sample(two) == 0 for _ in range(n)) / n
    assert abs(f - 0.75) < 0.015


def test_xorshift_rng_first_values():
    # xorshift64* with multiplier 0x2545F4914F6CDD1D (crates/kernels/src/testutil.rs:12-17)
    M = (1 << 64) - 1

    def ref(seed, n):
        s, out = max(seed, 1), []
        for _ in range(n):
            s ^= s >> 12
            s ^= (s << 25) & M
            s ^= s >> 27
            out.append((s * 0x2545F4914F6CDD1D) & M)
        return out

    for seed in (0, 1, 11, 24):
        r = O.Rng(seed)
        assert [r.next_u64() for _ in range(8)] == ref(seed, 8)
    r = O.Rng(11)
    want = [np.float32(v >> 40) / np.float32(1 << 23) - np.float32(1.0) for v in ref(11, 5)]
    assert np.array_equal(r.vec(5, 1.0), np.array(want, dtype=np.float32))
    # random q4_0 matrix: scale exponents stay in 7..13 and sizes match
    m = O.Rng(5).qmatrix(O.Q4_0, 4, 64)
    assert m.size == 4 * 64 // 32 * 18
    ex = (m.reshape(-1, 18)[:, 1] >> 2) & 31
    assert ex.min() >= 7 and ex.max() <= 13


def test_rope_table_large_position():
    cos, sin = O.rope_table(1e6, 128, 3)
    assert cos[0] == 1.0 and sin[0] == 0.0
    assert cos[64] == np.float32(math.cos(1.0)) and sin[64] == np.float32(math.sin(1.0))
    inv = 1.0 / (1e6 ** (2 / 128))
    assert cos[2 * 64 + 1] == np.float32(math.cos(2 * inv))
