"""The allocation-free decode attention entry point against the regular one.

Some users of the library cannot allocate device memory at the point where they need attention: a thread
that is recording a CUDA graph, a plugin living inside someone else's memory budget, a serving loop that
must not touch the allocator. For them brasa_k_decode_attention_static keeps its scratch in a fixed array
inside the library. This test calls it through the C ABI twice in a row (the array keeps the previous
call's contents, so the second call shows that stale data does no harm) and expects exactly what
brasa_k_decode_attention produces with a caller-allocated scratch buffer, for every cache type. It runs
last so that a failure here cannot hide the other tests, and it does not depend on them."""

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_attention_matches_the_allocating_one():
    import brasa_b200 as B
    ctx = B.Context(0)
    try:
        K = B.Kernels(ctx)
        rng = O.Rng(41)
        hq, hkv, dim = 32, 8, 128
        for kv in (B.KvType.F16, B.KvType.Q8_0, B.KvType.F32):
            for pos0 in (700, 129):  # second call: fewer chunks than the first left behind in the array
                lk = pos0 + 1
                q = rng.vec(hq * dim, 2.0)
                k, v = rng.vec(lk * hkv * dim, 2.0), rng.vec(lk * hkv * dim, 3.0)
                if kv == B.KvType.F16:
                    kd, vd, kf, vf = k.astype(np.float16), v.astype(np.float16), None, None
                    kf, vf = kd.astype(np.float32), vd.astype(np.float32)
                elif kv == B.KvType.Q8_0:
                    kd, vd = O.quantize_kv_q8(k), O.quantize_kv_q8(v)
                    kf, vf = O.dequantize_kv_q8(kd), O.dequantize_kv_q8(vd)
                else:
                    kd, vd, kf, vf = k, v, k, v
                gq, gk, gv = ctx.buffer_from(q), ctx.buffer_from(kd), ctx.buffer_from(vd)
                want_buf, got_buf = ctx.buffer(hq * dim * 4), ctx.buffer(hq * dim * 4)
                part = ctx.buffer(B.decode_partials_len(hq, lk) * 4)
                shape = B.AttnShape(1, hq, hkv, dim, pos0, kv)
                cmd = ctx.command()
                K.decode_attention(cmd, gq, gk, gv, part, want_buf, shape)
                cmd.wait()
                got_buf.fill(0xFF)
                cmd = ctx.command()
                K.decode_attention_static(cmd, gq, gk, gv, got_buf, shape)
                cmd.wait()
                want, got = want_buf.download(np.float32), got_buf.download(np.float32)
                assert np.array_equal(got, want), (kv, pos0)  # same kernels, same order: same bits
                ref, vmax = O.attention(q, kf, vf, 1, hq, hkv, dim, pos0)
                assert np.max(np.abs(got - ref) / np.maximum(vmax, 1e-30)) <= 1e-5
        # beyond the fixed array: a clear refusal, nothing launched
        small = ctx.buffer(16)
        with pytest.raises(B.BrasaError) as e:
            cmd = ctx.command()
            try:
                K.decode_attention_static(cmd, small, small, small, small, B.AttnShape(1, 32, 8, 128, 8192, B.KvType.F16))
            finally:
                cmd.wait()
        assert e.value.code == B.EINVAL and "8192" in str(e.value)
        with pytest.raises(B.BrasaError):
            cmd = ctx.command()
            try:
                K.decode_attention_static(cmd, small, small, small, small, B.AttnShape(1, 128, 8, 128, 10, B.KvType.F16))
            finally:
                cmd.wait()
    finally:
        ctx.close()


def test_static_scratch_at_the_top_of_its_range():
    """64 query heads over 8 KV heads at position 8 191: the last chunk of the last head writes the last words of the
    fixed array. Same bits as the allocating entry point; one key more is refused."""
    import brasa_b200 as B
    ctx = B.Context(0)
    try:
        K = B.Kernels(ctx)
        rng = O.Rng(43)
        hq, hkv, dim, pos0 = 64, 8, 128, 8191
        lk = pos0 + 1
        q = rng.vec(hq * dim, 2.0)
        kd, vd = rng.vec(lk * hkv * dim, 2.0).astype(np.float16), rng.vec(lk * hkv * dim, 3.0).astype(np.float16)
        gq, gk, gv = ctx.buffer_from(q), ctx.buffer_from(kd), ctx.buffer_from(vd)
        want_buf, got_buf = ctx.buffer(hq * dim * 4), ctx.buffer(hq * dim * 4)
        part = ctx.buffer(B.decode_partials_len(hq, lk) * 4)
        shape = B.AttnShape(1, hq, hkv, dim, pos0, B.KvType.F16)
        for _ in range(2):
            cmd = ctx.command()
            K.decode_attention(cmd, gq, gk, gv, part, want_buf, shape)
            cmd.wait()
            got_buf.fill(0xFF)
            cmd = ctx.command()
            K.decode_attention_static(cmd, gq, gk, gv, got_buf, shape)
            cmd.wait()
            assert np.array_equal(got_buf.download(np.float32), want_buf.download(np.float32))
        ref, vmax = O.attention(q, kd.astype(np.float32), vd.astype(np.float32), 1, hq, hkv, dim, pos0)
        assert np.max(np.abs(got_buf.download(np.float32) - ref) / np.maximum(vmax, 1e-30)) <= 1e-5
        # the allocating entry point refuses a position whose key count does not fit 32 bits instead of launching nothing
        with pytest.raises(B.BrasaError) as e:
            cmd = ctx.command()
            try:
                K.decode_attention(cmd, gq, gk, gv, part, want_buf, B.AttnShape(1, hq, hkv, dim, 0xFFFFFFFF, B.KvType.F16))
            finally:
                cmd.wait()
        assert e.value.code == B.EINVAL
    finally:
        ctx.close()
