"""Two contexts on two devices in one process: everything a context sets up per device (opt-in shared memory of the
large kernels, the fixed scratch array of the allocation-free attention) must exist on both. Skipped with one GPU."""

import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


def device_count():
    import torch
    return torch.cuda.device_count()


def exercise(B, dev):
    """A tensor-core GEMM, the tensor-core prefill attention, decode attention (allocating and static) and the paged batch
    step of a small model on device `dev`, each against the oracle."""
    from oracle import brasa_format as BF
    import pathlib
    import tempfile
    ctx = B.Context(dev)
    try:
        K = B.Kernels(ctx)
        rng = O.Rng(7 + dev)

        def run(fn):
            cmd = ctx.command()
            fn(cmd)
            return cmd.wait()
        rows, cols, tokens = 256, 512, 200
        raw = rng.qmatrix(O.Q4_0, rows, cols)
        src, dst = ctx.buffer_from(raw), ctx.buffer(raw.nbytes)
        run(lambda c: K.repack(c, 0, src, dst, rows, cols))
        w = B.QMatrix(dst, B.WeightType.Q4_0, rows, cols, B.Layout.TILED)
        xh = rng.vec(tokens * cols, 1.0).astype(np.float16)
        gx, gy = ctx.buffer_from(xh), ctx.buffer(tokens * rows * 4)
        run(lambda c: K.gemm(c, w, gx, gy, tokens))
        want, s = O.matmul(O.Q4_0, raw, rows, cols, xh.astype(np.float32), f16_inputs=True)
        assert np.max(np.abs(gy.download(np.float32).reshape(tokens, rows) - want) / s) <= 1e-5
        x32 = xh[:cols].astype(np.float32)
        gx1, gy1 = ctx.buffer_from(x32), ctx.buffer(rows * 4)
        run(lambda c: K.gemv(c, w, gx1, gy1, 1))
        want1, s1 = O.matmul(O.Q4_0, raw, rows, cols, x32)
        assert np.max(np.abs(gy1.download(np.float32)[:rows] - want1[0]) / s1[0]) <= 1e-5

        hq, hkv, dim, ntok, pos0 = 8, 2, 128, 200, 60
        lk = pos0 + ntok
        q = rng.vec(ntok * hq * dim, 2.0)
        kd, vd = rng.vec(lk * hkv * dim, 2.0).astype(np.float16), rng.vec(lk * hkv * dim, 3.0).astype(np.float16)
        gq, gk, gv, go = ctx.buffer_from(q), ctx.buffer_from(kd), ctx.buffer_from(vd), ctx.buffer(q.size * 2)
        run(lambda c: K.flash_attention(c, gq, gk, gv, go, B.AttnShape(ntok, hq, hkv, dim, pos0, B.KvType.F16)))
        want16, vmax = O.attention(q, kd.astype(np.float32), vd.astype(np.float32), ntok, hq, hkv, dim, pos0, q16=True)
        oh = go.download(np.float16).astype(np.float32)
        d = np.maximum(np.abs(oh - want16) - np.abs(want16) * 2.0 ** -11, 0.0)
        assert float(np.max(d / np.maximum(vmax, 1e-30))) <= 1e-5

        q1 = rng.vec(hq * dim, 2.0)
        gq1, o1, o2 = ctx.buffer_from(q1), ctx.buffer(hq * dim * 4), ctx.buffer(hq * dim * 4)
        part = ctx.buffer(B.decode_partials_len(hq, lk) * 4)
        sh = B.AttnShape(1, hq, hkv, dim, lk - 1, B.KvType.F16)
        run(lambda c: K.decode_attention(c, gq1, gk, gv, part, o1, sh))
        run(lambda c: K.decode_attention_static(c, gq1, gk, gv, o2, sh))
        ref, vm = O.attention(q1, kd.astype(np.float32), vd.astype(np.float32), 1, hq, hkv, dim, lk - 1)
        assert np.array_equal(o1.download(np.float32), o2.download(np.float32))
        assert np.max(np.abs(o2.download(np.float32) - ref) / np.maximum(vm, 1e-30)) <= 1e-5

        with tempfile.TemporaryDirectory() as td:
            path = pathlib.Path(td) / "model.brasa"
            cfg = BF.tiny_config(layers=2, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=512)
            BF.write_brasa(path, cfg, BF.synth_weights(cfg, seed=3, std=0.05, norm_jitter=0.1))
            m = B.Qwen3.load(ctx, path, B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
            prompt = np.arange(40, dtype=np.uint32)
            lg, _ = m.forward(prompt, 0)
            first = int(np.argmax(lg[0]))
            dev_ids, _ = m.decode_greedy(first, 40, 6)  # the whole-token kernel on this device
            bt = B.Batch(m, max_seqs=3, num_pages=24, max_positions=128)
            bt.set_prefix(prompt[:32])
            for _ in range(3):
                bt.add_sequence(prompt[32:])
            ids, _ = bt.decode(6)
            bt.free()
            m.free()
            for s in range(3):
                assert [int(t) for t in ids[s]] == [first] + [int(t) for t in dev_ids]
    finally:
        ctx.close()


def test_the_same_kernels_on_two_devices_in_one_process():
    import brasa_b200 as B
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    exercise(B, 0)
    exercise(B, 1)
    exercise(B, 0)


def test_two_contexts_on_one_device_with_models_of_different_size():
    """The opt-in shared-memory size of a kernel is one value per device: a second context whose model asks for less must
    not take the first one's grant away. Two models of different widths decode alternately, each in its own context."""
    import pathlib
    import tempfile

    import brasa_b200 as B
    from oracle import brasa_format as BF
    shapes = [dict(layers=2, hidden=1024, heads=8, kv_heads=4, ffn=4096, vocab=512), dict(layers=2, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=512)]
    with tempfile.TemporaryDirectory() as td:
        ctxs, models, firsts, want = [], [], [], []
        try:
            for i, sh in enumerate(shapes):
                path = pathlib.Path(td) / f"model{i}.brasa"
                cfg = BF.tiny_config(**sh)
                BF.write_brasa(path, cfg, BF.synth_weights(cfg, seed=5 + i, std=0.05, norm_jitter=0.1))
                ctx = B.Context(0)
                ctxs.append(ctx)
                m = B.Qwen3.load(ctx, path, B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
                models.append(m)
                lg, _ = m.forward(np.arange(24, dtype=np.uint32), 0)
                firsts.append(int(np.argmax(lg[0])))
                want.append([int(t) for t in m.decode_greedy(firsts[i], 24, 5)[0]])
            for _ in range(2):  # alternate: each launch follows one of the other context
                for i, m in enumerate(models):
                    assert [int(t) for t in m.decode_greedy(firsts[i], 24, 5)[0]] == want[i]
        finally:
            for m in models:
                m.free()
            for c in ctxs:
                c.close()
