"""Tensor-parallel exchange and sharded decode on the GPU.

One device: the exchange kernels with two ranks that share the device (every rank's send queued before any rank's
receive, so no kernel waits for a later launch), and a whole model with a one-rank exchange attached. Two devices
(skipped otherwise): two processes, one shard each, against the unsplit model on one device.
"""

import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF

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
def untied_model(tmp_path_factory):
    d = tmp_path_factory.mktemp("tp_model")
    cfg = BF.tiny_config(layers=3, hidden=512, heads=8, kv_heads=2, ffn=1280, vocab=1024)
    cfg["tie_word_embeddings"] = False
    BF.write_brasa(d / "model.brasa", cfg, BF.synth_weights(cfg, seed=29, std=0.04, norm_jitter=0.1))
    return d / "model.brasa"


@pytest.mark.parametrize("n", [5120, 64 * 512, 2])
def test_allreduce_two_ranks_on_one_device(B, ctx, n):
    from brasa_b200.tp import TensorParallel
    K = B.Kernels(ctx)
    tps = TensorParallel.same_process([ctx, ctx], max(n, 2))
    try:
        rng = np.random.default_rng(n)
        x = rng.standard_normal(n).astype(np.float32)
        gx = [ctx.buffer_from(x.copy()) for _ in range(2)]
        gp = [ctx.buffer(n * 4) for _ in range(2)]
        for it in range(5):  # several exchanges: both parities of the buffer and growing exchange numbers
            parts = [rng.standard_normal(n).astype(np.float32) * (1 + r) for r in range(2)]
            for r in range(2):
                gp[r].upload(parts[r])
            cmd = ctx.command()
            for r in range(2):
                K.tp_allreduce_add(cmd, tps[r], gp[r], gx[r], gx[r], n, phase="push")
            for r in range(2):
                K.tp_allreduce_add(cmd, tps[r], gp[r], gx[r], gx[r], n, phase="gather")
            cmd.wait()
            x = x + (parts[0] + parts[1])  # rank order, then the residual: the kernel's order exactly
            for r in range(2):
                assert np.array_equal(gx[r].download(np.float32)[:n], x), (it, r)
        # without a residual the output is the plain sum
        cmd = ctx.command()
        out = [ctx.buffer(n * 4) for _ in range(2)]
        for r in range(2):
            K.tp_allreduce_add(cmd, tps[r], gp[r], None, out[r], n, phase="push")
        for r in range(2):
            K.tp_allreduce_add(cmd, tps[r], gp[r], None, out[r], n, phase="gather")
        cmd.wait()
        for r in range(2):
            assert np.array_equal(out[r].download(np.float32)[:n], parts[0] + parts[1])
    finally:
        for t in tps:
            t.free()


@pytest.mark.parametrize("rows,cols,world", [(512, 1024, 2), (2560, 2048, 4)])
def test_gemv_fused_with_the_exchange(B, ctx, rows, cols, world):
    """brasa_k_gemv_allreduce: a matrix split by columns over `world` ranks that share the device; every rank's GEMV
    writes its rows into all exchange buffers (queued first), the receives add them. Against the oracle's matmul of the
    whole matrix (1e-5 of sum |w x|), identical bits on every rank, and equal to the unfused GEMV + all-reduce."""
    from brasa_b200.tp import TensorParallel
    K = B.Kernels(ctx)
    rng = O.Rng(rows + world)
    raw = rng.qmatrix(O.Q4_0, rows, cols)
    x = rng.vec(cols, 1.0)
    resid = rng.vec(rows, 2.0)
    want, s = O.matmul(O.Q4_0, raw, rows, cols, x)
    per = cols // world
    blocks = raw.reshape(rows, cols // 32, 18)
    shards = []
    for r in range(world):
        part = np.ascontiguousarray(blocks[:, r * per // 32:(r + 1) * per // 32, :]).reshape(-1)
        src, dst = ctx.buffer_from(part), ctx.buffer(part.nbytes)
        cmd = ctx.command()
        K.repack(cmd, 0, src, dst, rows, per)
        cmd.wait()
        shards.append(B.QMatrix(dst, B.WeightType.Q4_0, rows, per, B.Layout.TILED))
    tps = TensorParallel.same_process([ctx] * world, rows)
    try:
        xs = [ctx.buffer_from(np.ascontiguousarray(x[r * per:(r + 1) * per])) for r in range(world)]
        gres = [ctx.buffer_from(resid.copy()) for _ in range(world)]
        outs = [ctx.buffer(rows * 4) for _ in range(world)]
        for it in range(3):  # both parities of the buffer
            cmd = ctx.command()
            for r in range(world):
                K.gemv_allreduce(cmd, tps[r], shards[r], xs[r], gres[r], outs[r], phase="push")
            for r in range(world):
                K.gemv_allreduce(cmd, tps[r], shards[r], xs[r], gres[r], outs[r], phase="gather")
            cmd.wait()
            got = [o.download(np.float32)[:rows] for o in outs]
            for r in range(1, world):
                assert np.array_equal(got[r], got[0])
            assert np.max(np.abs(got[0] - resid - want[0]) / s[0]) <= 2e-5  # world partial sums, each within 1e-5 of its share
        # the unfused sequence gives the same bits
        parts = [ctx.buffer(rows * 4) for _ in range(world)]
        outs2 = [ctx.buffer(rows * 4) for _ in range(world)]
        cmd = ctx.command()
        for r in range(world):
            K.gemv(cmd, shards[r], xs[r], parts[r], 1)
            K.tp_allreduce_add(cmd, tps[r], parts[r], gres[r], outs2[r], rows, phase="push")
        for r in range(world):
            K.tp_allreduce_add(cmd, tps[r], parts[r], gres[r], outs2[r], rows, phase="gather")
        cmd.wait()
        assert np.array_equal(outs2[0].download(np.float32)[:rows], got[0])
    finally:
        for t in tps:
            t.free()


def test_argmax_exchange_ties_and_nan(B, ctx):
    from brasa_b200.tp import TensorParallel
    K = B.Kernels(ctx)
    world, n = 4, 1000
    tps = TensorParallel.same_process([ctx] * world, 16)
    try:
        rng = np.random.default_rng(9)
        cases = []
        a = rng.standard_normal((world, n)).astype(np.float32)
        cases.append(a.copy())
        a[1, 17] = a[3, 5] = a.max() + 1.0  # equal maxima on two ranks: the lower global index wins
        cases.append(a.copy())
        a[0, :] = np.nan  # a rank with nothing but NaN never wins
        cases.append(a.copy())
        cases.append(np.full((world, n), -np.inf, np.float32))  # all -inf: index 0
        for c in cases:
            bufs = [ctx.buffer_from(c[r].copy()) for r in range(world)]
            outs = [ctx.buffer(4) for _ in range(world)]
            cmd = ctx.command()
            for r in range(world):
                K.tp_argmax(cmd, tps[r], bufs[r], n, r * n, outs[r], phase="push")
            for r in range(world):
                K.tp_argmax(cmd, tps[r], bufs[r], n, r * n, outs[r], phase="gather")
            cmd.wait()
            want = O.argmax(c.reshape(-1))
            for r in range(world):
                assert int(outs[r].download(np.uint32)[0]) == want
    finally:
        for t in tps:
            t.free()


def test_receive_without_a_send_gives_up_and_the_context_lives(B, ctx, untied_model):
    """A rank whose peer never sends: the receive runs out of polls by itself (nothing faults, nothing hangs), the
    call reports ETIMEOUT, and the same context runs the next exchange correctly. A model decoding on the same context
    with the whole-token kernel (whose activation words live across launches and are emptied after an abandoned wait)
    gives the same tokens before and after."""
    from brasa_b200.tp import TensorParallel
    K = B.Kernels(ctx)
    n = 512
    model = B.Qwen3.load(ctx, untied_model, B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16))
    prompt = np.random.default_rng(9).integers(0, 1024, size=24).astype(np.uint32)
    lg, _ = model.forward(prompt, 0)
    first = int(np.argmax(lg[0]))
    before = [int(t) for t in model.decode_greedy(first, 24, 7)[0]]  # an odd count: the next launch starts on the other copy
    tps = TensorParallel.same_process([ctx, ctx], n)
    try:
        tps[0].set_poll_limit(2000)
        part = ctx.buffer_from(np.ones(n, np.float32))
        out = ctx.buffer(n * 4)
        cmd = ctx.command()
        K.tp_allreduce_add(cmd, tps[0], part, None, out, n, phase="push")
        K.tp_allreduce_add(cmd, tps[0], part, None, out, n, phase="gather")  # rank 1 never pushed
        with pytest.raises(B.BrasaError) as err:
            cmd.wait()
        assert err.value.code == B.ETIMEOUT
        ctx.sync()  # the status word was cleared by the failed wait: the context is clean again
        assert [int(t) for t in model.decode_greedy(first, 24, 7)[0]] == before
        assert [int(t) for t in model.decode_greedy(first, 24, 7)[0]] == before
        # rank 1 catches up with the abandoned exchange (its own receive finds both ranks' words), then a full one
        cmd = ctx.command()
        K.tp_allreduce_add(cmd, tps[1], part, None, out, n, phase="push")
        K.tp_allreduce_add(cmd, tps[1], part, None, out, n, phase="gather")
        cmd.wait()
        assert np.array_equal(out.download(np.float32)[:n], np.full(n, 2.0, np.float32))
        outs = [ctx.buffer(n * 4) for _ in range(2)]
        cmd = ctx.command()
        for r in range(2):
            K.tp_allreduce_add(cmd, tps[r], part, None, outs[r], n, phase="push")
        for r in range(2):
            K.tp_allreduce_add(cmd, tps[r], part, None, outs[r], n, phase="gather")
        cmd.wait()
        for r in range(2):
            assert np.array_equal(outs[r].download(np.float32)[:n], np.full(n, 2.0, np.float32))
    finally:
        for t in tps:
            t.free()
        model.free()


@pytest.mark.parametrize("kv", ["F32", "F16"])
def test_one_rank_exchange_changes_nothing(B, ctx, untied_model, kv):
    from brasa_b200.tp import TensorParallel
    limits = B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=getattr(B.KvType, kv))
    ids = np.random.default_rng(5).integers(0, 1024, size=40).astype(np.uint32)
    plain = B.Qwen3.load(ctx, untied_model, limits)
    want, _ = plain.forward(ids, 0)
    want1, _ = plain.forward(ids[:1], 40)
    want_t, _ = plain.decode_greedy(int(ids[0]), 40, 12)

    def batch_of(model):
        g = np.random.default_rng(6)
        bt = B.Batch(model, max_seqs=10, num_pages=40, max_positions=64)
        bt.set_prefix(g.integers(0, 1024, size=16).astype(np.uint32))
        for k in (5, 11, 3, 7, 2, 9, 4, 6, 8, 10):  # ten sequences: the projections run as GEMMs
            bt.add_sequence(g.integers(0, 1024, size=k).astype(np.uint32))
        lg = bt.peek_logits()
        out, _ = bt.decode(6)
        bt.free()
        return lg, out

    want_bl, want_bids = batch_of(plain)
    plain.free()
    m = B.Qwen3.load(ctx, untied_model, limits)
    tp = TensorParallel(ctx, 0, 1, 64 * 512)
    m.set_tp(tp)
    try:
        got, _ = m.forward(ids, 0)
        got1, _ = m.forward(ids[:1], 40)
        toks, _ = m.decode_greedy(int(ids[0]), 40, 12)
        toks2, _ = m.decode_greedy(int(ids[0]), 40, 12)
        assert np.array_equal(got, want)
        assert np.abs(got1 - want1).max() <= 1e-5 * np.abs(want1).max()  # x + (W a) in one kernel or in two
        assert list(toks) == list(want_t) == list(toks2)
        got_bl, got_bids = batch_of(m)  # the batched path with the exchange in place of the residual adds
        assert np.array_equal(got_bl, want_bl) and np.array_equal(got_bids, want_bids)
    finally:
        m.free()
        tp.free()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("kv", ["F32", "F16"])
def test_two_processes_two_devices_match_the_unsplit_model(B, ctx, untied_model, tmp_path, kv):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from brasa_b200 import tp as TP
    outs = [tmp_path / f"shard{r}.brasa" for r in range(2)]
    TP.split_model(untied_model, outs)
    n_prompt, steps = 40, 12
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
           str(_free_port()), os.path.join(os.path.dirname(__file__), "tp_worker.py"), str(tmp_path / "shard{rank}.brasa"), str(tmp_path),
           str(n_prompt), str(steps), kv]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    limits = B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=getattr(B.KvType, kv))
    ids = np.random.default_rng(5).integers(0, 1024, size=n_prompt).astype(np.uint32)
    m = B.Qwen3.load(ctx, untied_model, limits)
    try:
        if kv == "F32":
            m.set_prefill_precision(B.PrefillPrecision.F32)
        want, _ = m.forward(ids, 0)
        want1, _ = m.forward(ids[:1], n_prompt)
        want_t, _ = m.decode_greedy(int(ids[0]), n_prompt, steps)
        g = np.random.default_rng(6)
        prefix = g.integers(0, 1024, size=16).astype(np.uint32)
        own = [g.integers(0, 1024, size=int(k)).astype(np.uint32) for k in (5, 11, 3)]
        bt = B.Batch(m, max_seqs=3, num_pages=16, max_positions=64)
        bt.set_prefix(prefix)
        for o in own:
            bt.add_sequence(o)
        want_bl = bt.peek_logits()
        want_bids, _ = bt.decode(8)
        bt.free()
    finally:
        m.free()
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(2)]
    got = np.concatenate([r["logits"] for r in ranks], axis=1)
    got1 = np.concatenate([r["one"] for r in ranks], axis=1)
    assert [int(r["row0"]) for r in ranks] == [0, 512]
    # The split changes only the order of the sums over o_proj's and down_proj's columns. With an f32 cache the test
    # runs the f32 prefill, so everything is f32 and the model-level bound for f32 applies; with an f16 cache the
    # prefill rounds its GEMM inputs to f16 (PrefillPrecision::F16), where a last-bit difference in x can flip a
    # rounding: the bound is the reference's floor for that mode (crates/models/tests/forward.rs:40-55).
    tol = 1e-4 if kv == "F32" else 2e-3
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    assert np.abs(got1 - want1).max() <= tol * np.abs(want1).max()
    for r in ranks:
        assert list(r["toks"]) == list(want_t) and list(r["toks2"]) == list(want_t)
    # the batched path over paged KV: every rank chose the same tokens, and they are the unsplit model's
    got_bl = np.concatenate([r["batch_logits"] for r in ranks], axis=1)
    assert np.abs(got_bl - want_bl).max() <= tol * np.abs(want_bl).max()
    assert np.array_equal(ranks[0]["batch_ids"], ranks[1]["batch_ids"])
    assert np.array_equal(ranks[0]["batch_ids"], want_bids)
    # sampled: the ranks drew the same tokens, and each sequence's first one is the oracle sampler's choice on the
    # gathered logits of its prompt with that sequence's stream
    assert np.array_equal(ranks[0]["sampled_ids"], ranks[1]["sampled_ids"])
    if kv == "F32":  # (with f16 GEMM inputs a prompt prefilled whole and one prefilled behind the cached prefix differ in the last bits)
        full = np.concatenate([r["prompt_last"] for r in ranks], axis=1)
        for i in range(3):
            assert O.Sampler(temperature=0.7, top_k=0, top_p=0.95, seed=100 + i).sample(full[i]) == int(ranks[0]["sampled_ids"][i, 0])
    assert len({tuple(r) for r in ranks[0]["sampled_ids"].tolist()}) > 1
