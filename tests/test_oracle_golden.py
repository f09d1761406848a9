"""The oracle against golden files produced by the reference's Python tools
(tests/golden/make_golden.py): quantisers and dequantisers bit-exact, KV-Q8 rounding bit-exact,
RoPE and the whole-model forward within float32 round-off of tools/qwen3_ref.py."""

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF


@pytest.fixture(scope="module")
def quant(golden_dir):
    return np.load(golden_dir / "quant_cases.npz")


@pytest.mark.parametrize("name", ["q4_0", "q6_0", "q8_0"])
def test_quantisers_bit_exact(quant, name):
    q = O.QTYPE[name]
    got = O.quantize(q, quant["w"])
    assert np.array_equal(got, quant[name])
    deq = O.dequantize(q, quant[name], quant["w"].size).reshape(quant["w"].shape)
    assert np.array_equal(deq.view(np.uint32), quant[name + "_deq"].view(np.uint32))


def test_kv_q8_rounding_bit_exact(quant):
    got = O.dequantize_kv_q8(O.quantize_kv_q8(quant["kv"])).reshape(quant["kv"].shape)
    want = quant["kv_q8_rounded"]
    # the two differ only in the sign of zeros (q * d with q = -0.0 in torch)
    assert np.array_equal(got, want)
    assert np.array_equal(O.round_kv(O.KV_Q8, quant["kv"]), want)


def test_rope_matches_reference(golden_dir):
    g = np.load(golden_dir / "rope_cases.npz")
    cos, sin = O.rope_table(1e6, 128, int(g["pos"].max()) + 1)
    for i, p in enumerate(g["pos"]):
        y = O.rope_neox(g["x"][i], 5, 128, int(p), cos, sin).reshape(5, 128)
        x = g["x"][i]
        bound = 1e-6 * (np.abs(x) + np.abs(np.roll(x, 64, axis=1)))
        assert np.all(np.abs(y - g["y"][i]) <= bound + 1e-9)


def test_brasa_reader_and_writer_round_trip(golden_dir, tmp_path):
    f = BF.BrasaFile(golden_dir / "tiny" / "model.brasa")
    f.verify()
    assert f.config()["num_hidden_layers"] == 2
    assert f.tensors["model.embed_tokens.weight"]["dtype"] == "q6_0"
    assert f.tensors["model.layers.0.mlp.gate_proj.weight"]["dtype"] == "q4_0"
    assert f.tensors["model.norm.weight"]["dtype"] == "f32"
    assert all(t["offset"] % 16384 == 0 for t in f.meta["tensors"])
    # re-quantising the dequantised weights reproduces the file's bytes (quantiser fixed point)
    w = {n: f.get_f32(n) for n in f.tensors}
    BF.write_brasa(tmp_path / "again.brasa", f.config(), w)
    g = BF.BrasaFile(tmp_path / "again.brasa")
    g.verify()
    for n in f.tensors:
        assert f.tensors[n]["sha256"] == g.tensors[n]["sha256"], n
        assert f.tensors[n]["offset"] == g.tensors[n]["offset"], n
    bad = bytearray((tmp_path / "again.brasa").read_bytes())
    bad[g.tensors["model.norm.weight"]["offset"]] ^= 1
    (tmp_path / "bad.brasa").write_bytes(bad)
    with pytest.raises(ValueError):
        BF.BrasaFile(tmp_path / "bad.brasa").verify()


def _rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


# Distance allowed between the oracle (double accumulation) and tools/qwen3_ref.py (torch f32). With a
# rounded KV cache a value that lands within float round-off of a rounding boundary flips by one
# step and moves the logits; the reference documents this (docs/adr/0009-kv-cache-f16-y-q8.md:40-46,
# 105-109) and allows 1e-3 (f16) and 2e-2 (q8_0) for it in crates/models/tests/forward.rs:40-55.
TOL = {"f32": 5e-6, "f16": 5e-4, "q8_0": 5e-4}


@pytest.mark.parametrize("kv", ["f32", "f16", "q8_0"])
def test_whole_model_matches_qwen3_ref(golden_dir, kv):
    f = BF.BrasaFile(golden_dir / "tiny" / "model.brasa")
    g = np.load(golden_dir / "tiny" / f"ref_{kv}.npz")
    m = O.Qwen3Oracle(f, kv=kv, ctx=64)
    prompt = g["prompt"]
    tol = TOL[kv]
    logits, hid = m.forward(prompt, logit_rows=prompt.size, capture_hidden=True)
    assert _rel(hid[0], g["layer0"]) < tol
    assert _rel(hid[1], g["layer1"]) < tol
    assert _rel(logits, g["prefill_logits"]) < tol
    # layer-0 cache: same values as the reference's; rounded types may flip a few entries by one step
    mine, ref = m.k[0, :prompt.size].reshape(-1), g["k_cache0"][:prompt.size].reshape(-1)
    if kv == "f32":
        assert _rel(mine, ref) < 2e-6
    else:
        flips = mine != ref
        assert flips.mean() < 0.01
        assert np.all(np.abs(mine - ref)[flips] <= np.abs(ref[flips]) * 2.0 ** -9 + 1e-6)
    nxt = int(np.argmax(logits[-1]))
    for step in range(8):
        assert nxt == int(g["greedy"][step])
        lg = m.forward([nxt])
        assert _rel(lg[0], g["decode_logits"][step]) < tol
        nxt = int(np.argmax(lg[0]))
    # chunked prefill reaches the same state
    m.reset()
    m.forward(prompt[:16])
    tail = m.forward(prompt[16:], logit_rows=8)
    assert _rel(tail, g["chunked_tail_logits"]) < tol


def test_f16_prefill_mode_stays_close(golden_dir):
    f = BF.BrasaFile(golden_dir / "tiny" / "model.brasa")
    g = np.load(golden_dir / "tiny" / "ref_f16.npz")
    m = O.Qwen3Oracle(f, kv="f16", ctx=64)
    logits = m.forward(g["prompt"], logit_rows=1, f16_prefill=True)
    # the reference's own bound for f16 prefill + f16 KV is 2e-3 of max|logit|
    assert _rel(logits[0], g["prefill_logits"][-1]) < 2e-3
