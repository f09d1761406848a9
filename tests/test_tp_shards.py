"""Tensor-parallel shard files (CPU): splitting a model keeps every byte, and the split computes the same products.

The reference runs one device, so these check the construction itself: q/k/v and gate/up split by rows, o_proj and
down_proj by columns, lm_head by vocabulary rows, norms and the embedding table replicated.
"""

import numpy as np
import pytest

import oracle as O
from oracle import brasa_format as BF


@pytest.fixture(scope="module")
def full_model(tmp_path_factory):
    d = tmp_path_factory.mktemp("tp_full")
    cfg = BF.tiny_config(layers=2, hidden=512, heads=8, kv_heads=2, ffn=1280, vocab=1024)
    cfg["tie_word_embeddings"] = False
    BF.write_brasa(d / "model.brasa", cfg, BF.synth_weights(cfg, seed=23, std=0.04, norm_jitter=0.1))
    return d / "model.brasa", cfg


def tensors_of(path):
    from brasa_b200 import tp
    meta, raw = tp.read_container(path)
    return meta, {t["name"]: (t, np.asarray(raw[t["offset"]:t["offset"] + t["nbytes"]])) for t in meta["tensors"]}


def test_share_is_contiguous_and_covers_everything():
    from brasa_b200 import tp
    for total, world in ((100, 8), (8, 8), (5, 2), (151936, 8)):
        spans = [tp._share(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def test_qwen3_32b_splits_over_1_2_4_8_ranks():
    from brasa_b200 import synth, tp
    for world in (1, 2, 4, 8):
        ffn = heads = vocab = 0
        for r in range(world):
            c = tp.shard_config(synth.QWEN3_32B, r, world)
            assert c["intermediate_size"] % 256 == 0 and c["num_attention_heads"] == 8 * c["num_key_value_heads"]
            ffn += c["intermediate_size"]
            heads += c["num_attention_heads"]
            assert c["tp_vocab_offset"] == vocab
            vocab += c["tp_head_rows"]
        assert (ffn, heads, vocab) == (25600, 64, 151936)
    with pytest.raises(ValueError):
        tp.shard_config(synth.QWEN3_4B, 0, 2)  # tied lm_head


@pytest.mark.parametrize("world", [2])
def test_split_keeps_every_byte_and_the_products(full_model, tmp_path, world):
    import brasa_b200 as B
    from brasa_b200 import tp
    path, cfg = full_model
    outs = [tmp_path / f"shard{r}.brasa" for r in range(world)]
    cfgs = tp.split_model(path, outs)
    for o in outs:
        B.file_check(o, verify=True)  # structure and sha256 of every tensor
    _, full = tensors_of(path)
    shards = [tensors_of(o)[1] for o in outs]
    H, D = cfg["hidden_size"], cfg["head_dim"]
    rng = np.random.default_rng(3)
    for name, (t, data) in full.items():
        parts = [s[name] for s in shards]
        if t["dtype"] == "f32" or name == "model.embed_tokens.weight":
            for pt, pd in parts:
                assert pt["shape"] == t["shape"] and np.array_equal(pd, data), name
        elif name.endswith(("o_proj.weight", "down_proj.weight")):
            # column split: the full product is the sum of the shards' products over their own slice of x
            rows, cols = t["shape"]
            x = rng.standard_normal(cols).astype(np.float32)
            want = O.matmul(O.QTYPE[t["dtype"]], data, rows, cols, x)[0][0]
            got, c0 = np.zeros(rows, np.float64), 0
            for pt, pd in parts:
                pc = pt["shape"][1]
                got += O.matmul(O.QTYPE[t["dtype"]], pd, rows, pc, x[c0:c0 + pc])[0][0]
                c0 += pc
            assert c0 == cols
            assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 1e-6, name
            # and the blocks themselves are the full matrix's blocks
            bb = 18
            whole = data.reshape(rows, cols // 32, bb)
            assert np.array_equal(np.concatenate([pd.reshape(rows, -1, bb) for _, pd in parts], axis=1), whole), name
        else:  # row split: the shards' bytes in rank order are the full tensor
            assert np.array_equal(np.concatenate([pd for _, pd in parts]), data), name
            assert sum(pt["shape"][0] for pt, _ in parts) == t["shape"][0]
    assert [c["tp_vocab_offset"] for c in cfgs] == [0, 512]
    assert cfgs[0]["intermediate_size"] + cfgs[1]["intermediate_size"] == 1280 and cfgs[0]["intermediate_size"] == 768
    assert all(c["num_attention_heads"] == 4 and c["num_key_value_heads"] == 1 for c in cfgs)
    assert H == 512 and D == 128
