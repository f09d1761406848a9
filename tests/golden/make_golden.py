"""Generates the golden fixtures in this directory from the REFERENCE's own Python tools.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports tools/convert_brasa.py, tools/brasa_file.py and tools/qwen3_ref.py from that checkout
(nothing is copied) and writes:

  quant_cases.npz   f32 blocks -> q4_0 / q6_0 / q8_0 bytes (convert_brasa.quant_*), their
                    dequantised values (brasa_file.dequantize), and KV-Q8 rounded values
                    (qwen3_ref.round_kv_q8)
  tiny/model.brasa  a 2-layer random-init Qwen3 written by convert_brasa.main()
  tiny/ref_*.npz    Qwen3Ref logits / hidden states / greedy ids for KV f32, f16 and q8_0
  rope_cases.npz    qwen3_ref.rope on random vectors at positions 0, 3, 40944

The fixtures are small (about 1.5 MB in total) and are committed; the tests read only them.
"""

from __future__ import annotations

import json
import pathlib
import shutil
import sys
import tempfile

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent


def main() -> None:
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of a checkout of the reference repository>")
    ref = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(ref / "tools"))
    import brasa_file
    import convert_brasa
    import qwen3_ref
    from safetensors.numpy import save_file

    rng = np.random.default_rng(20240607)

    # ---- quantiser cases -------------------------------------------------------------------
    w = (rng.standard_normal((96, 32)) * 0.02).astype(np.float32)
    w[3] = 0.0                                     # zero block
    w[4] = np.linspace(-8, 7, 32, dtype=np.float32)  # exact integers, d = 1
    w[5, 7], w[5, 19] = 0.5, -0.5                  # tie on |max|: first index wins
    w[6] = (np.arange(32) - 15.5).astype(np.float32) * 0.125  # x/d exactly half-way
    w[7] = np.float32(1e-9)                        # scale underflows to 0 in f16
    w[8] = rng.standard_normal(32).astype(np.float32) * 300.0
    w[9, :] = 0.0
    w[9, 31] = -3.0
    flat = w.reshape(-1)
    out = {"w": w}
    for name, fn in (("q4_0", convert_brasa.quant_q4_0), ("q6_0", convert_brasa.quant_q6_0),
                     ("q8_0", convert_brasa.quant_q8_0)):
        b = np.frombuffer(fn(flat), dtype=np.uint8)
        out[name] = b
        out[name + "_deq"] = brasa_file.dequantize(name, b.copy(), list(w.shape))
    kv = (rng.standard_normal((40, 128)) * 3.0).astype(np.float32)
    kv[1, 32:64] = 0.0
    d = np.float32(np.float16(1.0 / 127.0))
    kv[2, :32] = (np.arange(32, dtype=np.float32) - 15.5) * d
    kv[2, 31] = 1.0
    kv[3, :32] = 3000.0
    out["kv"] = kv
    out["kv_q8_rounded"] = qwen3_ref.round_kv_q8(torch.from_numpy(kv)).numpy()
    np.savez_compressed(HERE / "quant_cases.npz", **out)

    # ---- rope ------------------------------------------------------------------------------
    x = rng.standard_normal((3, 5, 128)).astype(np.float32)
    pos = torch.tensor([0, 3, 40944])
    np.savez_compressed(HERE / "rope_cases.npz", x=x, pos=pos.numpy(),
                        y=qwen3_ref.rope(torch.from_numpy(x), pos, 1e6).numpy())

    # ---- tiny model through the reference converter and forward ----------------------------
    cfg = {"model_type": "qwen3", "tie_word_embeddings": True, "num_hidden_layers": 2,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "rms_norm_eps": 1e-6,
           "rope_theta": 1e6, "hidden_size": 256, "intermediate_size": 512, "vocab_size": 512,
           "max_position_embeddings": 4096}
    H, F, V, D = 256, 512, 512, 128
    qd, kvd = 4 * D, 2 * D

    def mat(r, c):
        return (rng.standard_normal((r, c)) * 0.05).astype(np.float32)

    def norm(n):
        return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)

    tensors = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": norm(H)}
    for i in range(2):
        p = f"model.layers.{i}."
        tensors.update({
            p + "input_layernorm.weight": norm(H), p + "post_attention_layernorm.weight": norm(H),
            p + "self_attn.q_norm.weight": norm(D), p + "self_attn.k_norm.weight": norm(D),
            p + "self_attn.q_proj.weight": mat(qd, H), p + "self_attn.k_proj.weight": mat(kvd, H),
            p + "self_attn.v_proj.weight": mat(kvd, H), p + "self_attn.o_proj.weight": mat(H, qd),
            p + "mlp.gate_proj.weight": mat(F, H), p + "mlp.up_proj.weight": mat(F, H),
            p + "mlp.down_proj.weight": mat(H, F)})
    with tempfile.TemporaryDirectory() as td:
        hf, dst = pathlib.Path(td) / "hf", pathlib.Path(td) / "out"
        hf.mkdir()
        (hf / "config.json").write_text(json.dumps(cfg))
        save_file(tensors, str(hf / "model.safetensors"))
        (hf / "model.safetensors.index.json").write_text(
            json.dumps({"weight_map": {k: "model.safetensors" for k in tensors}}))
        for n in ("tokenizer.json", "tokenizer_config.json"):
            (hf / n).write_text("{}")
        sys.argv = ["convert_brasa.py", str(hf), str(dst), "--source-repo", "synthetic/tiny",
                    "--source-commit", "0"]
        convert_brasa.main()
        tiny = HERE / "tiny"
        tiny.mkdir(exist_ok=True)
        shutil.copy(dst / "model.brasa", tiny / "model.brasa")
        (tiny / "config.json").write_text(json.dumps(cfg))

        prompt = torch.from_numpy(rng.integers(0, V, size=24).astype(np.int64))
        torch.manual_seed(0)
        for tag, kvt in (("f32", None), ("f16", torch.float16), ("q8_0", "q8_0")):
            m = qwen3_ref.Qwen3Ref(hf, brasa=dst / "model.brasa", kv_dtype=kvt)
            caches = [m.new_cache()]
            cap: dict = {}
            logits = m.forward_many([prompt], caches, capture=cap)[0]
            greedy, dec_logits = [], []
            nxt = int(logits[-1].argmax())
            for _ in range(8):
                greedy.append(nxt)
                lg = m.forward_many([torch.tensor([nxt])], caches)[0]
                dec_logits.append(lg[0].numpy())
                nxt = int(lg[0].argmax())
            # chunked prefill (16 + 8) must give the same last-row logits up to f32 reduction order
            caches2 = [m.new_cache()]
            m.forward_many([prompt[:16]], caches2)
            chunked = m.forward_many([prompt[16:]], caches2)[0]
            np.savez_compressed(
                tiny / f"ref_{tag}.npz", prompt=prompt.numpy().astype(np.uint32),
                prefill_logits=logits.numpy(), embed=cap["embed"][0].numpy(),
                layer0=cap[0][0].numpy(), layer1=cap[1][0].numpy(),
                greedy=np.array(greedy, dtype=np.uint32), decode_logits=np.stack(dec_logits),
                chunked_tail_logits=chunked.numpy(),
                k_cache0=caches[0][0][0].numpy(), v_cache0=caches[0][0][1].numpy())
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
