"""Generates the long-context golden fixtures from the REFERENCE's own forward (tools/qwen3_ref.py).

Run where the reference checkout is available:

    python tests/golden/make_golden_long.py /path/to/reference

The model is the committed tiny/model.brasa (written by make_golden.py through the reference's converter). A seeded
16 384-token prompt goes through Qwen3Ref.forward_many in 512-token chunks over an f16 and over a q8_0 KV cache,
followed by 8 greedy decode steps. Written per cache type to tiny/ref_long_<kv>.npz: the prompt, the logits of the
last prompt position, the 8 decode-step logits and the greedy ids. About 40 KB each.
"""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
PROMPT_TOKENS = 16384
CHUNK = 512
STEPS = 8


def main() -> None:
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_long.py <path of a checkout of the reference repository>")
    ref = pathlib.Path(sys.argv[1])
    sys.path.insert(0, str(ref / "tools"))
    import qwen3_ref

    tiny = HERE / "tiny"
    torch.set_num_threads(max(1, torch.get_num_threads()))
    prompt = np.random.default_rng(16384).integers(0, 512, size=PROMPT_TOKENS).astype(np.int64)
    for tag, kvt in (("f16", torch.float16), ("q8_0", "q8_0")):
        m = qwen3_ref.Qwen3Ref(tiny, brasa=tiny / "model.brasa", kv_dtype=kvt)
        caches = [m.new_cache()]
        logits = None
        for off in range(0, PROMPT_TOKENS, CHUNK):
            logits = m.forward_many([torch.from_numpy(prompt[off:off + CHUNK])], caches)[0]
        last = logits[-1].numpy().copy()
        nxt = int(logits[-1].argmax())
        greedy, dec = [], []
        for _ in range(STEPS):
            greedy.append(nxt)
            lg = m.forward_many([torch.tensor([nxt])], caches)[0]
            dec.append(lg[0].numpy().copy())
            nxt = int(lg[0].argmax())
        np.savez_compressed(tiny / f"ref_long_{tag}.npz", prompt=prompt.astype(np.uint16), prefill_last_logits=last,
                            decode_logits=np.stack(dec), greedy=np.array(greedy, dtype=np.uint32))
        print(tag, "done; top-1/top-2 gap at the last prompt position:", float(np.sort(last)[-1] - np.sort(last)[-2]))


if __name__ == "__main__":
    main()
