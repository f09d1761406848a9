"""One rank of the tensor-parallel parity test (launched by test_gpu_tp.py through torch.distributed.run).

argv: shard path pattern with {rank}, output directory, prompt length, decode steps. Every rank loads its shard,
connects the exchange over the process group (gloo on 127.0.0.1), runs a prefill and a device-resident greedy
decode, and writes its rows of the logits and the tokens it chose.
"""

import os
import pathlib
import sys

import numpy as np


def main():
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parents[1]))
    import torch.distributed as dist

    import brasa_b200 as B
    from brasa_b200.tp import TensorParallel

    pattern, out_dir, n_prompt, steps, kv_name = sys.argv[1], pathlib.Path(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    ctx = B.Context(local)
    limits = B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=getattr(B.KvType, kv_name))
    m = B.Qwen3.load(ctx, pattern.format(rank=rank), limits)
    tp = TensorParallel(ctx, rank, world, limits.max_tokens * m.cfg["hidden"])
    m.set_tp(tp)
    if kv_name == "F32":
        m.set_prefill_precision(B.PrefillPrecision.F32)
    ids = np.random.default_rng(5).integers(0, m.cfg["vocab"], size=n_prompt).astype(np.uint32)
    dist.barrier()
    logits, _ = m.forward(ids, 0)                      # prefill: GEMM path, all-reduce of [tokens, hidden]
    one, _ = m.forward(ids[:1], n_prompt)              # one token: the fused GEMV chain
    first = int(ids[0])
    dist.barrier()
    toks, _ = m.decode_greedy(first, n_prompt, steps)  # device-resident loop with the argmax exchange
    dist.barrier()
    toks2, _ = m.decode_greedy(first, n_prompt, steps)  # CUDA graph replay of the same steps
    # several sequences decoded together over paged KV (greedy: each row's best pair is exchanged between the ranks)
    g = np.random.default_rng(6)
    prefix = g.integers(0, m.cfg["vocab"], size=16).astype(np.uint32)
    own = [g.integers(0, m.cfg["vocab"], size=int(k)).astype(np.uint32) for k in (5, 11, 3)]
    bt = B.Batch(m, max_seqs=3, num_pages=16, max_positions=64)
    dist.barrier()
    bt.set_prefix(prefix)
    for o in own:
        dist.barrier()
        bt.add_sequence(o)
    dist.barrier()
    bl = bt.peek_logits()
    dist.barrier()
    bids, _ = bt.decode(8)
    bt.free()
    # the same sequences sampled: every rank gathers the rows' logits over the whole vocabulary and draws with the same streams
    params = B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=100)
    bt = B.Batch(m, max_seqs=3, num_pages=16, max_positions=64)
    dist.barrier()
    bt.set_prefix(prefix)
    for o in own:
        dist.barrier()
        bt.add_sequence(o, params)
    dist.barrier()
    sids, _ = bt.decode(8, params)
    bt.free()
    plast = []
    for o in own:  # this rank's rows of the logits each first token was drawn from
        dist.barrier()
        plast.append(m.forward(np.concatenate([prefix, o]), 0)[0][0])
    np.savez(out_dir / f"rank{rank}.npz", logits=logits, one=one, toks=toks, toks2=toks2, row0=m.cfg["head_row0"], batch_logits=bl, batch_ids=bids,
             sampled_ids=sids, prompt_last=np.stack(plast))
    dist.barrier()
    m.free()
    tp.free()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
