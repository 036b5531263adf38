"""Rank program for tests/test_tp_gpu.py: a mid-size model (hidden 2048) under tensor parallelism.
Prefill of 300 tokens (the projection -> reduce-scatter -> all-gather path), then decode steps (the in-kernel
combine), logits of the last prefill row and of every decode step.  World size 1 runs the same thing without a
process group: the oracle the parallel runs are compared with."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, preset, n_new = sys.argv[1], sys.argv[2], int(sys.argv[3])
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from phaseshift_b200.models.qwen35.config import Qwen35Config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_getter
    from phaseshift_b200.runtime.batch import SeqRows
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    cfg = Qwen35Config(vocab_size=8192, hidden_size=2048, intermediate_size=4096, num_hidden_layers=4,
                       linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128, linear_value_head_dim=128,
                       num_attention_heads=16, num_key_value_heads=4, head_dim=128, name="qwen35-mid")
    tp = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from phaseshift_b200.parallel.tp import TensorParallel
        tp = TensorParallel(dist.group.WORLD, dev)
    ew = build_engine_weights(cfg, random_getter(cfg, 0, dev), preset, dev, tp_rank=rank, tp_size=world)
    eng = Engine(ew, dev, StateConfig(max_slots=2, max_seq_len=512), tp=tp)
    prompt = torch.randint(0, cfg.vocab_size, (300,), generator=torch.Generator().manual_seed(5)).tolist()
    s = eng.open_sequence()
    logits = []
    toks, out = eng.step([SeqRows(s.slot, 0, prompt, (len(prompt) - 1,))], [s], want_logits=True, tap_layers=[0])
    logits.append(out.logits[0].float().clone())
    layer0 = out.taps[0][:len(prompt)].float().clone()
    tokens = [toks[0]]
    for _ in range(n_new):
        toks, out = eng.step([SeqRows(s.slot, s.position, [tokens[-1]], (0,))], [s], want_logits=True)
        logits.append(out.logits[0].float().clone())
        tokens.append(toks[0])
    lg = torch.stack(logits)
    # one row-parallel projection of 300 rows in isolation, through the model's own routing (pushed reduce-scatter +
    # owner reduce + all-gather) against fp32 partials summed by the library collective
    collective_err = 0.0
    if world > 1:
        W = ew.layers[0].down
        g = torch.Generator(device=dev).manual_seed(11)        # same activations on every rank, sliced like the weights
        xin = torch.randn(300, W.K * world, device=dev, generator=g).to(torch.bfloat16)[:, rank * W.K:(rank + 1) * W.K].contiguous()
        resid = torch.randn(300, W.N, device=dev, generator=g).to(torch.bfloat16)
        got, _ = eng.runner._row_parallel(xin, W, resid, "x_a", 300)
        part = eng.ops.linear(xin, W, name="chk_part", out_f32=True).clone()
        dist.all_reduce(part)
        ref = part.to(torch.bfloat16).float() + resid.float()
        collective_err = float((got[:300].float() - ref).norm() / ref.norm())
    disagreement = 0.0
    if world > 1:
        gl = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(gl, lg)
        disagreement = float(max((x - lg).abs().max() for x in gl))
    res = {"rank": rank, "tokens": tokens, "status": int(eng.ops.status[0]), "rank_disagreement": disagreement,
           "collective_err": collective_err,
           "stats": tp.stats if tp is not None else {}, "transport": tp.transport if tp is not None else "none",
           "graphs": len(eng.graphs)}
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, res)
    else:
        gathered = [res]
    if rank == 0:
        torch.save({"logits": lg.cpu(), "layer0": layer0.cpu()}, out_path + ".pt")
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
