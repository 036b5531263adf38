"""Rank program for tests/test_tp_gpu.py (run under torch.distributed.run, one rank per GPU)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, preset, n_new = sys.argv[1], sys.argv[2], int(sys.argv[3])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
    from phaseshift_b200.parallel.tp import TensorParallel
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], preset, dev, tp_rank=rank, tp_size=world)
    tp = TensorParallel(dist.group.WORLD, dev)
    eng = Engine(ew, dev, StateConfig(max_slots=1, max_seq_len=96), tp=tp)
    out = eng.generate(list(range(3, 27)), n_new, prefill_chunk=8)
    torch.cuda.synchronize()
    # stand-alone peer-memory all-reduce (both variants) against the library collective
    ar = {}
    if tp.transport == "fused":
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        for variant in ("peer", "multimem"):
            tp.use_multimem = variant == "multimem"
            errs = []
            for rows in (9, 300, 300):
                part = (torch.randn(rows, 512, device=dev, generator=g) * 0.5).to(torch.bfloat16)
                resid = torch.randn(rows, 512, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).to(torch.bfloat16)
                got = torch.empty_like(part)
                tp.peer_all_reduce(part, resid, got)
                ref = part.float()
                dist.all_reduce(ref)
                ref = ref.to(torch.bfloat16).float() + resid.float()
                errs.append(float((got.float() - ref).abs().max()))
                gl = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(gl, got)
                errs.append(float(max((x.float() - got.float()).abs().max() for x in gl)))     # ranks agree bit for bit
            ar[variant] = {"max_err": max(errs[0::2]), "rank_disagreement": max(errs[1::2]),
                           "status": int(tp._ar["status"][0]), "multicast": bool(tp._ar["mc_in"])}
    res = {"rank": rank, "tokens": out, "transport": tp.transport, "stats": tp.stats,
           "status": int(eng.ops.status[0]), "graphs": len(eng.graphs), "allreduce": ar}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
