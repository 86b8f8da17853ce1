"""Worker of tests/test_gpu_dp.py (one process per GPU, launched with torch.distributed.run).

Every rank builds the same small LM and draws its own tokens.  The data-parallel step (NCCL behind the C ABI,
per-layer buckets overlapped with the backward), run eagerly and as a captured CUDA graph, must leave on every rank
the mean of the per-rank gradients, which each rank also computes by itself by running every rank's tokens through
the single-GPU step."""
import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "photon-mamba2-llm_b200")); sys.path.insert(0, str(ROOT / "tests"))


def main():
    import pm_b200 as pm
    from oracle import mamba2_oracle as orc
    from util import block_params, cuda_params, randn, rel_err, to_pm_cfg
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)

    def say(msg):            # progress lines (flushed): a run that stops somewhere still shows where
        print(f"rank {rank}: {msg}", flush=True)
    dist.init_process_group("gloo")          # host channel for the id only; the gradients go through pmb_dp_*
    box = [pm.DataParallel.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    say("id exchanged")
    dp = pm.DataParallel(world, rank, box[0])
    say("communicator ready")
    hier = len(sys.argv) > 1 and sys.argv[1] == "hier"
    cfg = orc.Mamba2Config(d_model=64, d_state=8, d_head=16, n_heads=4, block_len=32)
    L, B, T, V = 3, 2, 64, 301
    layers = [block_params(cfg, seed=90 + i) for i in range(L + (2 if hier else 0))]
    kw = dict(level1_layers=2, group=4) if hier else {}
    lm = pm.FlatMamba(to_pm_cfg(cfg), L, V, B, T, **kw)
    lm.load(randn((V, 64), 17, 0.5).cuda(), [cuda_params(p) for p in layers], wproj=randn((64, 64), 18, 0.125).cuda() if hier else None)
    toks = [orc.lcg_batch(100 + r, B, T, V)[:2] for r in range(world)]
    mean = torch.zeros_like(lm.flat_grads)
    for ids, tg in toks:                                   # every rank's gradients, computed locally
        lm.step_device(ids.cuda(), tg.cuda())
        mean += lm.flat_grads
    mean /= world
    say("local reference done")
    ids, tg = (t.cuda() for t in toks[rank])
    lm.step_device_dp(ids, tg, dp)
    torch.cuda.synchronize()
    e_eager = rel_err(lm.flat_grads, mean)
    say(f"eager step done {e_eager:.2e}")
    step = lm.capture_step(dp=dp)
    say("captured")
    lm.flat_grads.zero_()
    step(ids, tg)
    torch.cuda.synchronize()
    e_graph = rel_err(lm.flat_grads, mean)
    ok = e_eager < 1e-6 and e_graph < 1e-6 and pm.device_status() == 0
    print(f"rank {rank}: eager {e_eager:.2e} graph {e_graph:.2e} {'OK' if ok else 'FAIL'}", flush=True)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    say("closing")
    del step                 # NCCL keeps a communicator alive while a captured graph uses it: graphs go first
    torch.cuda.synchronize()
    dp.close(); lm.close()
    dist.destroy_process_group()
    say("closed")
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
