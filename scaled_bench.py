"""The scaled synthetic model (dim 2048, 24 layers, 16 heads x 128, ffn 8192, vocab 50257,
ctx 4096, ~1.4B parameters, bf16 random init): ragged sequences with prompts uniform in
[128, 3072], each generating `--gen` tokens, continuous batching with `--max-seqs` in flight.

    python scaled_bench.py [--seqs 512] [--gen 128] [--max-seqs 64]
    torchrun --nproc-per-node N ... scaled_bench.py             # sequences sharded over N GPUs
    torchrun --nproc-per-node 2 ... scaled_bench.py --tp 2      # 2-way tensor parallel (NCCL all-reduce)

Data parallel: every rank owns a round-robin shard of the SAME sequence list (strong scaling, no
data-path collective). Tensor parallel: the two ranks run the same schedule in lock step.
One JSON line from rank 0.
"""
from __future__ import annotations

import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def opt(name, default):
    return type(default)(sys.argv[sys.argv.index(name) + 1]) if name in sys.argv else default


def main():
    import torch
    import torch.distributed as dist
    ak = entry.load_package()
    from akasha_core_b200 import sharding
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n_seqs, gen, max_seqs, tp = opt("--seqs", 512), opt("--gen", 128), opt("--max-seqs", 64), opt("--tp", 1)
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = ak.ModelConfig.scaled_1p4b()
    ctx = ak.Context(local)
    if tp > 1:
        assert world == tp, "tensor-parallel run: launch exactly --tp ranks"
        obj = [ak.Context.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        ctx.tp_init(tp, rank, obj[0])
    w = ak.ModelWeights(ctx, cfg, ak.AK_BF16)
    w.init_synthetic(seed=0, std=0.02)
    lens = ak.uniform_ints(n_seqs, 128, 3072, seed=5)
    mine = list(range(n_seqs)) if tp > 1 else sharding.shard_round_robin(n_seqs, rank, world)
    prompts = [ak.uniform_tokens(int(lens[i]), cfg.vocab_size, seed=50_000 + i) for i in mine]
    max_len = 3072 + gen
    eng = ak.Engine(ctx, w, max_seqs=max_seqs, max_seq_len=max_len, max_batch_tokens=max_seqs + 16384,
                    use_cuda_graph=True, attn_timing=True, async_steps=(tp == 1))

    def job():
        ids = [eng.submit(p, len(p) + gen) for p in prompts]
        eng.run_to_completion()
        n = sum(len(eng.poll(i, gen + 1)[0]) for i in ids)
        eng.clear_finished()
        return n

    # warm-up on a slice (captures the step graphs), then the timed pass
    warm = [eng.submit(p, len(p) + 4) for p in prompts[:max(2, max_seqs // 8)]]
    eng.run_to_completion()
    eng.clear_finished()
    eng.reset_stats()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = job()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.stats()
    ctx.check_device_status()
    if tp > 1:
        thr, units, secs = n / dt, n, dt
    else:
        thr, units, secs = sharding.aggregate(dist if world > 1 else None, n, dt, device=torch.device("cuda", local))
    if rank == 0:
        print(json.dumps({
            "workload": f"scaled 1.4B bf16, {n_seqs} seqs, prompts U[128,3072] seed 5, {gen} generated tokens each, "
                        f"{max_seqs} in flight per engine",
            "mode": f"tp{tp}" if tp > 1 else f"dp{world}", "n_gpus": world, "generated_tokens": units, "seconds": secs,
            "tok/s": thr, "prompt_tokens_rank0": int(sum(len(p) for p in prompts)),
            "rank0": {"steps": st["steps"], "decode_tokens": st["decode_tokens"], "prefill_tokens": st["prefill_tokens"],
                      "attn_GB/s": st["attn_bytes_total"] / max(1e-9, st["attn_ms_total"] * 1e-3) / 1e9,
                      "attn_us_layer0": 1e3 * st["attn_ms_total"] / max(1, st["attn_launches_timed"]),
                      # where rank 0's time goes: device time of its steps, host time spent launching them
                      "gpu_ms_total": st["step_gpu_ms_total"], "launch_host_ms_total": st["launch_host_ms_total"]}}))
    eng.close(); w.close(); ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
