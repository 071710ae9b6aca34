#!/usr/bin/env python
"""Headline benchmark: continuous-batching decode throughput of the 162M akasha-hall model.

Workload (one "step" = one full pass over it): 256 sequences, prompt lengths uniform in [16,448]
(seed 2), token ids uniform in [0,50257), each generating until its total length is 512, at most
64 sequences in flight, a finished sequence's slot refilled at once; paged KV cache with block
size 16; bf16 weights/KV/activations with fp32 accumulation; greedy sampling on the device.
Metric: generated tokens per second (prefill time of the admitted prompts is inside the timed
region). N GPUs = N independent engines, each with its own 256 sequences (weak scaling, no
data-path collective); value is the aggregate over ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`--impl reference` times the CPU restatement of the reference's own path (the oracle, all host
threads) on a bounded sample of the same workload: each step runs ONE sequence of the workload in
full (prefill of its prompt, then greedy decode to length 512), a different sequence every step,
so the prompt : generated mix of the sample follows the workload's.
`--cpu-config1` prints the reference CPU path's own configuration instead (batch 1, prompt of 64
ids from seed 1, 128 greedy decode steps): prefill ms and decode tok/s, single-thread and all threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

N_SEQS, MAX_SEQS, TOTAL_LEN, LEN_LO, LEN_HI = 256, 64, 512, 16, 448
WORKLOAD = ("continuous-batching decode, akasha-hall 162M (dim 768, 12 layers, 12x64 heads, ffn 3072, vocab 50257), "
            "256 seqs, 64 in flight, prompts U[16,448] seed 2, run to length 512, paged KV block 16, bf16 + fp32 acc")


def make_prompts(ak, rank: int):
    lens = ak.uniform_ints(N_SEQS, LEN_LO, LEN_HI, seed=2 + 1000 * rank)
    return [ak.uniform_tokens(int(l), 50257, seed=10_000 * (rank + 1) + i) for i, l in enumerate(lens)]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def workload_config(ak):
    """The `config` object of the JSON line: the same for both arms."""
    gen = sum(TOTAL_LEN - len(p) for p in make_prompts(ak, 0))
    return {"workload": WORKLOAD, "generated_tokens_per_step": gen,
            "l2": "working set per engine step (247 MB weights + ~0.9 GB KV) exceeds the 126 MB L2"}


def cpu_reference_arm(ak, steps: int, warmup: int):
    """The reference's CPU path (restated by the oracle), fp32, all host threads, on a bounded sample
    of the workload: one step = one sequence of the workload run in full (prefill of its prompt, then
    greedy decode until its length is 512), sequences taken in workload order, one after the other
    (the reference has no batching). Over a handful of steps the prompt : generated mix follows the
    workload's (prompts are uniform in [16, 448])."""
    orc = entry.load_oracle()
    cfg = ak.ModelConfig.akasha_hall_1()
    params = ak.synthetic_weights(cfg, seed=0, std=0.02)
    model = orc.Model(cfg.as_dict(), params)
    prompts = make_prompts(ak, 0)
    # every core this process may run on (a launcher may have exported OMP_NUM_THREADS=1: the oracle's own
    # maximum would then read 1)
    cores = max(orc.max_threads(), len(os.sched_getaffinity(0)))
    orc.set_threads(cores)

    def one_seq(i):
        p = prompts[i % len(prompts)]
        t0 = time.perf_counter()
        s = orc.Session(model, TOTAL_LEN)
        st, toks, _ = s.generate_greedy(p, TOTAL_LEN - len(p))
        return len(p), len(toks), time.perf_counter() - t0

    for i in range(warmup):
        one_seq(steps + i)
    n_prompt = gen = 0
    total = 0.0
    for i in range(steps):
        pl, g, t = one_seq(i)
        n_prompt += pl
        gen += g
        total += t
    sample = (f"{steps} of the workload's 256 sequences, each run in full (prompt prefill + greedy decode to length 512; "
              f"{n_prompt} prompt tokens, {gen} generated), one after the other, fp32 oracle, {cores} OpenMP threads")
    return {"value": gen / total, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step": 1e3 * total / steps}


def cpu_config1(ak):
    """The reference CPU backend's own configuration: 162M fp32, batch 1, prompt = 64 ids (seed 1), prefill then
    128 greedy decode steps; timed single-thread (the reference's CPU kernels are scalar loops) and on all threads."""
    orc = entry.load_oracle()
    cfg = ak.ModelConfig.akasha_hall_1()
    model = orc.Model(cfg.as_dict(), ak.synthetic_weights(cfg, seed=0, std=0.02))
    prompt = ak.uniform_tokens(64, cfg.vocab_size, seed=1)
    cores = max(orc.max_threads(), len(os.sched_getaffinity(0)))
    out = {"config": "akasha-hall 162M fp32, batch 1, prompt 64 ids (seed 1), 128 greedy decode steps, CPU oracle"}
    for name, th in (("single_thread", 1), ("all_threads", cores)):
        orc.set_threads(th)
        s = orc.Session(model, TOTAL_LEN)
        t0 = time.perf_counter()
        rc, logits = s.prefill(prompt)
        t1 = time.perf_counter()
        tok = int(np.argmax(logits))
        for _ in range(128):
            rc, logits = s.decode_step(tok)
            tok = int(np.argmax(logits))
        t2 = time.perf_counter()
        out[name] = {"threads": th, "prefill_ms": 1e3 * (t1 - t0), "decode_tok_s": 128 / (t2 - t1)}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-config1", action="store_true", help="print the reference CPU configuration's numbers and exit")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pin", action="store_true", help="multi-rank runs: do not pin each rank to its own host cores")
    ap.add_argument("--sync-steps", action="store_true", help="read every step's tokens before launching the next one")
    ap.add_argument("--chunked-prefill", action="store_true",
                    help="prefill a prompt admitted while others decode in 64-row chunks that ride in the decode launches")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Several ranks on one host: give each its own share of the host cores before any thread is created, so that one
    # rank's launch thread is never descheduled for another's (a host-side setting of this process, not of a GPU).
    cores_per_rank = None
    if world > 1 and not args.no_pin and args.impl != "reference" and hasattr(os, "sched_setaffinity"):
        cpus = sorted(os.sched_getaffinity(0))
        per = len(cpus) // world
        if per >= 1:
            os.sched_setaffinity(0, set(cpus[local_rank * per:(local_rank + 1) * per]))
            cores_per_rank = per
    ak = entry.load_package()

    if args.cpu_config1:
        if rank == 0:
            print(json.dumps(cpu_config1(ak)))
        return 0
    if args.impl == "reference":
        if rank != 0:
            return 0
        r = cpu_reference_arm(ak, max(1, args.steps), max(0, args.warmup))
        line = {"impl": "reference", "metric": "decode tok/s", "value": r["value"], "unit": "tok/s", "n_gpus": args.gpus,
                "steps": max(1, args.steps), "warmup": max(0, args.warmup), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(ak),
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    cfg = ak.ModelConfig.akasha_hall_1()
    ctx = ak.Context(local_rank)
    w = ak.ModelWeights(ctx, cfg, ak.AK_BF16)
    w.init_synthetic(seed=0, std=0.02)  # N(0, 0.02) matrices, N(1, 0.02) gains, generated on the device
    eng = ak.Engine(ctx, w, max_seqs=MAX_SEQS, max_seq_len=TOTAL_LEN, use_cuda_graph=not args.no_graph,
                    stop_on_eos=False, attn_timing=True, async_steps=not args.sync_steps,
                    prefill_chunk_rows=128 - MAX_SEQS if args.chunked_prefill else 0)
    prompts = make_prompts(ak, rank)
    gen_per_job = sum(TOTAL_LEN - len(p) for p in prompts)
    ext = torch.cuda.ExternalStream(ctx.stream, device=local_rank)

    CHECK = (0, 63, 64, 150, N_SEQS - 1)   # sequences whose ids the two timed legs must agree on

    def job(collect: bool):
        """One pass through the public API: submit (host prompts), step until done, poll outputs."""
        ids = [eng.submit(p, TOTAL_LEN) for p in prompts]
        eng.run_to_completion()
        n, kept = 0, {}
        if collect:
            for k, i in enumerate(ids):
                t, fin = eng.poll(i, TOTAL_LEN)
                assert fin
                n += len(t)
                if k in CHECK:
                    kept[k] = t
        eng.clear_finished()
        return n, kept

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 0)):
        job(False)
    leg1_ids = {}
    ctx.check_device_status()

    # ---- leg 1: device-timed (CUDA events on the engine's stream), prompts queued before the timer
    eng.reset_stats()
    launches0 = ak.launch_count()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms = 0.0
    for _ in range(args.steps):
        ids = [eng.submit(p, TOTAL_LEN) for p in prompts]
        with torch.cuda.stream(ext):
            e0.record()
        eng.run_to_completion()
        with torch.cuda.stream(ext):
            e1.record()
        e1.synchronize()
        dev_ms += e0.elapsed_time(e1)
        leg1_ids = {k: eng.poll(ids[k], TOTAL_LEN)[0] for k in CHECK}   # after the timer
        eng.clear_finished()
    barrier()
    st = eng.stats()
    eager_launches = ak.launch_count() - launches0

    # ---- leg 2: end to end through the public API with host buffers (wall clock incl. copies)
    barrier()
    t0 = time.perf_counter()
    got = 0
    for _ in range(args.steps):
        n, leg2_ids = job(True)
        got += n
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    assert got == gen_per_job * args.steps
    # same engine, same prompts: the device-timed leg and the end-to-end leg must have generated the same ids
    for k in CHECK:
        assert leg1_ids[k].tolist() == leg2_ids[k].tolist(), f"sequence {k}: ids differ between the two timed legs"
    st2 = eng.stats()
    ctx.check_device_status()

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms_max, e2e_ms_max = times.tolist()
    # per rank, so that a scaling loss can be attributed: the device-timed leg (ms per job), the GPU time of the
    # rank's own steps and the host time it spent launching them
    mine = torch.tensor([dev_ms / args.steps, st["step_gpu_ms_total"] / args.steps, st["launch_host_ms_total"] / args.steps],
                        dtype=torch.float64, device="cuda")
    per_rank = [mine.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    per_rank = [[round(v, 2) for v in t.tolist()] for t in per_rank]
    total_gen = gen_per_job * args.steps * world
    value = total_gen / (dev_ms_max / 1e3)
    e2e_value = total_gen / (e2e_ms_max / 1e3)

    if rank == 0:
        peak, peak_kind = measured_peak_hbm()
        attn_ms = st["attn_ms_total"] / max(1, st["attn_launches_timed"])
        attn_bytes = st["attn_bytes_total"] / max(1, st["attn_launches_timed"])
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9 if attn_ms > 0 else 0.0
        steps_per_job = st["steps"] / args.steps
        # whole decode step against the HBM roofline: every weight once, the K/V of all 12 layers, the appends
        n_dec = max(1, st["decode_steps_timed"])
        step_ms = st["decode_step_gpu_ms_total"] / n_dec
        step_bytes = st["decode_step_bytes_total"] / n_dec
        step_achieved = step_bytes / (step_ms * 1e-3) / 1e9 if step_ms > 0 else 0.0
        line = {
            "metric": "decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(ak),
            "e2e": {"value": e2e_value, "unit": "tok/s",
                    "h2d_bytes_per_step": (st2["h2d_bytes"] - st["h2d_bytes"]) / args.steps,
                    "d2h_bytes_per_step": (st2["d2h_bytes"] - st["d2h_bytes"]) / args.steps},
            "gpu_launches": int(st["kernel_launches"]),
            "roofline": {"bound": "hbm", "kernel": "attn_decode_paged_kernel<bf16,64,2> (layer 0, every decode-only step)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind,
                         # two CUDA events per step, recorded on a side stream of the captured step: "the qkv projection
                         # before it has completed" and "the attention launch has completed". The kernel keeps its
                         # launch overlap: its CTAs are resident and have requested their first K/V tiles before the
                         # first event, so this is the launch's share of the step's critical path, shorter than the
                         # same launch timed alone (16.1 us, 0.69 of peak: python microbench.py attn --rows 64 --min-len 232)
                         "timing": "events on a side stream inside the captured step: predecessor complete -> launch complete",
                         # DRAM bytes per launch: 1.059 x the algorithmic bytes, the ratio ncu measured
                         # (dram__bytes_read.sum + dram__bytes_write.sum) on a smaller launch of the same
                         # kernel; traffic grows in proportion to the K/V bytes
                         "traffic": 1.059 * attn_bytes,
                         "bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms, "launches_timed": st["attn_launches_timed"],
                         # the whole decode-only engine step (a captured graph of ~100 launches) against the same peak
                         "step": {"achieved": step_achieved, "frac": step_achieved / peak, "unit": "GB/s",
                                  "bytes_per_step": step_bytes, "ms_per_step": step_ms, "steps_timed": st["decode_steps_timed"]}},
            "clocks": clocks,
            "engine": {"decode_tokens": st["decode_tokens"], "prefill_tokens": st["prefill_tokens"],
                       "graph_launches": st["graph_launches"], "eager_steps": st["eager_steps"],
                       "host_counted_launches": int(eager_launches), "engine_steps_per_job": steps_per_job,
                       "cuda_graph": not args.no_graph, "async_steps": not args.sync_steps,
                       "chunked_prefill": args.chunked_prefill, "host_cores_per_rank": cores_per_rank,
                       # rank 0, per job (one pass over the 256 sequences): where the time goes
                       "gpu_ms_per_job": st["step_gpu_ms_total"] / args.steps,
                       "launch_host_ms_per_job": st["launch_host_ms_total"] / args.steps,
                       "per_rank_ms_per_job": {"columns": ["device_timed_leg", "gpu_steps", "launch_host"], "ranks": per_rank},
                       "ids_checked_between_legs": list(CHECK)},
        }
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_arm(ak, 4, 0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    eng.close(); w.close(); ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
