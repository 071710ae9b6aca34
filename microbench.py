"""Kernel microbenchmarks (one JSON line per kernel), timed with CUDA events on the launching stream.

    python microbench.py [attn] [gemm] [norm] [engine] [--iters N] [--small]
                                          [--rows R] [--splits S] [--min-len L] [--max-len L]   (attn only)
                                          [--n N]                                               (gemm only)

  attn : ragged paged decode attention, 1024 sequences, 12 heads x 64, KV lengths U[1,512] (seed 3),
         bf16 K/V ~ N(0,1), block 16.  Reports algorithmic GB/s against the measured HBM peak.
  gemm : tcgen05 bf16 GEMM, M = 32768, K = 768, N in {2304, 3072, 50257}. Reports TFLOP/s.
  norm : fused RMSNorm + RoPE (+ residual) on 32768 x 768 rows, f32 in / bf16 out. Reports GB/s.
  engine : steady-state decode steps of the 162M engine with 64 ragged sequences in flight
         (not in the default set; the launch sequence to hand to a profiler).
  session : batch-1 prefill + greedy decode through the session API, fp32 and bf16 (not in the default set).
  prefill : causal prefill attention over the paged pools, both model shapes (not in the default set). Reports TFLOP/s.

`--small` shrinks every case (for a profiler capture: inputs stay above the 126 MB L2 where it
matters, a few launches, well under a GB on the device).
Every input is larger than L2 or the buffers are rotated, so no iteration re-reads a warm cache.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _opt(name, default):
    """Value of a `--name value` command-line option."""
    return sys.argv[sys.argv.index(name) + 1] if name in sys.argv else default


def timed(torch, fn, iters, warmup=3):
    st = torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for _ in range(iters):
        fn()
    e1.record(st)
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_attn(ak, torch, iters, small):
    rows, heads, hd, max_blocks = (256 if small else 1024), 12, 64, 32
    rows = int(_opt("--rows", rows))
    splits = int(_opt("--splits", 0))      # 0 = the library's own plan
    lo = int(_opt("--min-len", 1))
    hi = int(_opt("--max-len", 512))
    lens = ak.uniform_ints(rows, lo, hi, seed=3)
    n_blocks = rows * max_blocks
    g = torch.Generator(device="cuda").manual_seed(3)
    # pools are rotated between launches so that together they exceed L2 (126 MB), as the 12 layers' pools do
    # inside the engine: every launch streams its K/V from HBM
    pool_bytes = 2 * n_blocks * heads * 16 * hd * 2
    n_sets = max(1, min(8, -(-512 * 1024 * 1024 // pool_bytes)))
    kps = [torch.randn(n_blocks, heads, 16, hd, device="cuda", generator=g).bfloat16() for _ in range(n_sets)]
    vps = [torch.randn(n_blocks, heads, 16, hd, device="cuda", generator=g).bfloat16() for _ in range(n_sets)]
    perm = torch.randperm(n_blocks, device="cuda", generator=g).to(torch.int32).reshape(rows, max_blocks)
    q = torch.randn(rows, heads * hd, device="cuda", generator=g).bfloat16()
    out = torch.empty_like(q)
    kv_lens = torch.from_numpy(lens.astype(np.int32)).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    nb = ak.ops.attn_decode_scratch_bytes(rows, heads, hd, max_blocks, splits, ak.AK_BF16)
    scratch = torch.zeros(max(nb, 16), dtype=torch.uint8, device="cuda")
    it = [0]

    def fn():
        i = it[0] % n_sets
        it[0] += 1
        ak.ops.attn_decode_paged(q, kps[i], vps[i], perm, kv_lens, out, rows, heads, hd, max_blocks, 0.125,
                                 ak.AK_BF16, splits, n_blocks, scratch, stream)
    ms = timed(torch, fn, iters)
    sumL = int(lens.sum())
    alg = sumL * heads * hd * 2 * 2 + rows * heads * hd * 2 * 2 + int(((lens + 15) // 16).sum()) * 4
    hbm, _, src = peaks()
    gbs = alg / (ms * 1e-3) / 1e9
    return {"kernel": "attn_decode_paged_kernel<bf16,64>", "rows": rows, "n_splits": splits or "auto", "pool_sets": n_sets,
            "sum_kv_len": sumL, "ms": ms, "algorithmic_bytes": alg, "GB/s": gbs, "peak_GB/s": hbm, "frac": gbs / hbm,
            "peak_source": src}


def bench_gemm(ak, torch, iters, small):
    res = []
    M, K = (4096 if small else 32768), 768
    _, tf, src = peaks()
    stream = torch.cuda.current_stream().cuda_stream
    only_n = int(_opt("--n", 0))            # one N only (a profiler capture of the full-size launch)
    for N in ((only_n,) if only_n else (2304, 3072, 50257)):
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        wt = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        ldc = (N + 7) // 8 * 8      # a row pitch of whole 16-byte vectors (50257 -> 50264)
        c = torch.empty(M, ldc, device="cuda", dtype=torch.bfloat16)
        fn = lambda: ak.ops.gemm_bf16(a, wt, c, M, N, K, ak.EPI_STORE_BF16, stream, ldc=ldc)
        ms = timed(torch, fn, max(3, iters // (8 if N > 10000 else 1)))
        fl = 2.0 * M * N * K
        t = fl / (ms * 1e-3) / 1e12
        res.append({"kernel": "gemm_bf16_kernel (tcgen05)", "m": M, "n": N, "k": K, "ldc": ldc, "ms": ms, "TFLOP/s": t,
                    "peak_TFLOP/s": tf, "frac": t / tf, "peak_source": src})
        del a, wt, c
    return res


def bench_skinny(ak, torch, iters, small):
    """The four per-layer GEMMs of a 64-row decode step, each as a chain of 12 launches over 12
    different weight sets (170 MB in total, more than L2) replayed from a CUDA graph, so that
    each launch sees the launch-to-launch overlap and the cold weights it sees inside the engine."""
    M = int(_opt("--m", 64))
    shapes = [("qkv", 2304, 768, ak.EPI_STORE_F32), ("out", 768, 768, ak.EPI_ADD_F32),
              ("up", 3072, 768, ak.EPI_SILU_BF16), ("down", 768, 3072, ak.EPI_ADD_F32)]
    res = []
    for name, N, K, epi in shapes:
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        wts = [(torch.randn(N, K, device="cuda") * 0.05).bfloat16() for _ in range(12)]
        pad = [torch.empty(9 * 1024 * 1024 // 2, device="cuda", dtype=torch.bfloat16) for _ in range(12)]  # spacing, as other layers' weights
        c = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if epi == ak.EPI_SILU_BF16 else torch.float32)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            stream = side.cuda_stream
            for wt in wts:
                ak.ops.gemm_bf16(a, wt, c, M, N, K, epi, stream)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(4):
                    for wt in wts:
                        ak.ops.gemm_bf16(a, wt, c, M, N, K, epi, torch.cuda.current_stream().cuda_stream)
            ms = timed(torch, g.replay, iters)
        res.append({"kernel": "gemm_bf16_kernel chain", "op": name, "m": M, "n": N, "k": K, "us_per_launch": 1e3 * ms / 48})
        del a, wts, c, pad
    return res


def bench_prefill(ak, torch, iters, small):
    """Causal prefill attention over the paged pools (tcgen05 kernel), the two model shapes: tensor-core flops
    4 * H * hd * sum(P^2 / 2) per launch against the measured bf16 peak."""
    res = []
    _, tf, src = peaks()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(7)
    cases = [("162M: 12 heads x 64, 32 prompts of 448", 12, 64, [448] * 32),
             ("162M: 12 heads x 64, 8 prompts of 2048", 12, 64, [2048] * (2 if small else 8)),
             ("1.4B: 16 heads x 128, 8 prompts of 2048", 16, 128, [2048] * (2 if small else 8)),
             ("1.4B: 16 heads x 128, ragged U[128,3072] x 16", 16, 128, [int(v) for v in ak.uniform_ints(4 if small else 16, 128, 3072, seed=5)])]
    for name, H, hd, lens in cases:
        dim, n = H * hd, len(lens)
        max_blocks = (max(lens) + 15) // 16
        n_blocks = n * max_blocks
        kp = torch.randn(n_blocks, H, 16, hd, device="cuda", generator=g).bfloat16()
        vp = torch.randn(n_blocks, H, 16, hd, device="cuda", generator=g).bfloat16()
        tables = torch.randperm(n_blocks, device="cuda", generator=g).to(torch.int32).reshape(n, max_blocks)
        cu = np.zeros(n + 1, np.int32)
        cu[1:] = np.cumsum(lens)
        total = int(cu[-1])
        q = torch.randn(total, dim, device="cuda", generator=g).bfloat16()
        out = torch.empty_like(q)
        dcu = torch.from_numpy(cu).cuda()
        slot = torch.arange(n, dtype=torch.int32, device="cuda")
        scale = 1.0 / float(np.sqrt(hd))
        fn = lambda: ak.ops.attn_prefill_paged(q, kp, vp, tables, max_blocks, dcu, slot, out, n, max(lens), total, H, hd, scale,
                                               ak.AK_BF16, n_blocks, stream)
        ms = timed(torch, fn, max(3, iters // 4))
        fl = 4.0 * H * hd * sum(L * (L + 1) / 2 for L in lens)      # QK^T and PV over the causal half
        t = fl / (ms * 1e-3) / 1e12
        res.append({"kernel": "prefill_tc_kernel (tcgen05 causal attention)", "case": name, "prompt_tokens": total, "ms": ms,
                    "TFLOP/s": t, "peak_TFLOP/s": tf, "frac": t / tf, "peak_source": src})
        del kp, vp, q, out
    return res


def bench_norm(ak, torch, iters, small):
    rows, size, hd = (8192 if small else 32768), 768, 64
    nbuf = 4  # rotate buffers: 4 x (100 MB in + 50 MB out) > L2
    xs = [torch.randn(rows, size, device="cuda") for _ in range(nbuf)]
    rs = [torch.randn(rows, size, device="cuda") for _ in range(nbuf)]
    ys = [torch.empty(rows, size, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
    w = torch.ones(size, device="cuda")
    pos = (torch.arange(rows, device="cuda", dtype=torch.int32) % 512).contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    hbm, _, src = peaks()
    out = []
    for name, use_res, use_rope in (("rmsnorm", False, False), ("rmsnorm+rope", False, True),
                                    ("rmsnorm+rope+residual", True, True)):
        it = [0]

        def fn():
            i = it[0] % nbuf
            it[0] += 1
            ak.ops.rmsnorm_rope_residual(xs[i], rs[i] if use_res else None, w, ys[i], pos if use_rope else None, rows,
                                         size, 1e-5, hd if use_rope else 0, ak.AK_BF16, stream)
        ms = timed(torch, fn, iters)
        alg = rows * size * (4 + 2) + (rows * size * 8 if use_res else 0)
        gbs = alg / (ms * 1e-3) / 1e9
        out.append({"kernel": f"rmsnorm_rows_kernel ({name})", "rows": rows, "size": size, "ms": ms,
                    "algorithmic_bytes": alg, "GB/s": gbs, "peak_GB/s": hbm, "frac": gbs / hbm, "peak_source": src})
    return out


def bench_engine(ak, torch, iters, small):
    """Steady-state decode steps of the 162M engine (64 sequences in flight, ragged lengths):
    the launch sequence a profiler should look at. Admits 64 prompts, runs `warm` steps, then
    times `iters` decode-only steps (captured graph) with host wall clock around each step."""
    import time
    cfg = ak.ModelConfig.akasha_hall_1()
    ctx = ak.Context(0)
    w = ak.ModelWeights(ctx, cfg, ak.AK_BF16)
    w.init_synthetic(0, 0.02)
    eng = ak.Engine(ctx, w, max_seqs=64, max_seq_len=512, use_cuda_graph=True, attn_timing=True)
    lens = ak.uniform_ints(63 if "--mixed" in sys.argv else 64, 16, 448, seed=2)
    for i, l in enumerate(lens):
        eng.submit(ak.uniform_tokens(int(l), cfg.vocab_size, seed=100 + i), 512)
    warm = 4 if small else 40
    for _ in range(warm):
        eng.step()
    eng.reset_stats()
    t0 = time.perf_counter()
    for _ in range(iters):
        eng.step()
    dt = (time.perf_counter() - t0) / iters
    st = eng.stats()
    mixed = None
    if "--mixed" in sys.argv:
        # a steady-state admission: one more 232-token prompt joins 63 running sequences
        mixed = []
        for rep in range(3):
            eng.submit(ak.uniform_tokens(232, cfg.vocab_size, seed=999 + rep), 232 + 3)
            t1 = time.perf_counter()
            eng.step()
            mixed.append((time.perf_counter() - t1) * 1e3)
            for _ in range(4):
                eng.step()
    out = {"kernel": "engine decode step (162M, 64 seqs)", "ms_per_step": dt * 1e3, "tok/s": 64 / dt,
           "kernels_per_step": st["kernel_launches"] / max(1, st["steps"]),
           "attn_us_layer0": 1e3 * st["attn_ms_total"] / max(1, st["attn_launches_timed"]),
           "attn_GB/s": st["attn_bytes_total"] / max(1e-9, st["attn_ms_total"] * 1e-3) / 1e9,
           "gpu_ms_per_step": st["step_gpu_ms_total"] / max(1, st["steps"]),
           "graph_launch_host_ms_per_step": st["launch_host_ms_total"] / max(1, st["graph_launches"])}
    if mixed:
        out["mixed_step_ms"] = mixed   # first entry includes the bucket's graph capture
    eng.close(); w.close(); ctx.close()
    return out


def bench_session(ak, torch, iters, small):
    """Batch-1 generation with the session API (the reference's own use: one sequence, one token per
    step): 162M model, 512-token prompt, then 384 greedy decode steps (context 1024), in fp32 parity mode
    and in bf16. Per decode step the weights are streamed once (494.2 MB fp32 / 247.1 MB bf16) plus the
    sequence's K/V; the fraction is that stream against the measured HBM peak. Wall clock around the
    library's own generate loop (prefill timed apart)."""
    import time
    cfg = ak.ModelConfig.akasha_hall_1()
    hbm, _, src = peaks()
    n_prompt, n_new = (128, 64) if small else (512, 384)
    prompt = ak.uniform_tokens(n_prompt, cfg.vocab_size, seed=1)
    out = []
    for name, dt, esz in (("f32", ak.AK_F32, 4), ("bf16", ak.AK_BF16, 2)):
        ctx = ak.Context(0)
        w = ak.ModelWeights(ctx, cfg, dt)
        w.init_synthetic(0, 0.02)
        s = ak.InferenceSession(ctx, w, 1024)
        best = None
        for rep in range(2):   # the first pass captures the decode graph
            s.replace_cache()
            t0 = time.perf_counter()
            tok = s.prefill(prompt, want_logits=False)
            t1 = time.perf_counter()
            for _ in range(n_new):
                tok = s.decode_step(tok, want_logits=False)
            t2 = time.perf_counter()
            best = (t1 - t0, t2 - t1)
        pf_s, dec_s = best
        w_bytes = 123_551_232 * esz
        kv_bytes = (n_prompt + n_new / 2) * 18_432 * esz
        gbs = (w_bytes + kv_bytes) * n_new / dec_s / 1e9
        out.append({"kernel": f"session batch-1 decode ({name})", "prompt": n_prompt, "decode_steps": n_new,
                    "prefill_ms": pf_s * 1e3, "decode_tok/s": n_new / dec_s, "us_per_token": 1e6 * dec_s / n_new,
                    "stream_bytes_per_token": w_bytes + kv_bytes, "GB/s": gbs, "peak_GB/s": hbm, "frac": gbs / hbm,
                    "peak_source": src})
        s.close(); w.close(); ctx.close()
    return out


def main():
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    ak = entry.load_package()
    args = [a for a in sys.argv[1:] if a in ("attn", "gemm", "norm", "engine", "skinny", "session", "prefill")]
    iters = int(_opt("--iters", 20))
    small = "--small" in sys.argv
    which = args or ["attn", "gemm", "norm"]
    torch.cuda.set_device(0)
    for w in which:
        r = {"attn": bench_attn, "gemm": bench_gemm, "norm": bench_norm, "engine": bench_engine, "skinny": bench_skinny, "session": bench_session, "prefill": bench_prefill}[w](ak, torch, iters, small)
        for line in (r if isinstance(r, list) else [r]):
            print(json.dumps(line))
    torch.cuda.synchronize()
    ak.check(ak.lib().ak_check_device_status(None))


if __name__ == "__main__":
    main()
