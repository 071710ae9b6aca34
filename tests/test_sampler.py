"""`sample_token` (src/nn/sampling.rs): the oracle against the reference's own KATs on CPU, and
the on-device sampler against the oracle with the same uniform draws on GPU."""
import numpy as np
import pytest

LOGITS = np.array([1.0, 4.0, 2.0, 8.0, 3.0], np.float32)   # src/nn/sampling.rs:97


def test_oracle_sampler_kats(orc):
    rs = [i / 20.0 for i in range(20)]
    assert all(orc.sample_token(LOGITS, 0.0, 0, 1.0, r=r) == 3 for r in rs)          # zero_temperature_is_greedy
    assert all(orc.sample_token(LOGITS, 1.5, 1, 1.0, r=r) == 3 for r in rs)          # top_k_one_is_greedy
    assert all(orc.sample_token(LOGITS, 2.0, 2, 1.0, r=r) in (3, 1) for r in rs)     # top_k_restricts_candidates
    assert all(orc.sample_token(LOGITS, 1.0, 0, 0.01, r=r) == 3 for r in rs)         # tiny_top_p_is_greedy
    seen = {orc.sample_token(LOGITS, 100.0, 0, 1.0, r=(i + 0.5) / 2000.0) for i in range(2000)}
    assert seen == {0, 1, 2, 3, 4}                                                   # filters_off_can_reach_every_token
    assert orc.sample_token(LOGITS, 0.0, 0, 1.0, seen=[3], penalty=100.0) == 1       # repetition penalty demotes


@pytest.mark.gpu
def test_device_sampler_matches_oracle(ak, orc, torch_cuda):
    torch = torch_cuda
    rows, V = 12, 50257
    rng = np.random.default_rng(7)
    logits = (rng.standard_normal((rows, V)) * 2.0).astype(np.float32)
    logits[3, 100] = logits[3, 50] = logits[3].max() + 1.0   # tie at the top: index order decides
    seen_lists = [rng.integers(0, V, size=rng.integers(1, 300)).astype(np.uint32) for _ in range(rows)]
    off = np.zeros(rows + 1, np.uint32)
    off[1:] = np.cumsum([len(s) for s in seen_lists])
    seen = np.concatenate(seen_lists)
    d_logits = torch.from_numpy(logits).cuda()
    d_seen = torch.from_numpy(seen.view(np.int32)).cuda()
    d_off = torch.from_numpy(off.view(np.int32)).cuda()
    # top_k = 0 is "no truncation" (src/nn/sampling.rs:41-43): the whole vocabulary is the candidate list
    for (T, k, p, pen) in [(0.8, 40, 0.95, 1.15), (1.5, 1, 1.0, 1.0), (2.0, 2, 1.0, 1.0), (1.0, 64, 0.01, 1.0),
                           (0.0, 40, 0.95, 100.0), (100.0, 1000, 1.0, 1.0),
                           (1.0, 0, 1.0, 1.0), (0.8, 0, 0.95, 1.15), (100.0, 0, 1.0, 1.0), (1.0, 0, 0.01, 1.0), (0.3, 0, 0.5, 1.0)]:
        for step in range(4):
            out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
            ak.ops.sample_token(d_logits, rows, V, out, T, k, p, 1234, step, d_seen, d_off, pen)
            torch.cuda.synchronize()
            got = out.cpu().numpy().astype(np.int64)
            for r in range(rows):
                u = ak.ops.sampler_uniform(1234, step, r)
                want = orc.sample_token(logits[r], T, k, p, seen_lists[r], pen, r=u)
                assert got[r] == want, (T, k, p, pen, step, r, got[r], want)
    # the --chat defaults (src/main.rs:160-162) draw different tokens for different steps
    picks = set()
    for step in range(40):
        out = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ak.ops.sample_token(d_logits, rows, V, out, 0.8, 40, 0.95, 99, step)
        picks.add(int(out[0]))
    assert len(picks) > 3
    with pytest.raises(ak.AkashaError):
        ak.ops.sample_token(d_logits, rows, V, out, 1.0, 5000, 1.0, 1, 0)  # 1024 < top_k < vocabulary: not offered on the device


@pytest.mark.gpu
@pytest.mark.parametrize("settings", [(0.8, 40, 0.95, 1.15), (0.0, 0, 1.0, 3.0), (1.3, 5, 1.0, 1.0)])
def test_session_generate_samples_like_the_reference_loop(ak, orc, ctx, settings):
    """`generate` with the sampler on the device (src/nn/inference.rs:264-326): every token is what
    `sample_token` returns for the oracle's logits of that step, the history so far (prompt + generated)
    and the same uniform draw; fp32 parity mode, teacher-forced with the GPU's own tokens."""
    T, k, p, pen = settings
    cfg = ak.ModelConfig(300, 64, 2, 2, 64)
    params = ak.synthetic_weights(cfg, seed=21, std=0.35)     # large weights: a peaked next-token distribution
    w = ak.ModelWeights.from_params(ctx, cfg, params, ak.AK_F32)
    prompt = ak.uniform_tokens(9, cfg.vocab_size, seed=4)
    s = ak.InferenceSession(ctx, w, 48)
    got = s.generate(prompt, 30, stop_on_eos=False, temperature=T, top_k=k, top_p=p, repetition_penalty=pen, seed=77)
    assert len(got) == 30
    om = orc.Model(cfg.as_dict(), params)
    os_ = orc.Session(om, 48)
    rc, logits = os_.prefill(prompt)
    hist = list(prompt)
    for i, tok in enumerate(got):
        want = orc.sample_token(logits, T, k, p, hist, pen, r=ak.ops.sampler_uniform(77, i, 0))
        assert want == int(tok), f"token {i}: device {int(tok)}, reference loop {want}"
        hist.append(int(tok))
        rc, logits = os_.decode_step(int(tok))
    if T > 0:
        other = s2 = None
        s.reset_cache()
        other = s.generate(prompt, 30, stop_on_eos=False, temperature=T, top_k=k, top_p=p, repetition_penalty=pen, seed=78)
        assert len(other) == 30   # another seed is another stream of draws (it may or may not differ on a peaked model)
    s.close(); w.close()
