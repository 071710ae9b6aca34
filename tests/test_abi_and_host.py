"""CPU: the C-ABI library loads and exports every symbol the header declares (no compute calls),
the meta structs have the reference's layout, and the host-side helpers behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        names += re.findall(r"AK_API\s+[\w\s\*]+?\b(ak_\w+)\s*\(", text)
    return names


def test_every_declared_symbol_is_exported(ak):
    L = ak.lib()
    names = _declared_functions()
    assert len(names) >= 60
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert b"sm_100a" in L.ak_version()


def test_every_bound_prototype_is_declared(ak):
    declared = set(_declared_functions())
    assert set(ak._PROTOS) <= declared


def test_meta_struct_layouts(ak):
    # src/nn/ops/meta.rs: all members are 4 bytes, #[repr(C)]
    assert C.sizeof(ak.MatMulMeta) == 12 and C.sizeof(ak.NormMeta) == 12
    assert C.sizeof(ak.HeadMoveMeta) == 16 and C.sizeof(ak.AttnCachedMeta) == 12
    assert C.sizeof(ak.SoftmaxRectMeta) == 12 and C.sizeof(ak.RopeMeta) == 16
    assert C.sizeof(ak.RopeOffsetMeta) == 16 and C.sizeof(ak.CacheWriteMeta) == 12
    assert C.sizeof(ak.EmbeddingMeta) == 12 and C.sizeof(ak.FlashAttnMeta) == 20
    m = ak.FlashAttnMeta(5, 6, 7, 0.5, 9)
    raw = bytes(m)
    assert np.frombuffer(raw[:12], np.uint32).tolist() == [5, 6, 7]
    assert np.frombuffer(raw[12:16], np.float32)[0] == 0.5 and np.frombuffer(raw[16:], np.uint32)[0] == 9


def test_errors_without_gpu_are_loud(ak):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(ak.AkashaError) as e:
        ak.Context(0)
    assert e.value.code in (100, 101)


def test_model_config_mirror(ak):
    c = ak.ModelConfig.akasha_hall_1()  # src/config.rs:54-56
    assert (c.vocab_size, c.dim, c.num_heads, c.num_layers, c.seq_len) == (50257, 768, 12, 12, 512)
    assert c.ffn_hidden == 3072 and c.eos_token == 50256 and c.head_dim == 64 and abs(c.norm_eps - 1e-5) < 1e-12
    assert c.n_params == 162_148_608
    assert len(c.param_shapes()) == 1 + 6 * 12 + 2
    assert c.param_shapes()[2] == (768, 2304) and c.param_shapes()[-1] == (768, 50257)
    p = ak.ModelConfig.pidgeon()
    assert p.head_dim == 64 and p.num_layers == 8
    s = ak.ModelConfig.scaled_1p4b()
    assert s.head_dim == 128 and s.n_params == 1_413_912_576
    with pytest.raises(AssertionError):
        ak.ModelConfig(10, 30, 4, 1, 8)


def test_synthetic_inputs_are_deterministic(ak):
    cfg = ak.ModelConfig(97, 32, 4, 2, 16)
    a = ak.synthetic_weights(cfg, seed=0)
    b = ak.synthetic_weights(cfg, seed=0)
    c = ak.synthetic_weights(cfg, seed=1)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    assert not np.array_equal(a[0], c[0])
    assert [x.shape for x in a] == cfg.param_shapes()
    big = ak.normal_f32(200000, 0, 3, 0.0, 0.02)
    assert abs(big.mean()) < 3e-4 and abs(big.std() - 0.02) < 3e-4
    gains = a[1]
    assert abs(gains.mean() - 1.0) < 0.02
    t = ak.uniform_tokens(1000, 50257, 1)
    assert t.dtype == np.uint32 and t.max() < 50257 and len(set(t.tolist())) > 900
    lens = ak.uniform_ints(256, 16, 448, 2)
    assert lens.min() >= 16 and lens.max() <= 448


def test_error_names(ak):
    e = ak.AkashaError(3, "context window is full (16 tokens)")
    assert e.kind == "ContextFull" and "full" in str(e)


def _struct_fields(name):
    """Member names of `typedef struct <name> { ... } <name>;` in the public header, in order."""
    text = open(os.path.join(ROOT, "include", "akasha_b200.h")).read()
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split(";"):
        m = re.match(r"\s*(?:uint32_t|uint64_t|float|double|int32_t)\s+(.*)", decl.strip(), re.S)
        if m:
            names += [n.strip() for n in m.group(1).split(",")]
    return names


def test_engine_structs_match_the_header(ak):
    """The ctypes mirrors of the engine's config and statistics structs list the header's members in
    the header's order (a member added on one side only would shift every later one)."""
    assert [f for f, _ in ak.EngineConfig._fields_] == _struct_fields("ak_engine_config")
    assert [f for f, _ in ak.EngineStats._fields_] == _struct_fields("ak_engine_stats")
    assert C.sizeof(ak.EngineConfig) == 4 * len(ak.EngineConfig._fields_)


def test_reference_arm_uses_every_core_under_a_launcher():
    """`bench.py --impl reference` prints one JSON line from the CPU oracle and does not let a
    launcher's OMP_NUM_THREADS=1 shrink it to one thread."""
    import json
    import subprocess
    import sys
    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode tok/s" and d["value"] > 0
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0)) and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
