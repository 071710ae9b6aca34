"""AKV3 checkpoint reader (src/nn/checkpoint.rs). The header reader runs on CPU; loading tensors
into device weights is a GPU test."""
import struct

import numpy as np
import pytest


def test_header_roundtrip_and_bad_magic(ak, tmp_path):
    cfg = ak.ModelConfig(97, 32, 4, 2, 16)
    params = ak.synthetic_weights(cfg, seed=3, std=0.1)
    p = str(tmp_path / "m.v3.bin")
    ak.akv3_write(p, cfg, params, train_step=440000, schedule_step=77)
    got, step = ak.akv3_read_header(p)
    assert (got.vocab_size, got.dim, got.num_heads, got.num_layers, got.seq_len, got.ffn_hidden) == (97, 32, 4, 2, 16, 128)
    assert got.eos_token == 96 and step == 440000
    raw = open(p, "rb").read()
    # layout: magic, then the fixed-int little-endian fields, then u64 tensor count
    assert raw[:4] == b"AKV3"
    assert struct.unpack_from("<IIIQIIQI", raw, 4) == (97, 32, 4, 2, 16, 128, 440000, 77)
    assert struct.unpack_from("<Q", raw, 4 + 40)[0] == len(params) == 15
    bad = str(tmp_path / "bad.bin")
    open(bad, "wb").write(b"AKV2" + raw[4:])
    with pytest.raises(ak.AkashaError) as e:
        ak.akv3_read_header(bad)
    assert "not a v3 checkpoint" in str(e.value)
    with pytest.raises(ak.AkashaError) as e:
        ak.akv3_read_header(str(tmp_path / "missing.bin"))
    assert e.value.kind == "NotFound"


@pytest.mark.gpu
def test_load_into_weights_and_mismatch_errors(ak, ctx, tmp_path):
    cfg = ak.ModelConfig(97, 32, 4, 2, 16)
    params = ak.synthetic_weights(cfg, seed=3, std=0.1)
    moments = [(np.zeros_like(p), np.ones_like(p)) for p in params]
    p = str(tmp_path / "m.v3.bin")
    ak.akv3_write(p, cfg, params, train_step=12, moments=moments)
    w = ak.ModelWeights(ctx, cfg, ak.AK_F32)
    assert w.load_akv3(p) == 12
    assert all(np.array_equal(a, b) for a, b in zip(params, w.params()))
    w.close()
    # architecture mismatch (src/nn/checkpoint.rs:127-133)
    other = ak.ModelWeights(ctx, ak.ModelConfig(97, 32, 4, 3, 16), ak.AK_F32)
    with pytest.raises(ak.AkashaError) as e:
        other.load_akv3(p)
    assert "architecture mismatch" in str(e.value)
    other.close()
    # a tensor of the wrong length (src/nn/checkpoint.rs:176-183)
    broken = [q.copy() for q in params]
    broken[2] = broken[2].reshape(-1)[:-1]
    pb = str(tmp_path / "broken.bin")
    ak.akv3_write(pb, cfg, broken)
    w2 = ak.ModelWeights(ctx, cfg, ak.AK_F32)
    with pytest.raises(ak.AkashaError) as e:
        w2.load_akv3(pb)
    assert "checkpoint tensor 2 has" in str(e.value)
    w2.close()
