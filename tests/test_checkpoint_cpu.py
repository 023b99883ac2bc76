"""Quantized-checkpoint format (CPU): host quantizers bit-exact against the oracle, tile packing through the
library's host packers, container round trip, and readability by the stock `safetensors` package (the same
container the reference parses, xn-core/src/safetensors.rs)."""
import json
import os

import numpy as np
import pytest

from xn_b200 import checkpoint as ck


def _weights(seed, n, k, scale=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * scale).astype(np.float32)
    w[1, :32] = 0.0          # an all-zero block (scale 0)
    w[2, 5] = 7.5 * w[2, :32].max() if n > 2 else w[0, 0]   # a clear block maximum
    return w


@pytest.mark.parametrize("n,k", [(48, 256), (41, 384)])
def test_host_block_quantizers_match_oracle_bit_exact(oracle, n, k):
    w = _weights(3, n, k)
    for qmax, ofn in ((7, oracle.quantize_q4), (127, oracle.quantize_q8)):
        q, s = ck.quantize_blocks_host(w, 32, qmax)
        q0, s0 = ofn(w)
        assert np.array_equal(q, q0)
        assert np.array_equal(s.view(np.uint32), np.asarray(s0, dtype=np.float32).reshape(s.shape).view(np.uint32))


def test_host_e4m3_encoder_matches_oracle_on_every_boundary(oracle):
    # all representable values, their midpoints (ties), neighbours of the midpoints, subnormals, saturation, signs
    table = oracle.e4m3_decode_table()
    pos = np.array(sorted(set(float(v) for v in table[:0x7F])), dtype=np.float64)
    mids = (pos[:-1] + pos[1:]) / 2
    pts = np.concatenate([pos, mids, np.nextafter(mids.astype(np.float32), np.float32(np.inf)),
                          np.nextafter(mids.astype(np.float32), np.float32(-np.inf)),
                          [448.0, 464.0, 465.0, 480.0, 1e6, 1e-12, 2 ** -10, 2 ** -9, 1.5 * 2 ** -9]]).astype(np.float32)
    pts = np.concatenate([pts, -pts])
    assert np.array_equal(ck.f32_to_e4m3_host(pts), oracle.f32_to_e4m3(pts))
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(20000) * rng.choice([1e-3, 0.1, 1.0, 30.0, 300.0], 20000)).astype(np.float32)
    assert np.array_equal(ck.f32_to_e4m3_host(x), oracle.f32_to_e4m3(x))


def test_host_fp8_channel_quantizer_matches_oracle(oracle):
    w = _weights(7, 40, 320, scale=0.05)
    w[3] = 0.0  # an all-zero channel
    q, s = ck.quantize_fp8_channel_host(w)
    q0, s0 = oracle.quantize_fp8_channel(w)
    assert np.array_equal(q, q0)
    assert np.array_equal(s.view(np.uint32), s0.view(np.uint32))


def test_tile_packing_matches_oracle(oracle):
    w = _weights(9, 41, 384)
    q, s = ck.quantize_blocks_host(w, 32, 7)
    assert np.array_equal(ck.pack_q4_host(q, s), oracle.pack_q4(q, s))
    q8, s8 = ck.quantize_blocks_host(w, 32, 127)
    assert np.array_equal(ck.pack_q8_host(q8, s8), oracle.pack_q8(q8, s8))


def test_checkpoint_round_trip_and_foreign_reader(tmp_path, oracle):
    rng = np.random.default_rng(11)
    weights = {"layers.0.in_proj": _weights(1, 48, 256), "layers.0.out_proj": _weights(2, 32, 128),
               "layers.0.ffn_up": _weights(4, 64, 256), "layers.0.norm.alpha": rng.standard_normal(256).astype(np.float32)}
    schemes = {"layers.0.in_proj": "q4", "layers.0.out_proj": "q8", "layers.0.ffn_up": "fp8"}
    bias = rng.standard_normal(48).astype(np.float32)
    path = os.path.join(tmp_path, "model.q.safetensors")
    ck.save_quantized(path, weights, schemes, extra={"layers.0.in_proj.bias": bias})
    linears, others = ck.load_quantized(path)
    assert set(linears) == set(schemes)
    q, s = oracle.quantize_q4(weights["layers.0.in_proj"])
    assert np.array_equal(linears["layers.0.in_proj"]["q4"], oracle.pack_q4(q, s))
    assert (linears["layers.0.in_proj"]["n"], linears["layers.0.in_proj"]["k"]) == (48, 256)
    q8, s8 = oracle.quantize_q8(weights["layers.0.out_proj"])
    assert np.array_equal(linears["layers.0.out_proj"]["q8"], oracle.pack_q8(q8, s8))
    qf, sf = oracle.quantize_fp8_channel(weights["layers.0.ffn_up"])
    assert np.array_equal(linears["layers.0.ffn_up"]["fp8"], qf)
    assert np.array_equal(linears["layers.0.ffn_up"]["fp8_scale"], sf)
    assert np.array_equal(others["layers.0.norm.alpha"], weights["layers.0.norm.alpha"])
    assert np.array_equal(others["layers.0.in_proj.bias"], bias)
    # the file is an ordinary safetensors file: the stock reader sees the same bytes
    st = pytest.importorskip("safetensors.numpy")
    foreign = st.load_file(path)
    assert np.array_equal(foreign["layers.0.in_proj.q4"], linears["layers.0.in_proj"]["q4"])
    assert foreign["layers.0.ffn_up.fp8"].dtype == np.uint8 and foreign["layers.0.ffn_up.fp8"].shape == (64, 256)
    from safetensors import safe_open
    with safe_open(path, framework="np") as f:
        md = f.metadata()
    assert md["xn_mm.format_version"] == ck.FORMAT_VERSION
    assert json.loads(md["xn_mm.layers.0.in_proj"]) == {"scheme": "q4", "n": 48, "k": 256, "block": 32}


def test_reader_rejects_damaged_files(tmp_path):
    path = os.path.join(tmp_path, "a.safetensors")
    ck.save_quantized(path, {"w": _weights(1, 16, 128)}, {"w": "q4"})
    raw = open(path, "rb").read()
    bad = os.path.join(tmp_path, "b.safetensors")
    open(bad, "wb").write(raw[:-100])  # truncated data
    with pytest.raises(ValueError):
        ck.load_quantized(bad)
    open(bad, "wb").write(raw[:4])  # truncated header
    with pytest.raises(ValueError):
        ck.load_quantized(bad)
    tensors, meta = ck.read_safetensors(path)
    meta["xn_mm.format_version"] = "999"
    ck.write_safetensors(bad, tensors, meta)
    with pytest.raises(ValueError):
        ck.load_quantized(bad)
    with pytest.raises(ValueError):
        ck.quantize_blocks_host(np.zeros((4, 100), np.float32), 32, 7)  # k not a multiple of the block
