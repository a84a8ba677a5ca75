"""Layer files of a QTIP checkpoint: the library's writer and reader against the reference's own container writer
(src/safetensors.cpp) and the reference runtime's loader (load_linear, runtime/src/qtip.cpp:231-289). Host code only."""
import struct

import numpy as np
import pytest


def make_layer(pkg, hidden, intermediate, seed):
    s = pkg.synth
    rng = np.random.default_rng(seed)
    shapes = {"self_attn.q_proj": (hidden, hidden), "mlp.gate_proj": (intermediate, hidden),
              "mlp.down_proj": (hidden, intermediate)}
    out = {}
    for i, (name, (m, n)) in enumerate(shapes.items()):
        out[name] = {"m": m, "n": n, "trellis": s.random_trellis(m, n, seed + i).reshape(-1, 32),
                     "SU": s.f32_to_bf16_bits(s.signs(n, seed + 10 + i)),
                     "SV": (s.signs(m, seed + 20 + i) * np.float32(0.01 + rng.random())).astype(np.float32),
                     "tlut": s.seeded_tlut(1).view(np.uint16)}
    return out


def test_round_trip_through_the_library(pkg, tmp_path):
    layer = make_layer(pkg, 128, 256, 3)
    path = tmp_path / "layer_7.safetensors"
    pkg.checkpoint.write_layer_file(path, 7, layer)
    for name, t in layer.items():
        got = pkg.checkpoint.read_layer_linear(path, 7, name, t["m"], t["n"])
        assert np.array_equal(got["trellis"], t["trellis"]) and np.array_equal(got["SV"], t["SV"])
        assert np.array_equal(got["SU"], pkg.synth.bf16_bits_to_f32(t["SU"])) and np.array_equal(got["tlut"], t["tlut"])
    with pytest.raises(pkg.QtipError):  # wrong geometry for the stored tensor
        pkg.checkpoint.read_layer_linear(path, 7, "self_attn.q_proj", 128, 256)
    with pytest.raises(pkg.QtipError):  # no such layer in the file
        pkg.checkpoint.read_layer_linear(path, 8, "self_attn.q_proj", 128, 128)


def test_file_loads_in_the_reference_runtime_and_equals_its_writer(pkg, reference, tmp_path):
    hidden, intermediate = 128, 256
    layer = make_layer(pkg, hidden, intermediate, 5)
    ours, theirs = tmp_path / "ours.safetensors", tmp_path / "theirs.safetensors"
    pkg.checkpoint.write_layer_file(ours, 2, layer)
    tl = next(iter(layer.values()))["tlut"]
    reference.write_layer_file(theirs, 2, {k: (t["m"], t["n"], t["trellis"], t["SU"], t["SV"]) for k, t in layer.items()}, tl)
    assert ours.read_bytes() == theirs.read_bytes()  # same header text, same tensor order, same bytes
    for name, t in layer.items():
        # a file written here through the reference runtime's loader (all of its checks pass) ...
        got = reference.load_linear(ours, 2, name, hidden, intermediate, 1, 64, t["m"], t["n"])
        assert np.array_equal(got["trellis"], t["trellis"]) and np.array_equal(got["SV"], t["SV"])
        assert np.array_equal(got["SU"], pkg.synth.bf16_bits_to_f32(t["SU"])) and np.array_equal(got["tlut"], t["tlut"])
        # ... and a file written by the reference's writer through this library's reader
        mine = pkg.checkpoint.read_layer_linear(theirs, 2, name, t["m"], t["n"])
        for k in ("trellis", "SU", "SV", "tlut"):
            assert np.array_equal(mine[k], got[k])


def test_loader_checks(pkg, tmp_path):
    """rcp != 0 and non-finite vectors are refused, like the runtime's loader does."""
    layer = {"self_attn.q_proj": make_layer(pkg, 64, 64, 9)["self_attn.q_proj"]}
    path = tmp_path / "l.safetensors"
    pkg.checkpoint.write_layer_file(path, 0, layer)
    raw = bytearray(path.read_bytes())
    hl = struct.unpack("<Q", raw[:8])[0]
    import json
    header = json.loads(raw[8:8 + hl])
    b, e = header["model.layers.0.self_attn.q_proj.rcp"]["data_offsets"]
    bad = bytearray(raw)
    bad[8 + hl + b:8 + hl + e] = struct.pack("<q", 1)
    (tmp_path / "rcp.safetensors").write_bytes(bad)
    with pytest.raises(pkg.QtipError) as err:
        pkg.checkpoint.read_layer_linear(tmp_path / "rcp.safetensors", 0, "self_attn.q_proj", 64, 64)
    assert "rcp" in str(err.value)
    b, e = header["model.layers.0.self_attn.q_proj.SV"]["data_offsets"]
    bad = bytearray(raw)
    bad[8 + hl + b:8 + hl + b + 4] = struct.pack("<f", float("inf"))
    (tmp_path / "sv.safetensors").write_bytes(bad)
    with pytest.raises(pkg.QtipError):
        pkg.checkpoint.read_layer_linear(tmp_path / "sv.safetensors", 0, "self_attn.q_proj", 64, 64)
    inf_sv = dict(layer["self_attn.q_proj"])
    inf_sv["SV"] = inf_sv["SV"].copy()
    inf_sv["SV"][3] = np.nan
    with pytest.raises(pkg.QtipError):
        pkg.checkpoint.write_layer_file(tmp_path / "x.safetensors", 0, {"self_attn.q_proj": inf_sv})
    assert not (tmp_path / "x.safetensors").exists()
