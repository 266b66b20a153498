"""Host-side pieces of the Lazilorn path that need no GPU: the oracle agrees with itself (whole prompt against token by token, the
mask rule), config.json becomes the right layer program, the safetensors reader round-trips, the registry picks by architecture."""
import json
import os

import numpy as np
import pytest

import lazilorn_oracle as O
import lazilorn_synth as S


def test_oracle_prompt_equals_token_by_token():
    cfg = S.config([S.parallel_layer(window=5, keep_first=2), S.delta_layer(conv=3, ff=40)], loop=(0, 2, 2))
    w = S.random_weights(cfg, 1)
    m = O.Model(cfg, w)
    toks = [int(t) for t in np.random.default_rng(2).integers(0, cfg["vocab"], 23)]
    whole = m.forward(toks)
    st = m.new_state()
    parts = np.concatenate([m.step(st, toks[:9]), m.step(st, toks[9:11])] + [m.step(st, [t]) for t in toks[11:]])
    assert np.abs(whole - parts).max() < 1e-9 * np.abs(whole).max()
    assert st["pos"] == len(toks)


def test_mask_rule():
    assert O.visible(10, 10, 1, 0) and not O.visible(10, 9, 1, 0)
    assert O.visible(10, 3, 8, 0) and not O.visible(10, 2, 8, 0)           # i - j < size
    assert O.visible(100, 3, 8, 4) and not O.visible(100, 4, 8, 4)         # j < keep_first
    assert not O.visible(2, 3, 8, 4)                                       # never ahead
    # kept tokens and the window may overlap early in a sequence: each key counts once
    q = np.ones((1, 1, 2)); k = np.zeros((6, 1, 2)); v = np.arange(6.0).reshape(6, 1, 1)
    out = O.windowed_attention(q, k, v, [5], np.arange(6), 1.0, 4, 3)
    assert abs(out[0, 0, 0] - np.mean([0, 1, 2, 3, 4, 5])) < 1e-12


def test_layer_run_order_and_step_vectors():
    cfg = S.config([S.delta_layer()] * 5, loop=(1, 4, 3))
    m = O.Model(cfg, S.random_weights(cfg, 0))
    assert m.runs == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    cfg = S.config([S.delta_layer()] * 2, loop=(0, 0, 1))
    assert O.Model(cfg, S.random_weights(cfg, 0)).runs == [0, 1]


def test_parse_config_reads_every_constant():
    from llama_gguf_b200 import lazilorn, COMPUTE_BF16, COMPUTE_F32, MIX_GATED_DELTA, MIX_WINDOW_MEMORY, InvalidArgument, Unsupported

    cfg = S.config([S.parallel_layer(heads=6, kv_heads=3, dim=20, vdim=28, window=13, keep_first=5, scale=0.37, mheads=5, mdim=12, mvdim=36,
                                     cap=9.5, left_scale=0.25, right_scale=1.75, ff=88),
                    S.delta_layer(heads=8, kv_heads=4, dim=12, vdim=20, conv=5, ff=0)],
                   width=80, vocab=123, loop=(1, 2, 4), eps=3e-6, embed_scale=7.5, logit_scale=0.125)
    prog, layers = lazilorn.parse_config(cfg, 777, 5, "float32")
    assert prog == {"width": 80, "vocab": 123, "max_seq_len": 777, "max_batch": 5, "norm_eps": 3e-6, "embed_scale": 7.5, "logit_scale": 0.125,
                    "pos_sinusoid": 1, "loop_start": 1, "loop_stop": 2, "loop_times": 4, "compute": COMPUTE_F32}
    assert layers[0]["mixer"] == MIX_WINDOW_MEMORY and layers[0]["ff"] == 88
    assert layers[0]["attn"] == {"heads": 6, "kv_heads": 3, "dim": 20, "vdim": 28, "window": 13, "keep_first": 5, "scale": 0.37, "qk_norm": 1,
                                 "out_gate": 1}
    assert layers[0]["mem"] == {"heads": 5, "dim": 12, "vdim": 36, "gate_cap": 9.5}
    assert (layers[0]["attn_scale"], layers[0]["mem_scale"]) == (0.25, 1.75)
    assert layers[1] == {"ff": 0, "mixer": MIX_GATED_DELTA, "delta": {"heads": 8, "kv_heads": 4, "dim": 12, "vdim": 20, "conv": 5}}
    assert lazilorn.parse_config(cfg, 8, 1)[0]["compute"] == COMPUTE_BF16
    with pytest.raises(InvalidArgument):
        lazilorn.parse_config(dict(cfg, architecture="llama"), 8, 1)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(Unsupported):
        lazilorn.parse_config(bad, 8, 1)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(Unsupported):
        lazilorn.parse_config(bad, 8, 1)


def test_safetensors_round_trip(tmp_path):
    from llama_gguf_b200.safetensors_io import BF16, F32, SafetensorsFile, bf16_bits, bf16_to_f32, write_safetensors

    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    b = bf16_bits(rng.standard_normal(11).astype(np.float32))
    t = np.arange(6, dtype=np.int32).reshape(2, 3)
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, {"a": a, "b.c": b, "table": t})
    with SafetensorsFile(p) as f:
        assert sorted(f.names()) == ["a", "b.c", "table"]
        gg, shape, arr = f.tensor("a")
        assert gg == F32 and shape == (5, 7) and np.array_equal(arr, a)
        gg, shape, arr = f.tensor("b.c")
        assert gg == BF16 and shape == (11,) and np.array_equal(arr, b)
        gg, shape, arr = f.tensor("table")
        assert gg is None and np.array_equal(arr, t)
        del arr
    # bf16 rounding: to nearest, ties to even; exact values survive
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], dtype=np.float32)
    y = bf16_to_f32(bf16_bits(x))
    assert y[0] == 1.0 and y[1] == 1.0 and y[2] == 1.015625 and y[3] == -2.5
    with open(p, "r+b") as f:
        f.write((1 << 40).to_bytes(8, "little"))
    with pytest.raises(ValueError):
        SafetensorsFile(p)


def test_registry_picks_by_architecture(tmp_path):
    from llama_gguf_b200 import registry, Unsupported

    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architecture": "Lazilorn"}))
    assert registry.architecture_of(str(d)) == "Lazilorn"
    assert "Lazilorn" in registry.LOADERS
    (d / "config.json").write_text(json.dumps({"architecture": "Nothing"}))
    with pytest.raises(Unsupported):
        registry.load_model(str(d))


def test_trace_runner_is_executable():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "bin", "trace_run")
    assert os.access(p, os.X_OK)
