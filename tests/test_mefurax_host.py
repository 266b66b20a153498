"""Host-side pieces of the Mefurax path that need no GPU: the oracle agrees with itself (whole prompt against portions, the mask rules,
the router), config.json becomes the right layer program, the list of tensors follows the config, the registry picks by architecture."""
import json

import numpy as np
import pytest

import mefurax_oracle as O
import mefurax_synth as S


def test_oracle_prompt_equals_portions():
    cfg = S.config([S.layer_b(mlp=S.dense(40)), S.layer_a(window=5, conv=3, mlp=S.moe())])
    w = S.random_weights(cfg, 1)
    m = O.Model(cfg, w)
    toks = [int(t) for t in np.random.default_rng(2).integers(0, cfg["vocab"], 23)]
    whole = m.forward(toks)
    st = m.new_state()
    parts = np.concatenate([m.step(st, toks[:9]), m.step(st, toks[9:11])] + [m.step(st, [t]) for t in toks[11:]])
    assert np.abs(whole - parts).max() < 1e-9 * np.abs(whole).max()
    assert st["n"] == len(toks)


def test_mask_rules():
    assert O.sees_window(10, 10, 1) and not O.sees_window(10, 9, 1)
    assert O.sees_window(10, 3, 8) and not O.sees_window(10, 2, 8) and not O.sees_window(2, 3, 8)
    assert O.sees_chunk(15, 8, 8) and not O.sees_chunk(16, 15, 8) and O.sees_chunk(16, 16, 8)
    assert not O.sees_chunk(9, 10, 8) and O.sees_chunk(7, 0, 8)


def test_small_pieces():
    # filter: the last tap meets the current input, zeros before the start
    f = np.array([[1.0, 10.0, 100.0]])
    hist = [np.array([1.0]), np.array([2.0]), np.array([3.0])]
    assert O.filter_step(hist[:1], f)[0] == 100.0
    assert O.filter_step(hist[:2], f)[0] == 10.0 + 200.0
    assert O.filter_step(hist, f)[0] == 1.0 + 20.0 + 300.0
    # rotation: pairs (0, 1), (2, 3); lengths stay, channels beyond dims stay; position 0 is the identity
    v = np.array([1.0, 0.0, 0.0, 2.0, 5.0, 6.0])
    r = O.rotate_pairs(v, 3, 4, 100.0)
    assert np.allclose(r[:2], [np.cos(3.0), np.sin(3.0)]) and np.allclose(r[2:4], [-2 * np.sin(0.3), 2 * np.cos(0.3)]) and np.array_equal(r[4:], v[4:])
    assert np.array_equal(O.rotate_pairs(v, 0, 4, 100.0), v)
    # router: largest logits, the lower index among equals, weights sum to one over the chosen only
    idx, wts = O.route(np.array([0.5, 2.0, 2.0, -1.0]), 2)
    assert idx == [1, 2] and np.allclose(wts, [0.5, 0.5])
    idx, wts = O.route(np.array([0.0, 1.0, 3.0]), 3)
    assert idx == [2, 1, 0] and abs(sum(wts) - 1) < 1e-12
    assert abs(O.distance_slope(7, 8) - 2.0 ** -8) < 1e-15 and abs(O.distance_slope(0, 8) - 0.5) < 1e-15
    assert abs(O.soft_cap(1000.0, 12.5) - 12.5) < 1e-9
    assert abs(O.gelu_tanh(np.array([1.0]))[0] - 0.8411919906082768) < 1e-12


def test_parse_config_reads_every_constant():
    from llama_gguf_b200 import (COMPUTE_BF16, COMPUTE_F32, FF_GATED_GELU, FF_MOE, FF_RELU2, GATE_HEAD, GATE_NONE, MASK_CHUNK, MASK_WINDOW,
                                 MIX_SOFTMAX_ATTN, QKNORM_HEAD_UNIT, QKNORM_WHOLE_WEIGHT, VMIX_BLEND, VMIX_NONE, VMIX_SOURCE, InvalidArgument,
                                 Unsupported, mefurax)

    cfg = S.config([S.layer_a(heads=6, kv_heads=3, dim=20, vdim=28, window=13, conv=5, scale=0.37, v_mix=False, mlp=None),
                    S.layer_b(heads=8, kv_heads=2, dim=12, vdim=42, chunk=9, rot_dims=6, rot_base=123.0, softcap=7.5, scale=0.21, v_mix=True,
                              mlp=S.dense(88)),
                    S.layer_a(heads=3, kv_heads=3, dim=8, vdim=28, v_mix=True, mlp=S.moe(experts=7, top=3, ff=18, shared=0))],
                   width=80, vocab=123, eps=3e-6, alpha=2.25)
    prog, layers = mefurax.parse_config(cfg, 777, 5, "float32")
    assert prog == {"width": 80, "vocab": 123, "max_seq_len": 777, "max_batch": 5, "norm_eps": 3e-6, "embed_scale": 1.0, "logit_scale": 1.0,
                    "pos_sinusoid": 0, "loop_start": 0, "loop_stop": 0, "loop_times": 1, "compute": COMPUTE_F32, "post_norm": 1,
                    "residual_alpha": 2.25, "norm_weight_offset": 1.0}
    assert all(L["mixer"] == MIX_SOFTMAX_ATTN for L in layers)
    assert layers[0]["sattn"] == {"heads": 6, "kv_heads": 3, "dim": 20, "vdim": 28, "mask_size": 13, "scale": 0.37, "v_mix": VMIX_NONE,
                                  "mask": MASK_WINDOW, "qkv_bias": 1, "conv": 5, "qk_norm": QKNORM_WHOLE_WEIGHT, "rot_dims": 0, "rot_base": 0.0,
                                  "softcap": 0.0, "dist_bias_exp": 8.0, "out_gate": GATE_NONE}
    assert (layers[0]["ff"], layers[0]["ff_kind"]) == (0, FF_RELU2)
    assert layers[1]["sattn"] == {"heads": 8, "kv_heads": 2, "dim": 12, "vdim": 42, "mask_size": 9, "scale": 0.21, "v_mix": VMIX_SOURCE,
                                  "mask": MASK_CHUNK, "qkv_bias": 0, "conv": 0, "qk_norm": QKNORM_HEAD_UNIT, "rot_dims": 6, "rot_base": 123.0,
                                  "softcap": 7.5, "dist_bias_exp": 0.0, "out_gate": GATE_HEAD}
    assert (layers[1]["ff"], layers[1]["ff_kind"]) == (88, FF_GATED_GELU)
    assert layers[2]["sattn"]["v_mix"] == VMIX_BLEND
    assert layers[2]["ff_kind"] == FF_MOE and layers[2]["moe"] == {"experts": 7, "top": 3, "expert_ff": 18, "shared_ff": 0}
    assert mefurax.parse_config(cfg, 8, 1)[0]["compute"] == COMPUTE_BF16
    with pytest.raises(InvalidArgument):
        mefurax.parse_config(dict(cfg, architecture="llama"), 8, 1)
    for key, val in (("type", "conv"), ("mlp", {"kind": "sparse"})):
        bad = json.loads(json.dumps(cfg))
        bad["layers"][1][key] = val
        with pytest.raises(Unsupported):
            mefurax.parse_config(bad, 8, 1)


def test_tensor_list_follows_the_config():
    from llama_gguf_b200 import mefurax

    cfg = S.config([S.layer_a(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, v_mix=True, mlp=S.moe(experts=3, top=2, ff=10, shared=6)),
                    S.layer_b(heads=2, kv_heads=1, dim=16, vdim=24, v_mix=True, mlp=None)], width=32, vocab=50)
    t = mefurax.tensor_shapes(cfg)
    assert t["l0.mix.q"] == (32, 32) and t["l0.mix.k.b"] == (16,) and t["l0.mix.v.conv"] == (24, 3) and t["l0.mix.q.norm"] == (32,)
    assert t["l0.mix.o"] == (32, 48) and "l0.mix.g" not in t and "l0.mix.vmix" not in t
    assert t["l0.mlp.router"] == (3, 32) and t["l0.mlp.e2.down"] == (32, 10) and t["l0.mlp.shared.up"] == (6, 32) and "l0.mlp.e3.up" not in t
    assert t["l1.mix.g"] == (2, 32) and t["l1.mix.vmix"] == () and "l1.mix.q.b" not in t and "l1.norm2" not in t
    assert set(S.random_weights(cfg, 0)) == set(t) | {"l0.mix.vmix"}


def test_registry_knows_the_architecture(tmp_path):
    from llama_gguf_b200 import registry

    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"architecture": "Mefurax"}))
    assert registry.architecture_of(str(d)) == "Mefurax"
    assert "Mefurax" in registry.LOADERS and "Lazilorn" in registry.LOADERS
