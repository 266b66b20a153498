"""Small Lazilorn configurations with random weights for the tests, and the glue between the library and the oracle.

Weights are drawn in float32 and rounded to bfloat16-representable values, so that the library (either compute mode) and the
float64 oracle hold exactly the same numbers."""
import numpy as np

import llama_gguf_b200 as B
from llama_gguf_b200 import lazilorn
from llama_gguf_b200.safetensors_io import bf16_bits, bf16_to_f32


def parallel_layer(heads=2, kv_heads=1, dim=24, vdim=40, window=8, keep_first=3, scale=None, mheads=2, mdim=16, mvdim=24, cap=15.0,
                   left_scale=0.7, right_scale=1.1, ff=80):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "mask": {"size": window, "keep_first": keep_first}, "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": mheads, "dim": mdim, "vdim": mvdim, "gate_cap": cap},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=0):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=64, vocab=96, loop=(0, 0, 1), eps=1e-5, embed_scale=3.0, logit_scale=0.7):
    return {"architecture": "Lazilorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "logit_scale": logit_scale, "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}, "layers": layers}


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    lp = cfg["loop"]
    if lp["stop"] > lp["start"]:
        out["loop.step"] = (lp["times"], W)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        out[p + "norm1"] = (W,)
        if L["type"] == "parallel":
            le, ri = m["left"], m["right"]
            q = p + "mix.left."
            out.update({q + "q": (le["heads"] * le["dim"], W), q + "k": (le["kv_heads"] * le["dim"], W), q + "v": (le["kv_heads"] * le["vdim"], W),
                        q + "q.norm": (le["dim"],), q + "k.norm": (le["dim"],), q + "g": (le["heads"] * le["vdim"], W),
                        q + "o": (W, le["heads"] * le["vdim"])})
            r = p + "mix.right."
            out.update({r + "q": (ri["heads"] * ri["dim"], W), r + "k": (ri["heads"] * ri["dim"], W), r + "v": (ri["heads"] * ri["vdim"], W),
                        r + "g": (ri["heads"] * ri["vdim"], W), r + "o": (W, ri["heads"] * ri["vdim"]), r + "norm": (ri["heads"] * ri["vdim"],),
                        r + "i": (ri["heads"], W), r + "i.b": (ri["heads"],), r + "f": (ri["heads"], W), r + "f.b": (ri["heads"],)})
        else:
            x = p + "mix."
            qk, vv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({x + "q": (qk, W), x + "q.conv": (qk, m["conv"]), x + "k": (qk, W), x + "k.conv": (qk, m["conv"]),
                        x + "v": (vv, W), x + "v.conv": (vv, m["conv"]), x + "b": (m["heads"], W), x + "A_log": (m["heads"],),
                        x + "norm": (m["vdim"],), x + "a": (m["heads"], W), x + "dt_bias": (m["heads"],), x + "g": (vv, W), x + "o": (W, vv)})
        if L["mlp"]:
            out.update({p + "norm2": (W,), p + "mlp.up": (L["mlp"]["ff"], W), p + "mlp.down": (W, L["mlp"]["ff"])})
    return out


def random_weights(cfg, seed=0):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name == "final.norm" or name.endswith(".norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "conv":
            a = 0.5 * rng.standard_normal(shape)
        elif name.endswith("i.b"):
            a = rng.uniform(-1.0, 1.0, shape)
        elif name.endswith("f.b"):
            a = rng.uniform(1.0, 4.0, shape)
        elif last == "A_log":
            a = rng.uniform(-2.0, 0.5, shape)
        elif last == "dt_bias":
            a = rng.uniform(-2.0, 1.0, shape)
        elif name == "loop.step":
            a = 0.3 * rng.standard_normal(shape)
        elif name == "embed":
            a = 0.5 * rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) * (2.0 / np.sqrt(shape[-1]))
        w[name] = bf16_to_f32(bf16_bits(a.astype(np.float32))).reshape(shape)
    return w


def gpu_model(cfg, weights, compute="float32", max_seq_len=256, max_batch=4, taps=False):
    program, layers = lazilorn.parse_config(cfg, max_seq_len, max_batch, compute)
    tensors = {n: (B.F32, list(reversed(a.shape)), np.ascontiguousarray(a, dtype=np.float32)) for n, a in weights.items()}
    return B.LayerProgramInference(program, layers, tensors, taps=taps)


def rel_err(got, want):
    """Row-wise: rms of the difference (mean removed) over the rms of the wanted row (mean removed); the largest row."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    s = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((s * s).mean(-1) + 1e-30)))
