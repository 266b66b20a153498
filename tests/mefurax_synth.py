"""Small Mefurax configurations with random weights for the tests, and the glue between the library and the oracle.

Weights are drawn in float32 and rounded to bfloat16-representable values, so that the library (either compute mode) and the float64
oracle hold exactly the same numbers."""
import numpy as np

import llama_gguf_b200 as B
from llama_gguf_b200 import mefurax
from llama_gguf_b200.safetensors_io import bf16_bits, bf16_to_f32


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, shared=40):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer_a(heads=4, kv_heads=2, dim=24, vdim=40, window=9, conv=3, scale=None, v_mix=True, mlp=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "conv": conv,
                      "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix},
            "mlp": mlp}


def layer_b(heads=4, kv_heads=2, dim=24, vdim=40, chunk=7, rot_dims=16, rot_base=1000.0, softcap=5.0, scale=None, v_mix=True, mlp=None):
    return {"type": "attention_2",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                      "rot": {"dims": rot_dims, "base": rot_base}, "softcap": softcap,
                      "scale": scale if scale is not None else 2.0 * dim ** -0.5, "v_mix": v_mix},
            "mlp": mlp}


def config(layers, width=64, vocab=96, eps=1e-5, alpha=1.7):
    return {"architecture": "Mefurax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}


def random_weights(cfg, seed=0):
    rng = np.random.default_rng(seed)
    shapes = dict(mefurax.tensor_shapes(cfg))
    for i, L in enumerate(cfg["layers"]):          # the file of a model holds '.vmix' for every blending layer, the first included
        if L["mixer"].get("v_mix"):
            shapes["l%d.mix.vmix" % i] = ()
    w = {}
    for name, shape in shapes.items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            a = 0.25 * rng.standard_normal(shape)                 # stored around zero
        elif name.endswith(".q.norm") or name.endswith(".k.norm"):
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "conv":
            a = 0.6 * rng.standard_normal(shape)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif last == "vmix":
            a = rng.uniform(0.2, 0.7, shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif last == "router":
            a = rng.standard_normal(shape) * (6.0 / np.sqrt(shape[-1]))
        else:
            a = rng.standard_normal(shape) * (2.0 / np.sqrt(shape[-1]))
        w[name] = bf16_to_f32(bf16_bits(np.asarray(a, dtype=np.float32))).reshape(shape)
    return w


def gpu_model(cfg, weights, compute="float32", max_seq_len=256, max_batch=4, taps=False):
    program, layers = mefurax.parse_config(cfg, max_seq_len, max_batch, compute)
    tensors = {n: (B.F32, list(reversed(a.shape)) if a.shape else [1], np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
                   if not a.shape else np.ascontiguousarray(a, dtype=np.float32)) for n, a in weights.items()}
    return B.LayerProgramInference(program, layers, tensors, taps=taps)


def rel_err(got, want):
    """Row-wise: rms of the difference (mean removed) over the rms of the wanted row (mean removed); the largest row."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    s = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((s * s).mean(-1) + 1e-30)))
