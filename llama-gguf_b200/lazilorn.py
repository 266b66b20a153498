"""Lazilorn: a small hybrid decoder.  config.json -> the library's layer program; model.safetensors -> its tensors.

The design in the library's terms (include/llama_b200.h, "layer-program models"):
  * embedding row * embedding.scale + sinusoidal position vector;
  * `layers`: each entry has a `type` -- "parallel" = B200_MIX_WINDOW_MEMORY (windowed softmax attention with kept first tokens,
    q/k norm, sigmoid output gate, beside a matrix memory; summed with left_scale / right_scale) or "delta" = B200_MIX_GATED_DELTA
    (gated delta rule behind short causal convolutions) -- and `mlp`: null or {"kind": "dense", "ff": n} (relu^2 feed-forward);
  * `loop`: layers start .. stop-1 run `times` times with the same weights and a state of their own per pass; `loop.step[t]` is
    added to the stream before pass t;
  * final norm, head, logits * logit_scale.
Tensor names are the file's own (`l<i>.norm1`, `l<i>.mix.left.q`, ..., `embed`, `head`, `final.norm`, `loop.step`): the library takes
them as they are."""
import json
import os

from . import COMPUTE_BF16, COMPUTE_F32, MIX_GATED_DELTA, MIX_WINDOW_MEMORY, InvalidArgument, LayerProgramInference, Unsupported
from .safetensors_io import SafetensorsFile

ARCHITECTURE = "Lazilorn"


def parse_config(cfg, max_seq_len, max_batch, compute="bfloat16"):
    """config.json (dict) -> (program dict, layer dicts) for LayerProgramInference.  Every size and constant is read from cfg."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise InvalidArgument(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    if compute not in ("bfloat16", "float32"):
        raise Unsupported(f"compute {compute!r}: bfloat16 or float32")
    loop = cfg.get("loop") or {}
    program = {
        "width": int(cfg["width"]), "vocab": int(cfg["vocab"]), "max_seq_len": int(max_seq_len), "max_batch": int(max_batch),
        "norm_eps": float(cfg["norm"]["eps"]), "embed_scale": float(cfg["embedding"]["scale"]),
        "logit_scale": float(cfg.get("logit_scale", 1.0)), "pos_sinusoid": 1,
        "loop_start": int(loop.get("start", 0)), "loop_stop": int(loop.get("stop", 0)), "loop_times": int(loop.get("times", 1)),
        "compute": COMPUTE_F32 if compute == "float32" else COMPUTE_BF16,
    }
    layers = []
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        mlp = L.get("mlp")
        if mlp is not None and mlp.get("kind") != "dense":
            raise Unsupported(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        d = {"ff": int(mlp["ff"]) if mlp else 0}
        if L["type"] == "parallel":
            le, ri = m["left"], m["right"]
            d.update(mixer=MIX_WINDOW_MEMORY, attn_scale=float(m["left_scale"]), mem_scale=float(m["right_scale"]),
                     attn={"heads": int(le["heads"]), "kv_heads": int(le["kv_heads"]), "dim": int(le["dim"]), "vdim": int(le["vdim"]),
                           "window": int(le["mask"]["size"]), "keep_first": int(le["mask"]["keep_first"]), "scale": float(le["scale"]),
                           "qk_norm": 1, "out_gate": 1},
                     mem={"heads": int(ri["heads"]), "dim": int(ri["dim"]), "vdim": int(ri["vdim"]), "gate_cap": float(ri["gate_cap"])})
        elif L["type"] == "delta":
            d.update(mixer=MIX_GATED_DELTA,
                     delta={"heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
                            "conv": int(m["conv"])})
        else:
            raise Unsupported(f"layer {i}: mixer type {L['type']!r}")
        layers.append(d)
    return program, layers


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this config holds (what model.safetensors must contain)."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    lp = cfg.get("loop") or {}
    if lp.get("stop", 0) > lp.get("start", 0):
        out["loop.step"] = (lp.get("times", 1), W)
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
        if L.get("mlp"):
            out.update({p + "norm2": (W,), p + "mlp.up": (L["mlp"]["ff"], W), p + "mlp.down": (W, L["mlp"]["ff"])})
    return out


def load(model_dir, max_seq_len=4096, max_batch=8, compute="bfloat16", device=0, taps=False):
    """A folder with config.json and model.safetensors -> a finalized context."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    program, layers = parse_config(cfg, max_seq_len, max_batch, compute)
    st = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))

    want = tensor_shapes(cfg)
    missing = sorted(set(want) - set(st.names()))
    if missing:
        raise InvalidArgument(f"{model_dir}: model.safetensors lacks {missing[:4]}{' ...' if len(missing) > 4 else ''}")
    for name, shape in want.items():
        if tuple(st.shape(name)) != tuple(shape):
            raise InvalidArgument(f"{model_dir}: tensor {name} has shape {st.shape(name)}, the config wants {tuple(shape)}")

    def feeder(upload):
        for name in st.names():
            if name not in want:
                continue
            gg, shape, arr = st.tensor(name)
            if gg is None:
                continue                      # integer tables: this design has none the engine reads
            upload(name, gg, list(reversed(shape)) if shape else [1], arr)

    try:
        gpu = LayerProgramInference(program, layers, device=device, taps=taps, feeder=feeder)
    finally:
        try:
            st.close()
        except BufferError:
            pass
    gpu.arch = ARCHITECTURE
    gpu.config = cfg
    return gpu
