"""Mefurax: a small attention-only decoder with two kinds of softmax mixer, norm after the residual sum, dense and mixture-of-experts
feed-forward layers.  config.json -> the library's layer program; model.safetensors -> its tensors.

The design in the library's terms (include/llama_b200.h, "layer-program models"):
  * x = embedding row; every layer is x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)) with alpha = `postln_alpha`
    (program.post_norm, residual_alpha); norm weights are stored around zero (norm_weight_offset = 1);
  * `layers[i].type` picks the options of B200_MIX_SOFTMAX_ATTN:
      "attention"    biases on q / k / v, a short causal convolution (`conv` taps) behind the projection, one RMS norm over the whole
                     of q (and of k) with a weight per channel, no rotation, a distance bias 2^(-8 (h + 1) / heads) (i - j) taken off
                     the scaled score, sliding window of mask.size positions;
      "attention_2"  no biases, rotary positions on the first rot.dims channels of every head (interleaved pairs), then a per-head RMS
                     norm without weight, soft cap on the scaled score, chunks of mask.size positions, one sigmoid gate per head;
    both: grouped K/V heads, `scale` from the config, value blending (`v_mix`): the first such layer is the source, every later one
    caches (1 - l) v + l v_source with l = its '.vmix';
  * `mlp`: null, {"kind": "dense", "ff"} = gated tanh-GELU, or {"kind": "moe", "router": {experts, top}, "expert": {ff}, "shared": {ff}};
  * final norm, head.
Tensor names are the file's own (`l<i>.norm1`, `l<i>.mix.q`, `l<i>.mix.q.b`, `l<i>.mlp.e<j>.up`, ..., `embed`, `head`, `final.norm`)."""
import json
import os

from . import (COMPUTE_BF16, COMPUTE_F32, FF_GATED_GELU, FF_MOE, FF_RELU2, GATE_HEAD, GATE_NONE, MASK_CHUNK, MASK_WINDOW, MIX_SOFTMAX_ATTN,
               QKNORM_HEAD_UNIT, QKNORM_WHOLE_WEIGHT, VMIX_BLEND, VMIX_NONE, VMIX_SOURCE, InvalidArgument, LayerProgramInference, Unsupported)
from .safetensors_io import SafetensorsFile

ARCHITECTURE = "Mefurax"
DIST_BIAS_EXP = 8.0     # head h of "attention" takes 2^(-8 (h + 1) / heads) per position of distance off its scores


def parse_config(cfg, max_seq_len, max_batch, compute="bfloat16"):
    """config.json (dict) -> (program dict, layer dicts) for LayerProgramInference.  Every size and constant is read from cfg."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise InvalidArgument(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    if compute not in ("bfloat16", "float32"):
        raise Unsupported(f"compute {compute!r}: bfloat16 or float32")
    program = {
        "width": int(cfg["width"]), "vocab": int(cfg["vocab"]), "max_seq_len": int(max_seq_len), "max_batch": int(max_batch),
        "norm_eps": float(cfg["norm"]["eps"]), "embed_scale": 1.0, "logit_scale": 1.0, "pos_sinusoid": 0,
        "loop_start": 0, "loop_stop": 0, "loop_times": 1, "compute": COMPUTE_F32 if compute == "float32" else COMPUTE_BF16,
        "post_norm": 1, "residual_alpha": float(cfg["postln_alpha"]), "norm_weight_offset": 1.0,
    }
    layers, have_source = [], False
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        a = {"heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
             "mask_size": int(m["mask"]["size"]), "scale": float(m["scale"])}
        if m.get("v_mix"):
            a["v_mix"] = VMIX_BLEND if have_source else VMIX_SOURCE
            have_source = True
        else:
            a["v_mix"] = VMIX_NONE
        if L["type"] == "attention":
            a.update(mask=MASK_WINDOW, qkv_bias=1, conv=int(m.get("conv", 0)), qk_norm=QKNORM_WHOLE_WEIGHT, rot_dims=0, rot_base=0.0,
                     softcap=0.0, dist_bias_exp=DIST_BIAS_EXP, out_gate=GATE_NONE)
        elif L["type"] == "attention_2":
            rot = m.get("rot") or {}
            a.update(mask=MASK_CHUNK, qkv_bias=0, conv=0, qk_norm=QKNORM_HEAD_UNIT, rot_dims=int(rot.get("dims", 0)),
                     rot_base=float(rot.get("base", 0.0)), softcap=float(m.get("softcap", 0.0)), dist_bias_exp=0.0, out_gate=GATE_HEAD)
        else:
            raise Unsupported(f"layer {i}: mixer type {L['type']!r}")
        d = {"mixer": MIX_SOFTMAX_ATTN, "sattn": a, "ff": 0, "ff_kind": FF_RELU2}
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind") == "dense":
                d.update(ff=int(mlp["ff"]), ff_kind=FF_GATED_GELU)
            elif mlp.get("kind") == "moe":
                sh = mlp.get("shared") or {}
                d.update(ff_kind=FF_MOE, moe={"experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
                                              "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": int(sh.get("ff", 0))})
            else:
                raise Unsupported(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    return program, layers


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this config must hold ('.vmix' of the first blending layer is in the file but unused)."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    seen_source = False
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        x = p + "mix."
        nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        out[p + "norm1"] = (W,)
        out.update({x + "q": (nq, W), x + "k": (nk, W), x + "v": (nv, W), x + "o": (W, m["heads"] * m["vdim"])})
        if m.get("v_mix"):
            if seen_source:
                out[x + "vmix"] = ()
            seen_source = True
        if L["type"] == "attention":
            out.update({x + "q.b": (nq,), x + "k.b": (nk,), x + "v.b": (nv,), x + "q.norm": (nq,), x + "k.norm": (nk,)})
            if m.get("conv", 0) > 0:
                out.update({x + "q.conv": (nq, m["conv"]), x + "k.conv": (nk, m["conv"]), x + "v.conv": (nv, m["conv"])})
        else:
            out[x + "g"] = (m["heads"], W)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                out.update({p + "mlp.e%d.up" % e: (ff, W), p + "mlp.e%d.down" % e: (W, ff)})
            if (mlp.get("shared") or {}).get("ff", 0) > 0:
                out.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"])})
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
    # a layer without feed-forward may still carry its second norm; the library applies it when it is there
    extra = {"l%d.norm2" % i for i, L in enumerate(cfg["layers"]) if L.get("mlp") is None} & set(st.names())

    def feeder(upload):
        for name in st.names():
            if name not in want and name not in extra:
                continue
            gg, shape, arr = st.tensor(name)
            if gg is None:
                continue
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
